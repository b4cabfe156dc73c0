// LayerNorm forward / backward with the rows prefetched through shared memory.
//
// One persistent CTA per SM.  Every thread copies the 16-byte packets it is going to work on
// itself, several rows ahead, with asynchronous 16-byte copies (cp.async, the load/store-unit
// path) into its own slots of a shared-memory ring, and picks them up with cp.async.wait_group.
// The data in flight per SM is the size of the ring (130-200 KB) instead of what the registers
// can hold, and since a thread only ever reads slots it filled itself the ring needs no barrier
// of its own: nothing in these kernels waits on another thread except the block-wide row sums of
// the backward pass.
//
// (An earlier version filled the ring with untiled bulk copies, cp.async.bulk + mbarrier.  With
// all of a stage's bytes behind one bulk request per row it streamed at most ~17 GB/s per SM from
// DRAM, 2.6 TB/s over the chip, however many stages were in flight; the per-thread 16-byte copies
// keep many more requests outstanding.)
//
// Results go straight from registers to global memory with 128-bit streaming stores.
#pragma once

#include "brk_common.cuh"

namespace brk {

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {      // at most N of this thread's groups still pending
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float ln_guard_gamma(float g, float eps) { return g >= 0.0f ? g + eps : g - eps; }

// One 16-byte packet of y = xhat * gamma + beta with xhat = x * rstd + shift.  fp32 tensors: all in fp32.
// fp16 tensors: xhat in fp32, rounded to half, then one packed half2 fma with gamma and beta as they lie in
// shared memory -- a quarter of the instructions of converting gamma and beta to fp32 for every row, for at
// most one more unit in the last place of the fp16 result.
template <typename T>
__device__ __forceinline__ uint4 ln_affine_packet(const Vec<T>& x, float rstd, float shift, const uint4& gamma, const uint4& beta);

template <>
__device__ __forceinline__ uint4 ln_affine_packet<float>(const Vec<float>& x, float rstd, float shift, const uint4& gamma,
                                                         const uint4& beta) {
    Vec<float> g, b, o;
    g.unpack(gamma);
    b.unpack(beta);
#pragma unroll
    for (int e = 0; e < 4; e++) o.v[e] = fmaf(fmaf(x.v[e], rstd, shift), g.v[e], b.v[e]);
    return o.pack();
}

template <>
__device__ __forceinline__ uint4 ln_affine_packet<__half>(const Vec<__half>& x, float rstd, float shift, const uint4& gamma,
                                                          const uint4& beta) {
    uint4 out;
    const __half2* g = reinterpret_cast<const __half2*>(&gamma);
    const __half2* b = reinterpret_cast<const __half2*>(&beta);
    __half2* o = reinterpret_cast<__half2*>(&out);
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const __half2 xh = __floats2half2_rn(fmaf(x.v[2 * e], rstd, shift), fmaf(x.v[2 * e + 1], rstd, shift));
        o[e] = __hfma2(xh, g[e], b[e]);
    }
    return out;
}

// ------------------------------------------------------------------------------------------
// forward: a team of WPR warps per row (each lane holds NV packets of it); every team owns DEPTH row
// slots and keeps DEPTH rows in flight.  With WPR = 2 the two warps of a team exchange their partial
// sums through shared memory around a 64-thread named barrier; twice the warps per SM at half the
// registers each keep the instruction issue busier than one warp per row does.
// ------------------------------------------------------------------------------------------
constexpr int LNR_FWD_TEAMS = 8;      // rows in work per CTA

template <int WPR>
__device__ __forceinline__ float lnr_team_sum(float v, float* xch, int team, int member, int lane, int slot) {
    v = warp_sum(v);
    if (WPR == 1) return v;
    // xch[slot][team][member]; the slot alternates between the two sums of a row, so a value is never
    // overwritten before the partner has read it (see the barrier order in the kernel)
    float* mine = xch + (slot * LNR_FWD_TEAMS + team) * WPR;
    if (lane == 0) mine[member] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(32 * WPR) : "memory");
    float t = 0.0f;
#pragma unroll
    for (int m = 0; m < WPR; m++) t += mine[m];      // same order in every member: identical totals
    return t;
}

template <typename T, int NV, int DEPTH, int WPR>
__global__ void __launch_bounds__(LNR_FWD_TEAMS * WPR * 32, 1)
ln_fwd_ring_kernel(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows, int hidden,
                   float eps) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float xch[2 * LNR_FWD_TEAMS * WPR];
    const int nvec = hidden / VN;
    const size_t row_bytes = (size_t)nvec * 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int team = warp / WPR, member = warp % WPR;
    pdl_wait();
    uint4* s_gamma = reinterpret_cast<uint4*>(smem_raw);
    uint4* s_beta = s_gamma + nvec;
    unsigned char* my_ring = smem_raw + 2 * row_bytes + (size_t)team * DEPTH * row_bytes;      // this team's DEPTH row slots

    // rows of this team: first + n * step, n = 0 .. nrows-1 (rows interleaved over all teams of the grid)
    const int64_t first = (int64_t)blockIdx.x * LNR_FWD_TEAMS + team;
    const int64_t step = (int64_t)gridDim.x * LNR_FWD_TEAMS;
    const int64_t nrows = rows > first ? (rows - first + step - 1) / step : 0;
    // packets of this lane: (i * WPR + member) * 32 + lane, i = 0 .. NV-1

    auto prefetch = [&](int64_t n, int slot) {      // one commit group per call, empty past the end
        if (n < nrows) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (first + n * step) * hidden);
            uint4* dst = reinterpret_cast<uint4*>(my_ring + (size_t)slot * row_bytes);
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int idx = (i * WPR + member) * 32 + lane;
                if (idx < nvec) cp_async_16(dst + idx, src + idx);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int d = 0; d < DEPTH; d++) prefetch(d, d);

    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        s_gamma[i] = reinterpret_cast<const uint4*>(gamma)[i];
        s_beta[i] = reinterpret_cast<const uint4*>(beta)[i];
    }
    __syncthreads();

    const float inv_h = 1.0f / (float)hidden;
    int slot = 0;
    for (int64_t n = 0; n < nrows; n++) {
        cp_async_wait<DEPTH - 1>();      // row n has landed (each lane waits for, and then reads, its own packets)
        const uint4* sp = reinterpret_cast<const uint4*>(my_ring + (size_t)slot * row_bytes);
        Vec<T> xv[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int idx = (i * WPR + member) * 32 + lane;
            if (idx < nvec) {
                xv[i].unpack(sp[idx]);
            } else {
#pragma unroll
                for (int e = 0; e < VN; e++) xv[i].v[e] = 0.0f;
            }
        }
        const int64_t row = first + n * step;
        T* yr = y + row * hidden;
        // four partial sums each: the additions of one lane do not form a single dependent chain
        float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < NV; i++)
#pragma unroll
            for (int e = 0; e < VN; e++) sm[e & 3] += xv[i].v[e];
        const float mu = lnr_team_sum<WPR>((sm[0] + sm[1]) + (sm[2] + sm[3]), xch, team, member, lane, 0) * inv_h;
        // every packet of the slot has been read and used by now: refill it with the row DEPTH ahead
        prefetch(n + DEPTH, slot);
        if (++slot == DEPTH) slot = 0;
        float qs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < NV; i++) {
            if ((i * WPR + member) * 32 + lane < nvec) {
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    const float d = xv[i].v[e] - mu;
                    qs[e & 3] = fmaf(d, d, qs[e & 3]);
                }
            }
        }
        const float v = lnr_team_sum<WPR>((qs[0] + qs[1]) + (qs[2] + qs[3]), xch, team, member, lane, 1) * inv_h + eps;
        const float rstd = rsqrtf(v);
        const float shift = -mu * rstd;      // xhat = x * rstd + shift
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int idx = (i * WPR + member) * 32 + lane;
            if (idx < nvec) __stcs(reinterpret_cast<uint4*>(yr + idx * VN), ln_affine_packet<T>(xv[i], rstd, shift, s_gamma[idx], s_beta[idx]));
        }
        if (lane == 0 && member == 0) {
            if (mean) mean[row] = mu;
            if (var) var[row] = v;
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
}

// Row slots per team that fit next to gamma and beta: 3, 2 or 0 (= rows too large or too small for this kernel).
static int lnr_fwd_depth(size_t row_bytes) {
    const size_t budget = 208 * 1024;
    if (row_bytes < 2048) return 0;
    if ((2 + 3 * LNR_FWD_TEAMS) * row_bytes <= budget) return 3;
    if ((2 + 2 * LNR_FWD_TEAMS) * row_bytes <= budget) return 2;
    return 0;
}

template <typename T, int NV, int DEPTH, int WPR>
static int launch_ln_fwd_ring_d(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows,
                                int hidden, float eps, cudaStream_t st) {
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const size_t smem = (2 + (size_t)DEPTH * LNR_FWD_TEAMS) * row_bytes;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ln_fwd_ring_kernel<T, NV, DEPTH, WPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "ln_fwd_ring smem attribute");
        return BRK_CUDA_ERROR;
    }
    const int64_t want = (rows + LNR_FWD_TEAMS - 1) / LNR_FWD_TEAMS;
    const int64_t cap = sm_count();
    const int grid = (int)(want < cap ? want : cap);
    cudaError_t le = launch_pdl(ln_fwd_ring_kernel<T, NV, DEPTH, WPR>, grid, LNR_FWD_TEAMS * WPR * 32, smem, st, x, gamma, beta, y, mean,
                                var, rows, hidden, eps);
    if (le != cudaSuccess) {
        set_cuda_error(le, "ln_fwd_ring_kernel");
        return BRK_CUDA_ERROR;
    }
    return launch_status("ln_fwd_ring_kernel");
}

// NV = 16-byte packets per lane with one warp per row; rows of 8 and more packets per lane are shared by two warps.
template <typename T, int NV>
static int launch_ln_fwd_ring(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows,
                              int hidden, float eps, cudaStream_t st) {
    constexpr int WPR = NV >= 8 ? 2 : 1;
    if (lnr_fwd_depth((size_t)hidden * sizeof(T)) == 3)
        return launch_ln_fwd_ring_d<T, NV / WPR, 3, WPR>(x, gamma, beta, y, mean, var, rows, hidden, eps, st);
    return launch_ln_fwd_ring_d<T, NV / WPR, 2, WPR>(x, gamma, beta, y, mean, var, rows, hidden, eps, st);
}

// ------------------------------------------------------------------------------------------
// backward: every thread owns NVT 16-byte column groups of every row; a stage is R rows of (dy, y).
// All threads meet at one barrier per stage for the block-wide row sums.
// ------------------------------------------------------------------------------------------
constexpr int LNR_BWD_MAX_THREADS = 512;      // (two CTAs of 256 threads with twice the columns per thread measured 30 % slower)

// Block-wide sums of Q values per thread in two steps around one barrier.
// Step 1 (before the barrier): every warp reduces its Q values and stores them at rp[q * 32 + warp].
// Step 2 (after the barrier): every thread gets the Q block totals in v[].
// For Q = 4 the values share their shuffles: after exchanging halves twice each lane carries one value,
// so a warp needs 6 shuffles instead of 20, and the second step reduces two values per lane over 16 lanes
// (at most 16 warps) and broadcasts, 12 shuffles instead of 20.
template <int Q>
__device__ __forceinline__ void lnr_warp_reduce_store(const float (&v)[Q], float* rp, int lane, int warp) {
#pragma unroll
    for (int q = 0; q < Q; q++) {
        const float w = warp_sum(v[q]);
        if (lane == 0) rp[q * 32 + warp] = w;
    }
}
template <>
__device__ __forceinline__ void lnr_warp_reduce_store<4>(const float (&v)[4], float* rp, int lane, int warp) {
    const bool hi16 = (lane & 16) != 0;
    // lanes 0-15 go on with (v0, v1), lanes 16-31 with (v2, v3)
    float a = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
    float b = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
    const bool hi8 = (lane & 8) != 0;
    // of those, lanes with bit 3 clear go on with the first, the others with the second
    float c = (hi8 ? b : a) + __shfl_xor_sync(0xffffffffu, hi8 ? a : b, 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    // lane 0 holds v0, lane 8 v1, lane 16 v2, lane 24 v3
    if ((lane & 7) == 0) rp[(lane >> 3) * 32 + warp] = c;
}

template <int Q>
__device__ __forceinline__ void lnr_block_totals(float (&v)[Q], const float* rp, int lane, int nwarp) {
#pragma unroll
    for (int q = 0; q < Q; q++) {
        const float t = lane < nwarp ? rp[q * 32 + lane] : 0.0f;
        v[q] = warp_sum(t);
    }
}
template <>
__device__ __forceinline__ void lnr_block_totals<4>(float (&v)[4], const float* rp, int lane, int nwarp) {
    if (nwarp > 16) {      // not reached with at most 512 threads; kept correct for any block size
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float t = lane < nwarp ? rp[q * 32 + lane] : 0.0f;
            v[q] = warp_sum(t);
        }
        return;
    }
    const int w = lane & 15, half = lane >> 4;
    float a = w < nwarp ? rp[half * 32 + w] : 0.0f;            // value 0 (lanes 0-15) / value 1 (lanes 16-31)
    float b = w < nwarp ? rp[(2 + half) * 32 + w] : 0.0f;      // value 2 / value 3
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    v[0] = __shfl_sync(0xffffffffu, a, 0);
    v[1] = __shfl_sync(0xffffffffu, a, 16);
    v[2] = __shfl_sync(0xffffffffu, b, 0);
    v[3] = __shfl_sync(0xffffffffu, b, 16);
}

template <typename T, int NVT>
struct LnrBwdRows {      // rows per stage: two while a thread's columns fit 8 floats per array, else one
    static constexpr int R = (NVT * Vec<T>::N <= 8) ? 2 : 1;
};

template <typename T, int NVT, int DEPTH>
__global__ void __launch_bounds__(LNR_BWD_MAX_THREADS, 1)
ln_bwd_ring_kernel(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, const T* res, T* dx, float* partial,
                   int64_t rows, int hidden, float eps) {
    constexpr int VN = Vec<T>::N;
    constexpr int R = LnrBwdRows<T, NVT>::R;
    constexpr int RED = (2 * R + 1) * 32;      // per phase: 2R row sums x 32 warps, then rstd of the R rows
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nvec = hidden / VN;
    const size_t row_bytes = (size_t)nvec * 16;
    const size_t stage_bytes = (size_t)R * 2 * row_bytes;      // [R][dy, y][nvec packets]
    unsigned char* ring = smem_raw;
    float* red = reinterpret_cast<float*>(ring + (size_t)DEPTH * stage_bytes);      // [2][RED]
    const int nthreads = (int)blockDim.x;      // a multiple of 32
    const int nwarp = nthreads >> 5;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();

    // Row groups of this CTA: group blockIdx.x + j * gridDim.x holds rows group*R .. group*R + R-1.  Everything that
    // walks over the groups (first row, byte offsets) is advanced by a constant per step instead of recomputed.
    const int64_t stride_rows = (int64_t)gridDim.x * R;
    const size_t stride_bytes = (size_t)stride_rows * row_bytes;
    const int64_t first_row = (int64_t)blockIdx.x * R;

    bool own[NVT];
    uint32_t off[NVT];      // byte offset of this thread's packets inside a row
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        own[i] = i * nthreads + tid < nvec;
        off[i] = (uint32_t)(i * nthreads + tid) * 16u;
    }

    // prefetch cursor: first row / source addresses of the next group to copy
    int64_t pf_row = first_row;
    const unsigned char* pf_dy = reinterpret_cast<const unsigned char*>(dy) + (size_t)first_row * row_bytes;
    const unsigned char* pf_y = reinterpret_cast<const unsigned char*>(y) + (size_t)first_row * row_bytes;
    auto prefetch = [&](int stage) {      // this thread's packets of the next group; one commit group per call, empty past the end
        unsigned char* dst = ring + (size_t)stage * stage_bytes;
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (pf_row + r < rows) {
#pragma unroll
                for (int i = 0; i < NVT; i++) {
                    if (own[i]) {
                        cp_async_16(dst + (size_t)(2 * r) * row_bytes + off[i], pf_dy + (size_t)r * row_bytes + off[i]);
                        cp_async_16(dst + (size_t)(2 * r + 1) * row_bytes + off[i], pf_y + (size_t)r * row_bytes + off[i]);
                    }
                }
            }
        }
        cp_async_commit();
        pf_row += stride_rows;
        pf_dy += stride_bytes;
        pf_y += stride_bytes;
    };
#pragma unroll
    for (int d = 0; d < DEPTH; d++) prefetch(d);

    const float inv_h = 1.0f / (float)hidden;
    float gam[NVT][VN], cofs[NVT][VN], ginv[NVT][VN], acc_g[NVT][VN], acc_b[NVT][VN];
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        const int idx = i * nthreads + tid;
        Vec<T> g, b;
        if (own[i]) {
            g.load(gamma + idx * VN);
            b.load(beta + idx * VN);
        }
#pragma unroll
        for (int e = 0; e < VN; e++) {
            gam[i][e] = own[i] ? g.v[e] : 0.0f;
            ginv[i][e] = own[i] ? 1.0f / ln_guard_gamma(g.v[e], eps) : 0.0f;
            cofs[i][e] = own[i] ? -b.v[e] * ginv[i][e] : 0.0f;      // xhat = y * ginv + cofs
            acc_g[i][e] = 0.0f;
            acc_b[i][e] = 0.0f;
        }
    }

    // Threads 0 .. R-1 look after var: thread r fetches var of row r of the group two steps ahead (a load issued where
    // the value is needed would put its whole latency on the critical path of every step, since all threads meet at a
    // barrier per step) and hands rsqrt(var) to the block through shared memory together with the row sums.
    const bool var_thread = tid < R;
    const float* var_ptr = var + first_row + tid;      // row of this thread in the current group
    auto load_var = [&](int ahead) {
        return (var_thread && first_row + tid + (int64_t)ahead * stride_rows < rows) ? __ldg(var_ptr + (int64_t)ahead * stride_rows) : 1.0f;
    };
    float var0 = load_var(0), var1 = load_var(1);
    int64_t rows_left = rows - first_row;      // rows from the current group's first row to the end

    int phase = 0, stage = 0;
    unsigned char* dx_row = reinterpret_cast<unsigned char*>(dx) + (size_t)first_row * row_bytes;
    // optional residual added to dx (res may be dx itself: a thread reads exactly the packets it writes, before it writes)
    const unsigned char* res_row = res ? reinterpret_cast<const unsigned char*>(res) + (size_t)first_row * row_bytes : nullptr;
    for (; rows_left > 0; rows_left -= stride_rows, dx_row += stride_bytes, var_ptr += stride_rows, phase ^= 1) {
        const float var2 = (var_thread && rows_left - tid > 2 * stride_rows) ? __ldg(var_ptr + 2 * stride_rows) : 1.0f;
        cp_async_wait<DEPTH - 1>();      // the current group has landed (this thread's own packets)
        const unsigned char* sp = ring + (size_t)stage * stage_bytes;
        Vec<T> vdy[R][NVT], vy[R][NVT];
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                if (own[i] && r < rows_left) {
                    vdy[r][i].unpack(*reinterpret_cast<const uint4*>(sp + (size_t)(2 * r) * row_bytes + off[i]));
                    vy[r][i].unpack(*reinterpret_cast<const uint4*>(sp + (size_t)(2 * r + 1) * row_bytes + off[i]));
                } else {
#pragma unroll
                    for (int e = 0; e < VN; e++) {
                        vdy[r][i].v[e] = 0.0f;
                        vy[r][i].v[e] = 0.0f;
                    }
                }
            }
        }

        float sums[2 * R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            float a = 0.0f, b = 0.0f;
#pragma unroll
            for (int i = 0; i < NVT; i++)
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    // vy becomes xhat and vdy becomes dy * gamma; a row past the end has dy = 0 and adds nothing.  The
                    // column sums do not depend on the row sums, so they are taken here, before the barrier.
                    const float xhat = fmaf(vy[r][i].v[e], ginv[i][e], cofs[i][e]);
                    const float d = vdy[r][i].v[e];
                    const float g = d * gam[i][e];
                    vy[r][i].v[e] = xhat;
                    vdy[r][i].v[e] = g;
                    a += g;
                    b = fmaf(g, xhat, b);
                    acc_g[i][e] = fmaf(xhat, d, acc_g[i][e]);
                    acc_b[i][e] += d;
                }
            sums[2 * r] = a;
            sums[2 * r + 1] = b;
        }
        // the residual packets are fetched here so that their latency passes behind the block-wide sums
        uint4 vres[R][NVT];
        if (res_row) {
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int i = 0; i < NVT; i++)
                    vres[r][i] = (own[i] && r < rows_left) ? __ldcs(reinterpret_cast<const uint4*>(res_row + (size_t)r * row_bytes + off[i]))
                                                           : make_uint4(0u, 0u, 0u, 0u);
        }
        // this thread's packets of the stage have been read and used by now: refill them with the group DEPTH ahead
        prefetch(stage);
        if (++stage == DEPTH) stage = 0;
        float* rp = red + phase * RED;
        lnr_warp_reduce_store<2 * R>(sums, rp, lane, warp);
        if (var_thread) rp[2 * R * 32 + tid] = rsqrtf(var0);
        __syncthreads();
        lnr_block_totals<2 * R>(sums, rp, lane, nwarp);
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r >= rows_left) continue;
            // dx = (g - mean(g) - xhat * mean(g * xhat)) * rstd = g * rstd + (xhat * c2 + c1)
            const float rstd = rp[2 * R * 32 + r];
            const float c1 = -sums[2 * r] * inv_h * rstd, c2 = -sums[2 * r + 1] * inv_h * rstd;
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                if (!own[i]) continue;
                Vec<T> o;
#pragma unroll
                for (int e = 0; e < VN; e++) o.v[e] = fmaf(vdy[r][i].v[e], rstd, fmaf(vy[r][i].v[e], c2, c1));
                if (res_row) {
                    Vec<T> a;
                    a.unpack(vres[r][i]);
#pragma unroll
                    for (int e = 0; e < VN; e++) o.v[e] += a.v[e];
                }
                __stcs(reinterpret_cast<uint4*>(dx_row + (size_t)r * row_bytes + off[i]), o.pack());
            }
        }
        if (res_row) res_row += stride_bytes;
        var0 = var1;
        var1 = var2;
    }
    cp_async_wait<0>();
    // the kernel that adds up the partial rows may start its launch now; it waits for this grid to finish before it reads
    pdl_launch_dependents();

    float* pg = partial + (size_t)blockIdx.x * 2 * hidden;
    float* pb = pg + hidden;
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        if (!own[i]) continue;
        const int idx = i * nthreads + tid;
#pragma unroll
        for (int e = 0; e < VN; e += 4) {
            *reinterpret_cast<float4*>(pg + idx * VN + e) = make_float4(acc_g[i][e], acc_g[i][e + 1], acc_g[i][e + 2], acc_g[i][e + 3]);
            *reinterpret_cast<float4*>(pb + idx * VN + e) = make_float4(acc_b[i][e], acc_b[i][e + 1], acc_b[i][e + 2], acc_b[i][e + 3]);
        }
    }
}

// Stages in flight: 6, 3 or 0 (= rows too large or too small for this kernel).
template <typename T, int NVT>
static int lnr_bwd_depth(size_t row_bytes) {
    const size_t budget = 200 * 1024;
    const size_t stage = (size_t)LnrBwdRows<T, NVT>::R * 2 * row_bytes;
    if (row_bytes < 2048) return 0;
    if (6 * stage <= budget) return 6;
    if (3 * stage <= budget) return 3;
    return 0;
}

template <typename T, int NVT>
static int lnr_bwd_grid(int64_t rows) {
    constexpr int R = LnrBwdRows<T, NVT>::R;
    const int64_t groups = (rows + R - 1) / R;
    const int64_t cap = sm_count();
    return (int)(groups < cap ? groups : cap);
}

template <typename T, int NVT, int DEPTH>
static int launch_ln_bwd_ring_d(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, const T* res, T* dx, float* partial,
                                int64_t rows, int hidden, float eps, int grid, cudaStream_t st) {
    constexpr int VN = Vec<T>::N;
    constexpr int R = LnrBwdRows<T, NVT>::R;
    const int nvec = hidden / VN;
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const int threads = ((nvec + NVT - 1) / NVT + 31) / 32 * 32;
    const size_t smem = (size_t)DEPTH * R * 2 * row_bytes + 2 * (2 * R + 1) * 32 * sizeof(float);
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ln_bwd_ring_kernel<T, NVT, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "ln_bwd_ring smem attribute");
        return BRK_CUDA_ERROR;
    }
    cudaError_t le = launch_pdl(ln_bwd_ring_kernel<T, NVT, DEPTH>, grid, threads, smem, st, dy, gamma, beta, var, y, res, dx, partial, rows,
                                hidden, eps);
    if (le != cudaSuccess) {
        set_cuda_error(le, "ln_bwd_ring_kernel");
        return BRK_CUDA_ERROR;
    }
    return launch_status("ln_bwd_ring_kernel");
}

// Returns the number of CTAs (= partial rows written) through *grid_out.
template <typename T, int NVT>
static int launch_ln_bwd_ring(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, const T* res, T* dx, float* partial,
                              int64_t rows, int hidden, float eps, int* grid_out, cudaStream_t st) {
    const int grid = lnr_bwd_grid<T, NVT>(rows);
    *grid_out = grid;
    if (lnr_bwd_depth<T, NVT>((size_t)hidden * sizeof(T)) == 6)
        return launch_ln_bwd_ring_d<T, NVT, 6>(dy, gamma, beta, var, y, res, dx, partial, rows, hidden, eps, grid, st);
    return launch_ln_bwd_ring_d<T, NVT, 3>(dy, gamma, beta, var, y, res, dx, partial, rows, hidden, eps, grid, st);
}

}  // namespace brk
