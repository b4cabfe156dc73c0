// LayerNorm forward / backward with the rows staged through a shared-memory ring.
//
// One persistent CTA per SM.  One thread streams the CTA's rows into a ring of stages with
// untiled bulk-asynchronous copies (cp.async.bulk, completion counted on an mbarrier per stage);
// the consumer warps read the rows from shared memory, so the amount of data in flight per SM is
// the size of the ring (100-200 KB) instead of what the consumers' registers can hold, and the
// load latency is hidden behind the rows that are being worked on.  Results go straight from
// registers to global memory with 128-bit stores.
//
// Stage protocol of the forward kernel (k = how many times the stage has been used before):
//   producer: wait empty[s] for use k-1 (skipped for k = 0), arrive.expect_tx on full[s], copies
//   consumer: wait full[s] with parity k & 1, move the data to registers, arrive on empty[s]
// Every wait is bounded; a wait that gives up raises g_ln_error and the thread stops using the ring.
#pragma once

#include "brk_common.cuh"
#include "brk_ptx.cuh"

namespace brk {

__device__ int g_ln_error = 0;

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
// forward: a stage is one row; consumer warp w takes the CTA's rows w, w + 8, ...
// ------------------------------------------------------------------------------------------
constexpr int LNR_FWD_WARPS = 8;
constexpr int LNR_FWD_THREADS = (LNR_FWD_WARPS + 1) * 32;
constexpr int LNR_FWD_MAX_STAGES = 16;

template <typename T, int NV>
__global__ void __launch_bounds__(LNR_FWD_THREADS, 1)
ln_fwd_ring_kernel(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows, int hidden,
                   float eps, int stages) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nvec = hidden / VN;
    const uint32_t row_bytes = (uint32_t)nvec * 16u;
    unsigned char* ring = smem_raw;
    uint4* s_gamma = reinterpret_cast<uint4*>(ring + (size_t)stages * row_bytes);
    uint4* s_beta = s_gamma + nvec;
    uint64_t* full = reinterpret_cast<uint64_t*>(s_beta + nvec);
    uint64_t* empty = full + stages;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // rows of this CTA: blockIdx.x + j * gridDim.x, j = 0 .. nj-1
    const int64_t nj = rows > (int64_t)blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const bool producer = warp == LNR_FWD_WARPS && lane == 0;

    if (producer) {      // barriers, then the first fill of every stage, before anything else is waited for
        for (int s = 0; s < stages; s++) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::fence_barrier_init();
        for (int64_t j = 0; j < nj && j < stages; j++) {
            ptx::mbar_arrive_expect_tx(&full[j], row_bytes);
            ptx::bulk_load_1d(ring + (size_t)j * row_bytes, x + ((int64_t)blockIdx.x + j * gridDim.x) * hidden, row_bytes, &full[j]);
        }
    }
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        s_gamma[i] = reinterpret_cast<const uint4*>(gamma)[i];
        s_beta[i] = reinterpret_cast<const uint4*>(beta)[i];
    }
    __syncthreads();      // barriers initialised, gamma and beta staged

    if (warp == LNR_FWD_WARPS) {
        if (lane == 0) {
            int s = 0;            // stage of row j; k = how often it has been used before (j = k * stages + s)
            uint32_t k = 1;
            for (int64_t j = stages; j < nj; j++) {
                if (!ptx::mbar_wait(&empty[s], (k - 1) & 1)) {
                    atomicExch(&g_ln_error, 1);
                    break;
                }
                const int64_t row = (int64_t)blockIdx.x + j * gridDim.x;
                ptx::mbar_arrive_expect_tx(&full[s], row_bytes);
                ptx::bulk_load_1d(ring + (size_t)s * row_bytes, x + row * hidden, row_bytes, &full[s]);
                if (++s == stages) {
                    s = 0;
                    k++;
                }
            }
        }
        return;
    }

    const float inv_h = 1.0f / (float)hidden;
    int s = warp % stages;      // stage of row j and how often it has been used before, kept without 64-bit divisions
    uint32_t k = (uint32_t)(warp / stages);
    for (int64_t j = warp; j < nj; j += LNR_FWD_WARPS, s += LNR_FWD_WARPS) {
        while (s >= stages) {
            s -= stages;
            k++;
        }
        bool ok = ptx::mbar_wait(&full[s], k & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) atomicExch(&g_ln_error, 2);
            break;
        }
        const uint4* sp = reinterpret_cast<const uint4*>(ring + (size_t)s * row_bytes);
        Vec<T> xv[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int idx = i * 32 + lane;
            if (idx < nvec) {
                xv[i].unpack(sp[idx]);
            } else {
#pragma unroll
                for (int e = 0; e < VN; e++) xv[i].v[e] = 0.0f;
            }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[s]);      // the row is in registers: the stage may be refilled

        const int64_t row = (int64_t)blockIdx.x + j * gridDim.x;
        T* yr = y + row * hidden;
        // four partial sums each: the additions of one lane do not form a single dependent chain
        float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < NV; i++)
#pragma unroll
            for (int e = 0; e < VN; e++) sm[e & 3] += xv[i].v[e];
        const float mu = warp_sum((sm[0] + sm[1]) + (sm[2] + sm[3])) * inv_h;
        float qs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < NV; i++) {
            if (i * 32 + lane < nvec) {
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    const float d = xv[i].v[e] - mu;
                    qs[e & 3] = fmaf(d, d, qs[e & 3]);
                }
            }
        }
        const float v = warp_sum((qs[0] + qs[1]) + (qs[2] + qs[3])) * inv_h + eps;
        const float rstd = rsqrtf(v);
        const float shift = -mu * rstd;      // xhat = x * rstd + shift
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int idx = i * 32 + lane;
            if (idx < nvec) __stcs(reinterpret_cast<uint4*>(yr + idx * VN), ln_affine_packet<T>(xv[i], rstd, shift, s_gamma[idx], s_beta[idx]));
        }
        if (lane == 0) {
            if (mean) mean[row] = mu;
            if (var) var[row] = v;
        }
    }
}

// Stages that fit next to gamma and beta; 0 = the ring does not fit this row size.
static int lnr_fwd_stages(size_t row_bytes) {
    const size_t budget = 200 * 1024;
    if (row_bytes < 2048 || 2 * row_bytes + 4 * row_bytes > budget) return 0;
    size_t s = (budget - 2 * row_bytes) / row_bytes;
    return (int)(s > LNR_FWD_MAX_STAGES ? LNR_FWD_MAX_STAGES : s);
}

template <typename T, int NV>
static int launch_ln_fwd_ring(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows,
                              int hidden, float eps, cudaStream_t st) {
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const int stages = lnr_fwd_stages(row_bytes);
    const size_t smem = (size_t)(stages + 2) * row_bytes + 2 * (size_t)stages * sizeof(uint64_t);
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ln_fwd_ring_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "ln_fwd_ring smem attribute");
        return BRK_CUDA_ERROR;
    }
    const int64_t cap = sm_count();
    const int grid = (int)(rows < cap ? rows : cap);
    ln_fwd_ring_kernel<T, NV><<<grid, LNR_FWD_THREADS, smem, st>>>(x, gamma, beta, y, mean, var, rows, hidden, eps, stages);
    return launch_status("ln_fwd_ring_kernel");
}

// ------------------------------------------------------------------------------------------
// backward: a stage is R rows of (dy, y); every thread owns NVT 16-byte column groups.
// All threads meet at one barrier per stage (the row sums are block-wide), and at that point every
// thread has moved its part of the stage to registers, so thread 0 refills the stage right there:
// no producer warp and no "empty" barriers are needed.
// ------------------------------------------------------------------------------------------
constexpr int LNR_BWD_MAX_THREADS = 512;
constexpr int LNR_BWD_MAX_STAGES = 6;
constexpr int LNR_BWD_CTAS_PER_SM = 1;      // (two CTAs of 256 threads with twice the columns per thread measured 30 % slower)

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
    static constexpr bool fits = NVT * Vec<T>::N <= 16;      // floats per per-column array in registers
};

template <typename T, int NVT>
__device__ __forceinline__ void lnr_bwd_fill(unsigned char* stage, uint64_t* full, const T* dy, const T* y, int64_t r0,
                                             int64_t rows, int hidden, uint32_t row_bytes) {
    constexpr int R = LnrBwdRows<T, NVT>::R;
    const int valid = (int)(rows - r0 < R ? rows - r0 : R);
    ptx::fence_proxy_async();      // the stage's previous contents were read through the generic proxy
    ptx::mbar_arrive_expect_tx(full, (uint32_t)valid * 2u * row_bytes);
    for (int r = 0; r < valid; r++) {
        ptx::bulk_load_1d(stage + (size_t)(2 * r) * row_bytes, dy + (r0 + r) * hidden, row_bytes, full);
        ptx::bulk_load_1d(stage + (size_t)(2 * r + 1) * row_bytes, y + (r0 + r) * hidden, row_bytes, full);
    }
}

template <typename T, int NVT>
__global__ void __launch_bounds__(LNR_BWD_MAX_THREADS, LNR_BWD_CTAS_PER_SM)
ln_bwd_ring_kernel(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, T* dx, float* partial,
                   int64_t rows, int hidden, float eps, int stages) {
    constexpr int VN = Vec<T>::N;
    constexpr int R = LnrBwdRows<T, NVT>::R;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nvec = hidden / VN;
    const uint32_t row_bytes = (uint32_t)nvec * 16u;
    const size_t stage_bytes = (size_t)R * 2 * row_bytes;
    unsigned char* ring = smem_raw;
    float* red = reinterpret_cast<float*>(ring + (size_t)stages * stage_bytes);      // [2][2R][32]
    uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * 2 * R * 32);
    const int nthreads = (int)blockDim.x;      // a multiple of 32
    const int nwarp = nthreads >> 5;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // row groups of this CTA: group blockIdx.x + j * gridDim.x holds rows group*R .. group*R + R-1
    const int64_t ngroups = (rows + R - 1) / R;
    const int64_t nj = ngroups > (int64_t)blockIdx.x ? (ngroups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (tid == 0) {
        for (int s = 0; s < stages; s++) ptx::mbar_init(&full[s], 1);
        ptx::fence_barrier_init();
        for (int64_t j = 0; j < nj && j < stages; j++)
            lnr_bwd_fill<T, NVT>(ring + (size_t)j * stage_bytes, &full[j], dy, y, ((int64_t)blockIdx.x + j * gridDim.x) * R, rows,
                                 hidden, row_bytes);
    }
    __syncthreads();      // the barriers are initialised before anybody waits on them

    const float inv_h = 1.0f / (float)hidden;
    float gam[NVT][VN], cofs[NVT][VN], ginv[NVT][VN], acc_g[NVT][VN], acc_b[NVT][VN];
    bool own[NVT];
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        const int idx = i * nthreads + tid;
        own[i] = idx < nvec;
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

    // var of the rows two stages ahead is fetched now: a global load issued where it is needed would put its
    // whole latency on the critical path of every stage (all threads meet at a barrier per stage)
    auto load_var = [&](int64_t jj, float (&out)[R]) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t row = ((int64_t)blockIdx.x + jj * gridDim.x) * R + r;
            out[r] = (jj < nj && row < rows) ? __ldg(var + row) : 1.0f;
        }
    };
    float var0[R], var1[R], var2[R];
    load_var(0, var0);
    load_var(1, var1);

    int phase = 0;
    bool dead = false;      // a wait gave up: keep meeting the others at the barrier, without data
    int s = 0;            // stage of group j; k = how often it has been used before
    uint32_t k = 0;
    for (int64_t j = 0; j < nj; j++, phase ^= 1) {
        load_var(j + 2, var2);
        if (!dead) {
            bool ok = ptx::mbar_wait(&full[s], k & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                dead = true;
                if (lane == 0) atomicExch(&g_ln_error, 4);
            }
        }
        const int64_t r0 = ((int64_t)blockIdx.x + j * gridDim.x) * R;
        const uint4* sp = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
        Vec<T> vdy[R][NVT], vy[R][NVT];
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                const int idx = i * nthreads + tid;
                if (own[i] && r0 + r < rows && !dead) {
                    vdy[r][i].unpack(sp[(size_t)(2 * r) * nvec + idx]);
                    vy[r][i].unpack(sp[(size_t)(2 * r + 1) * nvec + idx]);
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
                    // vy becomes xhat; a row past the end has dy = 0 and adds nothing
                    const float xhat = fmaf(vy[r][i].v[e], ginv[i][e], cofs[i][e]);
                    vy[r][i].v[e] = xhat;
                    const float g = vdy[r][i].v[e] * gam[i][e];
                    a += g;
                    b = fmaf(g, xhat, b);
                }
            sums[2 * r] = a;
            sums[2 * r + 1] = b;
        }
        float* rp = red + phase * (2 * R * 32);
        lnr_warp_reduce_store<2 * R>(sums, rp, lane, warp);
        __syncthreads();
        // every thread has its part of stage s in registers: refill it with the group `stages` ahead
        if (tid == 0 && j + stages < nj && !dead)
            lnr_bwd_fill<T, NVT>(ring + (size_t)s * stage_bytes, &full[s], dy, y, ((int64_t)blockIdx.x + (j + stages) * gridDim.x) * R,
                                 rows, hidden, row_bytes);
        lnr_block_totals<2 * R>(sums, rp, lane, nwarp);
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t row = r0 + r;
            if (row >= rows || dead) continue;
            const float mg = sums[2 * r] * inv_h, mgx = sums[2 * r + 1] * inv_h;
            const float rstd = rsqrtf(var0[r]);
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                if (!own[i]) continue;
                const int idx = i * nthreads + tid;
                Vec<T> o;
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    const float d = vdy[r][i].v[e];
                    const float xhat = vy[r][i].v[e];
                    o.v[e] = (d * gam[i][e] - mg - xhat * mgx) * rstd;
                    acc_g[i][e] = fmaf(xhat, d, acc_g[i][e]);
                    acc_b[i][e] += d;
                }
                o.store_stream(dx + row * hidden + idx * VN);
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            var0[r] = var1[r];
            var1[r] = var2[r];
        }
        if (++s == stages) {
            s = 0;
            k++;
        }
    }

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

template <typename T, int NVT>
static int lnr_bwd_stages(size_t row_bytes) {
    const size_t budget = 200 * 1024;
    const size_t stage = (size_t)LnrBwdRows<T, NVT>::R * 2 * row_bytes;
    if (row_bytes < 2048 || 2 * stage > budget) return 0;
    size_t s = budget / stage;
    return (int)(s > LNR_BWD_MAX_STAGES ? LNR_BWD_MAX_STAGES : s);
}

template <typename T, int NVT>
static int lnr_bwd_grid(int64_t rows) {
    constexpr int R = LnrBwdRows<T, NVT>::R;
    const int64_t groups = (rows + R - 1) / R;
    const int64_t cap = (int64_t)sm_count() * LNR_BWD_CTAS_PER_SM;
    return (int)(groups < cap ? groups : cap);
}

// Returns the number of CTAs (= partial rows written) through *grid_out.
template <typename T, int NVT>
static int launch_ln_bwd_ring(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, T* dx, float* partial,
                              int64_t rows, int hidden, float eps, int* grid_out, cudaStream_t st) {
    constexpr int VN = Vec<T>::N;
    constexpr int R = LnrBwdRows<T, NVT>::R;
    const int nvec = hidden / VN;
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const int stages = lnr_bwd_stages<T, NVT>(row_bytes);
    const int threads = ((nvec + NVT - 1) / NVT + 31) / 32 * 32;
    const size_t smem = (size_t)stages * R * 2 * row_bytes + 2 * 2 * R * 32 * sizeof(float) + (size_t)stages * sizeof(uint64_t);
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ln_bwd_ring_kernel<T, NVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "ln_bwd_ring smem attribute");
        return BRK_CUDA_ERROR;
    }
    const int grid = lnr_bwd_grid<T, NVT>(rows);
    *grid_out = grid;
    ln_bwd_ring_kernel<T, NVT><<<grid, threads, smem, st>>>(dy, gamma, beta, var, y, dx, partial, rows, hidden, eps, stages);
    return launch_status("ln_bwd_ring_kernel");
}

}  // namespace brk
