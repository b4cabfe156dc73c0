// LayerNorm forward / backward for sm_100a.  HBM-bound: every activation byte is read once and
// written once with 128-bit accesses.
//
// Forward: one warp per token row.  The row lives in registers (NV 16-byte packets per lane),
// mean and variance come from two register passes (no E[x^2]-mean^2 cancellation), gamma/beta
// are staged once per CTA in shared memory and the CTAs are persistent over rows.
//
// Backward: each thread of a CTA owns a fixed set of columns, CTAs stride over rows (R rows per
// step so one barrier serves several rows).  Per row the two row sums are block-reduced through
// shared memory, dx is written, and the thread adds its columns' dgamma/dbeta terms into
// registers.  At the end every CTA writes one partial row to the workspace and a second kernel
// reduces the partials in a fixed order (deterministic, no atomics).
#include <mutex>
#include <string>

#include "brk_common.cuh"
#include "layernorm_ring.cuh"

namespace brk {

// 0: kernels that prefetch the rows through shared memory where the row size allows them; 1: register-resident kernels only
static int g_ln_mode = 0;

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
constexpr int LN_FWD_WARPS = 4;

template <typename T, int NV>
__global__ void __launch_bounds__(LN_FWD_WARPS * 32)
ln_fwd_kernel(const T* x, const T* gamma, const T* beta, T* y,
              float* mean, float* var, int64_t rows, int hidden, float eps) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    T* s_gamma = reinterpret_cast<T*>(smem_raw);
    T* s_beta = s_gamma + hidden;
    const int nvec = hidden / VN;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        reinterpret_cast<uint4*>(s_gamma)[i] = reinterpret_cast<const uint4*>(gamma)[i];
        reinterpret_cast<uint4*>(s_beta)[i] = reinterpret_cast<const uint4*>(beta)[i];
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float inv_h = 1.0f / (float)hidden;
    for (int64_t row = (int64_t)blockIdx.x * LN_FWD_WARPS + warp; row < rows; row += (int64_t)gridDim.x * LN_FWD_WARPS) {
        const T* xr = x + row * hidden;
        T* yr = y + row * hidden;
        Vec<T> xv[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int idx = i * 32 + lane;
            if (idx < nvec) {
                xv[i].load_stream(xr + idx * VN);
            } else {
#pragma unroll
                for (int e = 0; e < VN; e++) xv[i].v[e] = 0.0f;
            }
        }
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++)
#pragma unroll
            for (int e = 0; e < VN; e++) s += xv[i].v[e];
        const float mu = warp_sum(s) * inv_h;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            if (i * 32 + lane < nvec) {
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    float d = xv[i].v[e] - mu;
                    q += d * d;
                }
            }
        }
        const float v = warp_sum(q) * inv_h + eps;
        const float rstd = rsqrtf(v);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int idx = i * 32 + lane;
            if (idx < nvec) {
                Vec<T> g, b, o;
                g.load(s_gamma + idx * VN);
                b.load(s_beta + idx * VN);
#pragma unroll
                for (int e = 0; e < VN; e++) o.v[e] = (xv[i].v[e] - mu) * rstd * g.v[e] + b.v[e];
                o.store_stream(yr + idx * VN);
            }
        }
        if (lane == 0) {
            if (mean) mean[row] = mu;
            if (var) var[row] = v;
        }
    }
}

// Any hidden size / alignment: one CTA per row, scalar accesses.
template <typename T>
__global__ void __launch_bounds__(256)
ln_fwd_generic_kernel(const T* x, const T* gamma, const T* beta, T* y,
                      float* mean, float* var, int64_t rows, int hidden, float eps) {
    __shared__ float red[64];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * hidden;
    T* yr = y + row * hidden;
    float s = 0.0f, z = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += to_f32(xr[i]);
    block_sum2(s, z, red);
    const float mu = s / (float)hidden;
    float q = 0.0f;
    z = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float d = to_f32(xr[i]) - mu;
        q += d * d;
    }
    block_sum2(q, z, red);
    const float v = q / (float)hidden + eps;
    const float rstd = rsqrtf(v);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        yr[i] = from_f32<T>((to_f32(xr[i]) - mu) * rstd * to_f32(gamma[i]) + to_f32(beta[i]));
    if (threadIdx.x == 0) {
        if (mean) mean[row] = mu;
        if (var) var[row] = v;
    }
}

template <typename T, int NV>
static int launch_ln_fwd(const T* x, const T* gamma, const T* beta, T* y, float* mean, float* var, int64_t rows,
                         int hidden, float eps, cudaStream_t st) {
    size_t smem = 2 * (size_t)hidden * sizeof(T);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(ln_fwd_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_cuda_error(e, "ln_fwd smem attribute");
            return BRK_CUDA_ERROR;
        }
    }
    int64_t want = (rows + LN_FWD_WARPS - 1) / LN_FWD_WARPS;
    int64_t cap = (int64_t)sm_count() * 8;
    int grid = (int)(want < cap ? want : cap);
    ln_fwd_kernel<T, NV><<<grid, LN_FWD_WARPS * 32, smem, st>>>(x, gamma, beta, y, mean, var, rows, hidden, eps);
    return launch_status("ln_fwd_kernel");
}

template <typename T>
static int ln_fwd_dispatch(const void* x_, const void* gamma_, const void* beta_, void* y_, float* mean, float* var,
                           int64_t rows, int64_t hidden, float eps, cudaStream_t st) {
    const T* x = (const T*)x_;
    const T* gamma = (const T*)gamma_;
    const T* beta = (const T*)beta_;
    T* y = (T*)y_;
    constexpr int VN = Vec<T>::N;
    bool fast = (hidden % VN == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta) &&
                hidden / VN <= 32 * 32 && 2 * hidden * sizeof(T) <= 200 * 1024;
    if (fast) {
        int nv = (int)((hidden / VN + 31) / 32);
        int h = (int)hidden;
        if (g_ln_mode == 0 && nv >= 4 && nv * VN <= 128 && lnr_fwd_depth((size_t)hidden * sizeof(T)) > 0) {
            if (nv <= 4) return launch_ln_fwd_ring<T, 4>(x, gamma, beta, y, mean, var, rows, h, eps, st);
            if (nv <= 8) return launch_ln_fwd_ring<T, 8>(x, gamma, beta, y, mean, var, rows, h, eps, st);
            if (nv <= 16) return launch_ln_fwd_ring<T, 16>(x, gamma, beta, y, mean, var, rows, h, eps, st);
            // 17 .. 32 packets per lane fit the registers only for fp32 (nv * VN <= 128 above): fp16 never gets here
            return launch_ln_fwd_ring<T, (VN == 4 ? 32 : 16)>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        }
        if (nv <= 1) return launch_ln_fwd<T, 1>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        if (nv <= 2) return launch_ln_fwd<T, 2>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        if (nv <= 4) return launch_ln_fwd<T, 4>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        if (nv <= 8) return launch_ln_fwd<T, 8>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        if (nv <= 16) return launch_ln_fwd<T, 16>(x, gamma, beta, y, mean, var, rows, h, eps, st);
        return launch_ln_fwd<T, 32>(x, gamma, beta, y, mean, var, rows, h, eps, st);
    }
    ln_fwd_generic_kernel<T><<<(unsigned)rows, 256, 0, st>>>(x, gamma, beta, y, mean, var, rows, (int)hidden, eps);
    return launch_status("ln_fwd_generic_kernel");
}

// ------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------
constexpr int LN_BWD_R = 2;  // rows per step

__device__ __forceinline__ float guard_gamma(float g, float eps) { return g >= 0.0f ? g + eps : g - eps; }

// NVT = 16-byte packets (column groups) owned by one thread.
template <typename T, int NVT>
__global__ void __launch_bounds__(512)
ln_bwd_kernel(const T* dy, const T* gamma, const T* beta,
              const float* var, const T* y, const T* res, T* dx,
              float* partial, int64_t rows, int hidden, float eps) {
    constexpr int VN = Vec<T>::N;
    constexpr int R = LN_BWD_R;
    __shared__ float red[2][2 * R][32];
    const int nvec = hidden / VN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float inv_h = 1.0f / (float)hidden;

    float gam[NVT][VN], bet[NVT][VN], ginv[NVT][VN], acc_g[NVT][VN], acc_b[NVT][VN];
    bool own[NVT];
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        int idx = i * blockDim.x + threadIdx.x;
        own[i] = idx < nvec;
        Vec<T> g, b;
        if (own[i]) {
            g.load(gamma + idx * VN);
            b.load(beta + idx * VN);
        }
#pragma unroll
        for (int e = 0; e < VN; e++) {
            gam[i][e] = own[i] ? g.v[e] : 0.0f;
            bet[i][e] = own[i] ? b.v[e] : 0.0f;
            ginv[i][e] = own[i] ? 1.0f / guard_gamma(g.v[e], eps) : 0.0f;
            acc_g[i][e] = 0.0f;
            acc_b[i][e] = 0.0f;
        }
    }

    int phase = 0;
    for (int64_t r0 = (int64_t)blockIdx.x * R; r0 < rows; r0 += (int64_t)gridDim.x * R, phase ^= 1) {
        Vec<T> vdy[R][NVT], vy[R][NVT];
        float sums[2 * R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t row = r0 + r;
            sums[2 * r] = 0.0f;
            sums[2 * r + 1] = 0.0f;
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                int idx = i * blockDim.x + threadIdx.x;
                if (own[i] && row < rows) {
                    vdy[r][i].load_stream(dy + row * hidden + idx * VN);
                    vy[r][i].load_stream(y + row * hidden + idx * VN);
                } else {
#pragma unroll
                    for (int e = 0; e < VN; e++) {
                        vdy[r][i].v[e] = 0.0f;
                        vy[r][i].v[e] = 0.0f;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int i = 0; i < NVT; i++)
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    // vy becomes xhat; columns this thread does not own contribute 0
                    float xhat = (vy[r][i].v[e] - bet[i][e]) * ginv[i][e];
                    vy[r][i].v[e] = xhat;
                    float g = vdy[r][i].v[e] * gam[i][e];
                    sums[2 * r] += g;
                    sums[2 * r + 1] += g * xhat;
                }
#pragma unroll
        for (int k = 0; k < 2 * R; k++) {
            float w = warp_sum(sums[k]);
            if (lane == 0) red[phase][k][warp] = w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 2 * R; k++) {
            float t = lane < nwarp ? red[phase][k][lane] : 0.0f;
            sums[k] = warp_sum(t);
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t row = r0 + r;
            if (row >= rows) continue;
            const float mg = sums[2 * r] * inv_h, mgx = sums[2 * r + 1] * inv_h;
            const float rstd = rsqrtf(var[row]);
#pragma unroll
            for (int i = 0; i < NVT; i++) {
                if (!own[i]) continue;
                int idx = i * blockDim.x + threadIdx.x;
                Vec<T> o;
#pragma unroll
                for (int e = 0; e < VN; e++) {
                    float d = vdy[r][i].v[e];
                    float xhat = vy[r][i].v[e];
                    o.v[e] = (d * gam[i][e] - mg - xhat * mgx) * rstd;
                    acc_g[i][e] += xhat * d;
                    acc_b[i][e] += d;
                }
                if (res) {      // res may be dx: this thread reads the packet it is about to write
                    Vec<T> a;
                    a.load_stream(res + row * hidden + idx * VN);
#pragma unroll
                    for (int e = 0; e < VN; e++) o.v[e] += a.v[e];
                }
                o.store_stream(dx + row * hidden + idx * VN);
            }
        }
    }
    float* pg = partial + (size_t)blockIdx.x * 2 * hidden;
    float* pb = pg + hidden;
#pragma unroll
    for (int i = 0; i < NVT; i++) {
        if (!own[i]) continue;
        int idx = i * blockDim.x + threadIdx.x;
#pragma unroll
        for (int e = 0; e < VN; e += 4) {
            *reinterpret_cast<float4*>(pg + idx * VN + e) = make_float4(acc_g[i][e], acc_g[i][e + 1], acc_g[i][e + 2], acc_g[i][e + 3]);
            *reinterpret_cast<float4*>(pb + idx * VN + e) = make_float4(acc_b[i][e], acc_b[i][e + 1], acc_b[i][e + 2], acc_b[i][e + 3]);
        }
    }
}

// out[j] = sum_p partial[p][j], j over 2*hidden (dgamma then dbeta).  32 columns x 16 partial lanes per CTA; each
// lane adds every 16th partial into four interleaved accumulators (independent loads in flight), and the lanes
// are combined in a fixed order (deterministic).
constexpr int LN_RED_LANES = 16;

template <typename T>
__global__ void __launch_bounds__(32 * LN_RED_LANES)
ln_bwd_reduce_kernel(const float* partial, T* dgamma, T* dbeta, int nparts, int hidden, int accumulate) {
    __shared__ float red[LN_RED_LANES][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + tx;
    // when launched as a programmatic dependent of the kernel that writes the partials: wait for that grid to
    // finish (returns at once otherwise)
    pdl_wait();
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    if (j < 2 * hidden) {
        const size_t stride = (size_t)2 * hidden;
        int p = ty;
        for (; p + 3 * LN_RED_LANES < nparts; p += 4 * LN_RED_LANES) {
            s0 += partial[(size_t)p * stride + j];
            s1 += partial[(size_t)(p + LN_RED_LANES) * stride + j];
            s2 += partial[(size_t)(p + 2 * LN_RED_LANES) * stride + j];
            s3 += partial[(size_t)(p + 3 * LN_RED_LANES) * stride + j];
        }
        for (; p < nparts; p += LN_RED_LANES) s0 += partial[(size_t)p * stride + j];
    }
    red[ty][tx] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (ty == 0 && j < 2 * hidden) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < LN_RED_LANES; k++) t += red[k][tx];
        T* out = j < hidden ? dgamma + j : dbeta + (j - hidden);
        if (accumulate) t += to_f32(*out);
        *out = from_f32<T>(t);
    }
    pdl_launch_dependents();
}

// Generic path: one CTA per row for dx; column sums by a thread-per-column kernel.
template <typename T>
__global__ void __launch_bounds__(256)
ln_bwd_dx_generic_kernel(const T* dy, const T* gamma, const T* beta, const float* var, const T* y, const T* res, T* dx,
                         int64_t rows, int hidden, float eps) {
    __shared__ float red[64];
    const int64_t row = blockIdx.x;
    const T* dyr = dy + row * hidden;
    const T* yr = y + row * hidden;
    float sg = 0.0f, sgx = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float gm = to_f32(gamma[i]);
        float xhat = (to_f32(yr[i]) - to_f32(beta[i])) / guard_gamma(gm, eps);
        float g = to_f32(dyr[i]) * gm;
        sg += g;
        sgx += g * xhat;
    }
    block_sum2(sg, sgx, red);
    const float mg = sg / (float)hidden, mgx = sgx / (float)hidden;
    const float rstd = rsqrtf(var[row]);
    __syncthreads();
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float gm = to_f32(gamma[i]);
        float xhat = (to_f32(yr[i]) - to_f32(beta[i])) / guard_gamma(gm, eps);
        float g = to_f32(dyr[i]) * gm;
        float o = (g - mg - xhat * mgx) * rstd;
        if (res) o += to_f32(res[row * hidden + i]);
        dx[row * hidden + i] = from_f32<T>(o);
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
ln_bwd_cols_generic_kernel(const T* dy, const T* gamma, const T* beta, const T* y, T* dgamma, T* dbeta,
                           int64_t rows, int hidden, float eps, int accumulate) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= hidden) return;
    float gi = 1.0f / guard_gamma(to_f32(gamma[j]), eps), b = to_f32(beta[j]);
    float ag = 0.0f, ab = 0.0f;
    for (int64_t r = 0; r < rows; r++) {
        float d = to_f32(dy[r * hidden + j]);
        ag += (to_f32(y[r * hidden + j]) - b) * gi * d;
        ab += d;
    }
    if (accumulate) {
        ag += to_f32(dgamma[j]);
        ab += to_f32(dbeta[j]);
    }
    dgamma[j] = from_f32<T>(ag);
    dbeta[j] = from_f32<T>(ab);
}

static int ln_bwd_grid(int64_t rows) {
    int64_t want = (rows + LN_BWD_R - 1) / LN_BWD_R;
    int64_t cap = (int64_t)sm_count() * 2;
    return (int)(want < cap ? want : cap);
}

template <typename T>
static int ln_bwd_dispatch(const void* dy_, const void* gamma_, const void* beta_, const float* var, const void* y_, const void* res_,
                           void* dgamma_, void* dbeta_, void* dx_, int64_t rows, int64_t hidden, float eps,
                           void* workspace, size_t workspace_bytes, int accumulate, cudaStream_t st) {
    const T* dy = (const T*)dy_;
    const T* gamma = (const T*)gamma_;
    const T* beta = (const T*)beta_;
    const T* y = (const T*)y_;
    const T* res = (const T*)res_;
    T* dgamma = (T*)dgamma_;
    T* dbeta = (T*)dbeta_;
    T* dx = (T*)dx_;
    constexpr int VN = Vec<T>::N;
    const int64_t nvec = hidden / VN;
    bool fast = (hidden % VN == 0) && nvec <= 2048 && aligned16(dy) && aligned16(y) && aligned16(dx) &&
                aligned16(gamma) && aligned16(beta) && aligned16(workspace) && aligned16(res);
    if (fast) {
        if (workspace == nullptr || workspace_bytes < brk_layernorm_bwd_workspace_bytes(rows, hidden)) return BRK_ATTR_ERROR;
        float* partial = (float*)workspace;
        int h = (int)hidden;
        const size_t row_bytes = (size_t)hidden * sizeof(T);
        // packets per thread: 1, 2 or 4 with at most 512 threads and 16 floats per per-column register array
        int rnvt = nvec <= LNR_BWD_MAX_THREADS ? 1 : (nvec <= 2 * LNR_BWD_MAX_THREADS ? 2 : 4);
        bool ring = nvec <= 4 * LNR_BWD_MAX_THREADS && rnvt * VN <= 16 &&
                    (rnvt == 1 ? lnr_bwd_depth<T, 1>(row_bytes) : rnvt == 2 ? lnr_bwd_depth<T, 2>(row_bytes) : lnr_bwd_depth<T, 4>(row_bytes)) > 0;
        if (g_ln_mode == 0 && ring) {
            int rgrid = 0;      // at most one CTA per SM: never more partial rows than the workspace was sized for
            int rc;
            if (rnvt == 1)
                rc = launch_ln_bwd_ring<T, 1>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps, &rgrid, st);
            else if (rnvt == 2)
                rc = launch_ln_bwd_ring<T, 2>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps, &rgrid, st);
            else
                rc = launch_ln_bwd_ring<T, (Vec<T>::N == 4 ? 4 : 2)>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps, &rgrid, st);
            if (rc) return rc;
            // programmatic dependent launch: the reduce kernel's launch overlaps the tail of the kernel above
            const float* cpartial = partial;
            cudaError_t le = launch_pdl(ln_bwd_reduce_kernel<T>, (2 * h + 31) / 32, 32 * LN_RED_LANES, 0, st, cpartial, dgamma, dbeta, rgrid, h, accumulate);
            if (le != cudaSuccess) {
                set_cuda_error(le, "ln_bwd_reduce_kernel");
                return BRK_CUDA_ERROR;
            }
            return launch_status("ln_bwd_reduce_kernel");
        }
        int grid = ln_bwd_grid(rows);
        int nvt = nvec <= 512 ? 1 : (nvec <= 1024 ? 2 : 4);
        int threads = (int)(((nvec + nvt - 1) / nvt + 31) / 32 * 32);
        if (nvt == 1)
            ln_bwd_kernel<T, 1><<<grid, threads, 0, st>>>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps);
        else if (nvt == 2)
            ln_bwd_kernel<T, 2><<<grid, threads, 0, st>>>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps);
        else
            ln_bwd_kernel<T, 4><<<grid, threads, 0, st>>>(dy, gamma, beta, var, y, res, dx, partial, rows, h, eps);
        int rc = launch_status("ln_bwd_kernel");
        if (rc) return rc;
        ln_bwd_reduce_kernel<T><<<(2 * h + 31) / 32, 32 * LN_RED_LANES, 0, st>>>(partial, dgamma, dbeta, grid, h, accumulate);
        return launch_status("ln_bwd_reduce_kernel");
    }
    // column sums first: dx may alias dy or y
    ln_bwd_cols_generic_kernel<T><<<(unsigned)((hidden + 127) / 128), 128, 0, st>>>(dy, gamma, beta, y, dgamma, dbeta, rows,
                                                                                  (int)hidden, eps, accumulate);
    int rc = launch_status("ln_bwd_cols_generic_kernel");
    if (rc) return rc;
    ln_bwd_dx_generic_kernel<T><<<(unsigned)rows, 256, 0, st>>>(dy, gamma, beta, var, y, res, dx, rows, (int)hidden, eps);
    return launch_status("ln_bwd_dx_generic_kernel");
}

}  // namespace brk

extern "C" int brk_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* var,
                                 int64_t rows, int64_t hidden, float eps, int dtype, void* stream) {
    if (!x || !gamma || !beta) return BRK_INPUT_ERROR;
    if (!y) return BRK_OUTPUT_ERROR;
    if (rows < 0 || hidden <= 0 || hidden > (1 << 30) || rows > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::ln_fwd_dispatch<float>(x, gamma, beta, y, mean, var, rows, hidden, eps, st);
    if (dtype == BRK_F16) return brk::ln_fwd_dispatch<__half>(x, gamma, beta, y, mean, var, rows, hidden, eps, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_layernorm_set_mode(int mode) {
    if (mode != 0 && mode != 1) return BRK_ATTR_ERROR;
    brk::g_ln_mode = mode;
    return BRK_OK;
}

extern "C" size_t brk_layernorm_bwd_workspace_bytes(int64_t rows, int64_t hidden) {
    if (rows <= 0 || hidden <= 0) return 0;
    // one partial row (dgamma then dbeta, fp32) per CTA; no kernel variant launches more than min(rows, 2 x SMs) CTAs
    const int64_t cap = (int64_t)brk::sm_count() * 2;
    return (size_t)(rows < cap ? rows : cap) * 2 * (size_t)hidden * sizeof(float);
}

extern "C" int brk_layernorm_bwd_residual(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                                          const void* residual, void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden,
                                          float eps, void* workspace, size_t workspace_bytes, int accumulate, int dtype,
                                          void* stream) {
    if (!dy || !gamma || !beta || !var || !y) return BRK_INPUT_ERROR;
    if (!dgamma || !dbeta || !dx) return BRK_OUTPUT_ERROR;
    if (rows < 0 || hidden <= 0 || hidden > (1 << 30) || rows > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32)
        return brk::ln_bwd_dispatch<float>(dy, gamma, beta, var, y, residual, dgamma, dbeta, dx, rows, hidden, eps, workspace,
                                           workspace_bytes, accumulate, st);
    if (dtype == BRK_F16)
        return brk::ln_bwd_dispatch<__half>(dy, gamma, beta, var, y, residual, dgamma, dbeta, dx, rows, hidden, eps, workspace,
                                            workspace_bytes, accumulate, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_layernorm_bwd(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                                 void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden, float eps,
                                 void* workspace, size_t workspace_bytes, int accumulate, int dtype, void* stream) {
    return brk_layernorm_bwd_residual(dy, gamma, beta, var, y, nullptr, dgamma, dbeta, dx, rows, hidden, eps, workspace,
                                      workspace_bytes, accumulate, dtype, stream);
}

// ------------------------------------------------------------------------------------------
// LayerNorm backward without a caller-provided workspace.
//
// Some hosts of this library cannot give the backward pass a scratch buffer at call time: a
// plugin that runs inside an engine which has already handed all device memory to its own pool,
// a process confined to a fixed memory quota on a shared GPU, or code that is reached while
// the engine is capturing a stream, where the allocation calls are not permitted.  For them the
// per-CTA partial column sums live in a fixed array that is part of the library image.
//
// The array is reserved on every GPU that loads the library and stays reserved until the process
// ends.  It is shared by all calls: each call overwrites exactly the part it reads back (every
// CTA stores a full row of partials before the reduce kernel runs), so nothing needs clearing
// between calls, but two calls whose kernels can overlap on the GPU (different streams, or
// different host threads without ordering) race on it.
// ------------------------------------------------------------------------------------------
namespace brk {

constexpr size_t LN_BWD_STATIC_BYTES = (size_t)16 << 20;  // 16 MiB: e.g. 296 CTAs x 2 x 4096 columns x 4 B = 9.25 MiB
static __device__ __align__(256) unsigned char g_ln_bwd_static_scratch[LN_BWD_STATIC_BYTES];

// In host code the array's name is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device and cached.
static void* g_ln_bwd_static_ptr[64] = {nullptr};
static std::mutex g_ln_bwd_static_mu;

static int ln_bwd_static_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice, "brk_layernorm_bwd_static: current device");
        return BRK_CUDA_ERROR;
    }
    std::lock_guard<std::mutex> lk(g_ln_bwd_static_mu);
    if (g_ln_bwd_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_ln_bwd_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_cuda_error(e, "brk_layernorm_bwd_static: cudaGetSymbolAddress");
            return BRK_CUDA_ERROR;
        }
        g_ln_bwd_static_ptr[dev] = p;
    }
    *out = g_ln_bwd_static_ptr[dev];
    return BRK_OK;
}

}  // namespace brk

extern "C" size_t brk_layernorm_bwd_static_capacity(void) { return brk::LN_BWD_STATIC_BYTES; }

extern "C" int brk_layernorm_bwd_static(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                                        void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden, float eps,
                                        int accumulate, int dtype, void* stream) {
    if (!dy || !gamma || !beta || !var || !y) return BRK_INPUT_ERROR;
    if (!dgamma || !dbeta || !dx) return BRK_OUTPUT_ERROR;
    if (rows < 0 || hidden <= 0 || hidden > (1 << 30) || rows > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (dtype != BRK_F32 && dtype != BRK_F16) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    const size_t need = brk_layernorm_bwd_workspace_bytes(rows, hidden);
    if (need > brk::LN_BWD_STATIC_BYTES) {
        brk::set_error_message("brk_layernorm_bwd_static: rows x hidden needs " + std::to_string(need) +
                               " bytes of scratch but the built-in array holds " + std::to_string(brk::LN_BWD_STATIC_BYTES) +
                               "; use brk_layernorm_bwd with a caller workspace");
        return BRK_ATTR_ERROR;
    }
    void* scratch = nullptr;
    int rc = brk::ln_bwd_static_address(&scratch);
    if (rc != BRK_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32)
        return brk::ln_bwd_dispatch<float>(dy, gamma, beta, var, y, nullptr, dgamma, dbeta, dx, rows, hidden, eps, scratch,
                                           brk::LN_BWD_STATIC_BYTES, accumulate, st);
    return brk::ln_bwd_dispatch<__half>(dy, gamma, beta, var, y, nullptr, dgamma, dbeta, dx, rows, hidden, eps, scratch,
                                        brk::LN_BWD_STATIC_BYTES, accumulate, st);
}
