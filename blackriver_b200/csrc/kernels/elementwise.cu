// Data-movement and small reduction kernels: broadcast add, fill, cast, [a,b,c,d]->[a,c,b,d]
// transpose, column sums, row softmax (unfused parity path), embedding gather, ALiBi / mask
// construction.  All HBM-bound; vectorised where shapes and alignment allow.
#include <math.h>

#include <mutex>
#include <string>

#include "brk_common.cuh"

namespace brk {

static std::mutex g_err_mu;
static std::string g_err = "";

void set_cuda_error(cudaError_t e, const char* where) {
    std::lock_guard<std::mutex> lk(g_err_mu);
    g_err = std::string(where) + ": " + cudaGetErrorString(e);
}

void set_error_message(const std::string& msg) {
    std::lock_guard<std::mutex> lk(g_err_mu);
    g_err = msg;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static inline int grid_for(int64_t work_items, int threads, int per_sm) {
    int64_t want = (work_items + threads - 1) / threads;
    int64_t cap = (int64_t)sm_count() * per_sm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

// ------------------------------------------------------------------------------------------
// c = a + b with broadcast of b (4-D).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
add_same_vec_kernel(const T* a, const T* b, T* c, int64_t nvec) {
    constexpr int VN = Vec<T>::N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        Vec<T> va, vb;
        va.load_stream(a + i * VN);
        vb.load_stream(b + i * VN);
#pragma unroll
        for (int e = 0; e < VN; e++) va.v[e] += vb.v[e];
        va.store_stream(c + i * VN);
    }
}

struct Dims4 {
    int64_t a[4];
    int64_t bs[4];
};

template <typename T>
__global__ void __launch_bounds__(256)
add_bcast_kernel(const T* a, const T* b, T* c, Dims4 d, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i;
        int64_t i3 = r % d.a[3]; r /= d.a[3];
        int64_t i2 = r % d.a[2]; r /= d.a[2];
        int64_t i1 = r % d.a[1]; r /= d.a[1];
        int64_t i0 = r;
        int64_t bi = i0 * d.bs[0] + i1 * d.bs[1] + i2 * d.bs[2] + i3 * d.bs[3];
        c[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[bi]));
    }
}

template <typename T>
static int add_dispatch(const void* a_, const void* b_, void* c_, const int64_t ad[4], const int64_t bd[4], cudaStream_t st) {
    const T* a = (const T*)a_;
    const T* b = (const T*)b_;
    T* c = (T*)c_;
    constexpr int VN = Vec<T>::N;
    int64_t n = ad[0] * ad[1] * ad[2] * ad[3];
    if (n == 0) return BRK_OK;
    bool same = true;
    for (int i = 0; i < 4; i++) {
        if (bd[i] != ad[i] && bd[i] != 1) return BRK_INPUT_ERROR;
        if (bd[i] != ad[i]) same = false;
    }
    if (same && n % VN == 0 && aligned16(a) && aligned16(b) && aligned16(c)) {
        add_same_vec_kernel<T><<<grid_for(n / VN, 256, 16), 256, 0, st>>>(a, b, c, n / VN);
        return launch_status("add_same_vec_kernel");
    }
    Dims4 d;
    int64_t stv = 1;
    for (int i = 3; i >= 0; i--) {
        d.a[i] = ad[i];
        d.bs[i] = (bd[i] == 1 && ad[i] != 1) ? 0 : stv;
        if (bd[i] == 1) d.bs[i] = 0;
        stv *= bd[i];
    }
    add_bcast_kernel<T><<<grid_for(n, 256, 16), 256, 0, st>>>(a, b, c, d, n);
    return launch_status("add_bcast_kernel");
}

// ------------------------------------------------------------------------------------------
// fill / cast
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* x, float value, int64_t n) {
    T v = from_f32<T>(value);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] = v;
}

template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_kernel(const S* src, D* dst, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = from_f32<D>(to_f32(src[i]));
}

// ------------------------------------------------------------------------------------------
// transpose 0213: y[a,c,b,:] = x[a,b,c,:]; rows of d elements are moved as 16-byte packets
// when d and the pointers allow it.
// ------------------------------------------------------------------------------------------
template <typename P>
__global__ void __launch_bounds__(256)
transpose_0213_kernel(const P* x, P* y, int64_t a, int64_t b, int64_t c, int64_t dp) {
    const int64_t n = a * b * c * dp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        // i indexes the OUTPUT [a,c,b,dp] so that stores are fully coalesced
        int64_t r = i;
        int64_t id = r % dp; r /= dp;
        int64_t ib = r % b; r /= b;
        int64_t ic = r % c; r /= c;
        int64_t ia = r;
        y[i] = x[((ia * b + ib) * c + ic) * dp + id];
    }
}

// ------------------------------------------------------------------------------------------
// column sums: out[j] = sum_i x[i,j].  Stage 1: CTAs of 32x8 threads each own 32 columns and a
// slice of rows; stage 2 is folded in by letting gridDim.y == 1 (rows are few thousands and the
// op is tiny next to the GEMMs it accompanies), so the result is deterministic.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* x, T* out, int64_t rows, int64_t cols, int accumulate) {
    __shared__ float tile[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t j = (int64_t)blockIdx.x * 32 + tx;
    float s = 0.0f;
    if (j < cols)
        for (int64_t i = ty; i < rows; i += 8) s += to_f32(x[i * cols + j]);
    tile[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && j < cols) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; k++) t += tile[k][tx];
        if (accumulate) t += to_f32(out[j]);
        out[j] = from_f32<T>(t);
    }
}

// Two-stage form for large inputs: stage 1 CTAs own 64 columns x a slice of rows (128-bit loads,
// 32 row lanes) and write fp32 partial sums [slices, cols] to scratch; stage 2 adds the slices in a
// fixed order.  Deterministic, and enough CTAs in flight to stream at HBM speed.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* x, float* partial, int64_t rows, int64_t cols, int64_t rows_per_slice) {
    constexpr int VN = Vec<T>::N;
    constexpr int CV = 64 / VN;                 // 16-byte packets across the 64 columns of this CTA
    constexpr int RL = 256 / CV;                // row lanes
    __shared__ float red[RL][65];
    const int cv = threadIdx.x % CV, rl = threadIdx.x / CV;
    const int64_t c0 = (int64_t)blockIdx.x * 64 + cv * VN;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slice;
    const int64_t r1 = min(rows, r0 + rows_per_slice);
    float acc[VN];
#pragma unroll
    for (int e = 0; e < VN; e++) acc[e] = 0.0f;
    pdl_wait();          // launched as a programmatic dependent: x is complete from here on
    if (c0 < cols) {
        int64_t r = r0 + rl;
        for (; r + 3 * RL < r1; r += 4 * RL) {
            Vec<T> v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u].load_stream(x + (r + u * RL) * cols + c0);
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < VN; e++) acc[e] += v[u].v[e];
        }
        for (; r < r1; r += RL) {
            Vec<T> v;
            v.load_stream(x + r * cols + c0);
#pragma unroll
            for (int e = 0; e < VN; e++) acc[e] += v.v[e];
        }
    }
#pragma unroll
    for (int e = 0; e < VN; e++) red[rl][cv * VN + e] = acc[e];
    __syncthreads();
    if (threadIdx.x < 64) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < RL; k++) t += red[k][threadIdx.x];
        const int64_t c = (int64_t)blockIdx.x * 64 + threadIdx.x;
        if (c < cols) partial[(int64_t)blockIdx.y * cols + c] = t;
    }
    pdl_launch_dependents();
}

// Stage 2: 32 columns x 8 slice lanes per CTA; every lane adds each 8th slice (independent loads in flight) and the
// lanes are combined in a fixed order.
constexpr int COLSUM_FINAL_LANES = 8;

template <typename T>
__global__ void __launch_bounds__(32 * COLSUM_FINAL_LANES)
colsum_final_kernel(const float* partial, T* out, int slices, int64_t cols, int accumulate) {
    __shared__ float red[COLSUM_FINAL_LANES][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t j = (int64_t)blockIdx.x * 32 + tx;
    pdl_wait();          // the partial sums are complete from here on
    float t = 0.0f;
    if (j < cols) {
#pragma unroll 4
        for (int s = ty; s < slices; s += COLSUM_FINAL_LANES) t += partial[(int64_t)s * cols + j];
    }
    red[ty][tx] = t;
    __syncthreads();
    if (ty == 0 && j < cols) {
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < COLSUM_FINAL_LANES; k++) sum += red[k][tx];
        if (accumulate) sum += to_f32(out[j]);
        out[j] = from_f32<T>(sum);
    }
    pdl_launch_dependents();
}

template <typename T>
static int colsum_ws_dispatch(const void* x, void* out, int64_t rows, int64_t cols, int accumulate, void* ws, size_t ws_bytes,
                              cudaStream_t st) {
    int64_t col_ctas = (cols + 63) / 64;
    int64_t slices = ((int64_t)sm_count() * 4 + col_ctas - 1) / col_ctas;
    if (slices > rows / 32) slices = rows / 32 > 0 ? rows / 32 : 1;
    if (slices > 64) slices = 64;
    if ((size_t)(slices * cols) * sizeof(float) > ws_bytes) return BRK_ATTR_ERROR;
    int64_t rps = (rows + slices - 1) / slices;
    // both stages are programmatic dependents of the kernel before them in the stream: their launches overlap its tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)col_ctas, (unsigned)slices);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, colsum_partial_kernel<T>, (const T*)x, (float*)ws, rows, cols, rps);
    if (le != cudaSuccess) {
        set_cuda_error(le, "colsum_partial_kernel");
        return BRK_CUDA_ERROR;
    }
    le = launch_pdl(colsum_final_kernel<T>, (int)((cols + 31) / 32), 32 * COLSUM_FINAL_LANES, 0, st, (const float*)ws, (T*)out,
                    (int)slices, cols, accumulate);
    if (le != cudaSuccess) {
        set_cuda_error(le, "colsum_final_kernel");
        return BRK_CUDA_ERROR;
    }
    return launch_status("colsum_final_kernel");
}

// ------------------------------------------------------------------------------------------
// row softmax forward / backward (one CTA per row; rows are attention score rows, T <= 2048)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const T* x, T* y, int64_t rows, int cols) {
    __shared__ float red[64];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * cols;
        T* yr = y + row * cols;
        float m = -INFINITY;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, to_f32(xr[j]));
        m = block_max(m, red);
        float s = 0.0f, z = 0.0f;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) s += __expf(to_f32(xr[j]) - m);
        block_sum2(s, z, red);
        const float inv = 1.0f / s;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) yr[j] = from_f32<T>(__expf(to_f32(xr[j]) - m) * inv);
        __syncthreads();
    }
}

template <typename T>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const T* dy, const T* out, T* dx, int64_t rows, int cols) {
    __shared__ float red[64];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* g = dy + row * cols;
        const T* p = out + row * cols;
        T* d = dx + row * cols;
        float dot = 0.0f, z = 0.0f;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) dot += to_f32(g[j]) * to_f32(p[j]);
        block_sum2(dot, z, red);
        for (int j = threadIdx.x; j < cols; j += blockDim.x) d[j] = from_f32<T>(to_f32(p[j]) * (to_f32(g[j]) - dot));
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// embedding gather: one warp per output row, 16-byte packets when possible
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
gather_kernel(const T* table, const int32_t* ids, T* out, int64_t n, int64_t hidden, int64_t vocab, int vec_ok) {
    constexpr int VN = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = wid; r < n; r += nw) {
        const int64_t id = ids[r];
        const bool ok = id >= 0 && id < vocab;
        const T* src = table + (ok ? id : 0) * hidden;
        T* dst = out + r * hidden;
        if (vec_ok) {
            const uint4 zero = make_uint4(0, 0, 0, 0);
            for (int64_t i = lane; i < hidden / VN; i += 32)
                reinterpret_cast<uint4*>(dst)[i] = ok ? reinterpret_cast<const uint4*>(src)[i] : zero;
        } else {
            for (int64_t i = lane; i < hidden; i += 32) dst[i] = ok ? src[i] : from_f32<T>(0.0f);
        }
    }
}

// ------------------------------------------------------------------------------------------
// ALiBi and additive mask, bit-exact with the host loops they restate.
// ------------------------------------------------------------------------------------------
__global__ void alibi_kernel(const double* slopes, float* alibi, int heads, int tokens) {
    const int64_t n = (int64_t)heads * tokens;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int j = (int)(i / tokens), k = (int)(i % tokens);
        alibi[i] = (float)((double)k * 1.0 * slopes[j]);
    }
}

// one CTA per (b, query row m): key n is open iff n <= m and every mask[b,0..n] != 0
__global__ void xmask_kernel(const int32_t* mask, float* xmask, int batch, int tokens) {
    __shared__ int first_pad;
    const int b = blockIdx.x / tokens;
    const int m = blockIdx.x % tokens;
    const int32_t* ms = mask + (int64_t)b * tokens;
    if (threadIdx.x == 0) first_pad = tokens;
    __syncthreads();
    int local = tokens;
    for (int n = threadIdx.x; n < tokens; n += blockDim.x)
        if (ms[n] == 0) {
            local = n;
            break;
        }
    atomicMin(&first_pad, local);
    __syncthreads();
    const int fp = first_pad;
    float* row = xmask + ((int64_t)b * tokens + m) * tokens;
    for (int n = threadIdx.x; n < tokens; n += blockDim.x) row[n] = (n <= m && n < fp) ? 0.0f : -3.402823466e+38f;
}

}  // namespace brk

using namespace brk;

extern "C" int brk_version(void) { return 1; }

extern "C" const char* brk_last_cuda_error(void) {
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lk(g_err_mu);
    copy = g_err;
    return copy.c_str();
}

extern "C" int brk_sm_count(void) { return sm_count(); }

extern "C" int brk_add_bcast(const void* a, const void* b, void* c, const int64_t adims[4], const int64_t bdims[4], int dtype,
                             void* stream) {
    if (!a || !b || !adims || !bdims) return BRK_INPUT_ERROR;
    if (!c) return BRK_OUTPUT_ERROR;
    for (int i = 0; i < 4; i++)
        if (adims[i] < 0 || bdims[i] < 0) return BRK_ATTR_ERROR;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return add_dispatch<float>(a, b, c, adims, bdims, st);
    if (dtype == BRK_F16) return add_dispatch<__half>(a, b, c, adims, bdims, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_fill(void* x, float value, int64_t n, int dtype, void* stream) {
    if (!x) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (value == 0.0f) {
        size_t bytes = (size_t)n * (dtype == BRK_F16 ? 2 : 4);
        cudaError_t e = cudaMemsetAsync(x, 0, bytes, st);
        if (e != cudaSuccess) {
            set_cuda_error(e, "brk_fill memset");
            return BRK_CUDA_ERROR;
        }
        return BRK_OK;
    }
    if (dtype == BRK_F32)
        fill_kernel<float><<<grid_for(n, 256, 16), 256, 0, st>>>((float*)x, value, n);
    else if (dtype == BRK_F16)
        fill_kernel<__half><<<grid_for(n, 256, 16), 256, 0, st>>>((__half*)x, value, n);
    else
        return BRK_ATTR_ERROR;
    return launch_status("fill_kernel");
}

extern "C" int brk_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream) {
    if (!src) return BRK_INPUT_ERROR;
    if (!dst) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int g = grid_for(n, 256, 16);
    if (src_dtype == BRK_F32 && dst_dtype == BRK_F16)
        cast_kernel<float, __half><<<g, 256, 0, st>>>((const float*)src, (__half*)dst, n);
    else if (src_dtype == BRK_F16 && dst_dtype == BRK_F32)
        cast_kernel<__half, float><<<g, 256, 0, st>>>((const __half*)src, (float*)dst, n);
    else if (src_dtype == dst_dtype && (src_dtype == BRK_F32 || src_dtype == BRK_F16)) {
        cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)n * (src_dtype == BRK_F16 ? 2 : 4), cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) {
            set_cuda_error(e, "brk_cast copy");
            return BRK_CUDA_ERROR;
        }
        return BRK_OK;
    } else
        return BRK_ATTR_ERROR;
    return launch_status("cast_kernel");
}

extern "C" int brk_transpose_0213(const void* x, void* y, int64_t a, int64_t b, int64_t c, int64_t d, int dtype, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!y) return BRK_OUTPUT_ERROR;
    if (x == y) return BRK_OUTPUT_ERROR;
    if (a < 0 || b < 0 || c < 0 || d < 0) return BRK_ATTR_ERROR;
    if (dtype != BRK_F32 && dtype != BRK_F16) return BRK_ATTR_ERROR;
    int64_t n = a * b * c * d;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t es = dtype == BRK_F16 ? 2 : 4;
    if ((d * es) % 16 == 0 && aligned16(x) && aligned16(y)) {
        int64_t dp = d * es / 16;
        transpose_0213_kernel<uint4><<<grid_for(n * es / 16, 256, 16), 256, 0, st>>>((const uint4*)x, (uint4*)y, a, b, c, dp);
    } else if (es == 4) {
        transpose_0213_kernel<uint32_t><<<grid_for(n, 256, 16), 256, 0, st>>>((const uint32_t*)x, (uint32_t*)y, a, b, c, d);
    } else {
        transpose_0213_kernel<uint16_t><<<grid_for(n, 256, 16), 256, 0, st>>>((const uint16_t*)x, (uint16_t*)y, a, b, c, d);
    }
    return launch_status("transpose_0213_kernel");
}

extern "C" int brk_colsum(const void* x, void* out, int64_t rows, int64_t cols, int accumulate, int dtype, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (rows < 0 || cols < 0) return BRK_ATTR_ERROR;
    if (cols == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned g = (unsigned)((cols + 31) / 32);
    if (dtype == BRK_F32)
        colsum_kernel<float><<<g, 256, 0, st>>>((const float*)x, (float*)out, rows, cols, accumulate);
    else if (dtype == BRK_F16)
        colsum_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (__half*)out, rows, cols, accumulate);
    else
        return BRK_ATTR_ERROR;
    return launch_status("colsum_kernel");
}

extern "C" size_t brk_colsum_workspace_bytes(int64_t rows, int64_t cols) {
    (void)rows;
    return cols > 0 ? (size_t)64 * (size_t)cols * sizeof(float) : 0;
}

extern "C" int brk_colsum_ws(const void* x, void* out, int64_t rows, int64_t cols, int accumulate, int dtype, void* workspace,
                             size_t workspace_bytes, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (rows < 0 || cols < 0) return BRK_ATTR_ERROR;
    if (cols == 0) return BRK_OK;
    const int64_t vn = dtype == BRK_F16 ? 8 : 4;
    const bool fast = workspace && rows >= 256 && cols % vn == 0 && aligned16(x) && aligned16(workspace) &&
                      (dtype == BRK_F16 || dtype == BRK_F32);
    if (!fast) return brk_colsum(x, out, rows, cols, accumulate, dtype, stream);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F16) return colsum_ws_dispatch<__half>(x, out, rows, cols, accumulate, workspace, workspace_bytes, st);
    return colsum_ws_dispatch<float>(x, out, rows, cols, accumulate, workspace, workspace_bytes, st);
}

extern "C" int brk_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int dtype, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!y) return BRK_OUTPUT_ERROR;
    if (rows < 0 || cols <= 0 || cols > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t cap = (int64_t)sm_count() * 8;
    int g = (int)(rows < cap ? rows : cap);
    if (dtype == BRK_F32)
        softmax_fwd_kernel<float><<<g, 256, 0, st>>>((const float*)x, (float*)y, rows, (int)cols);
    else if (dtype == BRK_F16)
        softmax_fwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (__half*)y, rows, (int)cols);
    else
        return BRK_ATTR_ERROR;
    return launch_status("softmax_fwd_kernel");
}

extern "C" int brk_softmax_bwd(const void* dy, const void* out, void* dx, int64_t rows, int64_t cols, int dtype, void* stream) {
    if (!dy || !out) return BRK_INPUT_ERROR;
    if (!dx) return BRK_OUTPUT_ERROR;
    if (rows < 0 || cols <= 0 || cols > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t cap = (int64_t)sm_count() * 8;
    int g = (int)(rows < cap ? rows : cap);
    if (dtype == BRK_F32)
        softmax_bwd_kernel<float><<<g, 256, 0, st>>>((const float*)dy, (const float*)out, (float*)dx, rows, (int)cols);
    else if (dtype == BRK_F16)
        softmax_bwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)dy, (const __half*)out, (__half*)dx, rows, (int)cols);
    else
        return BRK_ATTR_ERROR;
    return launch_status("softmax_bwd_kernel");
}

extern "C" int brk_embedding_gather(const void* table, const int32_t* ids, void* out, int64_t n, int64_t hidden, int64_t vocab,
                                    int dtype, void* stream) {
    if (!table || !ids) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (n < 0 || hidden <= 0 || vocab <= 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int g = grid_for(n * 32, 256, 8);
    if (dtype == BRK_F32) {
        int vec_ok = hidden % 4 == 0 && aligned16(table) && aligned16(out);
        gather_kernel<float><<<g, 256, 0, st>>>((const float*)table, ids, (float*)out, n, hidden, vocab, vec_ok);
    } else if (dtype == BRK_F16) {
        int vec_ok = hidden % 8 == 0 && aligned16(table) && aligned16(out);
        gather_kernel<__half><<<g, 256, 0, st>>>((const __half*)table, ids, (__half*)out, n, hidden, vocab, vec_ok);
    } else
        return BRK_ATTR_ERROR;
    return launch_status("gather_kernel");
}

extern "C" void brk_alibi_slopes(int heads, double* slopes_out) {
    // blackriver/train_bloom.cpp:61-66, evaluated in double exactly as written there
    double base = 3 - log2(heads * 1.0);
    base = -1 * pow(2.0, base);
    base = pow(2.0, base);
    for (int j = 0; j < heads; j++) slopes_out[j] = pow(base, (j + 1) * 1.0);
}

extern "C" int brk_alibi_build(const double* slopes_dev, float* alibi, int heads, int tokens, void* stream) {
    if (!slopes_dev) return BRK_INPUT_ERROR;
    if (!alibi) return BRK_OUTPUT_ERROR;
    if (heads <= 0 || tokens < 0) return BRK_ATTR_ERROR;
    if (tokens == 0) return BRK_OK;
    alibi_kernel<<<grid_for((int64_t)heads * tokens, 256, 8), 256, 0, (cudaStream_t)stream>>>(slopes_dev, alibi, heads, tokens);
    return launch_status("alibi_kernel");
}

extern "C" int brk_xmask_build(const int32_t* mask, float* xmask, int batch, int tokens, void* stream) {
    if (!mask) return BRK_INPUT_ERROR;
    if (!xmask) return BRK_OUTPUT_ERROR;
    if (batch < 0 || tokens < 0) return BRK_ATTR_ERROR;
    if (batch == 0 || tokens == 0) return BRK_OK;
    xmask_kernel<<<(unsigned)((int64_t)batch * tokens), 256, 0, (cudaStream_t)stream>>>(mask, xmask, batch, tokens);
    return launch_status("xmask_kernel");
}
