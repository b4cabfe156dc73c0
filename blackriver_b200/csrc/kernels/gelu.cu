// bloom GELU (tanh approximation) forward / backward.  Pure HBM streaming: 128-bit loads with
// several packets in flight per thread, fp32 math, streaming stores.
#include "brk_common.cuh"

namespace brk {

// Two tanh flavours.  PRECISE: tanh(u) = 1 - 2/(1+exp(2u)), exp through ex2.approx and the division
// through rcp.approx: absolute error ~1e-7, saturates correctly for |u| large (exp -> inf gives 1,
// exp -> 0 gives -1); used for fp32 tensors.  Otherwise the hardware tanh.approx.f32 (one SFU
// operation, relative error 2^-11, i.e. below half precision's own rounding); used for fp16 tensors,
// where two SFU operations and the longer instruction sequence per element would cost as much time as
// the memory traffic.
template <bool PRECISE>
__device__ __forceinline__ float fast_tanh(float u) {
    if (PRECISE) {
        float e = __expf(2.0f * u);
        return 1.0f - __fdividef(2.0f, e + 1.0f);
    } else {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
        return t;
    }
}

template <bool PRECISE>
__device__ __forceinline__ float gelu_f(float x) {
    const float x2 = x * x;
    const float t = fast_tanh<PRECISE>(x * fmaf(0.79788456f * 0.044715f, x2, 0.79788456f));
    const float hx = 0.5f * x;
    return fmaf(hx, t, hx);
}

template <bool PRECISE>
__device__ __forceinline__ float gelu_grad_f(float g, float x) {
    const float x2 = x * x;
    const float t = fast_tanh<PRECISE>(x * fmaf(0.79788456f * 0.044715f, x2, 0.79788456f));
    const float sech2 = fmaf(-t, t, 1.0f);
    const float dpoly = fmaf(0.1070322243f, x2, 0.79788456f);
    const float ff = fmaf(0.5f * x * sech2, dpoly, fmaf(0.5f, t, 0.5f));
    return ff * g;
}

template <typename T>
struct GeluPrecise {
    static constexpr bool value = true;
};
template <>
struct GeluPrecise<__half> {
    static constexpr bool value = false;
};

constexpr int GELU_UNROLL = 4;
constexpr int GELU_THREADS = 256;

template <typename T, bool BWD>
__global__ void __launch_bounds__(GELU_THREADS)
gelu_vec_kernel(const T* dy, const T* x, T* out, int64_t nvec) {
    constexpr int VN = Vec<T>::N;
    pdl_wait();
    const int64_t stride = (int64_t)gridDim.x * GELU_THREADS;
    for (int64_t base = (int64_t)blockIdx.x * GELU_THREADS + threadIdx.x; base < nvec; base += stride * GELU_UNROLL) {
        // the packets stay packed (4 registers each) until their turn: more loads in flight per register
        uint4 rx[GELU_UNROLL], rg[GELU_UNROLL];
#pragma unroll
        for (int u = 0; u < GELU_UNROLL; u++) {
            int64_t i = base + u * stride;
            if (i < nvec) {
                rx[u] = ld_raw_stream(x + i * VN);
                if (BWD) rg[u] = ld_raw_stream(dy + i * VN);
            }
        }
#pragma unroll
        for (int u = 0; u < GELU_UNROLL; u++) {
            int64_t i = base + u * stride;
            if (i < nvec) {
                Vec<T> vx, vg, o;
                vx.unpack(rx[u]);
                if (BWD) vg.unpack(rg[u]);
#pragma unroll
                for (int e = 0; e < VN; e++)
                    o.v[e] = BWD ? gelu_grad_f<GeluPrecise<T>::value>(vg.v[e], vx.v[e]) : gelu_f<GeluPrecise<T>::value>(vx.v[e]);
                o.store_stream(out + i * VN);
            }
        }
    }
    pdl_launch_dependents();
}

template <typename T, bool BWD>
__global__ void gelu_scalar_kernel(const T* dy, const T* x, T* out, int64_t begin, int64_t n) {
    int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float xv = to_f32(x[i]);
        out[i] = from_f32<T>(BWD ? gelu_grad_f<GeluPrecise<T>::value>(to_f32(dy[i]), xv) : gelu_f<GeluPrecise<T>::value>(xv));
    }
}

template <typename T, bool BWD>
static int gelu_dispatch(const void* dy_, const void* x_, void* out_, int64_t n, cudaStream_t st) {
    const T* dy = (const T*)dy_;
    const T* x = (const T*)x_;
    T* out = (T*)out_;
    constexpr int VN = Vec<T>::N;
    int64_t nvec = 0;
    if (aligned16(x) && aligned16(out) && (!BWD || aligned16(dy))) nvec = n / VN;
    if (nvec > 0) {
        int64_t want = (nvec + (int64_t)GELU_THREADS * GELU_UNROLL - 1) / ((int64_t)GELU_THREADS * GELU_UNROLL);
        int64_t cap = (int64_t)sm_count() * 16;
        int grid = (int)(want < cap ? want : cap);
        cudaError_t le = launch_pdl(gelu_vec_kernel<T, BWD>, grid, GELU_THREADS, 0, st, dy, x, out, nvec);
        if (le != cudaSuccess) {
            set_cuda_error(le, "gelu_vec_kernel");
            return BRK_CUDA_ERROR;
        }
        int rc = launch_status("gelu_vec_kernel");
        if (rc) return rc;
    }
    int64_t done = nvec * VN;
    if (done < n) {
        int64_t rest = n - done;
        gelu_scalar_kernel<T, BWD><<<(unsigned)((rest + 255) / 256), 256, 0, st>>>(dy, x, out, done, n);
        return launch_status("gelu_scalar_kernel");
    }
    return BRK_OK;
}

}  // namespace brk

extern "C" int brk_gelu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!y) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::gelu_dispatch<float, false>(nullptr, x, y, n, st);
    if (dtype == BRK_F16) return brk::gelu_dispatch<__half, false>(nullptr, x, y, n, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, int dtype, void* stream) {
    if (!dy || !x) return BRK_INPUT_ERROR;
    if (!dx) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::gelu_dispatch<float, true>(dy, x, dx, n, st);
    if (dtype == BRK_F16) return brk::gelu_dispatch<__half, true>(dy, x, dx, n, st);
    return BRK_ATTR_ERROR;
}
