// Parameter-side kernels of the training step: mixed-precision Adam (fp32 master weights and
// moments, fp16 working copy), embedding-gradient scatter-add, seeded normal initialisation.
// All HBM-bound streaming kernels.
#include "brk_common.cuh"

namespace brk {

// ------------------------------------------------------------------------------------------
// Adam, torch.optim.Adam semantics (no weight decay, no amsgrad):
//   g = grad * grad_scale;  m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2
//   w -= lr/(1-b1^t) * m / (sqrt(v)/sqrt(1-b2^t) + eps);  w16 = fp16(w)
// 28 bytes of traffic per parameter (2 grad + 12 read + 12 write + 2 fp16 weight).
// An element whose scaled gradient is not finite (an fp16 gradient that overflowed under the loss scale) is left
// untouched -- weight and moments keep their values instead of turning NaN for good -- and raises g_adam_nonfinite,
// which brk_adam_status() reports.
// ------------------------------------------------------------------------------------------
__device__ int g_adam_nonfinite = 0;

template <typename G>
__global__ void __launch_bounds__(256)
adam_kernel(float* w, float* m, float* v, const G* g, __half* w16, int64_t n, float step_size, float inv_bc2_sqrt, float beta1,
            float beta2, float eps, float grad_scale) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
        if (i + 3 < n) {
            float4 wv = *reinterpret_cast<float4*>(w + i), mv = *reinterpret_cast<float4*>(m + i), vv = *reinterpret_cast<float4*>(v + i);
            float gg[4];
#pragma unroll
            for (int e = 0; e < 4; e++) gg[e] = to_f32(g[i + e]) * grad_scale;
            float* wp = &wv.x; float* mp = &mv.x; float* vp = &vv.x;
            bool bad = false;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (!isfinite(gg[e])) {
                    bad = true;
                    continue;
                }
                mp[e] = beta1 * mp[e] + (1.0f - beta1) * gg[e];
                vp[e] = beta2 * vp[e] + (1.0f - beta2) * gg[e] * gg[e];
                wp[e] -= step_size * mp[e] / (sqrtf(vp[e]) * inv_bc2_sqrt + eps);
            }
            if (bad) g_adam_nonfinite = 1;
            *reinterpret_cast<float4*>(w + i) = wv;
            *reinterpret_cast<float4*>(m + i) = mv;
            *reinterpret_cast<float4*>(v + i) = vv;
            if (w16) {
                __half2 lo = __floats2half2_rn(wv.x, wv.y), hi = __floats2half2_rn(wv.z, wv.w);
                *reinterpret_cast<__half2*>(w16 + i) = lo;
                *reinterpret_cast<__half2*>(w16 + i + 2) = hi;
            }
        } else {
            for (int64_t j = i; j < n; j++) {
                float gj = to_f32(g[j]) * grad_scale;
                if (!isfinite(gj)) {
                    g_adam_nonfinite = 1;
                    continue;
                }
                float mj = beta1 * m[j] + (1.0f - beta1) * gj;
                float vj = beta2 * v[j] + (1.0f - beta2) * gj * gj;
                m[j] = mj;
                v[j] = vj;
                float wj = w[j] - step_size * mj / (sqrtf(vj) * inv_bc2_sqrt + eps);
                w[j] = wj;
                if (w16) w16[j] = __float2half_rn(wj);
            }
        }
    }
}

// table_g[ids[r], :] += dx[r, :]  (duplicated ids make the floating-point order run-dependent)
template <typename T>
__global__ void __launch_bounds__(256)
scatter_add_kernel(const T* dx, const int32_t* ids, T* table_g, int64_t n, int64_t hidden, int64_t vocab);

template <>
__global__ void __launch_bounds__(256)
scatter_add_kernel<__half>(const __half* dx, const int32_t* ids, __half* table_g, int64_t n, int64_t hidden, int64_t vocab) {
    const int64_t pairs = hidden / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pairs, c = (i % pairs) * 2;
        const int64_t id = ids[r];
        if (id < 0 || id >= vocab) continue;
        atomicAdd(reinterpret_cast<__half2*>(table_g + id * hidden + c), *reinterpret_cast<const __half2*>(dx + r * hidden + c));
    }
}

template <>
__global__ void __launch_bounds__(256)
scatter_add_kernel<float>(const float* dx, const int32_t* ids, float* table_g, int64_t n, int64_t hidden, int64_t vocab) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * hidden; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / hidden, c = i % hidden;
        const int64_t id = ids[r];
        if (id < 0 || id >= vocab) continue;
        atomicAdd(table_g + id * hidden + c, dx[i]);
    }
}

// counter-based generator: element i of stream `seed` depends on (seed, i) only, so the result is
// independent of the launch shape
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void __launch_bounds__(256) init_normal_kernel(T* x, int64_t n, float mean, float std, uint64_t seed) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n + 1) / 2; i += (int64_t)gridDim.x * blockDim.x) {
        uint64_t r = mix64(mix64(seed) ^ (uint64_t)i);
        float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);   // (0, 1)
        float u2 = (float)(uint32_t)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
        float rad = sqrtf(-2.0f * __logf(u1));
        float s, c;
        __sincosf(6.283185307179586f * u2, &s, &c);
        x[2 * i] = from_f32<T>(mean + std * rad * c);
        if (2 * i + 1 < n) x[2 * i + 1] = from_f32<T>(mean + std * rad * s);
    }
}

}  // namespace brk

using namespace brk;

extern "C" int brk_adam_step(void* master_w, void* m, void* v, const void* grad, int grad_dtype, void* w16, int64_t n, float lr,
                             float beta1, float beta2, float eps, int step, float grad_scale, void* stream) {
    if (!master_w || !m || !v || !grad) return BRK_INPUT_ERROR;
    if (n < 0 || step < 1) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    if ((reinterpret_cast<uintptr_t>(master_w) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) return BRK_ATTR_ERROR;
    if (w16 && (reinterpret_cast<uintptr_t>(w16) & 3)) return BRK_ATTR_ERROR;
    double bc1 = 1.0 - pow((double)beta1, (double)step), bc2 = 1.0 - pow((double)beta2, (double)step);
    float step_size = (float)((double)lr / bc1), inv_bc2_sqrt = (float)(1.0 / sqrt(bc2));
    int64_t want = (n / 4 + 255) / 256 + 1, cap = (int64_t)sm_count() * 16;
    int grid = (int)(want < cap ? want : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (grad_dtype == BRK_F16)
        adam_kernel<__half><<<grid, 256, 0, st>>>((float*)master_w, (float*)m, (float*)v, (const __half*)grad, (__half*)w16, n, step_size,
                                                  inv_bc2_sqrt, beta1, beta2, eps, grad_scale);
    else if (grad_dtype == BRK_F32)
        adam_kernel<float><<<grid, 256, 0, st>>>((float*)master_w, (float*)m, (float*)v, (const float*)grad, (__half*)w16, n, step_size,
                                                 inv_bc2_sqrt, beta1, beta2, eps, grad_scale);
    else
        return BRK_ATTR_ERROR;
    return launch_status("adam_kernel");
}

extern "C" int brk_embedding_scatter_add(const void* dx, const int32_t* ids, void* table_g, int64_t n, int64_t hidden, int64_t vocab,
                                         int dtype, void* stream) {
    if (!dx || !ids) return BRK_INPUT_ERROR;
    if (!table_g) return BRK_OUTPUT_ERROR;
    if (n < 0 || hidden <= 0 || vocab <= 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t cap = (int64_t)sm_count() * 16;
    if (dtype == BRK_F16) {
        if (hidden % 2 != 0 || (reinterpret_cast<uintptr_t>(dx) & 3) || (reinterpret_cast<uintptr_t>(table_g) & 3)) return BRK_ATTR_ERROR;
        int64_t want = (n * hidden / 2 + 255) / 256;
        scatter_add_kernel<__half><<<(int)(want < cap ? want : cap), 256, 0, st>>>((const __half*)dx, ids, (__half*)table_g, n, hidden, vocab);
    } else if (dtype == BRK_F32) {
        int64_t want = (n * hidden + 255) / 256;
        scatter_add_kernel<float><<<(int)(want < cap ? want : cap), 256, 0, st>>>((const float*)dx, ids, (float*)table_g, n, hidden, vocab);
    } else
        return BRK_ATTR_ERROR;
    return launch_status("scatter_add_kernel");
}

extern "C" int brk_init_normal(void* x, int64_t n, float mean, float std, uint64_t seed, int dtype, void* stream) {
    if (!x) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    if (n == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t want = ((n + 1) / 2 + 255) / 256, cap = (int64_t)sm_count() * 16;
    int grid = (int)(want < cap ? want : cap);
    if (dtype == BRK_F16) init_normal_kernel<__half><<<grid, 256, 0, st>>>((__half*)x, n, mean, std, seed);
    else if (dtype == BRK_F32) init_normal_kernel<float><<<grid, 256, 0, st>>>((float*)x, n, mean, std, seed);
    else return BRK_ATTR_ERROR;
    return launch_status("init_normal_kernel");
}

// Synchronous: 1 if an Adam launch since the last query skipped elements whose gradient was not finite.
extern "C" int brk_adam_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, brk::g_adam_nonfinite, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(brk::g_adam_nonfinite, &zero, sizeof(int));
    return v;
}
