// Vocabulary log-softmax + NLL (and its gradient) over materialised logits [rows, vocab].
//
// One CTA per row, CTAs persistent over rows.  Pass 1 streams the row once with 128-bit loads
// and keeps an online (max, sum-of-exp) pair per thread, so the maximum is never a separate
// pass; pairs are merged warp-wide by shuffles and CTA-wide through shared memory.  The
// forward-only form stops there (row loss = logsumexp - logit[target]).  The forward+gradient
// form makes a second sweep over the same row, which the first sweep left in L2 (the number of
// rows in flight is bounded so that they fit), and writes (softmax - onehot) * grad_scale.
// Rows whose target is outside [0, vocab) are ignored: their logits are never read and their
// gradient row is written as zeros.
#include "brk_common.cuh"

namespace brk {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int NLL_THREADS = 1024;
constexpr int NLL_UNROLL = 4;

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// merge (m2, s2) into (m, s); maxima are in natural units, -inf means "empty"
__device__ __forceinline__ void merge_ms(float& m, float& s, float m2, float s2) {
    float mm = fmaxf(m, m2);
    if (mm == -INFINITY) return;
    s = s * ex2f((m - mm) * LOG2E) + s2 * ex2f((m2 - mm) * LOG2E);
    m = mm;
}

template <typename T, bool VEC>
__device__ __forceinline__ void row_max_sum(const T* z, int64_t vocab, float& m_out, float& s_out, float* red) {
    constexpr int VN = Vec<T>::N;
    float m = -INFINITY, s = 0.0f;
    if (VEC) {
        const int64_t nvec = vocab / VN;
        for (int64_t base = threadIdx.x; base < nvec; base += (int64_t)NLL_THREADS * NLL_UNROLL) {
            uint4 raw[NLL_UNROLL];
            bool ok[NLL_UNROLL];
#pragma unroll
            for (int u = 0; u < NLL_UNROLL; u++) {
                int64_t i = base + (int64_t)u * NLL_THREADS;
                ok[u] = i < nvec;
                if (ok[u]) raw[u] = ld_raw(z + i * VN);
            }
#pragma unroll
            for (int u = 0; u < NLL_UNROLL; u++)
                if (ok[u]) {
                    Vec<T> v;
                    v.unpack(raw[u]);
                    float gm = v.v[0];
#pragma unroll
                    for (int e = 1; e < VN; e++) gm = fmaxf(gm, v.v[e]);
                    if (gm > m) {
                        s *= ex2f((m - gm) * LOG2E);  // m == -inf gives 0 * 0
                        m = gm;
                    }
                    const float mneg = -m * LOG2E;
#pragma unroll
                    for (int e = 0; e < VN; e++) s += ex2f(fmaf(v.v[e], LOG2E, mneg));
                }
        }
    } else {
        for (int64_t i = threadIdx.x; i < vocab; i += NLL_THREADS) {
            float x = to_f32(z[i]);
            if (x > m) {
                s *= ex2f((m - x) * LOG2E);
                m = x;
            }
            s += ex2f((x - m) * LOG2E);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        merge_ms(m, s, m2, s2);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
        red[warp] = m;
        red[32 + warp] = s;
    }
    __syncthreads();
    m = lane < NLL_THREADS / 32 ? red[lane] : -INFINITY;
    s = lane < NLL_THREADS / 32 ? red[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        merge_ms(m, s, m2, s2);
    }
    m_out = m;
    s_out = s;
}

template <typename T, bool VEC, bool BWD>
__global__ void __launch_bounds__(NLL_THREADS, 1)
nll_kernel(const T* logits, const int32_t* __restrict__ target, float* __restrict__ row_loss,
           float* __restrict__ row_lse, T* dlogits, int64_t rows, int64_t vocab, float grad_scale, const int32_t* __restrict__ count) {
    // with a device-side count of contributing rows the factor becomes grad_scale / count (mean over counted rows)
    if (count != nullptr) {
        const int32_t c = *count;
        grad_scale = grad_scale / (float)(c > 0 ? c : 1);
    }
    constexpr int VN = Vec<T>::N;
    __shared__ float red[64];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int32_t tg = target[row];
        const bool counted = tg >= 0 && (int64_t)tg < vocab;
        const T* z = logits + row * vocab;
        if (!counted) {
            if (threadIdx.x == 0) {
                row_loss[row] = 0.0f;
                if (row_lse) row_lse[row] = 0.0f;
            }
            if (BWD) {
                T* dz = dlogits + row * vocab;
                if (VEC) {
                    Vec<T> zero;
#pragma unroll
                    for (int e = 0; e < VN; e++) zero.v[e] = 0.0f;
                    for (int64_t i = threadIdx.x; i < vocab / VN; i += NLL_THREADS) zero.store_stream(dz + i * VN);
                } else {
                    for (int64_t i = threadIdx.x; i < vocab; i += NLL_THREADS) dz[i] = from_f32<T>(0.0f);
                }
            }
            continue;
        }
        float m, s;
        row_max_sum<T, VEC>(z, vocab, m, s, red);
        const float lse = m + __log2f(s) * LN2;
        if (threadIdx.x == 0) {
            row_loss[row] = lse - to_f32(z[tg]);
            if (row_lse) row_lse[row] = lse;
        }
        if (BWD) {
            __syncthreads();  // z[tg] was read above and dz may alias z
            T* dz = dlogits + row * vocab;
            const float lneg = -lse * LOG2E;
            if (VEC) {
                const int64_t nvec = vocab / VN;
                const int64_t tvec = tg / VN;
                const int te = tg % VN;
                for (int64_t base = threadIdx.x; base < nvec; base += (int64_t)NLL_THREADS * NLL_UNROLL) {
                    uint4 raw[NLL_UNROLL];
                    bool ok[NLL_UNROLL];
#pragma unroll
                    for (int u = 0; u < NLL_UNROLL; u++) {
                        int64_t i = base + (int64_t)u * NLL_THREADS;
                        ok[u] = i < nvec;
                        if (ok[u]) raw[u] = ld_raw_stream(z + i * VN);
                    }
#pragma unroll
                    for (int u = 0; u < NLL_UNROLL; u++)
                        if (ok[u]) {
                            int64_t i = base + (int64_t)u * NLL_THREADS;
                            Vec<T> v;
                            v.unpack(raw[u]);
#pragma unroll
                            for (int e = 0; e < VN; e++) v.v[e] = ex2f(fmaf(v.v[e], LOG2E, lneg)) * grad_scale;
                            if (i == tvec) {
#pragma unroll
                                for (int e = 0; e < VN; e++)
                                    if (e == te) v.v[e] -= grad_scale;
                            }
                            v.store_stream(dz + i * VN);
                        }
                }
            } else {
                for (int64_t i = threadIdx.x; i < vocab; i += NLL_THREADS) {
                    float p = ex2f(fmaf(to_f32(z[i]), LOG2E, lneg)) * grad_scale;
                    if (i == tg) p -= grad_scale;
                    dz[i] = from_f32<T>(p);
                }
            }
        }
    }
}

template <typename T, bool BWD>
static int nll_dispatch(const void* logits_, const int32_t* target, float* row_loss, float* row_lse, void* dlogits_,
                        int64_t rows, int64_t vocab, float grad_scale, const int32_t* count, cudaStream_t st) {
    const T* logits = (const T*)logits_;
    T* dlogits = (T*)dlogits_;
    constexpr int VN = Vec<T>::N;
    bool vec = (vocab % VN == 0) && aligned16(logits) && (!BWD || aligned16(dlogits));
    int64_t cap = (int64_t)sm_count();
    int grid = (int)(rows < cap ? rows : cap);
    if (vec)
        nll_kernel<T, true, BWD><<<grid, NLL_THREADS, 0, st>>>(logits, target, row_loss, row_lse, dlogits, rows, vocab, grad_scale, count);
    else
        nll_kernel<T, false, BWD><<<grid, NLL_THREADS, 0, st>>>(logits, target, row_loss, row_lse, dlogits, rows, vocab, grad_scale, count);
    return launch_status("nll_kernel");
}

// Single CTA, fixed summation order.
__global__ void __launch_bounds__(1024) sum_f32_kernel(const float* x, float* out, int64_t n) {
    __shared__ float red[64];
    float a = 0.0f, b = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) a += x[i];
    block_sum2(a, b, red);
    if (threadIdx.x == 0) out[0] = a;
}

// out[0] = (sum of x) / max(count, 1), single CTA, fixed order: the mean loss without a host round trip
__global__ void __launch_bounds__(1024) sum_div_f32_kernel(const float* x, const int32_t* count, float* out, int64_t n) {
    __shared__ float red[64];
    float a = 0.0f, b = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) a += x[i];
    block_sum2(a, b, red);
    if (threadIdx.x == 0) {
        const int32_t c = *count;
        out[0] = a / (float)(c > 0 ? c : 1);
    }
}

__global__ void signal_u32_kernel(volatile uint32_t* flag, uint32_t value) {
    __threadfence_system();
    *flag = value;
}

__global__ void loss_targets_kernel(const int32_t* ids, const int32_t* mask, int32_t* target, int32_t* count, int batch,
                                    int tokens) {
    // one CTA; the count is a popcount-style reduction in a fixed order
    __shared__ int red[32];
    int local = 0;
    const int64_t n = (int64_t)batch * tokens;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        int t = (int)(i % tokens);
        int32_t tg = -100;
        if (t < tokens - 1 && mask[i] != 0 && mask[i + 1] != 0) {
            tg = ids[i + 1];
            local++;
        }
        target[i] = tg;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x < 32) {
        int v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) count[0] = v;
    }
}

}  // namespace brk

extern "C" int brk_logsoftmax_nll_fwd(const void* logits, const int32_t* target, float* row_loss, float* row_lse,
                                      int64_t rows, int64_t vocab, int dtype, void* stream) {
    if (!logits || !target) return BRK_INPUT_ERROR;
    if (!row_loss) return BRK_OUTPUT_ERROR;
    if (rows < 0 || vocab <= 0 || vocab > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::nll_dispatch<float, false>(logits, target, row_loss, row_lse, nullptr, rows, vocab, 0.0f, nullptr, st);
    if (dtype == BRK_F16) return brk::nll_dispatch<__half, false>(logits, target, row_loss, row_lse, nullptr, rows, vocab, 0.0f, nullptr, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_logsoftmax_nll_fwd_bwd(const void* logits, const int32_t* target, float* row_loss, void* dlogits,
                                          int64_t rows, int64_t vocab, float grad_scale, int dtype, void* stream) {
    if (!logits || !target) return BRK_INPUT_ERROR;
    if (!row_loss || !dlogits) return BRK_OUTPUT_ERROR;
    if (rows < 0 || vocab <= 0 || vocab > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::nll_dispatch<float, true>(logits, target, row_loss, nullptr, dlogits, rows, vocab, grad_scale, nullptr, st);
    if (dtype == BRK_F16) return brk::nll_dispatch<__half, true>(logits, target, row_loss, nullptr, dlogits, rows, vocab, grad_scale, nullptr, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_logsoftmax_nll_fwd_bwd_counted(const void* logits, const int32_t* target, float* row_loss, void* dlogits,
                                                  int64_t rows, int64_t vocab, float scale_numerator, const int32_t* count,
                                                  int dtype, void* stream) {
    if (!logits || !target || !count) return BRK_INPUT_ERROR;
    if (!row_loss || !dlogits) return BRK_OUTPUT_ERROR;
    if (rows < 0 || vocab <= 0 || vocab > 0x7fffffffLL) return BRK_ATTR_ERROR;
    if (rows == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32) return brk::nll_dispatch<float, true>(logits, target, row_loss, nullptr, dlogits, rows, vocab, scale_numerator, count, st);
    if (dtype == BRK_F16) return brk::nll_dispatch<__half, true>(logits, target, row_loss, nullptr, dlogits, rows, vocab, scale_numerator, count, st);
    return BRK_ATTR_ERROR;
}

extern "C" int brk_sum_div_f32(const float* x, const int32_t* count, float* out, int64_t n, void* stream) {
    if (!x || !count) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    brk::sum_div_f32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(x, count, out, n);
    return brk::launch_status("sum_div_f32_kernel");
}

extern "C" int brk_signal_u32(uint32_t* flag, uint32_t value, void* stream) {
    if (!flag) return BRK_OUTPUT_ERROR;
    brk::signal_u32_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, value);
    return brk::launch_status("signal_u32_kernel");
}

extern "C" int brk_sum_f32(const float* x, float* out, int64_t n, void* stream) {
    if (!x) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (n < 0) return BRK_ATTR_ERROR;
    brk::sum_f32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(x, out, n);
    return brk::launch_status("sum_f32_kernel");
}

extern "C" int brk_loss_targets(const int32_t* ids, const int32_t* mask, int32_t* target, int32_t* count, int batch,
                                int tokens, void* stream) {
    if (!ids || !mask) return BRK_INPUT_ERROR;
    if (!target || !count) return BRK_OUTPUT_ERROR;
    if (batch < 0 || tokens < 0) return BRK_ATTR_ERROR;
    brk::loss_targets_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, mask, target, count, batch, tokens);
    return brk::launch_status("loss_targets_kernel");
}
