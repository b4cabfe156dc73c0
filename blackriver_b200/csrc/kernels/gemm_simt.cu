// General strided-batched GEMM on CUDA cores with fp32 accumulation.  This is the fp32 parity
// path (single-layer checks against the CPU oracle need full fp32 products, which the tensor
// cores do not provide) and the small/odd-shape fallback; throughput-critical fp16 GEMMs go
// through the tcgen05 kernels instead.
//
// 64x64 output tile per CTA, K step 16, 256 threads, 4x4 accumulators per thread, operands
// staged through shared memory; every access is bounds-checked so any m, n, k, stride and
// alignment is accepted.
#include "brk_common.cuh"

namespace brk {

constexpr int GT_M = 64, GT_N = 64, GT_K = 16;

template <typename T, bool TA, bool TB>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* A, const T* B, T* C, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                 int64_t sa, int64_t sb, int64_t sc, float alpha, float beta, const T* bias) {
    __shared__ float As[GT_K][GT_M + 4];
    __shared__ float Bs[GT_K][GT_N + 4];
    const int64_t bz = blockIdx.z;
    A += bz * sa;
    B += bz * sb;
    C += bz * sc;
    const int64_t m0 = (int64_t)blockIdx.y * GT_M, n0 = (int64_t)blockIdx.x * GT_N;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 rows x 4 cols
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < k; k0 += GT_K) {
#pragma unroll
        for (int it = 0; it < 4; it++) {
            int e = tid + it * 256;
            int ai, ak;
            if (TA) { ai = e & 63; ak = e >> 6; } else { ak = e & 15; ai = e >> 4; }
            int64_t gi = m0 + ai, gk = k0 + ak;
            float v = 0.0f;
            if (gi < m && gk < k) v = to_f32(TA ? A[gk * lda + gi] : A[gi * lda + gk]);
            As[ak][ai] = v;
            int bj, bk;
            if (TB) { bk = e & 15; bj = e >> 4; } else { bj = e & 63; bk = e >> 6; }
            int64_t gj = n0 + bj;
            gk = k0 + bk;
            v = 0.0f;
            if (gj < n && gk < k) v = to_f32(TB ? B[gj * ldb + gk] : B[gk * ldb + gj]);
            Bs[bk][bj] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GT_K; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int64_t gi = m0 + ty * 4 + i;
        if (gi >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int64_t gj = n0 + tx * 4 + j;
            if (gj >= n) continue;
            float v = alpha * acc[i][j];
            if (bias) v += to_f32(bias[gj]);
            if (beta != 0.0f) v += beta * to_f32(C[gi * ldc + gj]);
            C[gi * ldc + gj] = from_f32<T>(v);
        }
    }
}

template <typename T>
static int gemm_dispatch(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int ta, int tb, int64_t lda,
                         int64_t ldb, int64_t ldc, int64_t batch, int64_t sa, int64_t sb, int64_t sc, float alpha,
                         float beta, const void* bias, cudaStream_t st) {
    dim3 grid((unsigned)((n + GT_N - 1) / GT_N), (unsigned)((m + GT_M - 1) / GT_M), (unsigned)batch);
    if (grid.y > 65535 || grid.z > 65535) return BRK_ATTR_ERROR;
    const T* A = (const T*)a;
    const T* B = (const T*)b;
    T* C = (T*)c;
    const T* bs = (const T*)bias;
    if (!ta && !tb)
        gemm_simt_kernel<T, false, false><<<grid, 256, 0, st>>>(A, B, C, m, n, k, lda, ldb, ldc, sa, sb, sc, alpha, beta, bs);
    else if (!ta && tb)
        gemm_simt_kernel<T, false, true><<<grid, 256, 0, st>>>(A, B, C, m, n, k, lda, ldb, ldc, sa, sb, sc, alpha, beta, bs);
    else if (ta && !tb)
        gemm_simt_kernel<T, true, false><<<grid, 256, 0, st>>>(A, B, C, m, n, k, lda, ldb, ldc, sa, sb, sc, alpha, beta, bs);
    else
        gemm_simt_kernel<T, true, true><<<grid, 256, 0, st>>>(A, B, C, m, n, k, lda, ldb, ldc, sa, sb, sc, alpha, beta, bs);
    return launch_status("gemm_simt_kernel");
}

}  // namespace brk

extern "C" int brk_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                        int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t sa, int64_t sb, int64_t sc, float alpha,
                        float beta, const void* bias, int dtype, void* stream) {
    if (!a || !b) return BRK_INPUT_ERROR;
    if (!c) return BRK_OUTPUT_ERROR;
    if (m < 0 || n < 0 || k < 0 || batch < 0) return BRK_ATTR_ERROR;
    if (m == 0 || n == 0 || batch == 0) return BRK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BRK_F32)
        return brk::gemm_dispatch<float>(a, b, c, m, n, k, trans_a, trans_b, lda, ldb, ldc, batch, sa, sb, sc, alpha, beta, bias, st);
    if (dtype == BRK_F16)
        return brk::gemm_dispatch<__half>(a, b, c, m, n, k, trans_a, trans_b, lda, ldb, ldc, batch, sa, sb, sc, alpha, beta, bias, st);
    return BRK_ATTR_ERROR;
}
