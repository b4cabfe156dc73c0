// Fused causal attention forward with ALiBi and right-padding masks on the tcgen05 tensor cores.
//
//   S = Q K^T / sqrt(d) + slope_h * key_index,   keys allowed:  key <= query  and  key < len[b]
//   P = softmax(S),   O = P V
//
// Q, K, V are read in place from token-major activations ([batch*tokens, ld] with head h at
// columns h*d .. h*d+d-1, e.g. the three thirds of the fused QKV projection output), O is
// written token-major too, so the four [B,T,h,d] <-> [B,h,T,d] transposes of the unfused path
// and the T x T score / mask tensors never exist.  Also emitted: the row log-sum-exp [B,h,T]
// that the backward kernels need.
//
// One CTA per (128-query block, head, batch), 192 threads:
//   warp 0     TMA producer (Q once, then K / V tiles of 128 keys through 2-stage rings);
//   warp 1     issues tcgen05.mma: S = Q K_j^T into one of two TMEM score buffers, O += P V_j;
//   warps 2-5  one thread per query row: tcgen05.ld the scores, mask, exponentiate, write P as
//              fp16 into shared memory in the tensor core's swizzled operand layout.
// Softmax is two-sweep: sweep A accumulates the row maximum and normaliser over all key blocks,
// sweep B recomputes the scores and feeds normalised probabilities to the second contraction, so
// the output accumulator in TMEM never needs rescaling.  The score contraction runs twice; it is
// a third of the attention FLOPs, which are a few per cent of a decoder layer.
// Every mbarrier wait is bounded (see brk_ptx.cuh); a give-up raises g_attn_error.
#include <mutex>

#include "brk_common.cuh"
#include "brk_ptx.cuh"

namespace brk {

using namespace ptx;

constexpr int AT_BQ = 128;
constexpr int AT_BKV = 128;
constexpr int AT_THREADS = 192;

__device__ int g_attn_error = 0;

struct AttnFwdParams {
    __half* out;
    float* lse;            // [batch, heads, tokens], natural log
    const int32_t* lens;   // [batch] or null
    const float* slopes;   // [heads] or null
    int64_t ld_out;
    int batch, tokens, heads;
    float scale_log2;      // log2(e) / sqrt(d)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// byte offset of element (row, col) inside a [128 x 64*atoms] fp16 operand tile stored as
// 64-column atoms of 16 KB with 128-byte swizzle (the layout TMA writes and tcgen05 reads)
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
    const int atom = col >> 6, c = col & 63;
    return (uint32_t)(atom * 16384 + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1)));
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, AttnFwdParams p) {
    constexpr uint32_t TILE_BYTES = 128 * D * 2;          // Q, K, V tiles: 128 rows x D
    constexpr uint32_t P_BYTES = 128 * AT_BKV * 2;
    constexpr int KSTAGES = 2, VSTAGES = 2;
    constexpr uint32_t TMEM_COLS = 512;                   // S0 [0,128) S1 [128,256) O [256,256+D)
    constexpr uint32_t IDESC_S = make_idesc_f16_f32(128, AT_BKV, 0, 0);
    constexpr uint32_t IDESC_PV = make_idesc_f16_f32(128, D, 0, 1);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;
    unsigned char* sK = sQ + TILE_BYTES;
    unsigned char* sV = sK + KSTAGES * TILE_BYTES;
    unsigned char* sP = sV + VSTAGES * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
    uint64_t* q_full = bars;                 // 1
    uint64_t* k_full = bars + 1;             // KSTAGES
    uint64_t* k_empty = k_full + KSTAGES;
    uint64_t* v_full = k_empty + KSTAGES;    // VSTAGES
    uint64_t* v_empty = v_full + VSTAGES;
    uint64_t* s_full = v_empty + VSTAGES;    // 2
    uint64_t* s_empty = s_full + 2;          // 2
    uint64_t* p_full = s_empty + 2;          // 1
    uint64_t* p_empty = p_full + 1;          // 1
    uint64_t* o_full = p_empty + 1;          // 1
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(o_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy (late) query blocks are scheduled first
    const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int head = blockIdx.y, b = blockIdx.z;
    const int q0 = qblk * AT_BQ;
    const int len = p.lens ? min(max(p.lens[b], 0), p.tokens) : p.tokens;
    const int key_end = min(q0 + AT_BQ, len);                     // keys beyond are masked for every row of the tile
    const int nkb = key_end > 0 ? (key_end + AT_BKV - 1) / AT_BKV : 0;
    const int row_base = b * p.tokens;                             // first row of this sequence in the [B*T, ld] matrices
    const int col = head * D;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KSTAGES; s++) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VSTAGES; s++) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 128); }
        mbar_init(p_full, 128);
        mbar_init(p_empty, 1);
        mbar_init(o_full, 1);
        fence_barrier_init();
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;
    const uint32_t tmem_o = tmem_base + 256;

    if (nkb > 0) {
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                bool ok = true;
                mbar_arrive_expect_tx(q_full, TILE_BYTES);
#pragma unroll
                for (int a = 0; a < D / 64; a++) tma_load_2d(sQ + a * 16384, &tmap_q, q_full, col + a * 64, row_base + q0);
                uint32_t kit = 0, vit = 0;
                for (int sweep = 0; sweep < 2 && ok; sweep++) {
                    for (int j = 0; j < nkb && ok; j++) {
                        {
                            const int s = kit % KSTAGES;
                            ok = mbar_wait(&k_empty[s], ((kit / KSTAGES) & 1) ^ 1);
                            if (!ok) break;
                            mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
#pragma unroll
                            for (int a = 0; a < D / 64; a++)
                                tma_load_2d(sK + s * TILE_BYTES + a * 16384, &tmap_k, &k_full[s], col + a * 64, row_base + j * AT_BKV);
                            kit++;
                        }
                        if (sweep == 1) {
                            const int s = vit % VSTAGES;
                            ok = mbar_wait(&v_empty[s], ((vit / VSTAGES) & 1) ^ 1);
                            if (!ok) break;
                            mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
#pragma unroll
                            for (int a = 0; a < D / 64; a++)
                                tma_load_2d(sV + s * TILE_BYTES + a * 16384, &tmap_v, &v_full[s], col + a * 64, row_base + j * AT_BKV);
                            vit++;
                        }
                    }
                }
                if (!ok) atomicExch(&g_attn_error, 1);
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                bool ok = mbar_wait(q_full, 0);
                tcgen05_fence_after();
                const uint32_t q_addr = smem_u32(sQ);
                const uint32_t p_addr = smem_u32(sP);
                uint32_t kit = 0, vit = 0, sit = 0;   // K tiles consumed, V tiles consumed, score tiles produced
                auto issue_scores = [&](void) -> bool {
                    const int s = kit % KSTAGES, sb = sit & 1;
                    if (!mbar_wait(&s_empty[sb], ((sit >> 1) & 1) ^ 1)) return false;
                    if (!mbar_wait(&k_full[s], (kit / KSTAGES) & 1)) return false;
                    tcgen05_fence_after();
                    const uint32_t k_addr = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
                        umma_f16_ss(tmem_base + sb * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                                    make_smem_desc_sw128(k_addr + off, 16, 1024), IDESC_S, kk != 0 ? 1u : 0u);
                    }
                    umma_commit(&k_empty[s]);
                    umma_commit(&s_full[sb]);
                    kit++;
                    sit++;
                    return true;
                };
                // sweep A: scores only
                for (int j = 0; j < nkb && ok; j++) ok = issue_scores();
                // sweep B: scores one block ahead of the P V contraction
                if (ok) ok = issue_scores();
                for (int j = 0; j < nkb && ok; j++) {
                    if (j + 1 < nkb) ok = issue_scores();
                    if (!ok) break;
                    const int s = vit % VSTAGES;
                    ok = mbar_wait(&v_full[s], (vit / VSTAGES) & 1) && mbar_wait(p_full, j & 1);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t v_addr = smem_u32(sV + s * TILE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < AT_BKV / 16; kk++) {
                        // A = P [128 q x 128 keys], K-major; B = V [128 keys x D], d contiguous (MN-major)
                        const uint64_t da = make_smem_desc_sw128(p_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(v_addr + kk * 2048, 16384, 1024);
                        umma_f16_ss(tmem_o, da, db, IDESC_PV, (j | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&v_empty[s]);
                    umma_commit(p_empty);
                    vit++;
                }
                if (ok) umma_commit(o_full);
                if (!ok) atomicExch(&g_attn_error, 2);
            }
        } else {
            // ---------------- softmax / epilogue: one thread per query row ----------------
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;          // row inside the tile == TMEM lane
            const int qi = q0 + r;                       // query position in the sequence
            const int klimit = min(qi + 1, len);         // keys [0, klimit) are visible to this row
            const float slope2 = p.slopes ? p.slopes[head] * 1.4426950408889634f : 0.0f;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            float m = -INFINITY, l = 0.0f;
            uint32_t sit = 0;
            bool ok = true;
            // sweep A
            for (int j = 0; j < nkb && ok; j++, sit++) {
                const int sb = sit & 1;
                ok = mbar_wait(&s_full[sb], (sit >> 1) & 1);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < AT_BKV; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(lane_addr + sb * 128 + c0, v);
                    tmem_ld_wait();
                    const int kbase = j * AT_BKV + c0;
                    float t[32];
                    float cm = m;
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        const int kj = kbase + e;
                        t[e] = kj < klimit ? fmaf(__uint_as_float(v[e]), p.scale_log2, slope2 * (float)kj) : -INFINITY;
                        cm = fmaxf(cm, t[e]);
                    }
                    if (cm > m) {
                        l *= fast_exp2(m - cm);
                        m = cm;
                    }
                    if (m > -INFINITY) {
#pragma unroll
                        for (int e = 0; e < 32; e++) l += fast_exp2(t[e] - m);
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(&s_empty[sb]);
            }
            const float lse2 = (l > 0.0f) ? m + __log2f(l) : 0.0f;
            if (ok && qi < p.tokens && p.lse)
                p.lse[((int64_t)b * p.heads + head) * p.tokens + qi] = lse2 * 0.6931471805599453f;
            // sweep B
            for (int j = 0; j < nkb && ok; j++, sit++) {
                const int sb = sit & 1;
                ok = mbar_wait(&s_full[sb], (sit >> 1) & 1);
                if (!ok) break;
                if (j > 0) ok = mbar_wait(p_empty, (j - 1) & 1);   // previous P consumed by the tensor core
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < AT_BKV; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(lane_addr + sb * 128 + c0, v);
                    tmem_ld_wait();
                    const int kbase = j * AT_BKV + c0;
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint4 pk;
                        __half2* h2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int k0 = kbase + g * 8 + e * 2;
                            float p0 = k0 < klimit ? fast_exp2(fmaf(__uint_as_float(v[g * 8 + e * 2]), p.scale_log2, slope2 * (float)k0) - lse2) : 0.0f;
                            float p1 = k0 + 1 < klimit ? fast_exp2(fmaf(__uint_as_float(v[g * 8 + e * 2 + 1]), p.scale_log2, slope2 * (float)(k0 + 1)) - lse2) : 0.0f;
                            h2[e] = __floats2half2_rn(p0, p1);
                        }
                        *reinterpret_cast<uint4*>(sP + sw128_offset(r, c0 + g * 8)) = pk;
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(&s_empty[sb]);
                fence_proxy_async();          // make the generic-proxy writes of P visible to the tensor core
                mbar_arrive(p_full);
            }
            // epilogue: O -> fp16 -> global, token-major
            if (ok) ok = mbar_wait(o_full, 0);
            if (ok) {
                tcgen05_fence_after();
                __half* orow = p.out + (int64_t)(row_base + qi) * p.ld_out + col;
                const bool vec = (p.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(lane_addr + 256 + c0, v);
                    tmem_ld_wait();
                    if (qi < p.tokens) {
                        if (vec) {
#pragma unroll
                            for (int g = 0; g < 4; g++) {
                                Vec<__half> o;
#pragma unroll
                                for (int e = 0; e < 8; e++) o.v[e] = __uint_as_float(v[g * 8 + e]);
                                o.store(orow + c0 + g * 8);
                            }
                        } else {
                            for (int e = 0; e < 32; e++) orow[c0 + e] = __float2half_rn(__uint_as_float(v[e]));
                        }
                    }
                }
            }
            if (!ok && lane == 0) atomicExch(&g_attn_error, 3);
        }
    } else if (warp >= 2) {
        // no visible key for any row of this tile (len == 0): zero output, lse 0
        const int r = (warp & 3) * 32 + lane, qi = q0 + r;
        if (qi < p.tokens) {
            __half* orow = p.out + (int64_t)(row_base + qi) * p.ld_out + col;
            for (int e = 0; e < D; e++) orow[e] = __float2half_rn(0.0f);
            if (p.lse) p.lse[((int64_t)b * p.heads + head) * p.tokens + qi] = 0.0f;
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p, cudaStream_t st) {
    constexpr size_t smem = 1024 + (size_t)128 * D * 2 * 5 + 128 * AT_BKV * 2 + 256;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] { attr_err = cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "attn_fwd smem attribute");
        return BRK_CUDA_ERROR;
    }
    dim3 grid((unsigned)((p.tokens + AT_BQ - 1) / AT_BQ), (unsigned)p.heads, (unsigned)p.batch);
    attn_fwd_kernel<D><<<grid, AT_THREADS, smem, st>>>(tq, tk, tv, p);
    return launch_status("attn_fwd_kernel");
}

}  // namespace brk

extern "C" int brk_flash_attn_fwd(const void* q, const void* k, const void* v, int64_t ld_qkv, void* out, int64_t ld_out,
                                  float* lse, const int32_t* lens, const float* slopes, int batch, int tokens, int heads,
                                  int head_dim, void* stream) {
    using namespace brk;
    if (!q || !k || !v) return BRK_INPUT_ERROR;
    if (!out) return BRK_OUTPUT_ERROR;
    if (batch < 0 || tokens < 0 || heads <= 0 || (head_dim != 64 && head_dim != 128)) return BRK_ATTR_ERROR;
    if (ld_qkv % 8 != 0 || ld_qkv < (int64_t)heads * head_dim || ld_out < (int64_t)heads * head_dim) return BRK_ATTR_ERROR;
    if (batch == 0 || tokens == 0) return BRK_OK;
    if ((int64_t)batch * tokens > 0x7fffffff || heads > 65535 || batch > 65535) return BRK_ATTR_ERROR;
    const uint64_t rows = (uint64_t)batch * tokens, cols = (uint64_t)heads * head_dim;
    CUtensorMap tq, tk, tv;
    if (!make_tmap_2d_f16(&tq, q, rows, cols, (uint64_t)ld_qkv, 64, 128) || !make_tmap_2d_f16(&tk, k, rows, cols, (uint64_t)ld_qkv, 64, 128) ||
        !make_tmap_2d_f16(&tv, v, rows, cols, (uint64_t)ld_qkv, 64, 128)) {
        set_error_message("brk_flash_attn_fwd: could not encode a tensor map (pointers must be 16-byte aligned)");
        return BRK_CUDA_ERROR;
    }
    AttnFwdParams p;
    p.out = (__half*)out;
    p.lse = lse;
    p.lens = lens;
    p.slopes = slopes;
    p.ld_out = ld_out;
    p.batch = batch;
    p.tokens = tokens;
    p.heads = heads;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)head_dim));
    cudaStream_t st = (cudaStream_t)stream;
    if (head_dim == 128) return launch_attn_fwd<128>(tq, tk, tv, p, st);
    return launch_attn_fwd<64>(tq, tk, tv, p, st);
}

// Synchronous: non-zero if an attention kernel gave up on a bounded wait since the last query.
extern "C" int brk_flash_attn_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, brk::g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(brk::g_attn_error, &zero, sizeof(int));
    return v;
}
