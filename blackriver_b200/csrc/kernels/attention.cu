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
// Persistent CTAs (one per SM) walk the work items (128-query block, head, batch), 320 threads:
//   warp 0     TMA producer (Q per item, K / V tiles of 128 keys through 2-stage rings that run across items);
//   warp 1     issues tcgen05.mma: S = Q K_j^T into one of two TMEM score buffers, O += P V_j;
//   warps 2-9  two threads per query row (64 key columns each): tcgen05.ld the scores, mask, exponentiate, write P
//              as fp16 into one of two shared-memory tiles in the tensor core's swizzled operand layout.
// Softmax is online, in one sweep over the key blocks: each score and each exponential is computed
// once.  Probabilities are taken relative to a per-row reference maximum that moves only when the
// running maximum has run ahead of it by 2^8; only then is the output accumulator in tensor memory
// rescaled (read, multiplied, written back between two P V products), which after the first blocks
// of a row is rare.  The normaliser is applied once, in the epilogue.  With two score buffers and
// two probability tiles the tensor core computes S(j+1) and O += P(j-1) V while the row owners
// exponentiate block j.
// Every mbarrier wait is bounded (see brk_ptx.cuh); a give-up raises g_attn_error.
#include <mutex>

#include "brk_common.cuh"
#include "brk_ptx.cuh"
#include "brk_attn.cuh"

namespace brk {

using namespace ptx;

__device__ int g_attn_error = 0;

// Two row-owner warps per scheduler (warps 2..9): warps w and w + 4 own the same 32 tensor-memory lanes and split
// the columns of every tile between them; a single owner warp per scheduler cannot hide the latency of its own
// tensor-memory loads and exponentials.
constexpr int AT_FWD_THREADS = 64 + 256;

struct AttnFwdParams {
    __half* out;
    float* lse;            // [batch, heads, tokens], natural log
    const int32_t* lens;   // [batch] or null
    const float* slopes;   // [heads] or null
    int64_t ld_out;
    int batch, tokens, heads;
    float scale_log2;      // log2(e) / sqrt(d)
};

// Work items of the persistent attention kernels: (128-row block, head, batch) in the order of decreasing work -- the
// causal mask makes late blocks the long ones -- dealt to the CTAs in rounds that alternate direction (CTA c takes item
// c of the first round, item G-1-c of the second, ...), which evens out the totals without any atomic counter.
struct AttnTile {
    int blk, head, b;
};
__device__ __forceinline__ bool attn_tile(int round, int n_blk, int heads, int batch, AttnTile& t, bool late_blocks_first = true) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    const int hb = heads * batch;
    if (idx >= n_blk * hb) return false;
    t.blk = late_blocks_first ? n_blk - 1 - idx / hb : idx / hb;
    const int r = idx % hb;
    t.head = r % heads;
    t.b = r / heads;
    return true;
}

template <int D>
__global__ void __launch_bounds__(AT_FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, AttnFwdParams p) {
    constexpr uint32_t TILE_BYTES = 128 * D * 2;          // Q, K, V tiles: 128 rows x D
    constexpr uint32_t P_BYTES = 128 * AT_BKV * 2;
    constexpr int KSTAGES = 2, VSTAGES = 2;
    constexpr uint32_t TMEM_COLS = 512;                   // S0 [0,128) S1 [128,256) O [256,256+D)
    constexpr uint32_t IDESC_S = make_idesc_f16_f32(128, AT_BKV, 0, 0);
    constexpr uint32_t IDESC_PV = make_idesc_f16_f32(128, D, 0, 1);
    constexpr float RESCALE_STEP = 8.0f;                  // log2 units the row maximum may run ahead of the reference

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;
    unsigned char* sK = sQ + TILE_BYTES;
    unsigned char* sV = sK + KSTAGES * TILE_BYTES;
    unsigned char* sP = sV + VSTAGES * TILE_BYTES;        // two probability tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * P_BYTES);
    uint64_t* q_full = bars;                 // 1
    uint64_t* q_empty = bars + 1;            // 1
    uint64_t* k_full = bars + 2;             // KSTAGES
    uint64_t* k_empty = k_full + KSTAGES;
    uint64_t* v_full = k_empty + KSTAGES;    // VSTAGES
    uint64_t* v_empty = v_full + VSTAGES;
    uint64_t* s_full = v_empty + VSTAGES;    // 2
    uint64_t* s_empty = s_full + 2;          // 2
    uint64_t* p_full = s_empty + 2;          // 2
    uint64_t* p_empty = p_full + 2;          // 2
    uint64_t* o_full = p_empty + 2;          // 1
    uint64_t* o_empty = o_full + 1;          // 1
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(o_empty + 1);
    float* xch = reinterpret_cast<float*>(tmem_base_smem + 2);     // [2 halves][128 rows]: what the two owners of a row tell each other

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qblk = (p.tokens + AT_BQ - 1) / AT_BQ;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < KSTAGES; s++) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VSTAGES; s++) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; s++) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], 256);
            mbar_init(&p_full[s], 256);
            mbar_init(&p_empty[s], 1);
        }
        mbar_init(o_full, 1);
        mbar_init(o_empty, 256);
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

    // The CTA is persistent: every role walks the same list of work items; all barriers, the tensor memory and the
    // K / V rings live across items (running counters give buffer and phase), so the loads and the first scores of
    // the next item run under the epilogue of the current one.
    auto blocks_of = [&](const AttnTile& t) {
        const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
        const int key_end = min(t.blk * AT_BQ + AT_BQ, len);
        return key_end > 0 ? (key_end + AT_BKV - 1) / AT_BKV : 0;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            uint32_t kit = 0, tcount = 0;
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
                const int nkb = blocks_of(t);
                if (nkb == 0) continue;
                const int row_base = t.b * p.tokens, col = t.head * D;
                ok = mbar_wait(q_empty, (tcount & 1) ^ 1);          // the previous item's scores no longer read Q
                if (!ok) break;
                mbar_arrive_expect_tx(q_full, TILE_BYTES);
#pragma unroll
                for (int a = 0; a < D / 64; a++) tma_load_2d(sQ + a * 16384, &tmap_q, q_full, col + a * 64, row_base + t.blk * AT_BQ);
                for (int j = 0; j < nkb && ok; j++, kit++) {
                    const int s = kit % KSTAGES;
                    ok = mbar_wait(&k_empty[s], ((kit / KSTAGES) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
#pragma unroll
                    for (int a = 0; a < D / 64; a++)
                        tma_load_2d(sK + s * TILE_BYTES + a * 16384, &tmap_k, &k_full[s], col + a * 64, row_base + j * AT_BKV);
                    ok = mbar_wait(&v_empty[s], ((kit / VSTAGES) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
#pragma unroll
                    for (int a = 0; a < D / 64; a++)
                        tma_load_2d(sV + s * TILE_BYTES + a * 16384, &tmap_v, &v_full[s], col + a * 64, row_base + j * AT_BKV);
                }
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 1);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = true;
            const uint32_t q_addr = smem_u32(sQ);
            const uint32_t p_addr = smem_u32(sP);
            uint32_t it = 0, tcount = 0;          // key blocks issued so far (all items), items started
            // S(it) = Q K^T into score buffer it & 1 (free once the row owners have read the scores two blocks back)
            auto issue_scores = [&](uint32_t i) -> bool {
                const int s = i % KSTAGES, sb = i & 1;
                if (!mbar_wait(&s_empty[sb], ((i >> 1) & 1) ^ 1)) return false;
                if (!mbar_wait(&k_full[s], (i / KSTAGES) & 1)) return false;
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
                return true;
            };
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
                const int nkb = blocks_of(t);
                if (nkb == 0) continue;
                ok = mbar_wait(q_full, tcount & 1);
                if (!ok) break;
                tcgen05_fence_after();
                ok = issue_scores(it);
                for (int j = 0; j < nkb && ok; j++) {
                    if (j + 1 < nkb) ok = issue_scores(it + j + 1);      // the next scores run while the row owners work on S(j)
                    else umma_commit(q_empty);                           // last scores of the item issued: Q may be replaced
                    if (!ok) break;
                    const uint32_t i = it + j;
                    const int s = i % VSTAGES, pb = i & 1;
                    ok = mbar_wait(&v_full[s], (i / VSTAGES) & 1) && mbar_wait(&p_full[pb], (i >> 1) & 1);
                    if (ok && j == 0) ok = mbar_wait(o_empty, (tcount & 1) ^ 1);      // the previous item's output has been read
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t v_addr = smem_u32(sV + s * TILE_BYTES);
                    const uint32_t pj = p_addr + pb * P_BYTES;
#pragma unroll
                    for (int kk = 0; kk < AT_BKV / 16; kk++) {
                        // A = P [128 q x 128 keys], K-major; B = V [128 keys x D], d contiguous (MN-major)
                        const uint64_t da = make_smem_desc_sw128(pj + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(v_addr + kk * 2048, 16384, 1024);
                        umma_f16_ss(tmem_o, da, db, IDESC_PV, (j | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&v_empty[s]);
                    umma_commit(&p_empty[pb]);
                }
                if (ok) umma_commit(o_full);
                it += nkb;
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 2);
        }
    } else {
        // ---------------- softmax / epilogue: two threads per query row, 64 of the 128 key columns each ----------------
        // Online softmax in one sweep over the key blocks: probabilities are taken relative to a reference maximum
        // m_ref that is only moved (and the output accumulator rescaled) when the running maximum has run ahead of it
        // by more than RESCALE_STEP, so P stays within 2^RESCALE_STEP -- far inside fp16 -- and rescaling is rare.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;          // row inside the tile == TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int cbase = half * 64;                 // this thread's columns of a 128-key block
        bool ok = true;
        uint32_t it = 0, tcount = 0;
        // both owners of a row run the same steps and meet at the pair barrier in each of them, also after a bounded
        // wait gave up (the work is skipped, the barrier is not), so neither is left waiting for the other
        auto pair_barrier = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory"); };
        AttnTile t;
        for (int round = 0; attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
            const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
            const int nkb = blocks_of(t);
            const int q0 = t.blk * AT_BQ;
            const int qi = q0 + r;                       // query position in the sequence
            const int row_base = t.b * p.tokens, col = t.head * D;
            if (nkb == 0) {
                // no visible key for any row of this tile (len == 0): zero output, lse 0
                if (half == 0 && qi < p.tokens) {
                    __half* orow = p.out + (int64_t)(row_base + qi) * p.ld_out + col;
                    for (int e = 0; e < D; e++) orow[e] = __float2half_rn(0.0f);
                    if (p.lse) p.lse[((int64_t)t.b * p.heads + t.head) * p.tokens + qi] = 0.0f;
                }
                continue;
            }
            const int klimit = min(qi + 1, len);         // keys [0, klimit) are visible to this row
            const float slope2 = p.slopes ? p.slopes[t.head] * 1.4426950408889634f : 0.0f;
            float m_ref = -INFINITY, l = 0.0f;
            for (int j = 0; j < nkb; j++) {
                const uint32_t i = it + j;
                const int sb = i & 1;
                if (ok) ok = mbar_wait(&s_full[sb], (i >> 1) & 1);
                float tt[64];
                float bm = -INFINITY;
                const int kbase = j * AT_BKV + cbase;
                if (ok) {
                    tcgen05_fence_after();
                    // pass 1: scaled scores + ALiBi of this thread's 64 columns into registers, and their maximum;
                    // key kbase + e gets slope2 * (kbase + e) as one fused multiply-add on constants
                    const float base2 = slope2 * (float)kbase;
                    const bool plain = __all_sync(0xffffffffu, kbase + 64 <= klimit);     // no key of the chunk is masked for any row
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(lane_addr + sb * 128 + cbase + c * 32, v);
                        tmem_ld_wait();
                        if (plain) {
#pragma unroll
                            for (int e = 0; e < 32; e++) {
                                tt[c * 32 + e] = fmaf(__uint_as_float(v[e]), p.scale_log2, fmaf(slope2, (float)(c * 32 + e), base2));
                                bm = fmaxf(bm, tt[c * 32 + e]);
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; e++) {
                                const float x = fmaf(__uint_as_float(v[e]), p.scale_log2, fmaf(slope2, (float)(c * 32 + e), base2));
                                tt[c * 32 + e] = kbase + c * 32 + e < klimit ? x : -INFINITY;
                                bm = fmaxf(bm, tt[c * 32 + e]);
                            }
                        }
                    }
                    tcgen05_fence_before();
                    mbar_arrive(&s_empty[sb]);         // the scores are in registers: the tensor core may refill the buffer
                }
                xch[half * 128 + r] = bm;
                pair_barrier();
                bm = fmaxf(bm, xch[(half ^ 1) * 128 + r]);
                pair_barrier();               // the partner has read this thread's cell before it is written again
                if (!ok) continue;
                const bool move = bm > m_ref + RESCALE_STEP;          // also the first visible key of the row (m_ref = -inf)
                float factor = 1.0f;
                if (move) {
                    factor = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - bm);
                    m_ref = bm;
                    l *= factor;
                }
                if (j > 0 && __any_sync(0xffffffffu, move)) {
                    // the accumulator may only be touched between two P V products: wait for the previous one
                    ok = mbar_wait(&p_empty[(i - 1) & 1], ((i - 1) >> 1) & 1);
                    if (!ok) continue;
                    tcgen05_fence_after();
#pragma unroll 1
                    for (int d0 = half * (D / 2); d0 < (half + 1) * (D / 2); d0 += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(lane_addr + 256 + d0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
                        tmem_st_32x32b_x32(lane_addr + 256 + d0, v);
                    }
                    tmem_st_wait();
                    tcgen05_fence_before();
                }
                if (i >= 2) ok = mbar_wait(&p_empty[sb], ((i - 2) >> 1) & 1);   // P tile i & 1 consumed by the tensor core
                if (!ok) continue;
                unsigned char* pt = sP + sb * P_BYTES;
                // pass 2: probabilities relative to m_ref (a masked score is -inf and gives exactly 0)
#pragma unroll
                for (int g = 0; g < 8; g++) {
                    uint4 pk;
                    __half2* h2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float p0 = fast_exp2(tt[g * 8 + e * 2] - m_ref);
                        const float p1 = fast_exp2(tt[g * 8 + e * 2 + 1] - m_ref);
                        l += p0 + p1;
                        h2[e] = __floats2half2_rn(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(pt + sw128_offset(r, cbase + g * 8)) = pk;
                }
                fence_proxy_async();          // make the generic-proxy writes of P visible to the tensor core
                mbar_arrive(&p_full[sb]);
            }
            it += nkb;
            // the row's normaliser is the sum of its two owners' partial sums
            xch[half * 128 + r] = l;
            pair_barrier();
            l += xch[(half ^ 1) * 128 + r];
            pair_barrier();
            // epilogue: O / l -> fp16 -> global, token-major; log-sum-exp for the backward
            if (ok) ok = mbar_wait(o_full, tcount & 1);
            tcount++;
            if (ok) {
                tcgen05_fence_after();
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                if (half == 0 && qi < p.tokens && p.lse)
                    p.lse[((int64_t)t.b * p.heads + t.head) * p.tokens + qi] = l > 0.0f ? (m_ref + __log2f(l)) * 0.6931471805599453f : 0.0f;
                __half* orow = p.out + (int64_t)(row_base + qi) * p.ld_out + col;
                const bool vec = (p.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
#pragma unroll 1
                for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(lane_addr + 256 + c0, v);
                    tmem_ld_wait();
                    if (qi < p.tokens) {
                        if (vec) {
#pragma unroll
                            for (int g = 0; g < 4; g++) {
                                Vec<__half> o;
#pragma unroll
                                for (int e = 0; e < 8; e++) o.v[e] = __uint_as_float(v[g * 8 + e]) * inv;
                                o.store(orow + c0 + g * 8);
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; e++) orow[c0 + e] = __float2half_rn(__uint_as_float(v[e]) * inv);
                        }
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(o_empty);             // the accumulator may take the next item's first product
            }
        }
        if (!ok && lane == 0) atomicExch(&g_attn_error, 3);
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
    constexpr size_t smem = 1024 + (size_t)128 * D * 2 * 5 + 2 * 128 * AT_BKV * 2 + 192 + 2 * 128 * sizeof(float);
    static_assert(smem <= 232448, "the forward attention tile set must fit the 227 KB a CTA can have");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] { attr_err = cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "attn_fwd smem attribute");
        return BRK_CUDA_ERROR;
    }
    const int64_t items = (int64_t)((p.tokens + AT_BQ - 1) / AT_BQ) * p.heads * p.batch;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());       // persistent: one CTA per SM walks the items
    attn_fwd_kernel<D><<<grid, AT_FWD_THREADS, smem, st>>>(tq, tk, tv, p);
    return launch_status("attn_fwd_kernel");
}


// ==========================================================================================
// backward
//   delta_i = sum_d dO_i O_i                      (small pre-pass, [B,h,T] fp32)
//   P_ij  = exp(s_ij - lse_i)  (0 where masked)   recomputed from Q, K and the saved lse
//   dV_j  = sum_i P_ij dO_i            dP_ij = dO_i . V_j          dS_ij = P_ij (dP_ij - delta_i)
//   dQ_i  = (1/sqrt d) sum_j dS_ij K_j            dK_j = (1/sqrt d) sum_i dS_ij Q_i
// Two kernels with the forward's roles (TMA producer warp, one MMA-issuing thread, 128 row-owner threads), both
// software-pipelined over sub-blocks of 64 so that the tensor core always has the next scores to compute while the
// row owners exponentiate the current ones:
//   * the dK / dV kernel owns a 128-key block and walks the 64-query sub-blocks at or after it.  It works on the
//     TRANSPOSED scores, S^T = K Q^T and dP^T = V dO^T (keys on the tensor-memory lanes, 64 query columns), so a row
//     owner is a key: it writes P^T and dS^T rows, which are K-major A operands of dV += P^T dO and dK += dS^T Q as
//     they stand; the 64 queries' lse and delta come from shared memory;
//   * the dQ kernel owns a 128-query block and walks the 64-key sub-blocks before it: S = Q K^T, dP = dO V^T
//     (64 key columns), dS rows to shared memory, dQ += dS K.
// Both keep two score / dP buffers in tensor memory and two tiles of each shared-memory operand in flight.
// ==========================================================================================
struct AttnBwdParams {
    const float* lse;      // [B,h,T] natural log, from the forward
    const float* delta;    // [B,h,T]
    const int32_t* lens;
    const float* slopes;
    __half* dq;
    __half* dk;
    __half* dv;
    int64_t ld_g;
    int batch, tokens, heads;
    float scale_log2;      // log2(e)/sqrt(d)
    float scale;           // 1/sqrt(d)
};

constexpr int AT_SUB = 64;      // rows of the walked operand per pipeline step of the backward kernels

// delta = sum_d dO * O per (token row, head): d / 8 neighbouring lanes own one head of one row, 16 bytes of O and
// of dO each, and fold their partial sums with shuffles
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __half* out, const __half* dout, int64_t ld, float* delta, int batch, int tokens, int heads, int d) {
    const int lanes = d >> 3;                       // 16 for d = 128, 8 for d = 64
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t grp = t / lanes;                  // (row, head) index
    const int part = (int)(t % lanes);
    const int64_t total = (int64_t)batch * tokens * heads;
    float s = 0.0f;
    const bool live = grp < total;
    int h = 0;
    int64_t row = 0;
    if (live) {
        h = (int)(grp % heads);
        row = grp / heads;
        const uint4 a = *reinterpret_cast<const uint4*>(out + row * ld + (int64_t)h * d + part * 8);
        const uint4 c = *reinterpret_cast<const uint4*>(dout + row * ld + (int64_t)h * d + part * 8);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* ch = reinterpret_cast<const __half2*>(&c);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float2 x = __half22float2(ah[e]), y = __half22float2(ch[e]);
            s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
        }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (live && part == 0) {
        const int b = (int)(row / tokens), tk = (int)(row % tokens);
        delta[((int64_t)b * heads + h) * tokens + tk] = s;
    }
}

// writes 32 consecutive fp16 values of row r, columns [c0, c0+32) of a swizzled operand tile
__device__ __forceinline__ void store_tile_chunk(unsigned char* tile, int r, int c0, const float (&x)[32]) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint4 pk;
        __half2* h2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; e++) h2[e] = __floats2half2_rn(x[g * 8 + e * 2], x[g * 8 + e * 2 + 1]);
        *reinterpret_cast<uint4*>(tile + sw128_offset(r, c0 + g * 8)) = pk;
    }
}

// The backward kernels run two row-owner warps per scheduler (one warp alone cannot hide the latency of its own
// tensor-memory loads and exponentials): warps 2..9, where warps w and w + 4 own the same 32 tensor-memory lanes (a warp
// may only touch lanes 32 * (warp % 4) ...) and split the 64 columns of a sub-block between them.
constexpr int AT_BWD_THREADS = 64 + 256;
__device__ __forceinline__ void owners_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(AT_BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q64, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do64, AttnBwdParams p) {
    constexpr uint32_t KV_BYTES = 128 * D * 2;            // this block's K and V tiles
    constexpr uint32_t SUB_BYTES = AT_SUB * D * 2;        // a 64-query tile of Q or dO
    constexpr uint32_t PT_BYTES = 128 * AT_SUB * 2;       // P^T / dS^T tile: 128 keys x 64 queries
    constexpr uint32_t SUB_ATOM = AT_SUB * 128;           // bytes between the 64-column atoms of a 64-row tile
    constexpr uint32_t TMEM_COLS = 512;   // S^T x2 [0,128)  dP^T x2 [128,256)  dV [256,256+D)  dK [256+D,256+2D)
    constexpr uint32_t IDESC_ST = make_idesc_f16_f32(128, AT_SUB, 0, 0);
    constexpr uint32_t IDESC_ACC = make_idesc_f16_f32(128, D, 0, 1);
    constexpr int QS = 4;                                 // stages of the Q / dO ring

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sK = base;
    unsigned char* sV = sK + KV_BYTES;
    unsigned char* sQ = sV + KV_BYTES;                    // QS tiles: the streamed operand needs a ring deep enough to
    unsigned char* sDO = sQ + QS * SUB_BYTES;             // cover the latency of its loads (two stages left the kernel waiting for TMA)
    unsigned char* sPT = sDO + QS * SUB_BYTES;            // 1 tile (the owners hold the next one in registers meanwhile)
    unsigned char* sDST = sPT + PT_BYTES;                 // 1 tile
    float* stat = reinterpret_cast<float*>(sDST + PT_BYTES);          // [2][lse2 x 64 | delta x 64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(stat + 2 * 128);
    uint64_t* kv_full = bars;
    uint64_t* kv_empty = bars + 1;
    uint64_t* qdo_full = bars + 2;     // QS
    uint64_t* qdo_empty = bars + 6;    // QS
    uint64_t* s_full = bars + 10;      // 2
    uint64_t* s_empty = bars + 12;     // 2
    uint64_t* p_full = bars + 14;      // 1
    uint64_t* p_empty = bars + 15;     // 1
    uint64_t* acc_full = bars + 16;
    uint64_t* acc_empty = bars + 17;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 18);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kblk = (p.tokens + AT_BKV - 1) / AT_BKV;
    const int nsub = (p.tokens + AT_SUB - 1) / AT_SUB;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        mbar_init(kv_empty, 1);
        for (int i = 0; i < QS; i++) {
            mbar_init(&qdo_full[i], 1);
            mbar_init(&qdo_empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 256);
        }
        mbar_init(p_full, 256);
        mbar_init(p_empty, 1);
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 256);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    // persistent CTA: every role walks the same items (128-key block, head, batch), early key blocks -- the long ones --
    // first; a block no query can see (beyond the sequence's length) costs its owners only the zero fill
    auto steps_of = [&](const AttnTile& t) {
        const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
        return t.blk * AT_BKV < len ? nsub - (t.blk * AT_BKV) / AT_SUB : 0;
    };

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0, tcount = 0;
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_kblk, p.heads, p.batch, t, false); round++) {
                const int niter = steps_of(t);
                if (niter == 0) continue;
                const int k0 = t.blk * AT_BKV, sub0 = k0 / AT_SUB;
                const int row_base = t.b * p.tokens, col = t.head * D;
                ok = mbar_wait(kv_empty, (tcount & 1) ^ 1);       // the previous item's score products no longer read K / V
                if (!ok) break;
                mbar_arrive_expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
                for (int a = 0; a < D / 64; a++) {
                    tma_load_2d(sK + a * 16384, &tmap_k, kv_full, col + a * 64, row_base + k0);
                    tma_load_2d(sV + a * 16384, &tmap_v, kv_full, col + a * 64, row_base + k0);
                }
                for (int li = 0; li < niter && ok; li++, it++) {
                    const int qs = it % QS;
                    ok = mbar_wait(&qdo_empty[qs], ((it / QS) & 1) ^ 1);
                    if (!ok) break;
                    const int q0 = (sub0 + li) * AT_SUB;
                    mbar_arrive_expect_tx(&qdo_full[qs], 2 * SUB_BYTES);
#pragma unroll
                    for (int a = 0; a < D / 64; a++) {
                        tma_load_2d(sQ + qs * SUB_BYTES + a * SUB_ATOM, &tmap_q64, &qdo_full[qs], col + a * 64, row_base + q0);
                        tma_load_2d(sDO + qs * SUB_BYTES + a * SUB_ATOM, &tmap_do64, &qdo_full[qs], col + a * 64, row_base + q0);
                    }
                }
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 11);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            uint32_t it0 = 0, tcount = 0;
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_kblk, p.heads, p.batch, t, false); round++) {
                const int niter = steps_of(t);
                if (niter == 0) continue;
                ok = mbar_wait(kv_full, tcount & 1);
                // step li issues the transposed scores of sub-block li and then the accumulations of sub-block li - 1,
                // whose P^T / dS^T the row owners produced while the scores of li were being computed
                for (int li = 0; li <= niter && ok; li++) {
                    if (li < niter) {
                        const uint32_t i = it0 + li;
                        const int sb = i & 1, qs = i % QS;
                        ok = mbar_wait(&qdo_full[qs], (i / QS) & 1) && mbar_wait(&s_empty[sb], ((i >> 1) & 1) ^ 1);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t q_addr = smem_u32(sQ + qs * SUB_BYTES), do_addr = smem_u32(sDO + qs * SUB_BYTES);
#pragma unroll
                        for (int kk = 0; kk < D / 16; kk++)      // S^T = K Q^T : [128 keys x 64 queries]
                            umma_f16_ss(tmem_base + sb * AT_SUB, make_smem_desc_sw128(k_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                                        make_smem_desc_sw128(q_addr + (kk >> 2) * SUB_ATOM + (kk & 3) * 32, 16, 1024), IDESC_ST, kk != 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 0; kk < D / 16; kk++)      // dP^T = V dO^T
                            umma_f16_ss(tmem_base + 128 + sb * AT_SUB, make_smem_desc_sw128(v_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                                        make_smem_desc_sw128(do_addr + (kk >> 2) * SUB_ATOM + (kk & 3) * 32, 16, 1024), IDESC_ST, kk != 0 ? 1u : 0u);
                        umma_commit(&s_full[sb]);
                        if (li == niter - 1) umma_commit(kv_empty);      // last products of the item that read K / V
                    }
                    if (li >= 1) {
                        const int j = li - 1;
                        const uint32_t i = it0 + j;
                        const int qs = i % QS;
                        ok = mbar_wait(p_full, i & 1);
                        if (ok && j == 0) ok = mbar_wait(acc_empty, (tcount & 1) ^ 1);      // the previous item's dV / dK have been read
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t q_addr = smem_u32(sQ + qs * SUB_BYTES), do_addr = smem_u32(sDO + qs * SUB_BYTES);
                        const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sDST);
#pragma unroll
                        for (int kk = 0; kk < AT_SUB / 16; kk++)      // dV += P^T dO  (contraction over the 64 queries)
                            umma_f16_ss(tmem_base + 256, make_smem_desc_sw128(pt_addr + kk * 32, 16, 1024),
                                        make_smem_desc_sw128(do_addr + kk * 2048, SUB_ATOM, 1024), IDESC_ACC, (j | kk) != 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 0; kk < AT_SUB / 16; kk++)      // dK += dS^T Q
                            umma_f16_ss(tmem_base + 256 + D, make_smem_desc_sw128(dst_addr + kk * 32, 16, 1024),
                                        make_smem_desc_sw128(q_addr + kk * 2048, SUB_ATOM, 1024), IDESC_ACC, (j | kk) != 0 ? 1u : 0u);
                        umma_commit(&qdo_empty[qs]);
                        umma_commit(p_empty);
                    }
                }
                if (ok) umma_commit(acc_full);
                it0 += niter;
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 12);
        }
    } else {
        // ---------------- row owners: two threads per key, 32 of the 64 query columns each ----------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int c0 = half * 32;
        bool ok = true;
        uint32_t it0 = 0, tcount = 0;
        AttnTile t;
        for (int round = 0; attn_tile(round, n_kblk, p.heads, p.batch, t, false); round++) {
            const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
            const int niter = steps_of(t);
            const int k0 = t.blk * AT_BKV, sub0 = k0 / AT_SUB;
            const int row_base = t.b * p.tokens, col = t.head * D;
            const int kj = k0 + r;                               // this thread's key
            if (niter == 0) {
                if (half == 0 && kj < p.tokens) {
                    __half* dvrow = p.dv + (int64_t)(row_base + kj) * p.ld_g + col;
                    __half* dkrow = p.dk + (int64_t)(row_base + kj) * p.ld_g + col;
                    const uint4 z = make_uint4(0, 0, 0, 0);
                    for (int e = 0; e < D; e += 8) {
                        *reinterpret_cast<uint4*>(dvrow + e) = z;
                        *reinterpret_cast<uint4*>(dkrow + e) = z;
                    }
                }
                continue;
            }
            const bool k_ok = kj < len;
            const float slope2 = p.slopes ? p.slopes[t.head] * 1.4426950408889634f : 0.0f;
            const float bias2 = slope2 * (float)kj;              // the ALiBi term is constant along a key's row
            const int64_t stat_base = ((int64_t)t.b * p.heads + t.head) * p.tokens;
            for (int li = 0; li < niter; li++) {
                const uint32_t i = it0 + li;
                const int sb = i & 1;
                const int q0 = (sub0 + li) * AT_SUB;
                if (half == 0) {
                    // the sub-block's 64 lse (in log2 units) and 64 delta values, one per thread of the first four warps
                    const int qi = q0 + (r & 63);
                    float v = 0.0f;
                    if (qi < p.tokens) v = r < 64 ? p.lse[stat_base + qi] * 1.4426950408889634f : p.delta[stat_base + qi];
                    stat[sb * 128 + r] = v;
                }
                // Orders this step's writes after every thread's reads two steps ago.  Every owner warp reaches it in
                // every step, also one whose bounded wait gave up (it only skips the work), so nobody is left waiting.
                owners_barrier();
                if (ok) ok = mbar_wait(&s_full[sb], (i >> 1) & 1);
                if (!ok) continue;
                tcgen05_fence_after();
                const float4* lse4 = reinterpret_cast<const float4*>(stat + sb * 128 + c0);
                const float4* dlt4 = reinterpret_cast<const float4*>(stat + sb * 128 + 64 + c0);
                uint32_t sv[32], dv[32];
                tmem_ld_32x32b_x32(lane_addr + sb * AT_SUB + c0, sv);
                tmem_ld_32x32b_x32(lane_addr + 128 + sb * AT_SUB + c0, dv);
                tmem_ld_wait();
                float pr[32], ds[32];
                // a sub-block strictly below the diagonal, inside the sequence, needs no predicate at all
                const bool plain = __all_sync(0xffffffffu, k_ok && kj <= q0) && q0 + AT_SUB <= p.tokens;
                if (plain) {
#pragma unroll
                    for (int g = 0; g < 8; g++) {
                        const float4 l4 = lse4[g], d4 = dlt4[g];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float pe = fast_exp2(fmaf(__uint_as_float(sv[g * 4 + e]), p.scale_log2, bias2 - ls[e]));
                            pr[g * 4 + e] = pe;
                            ds[g * 4 + e] = pe * (__uint_as_float(dv[g * 4 + e]) - dd[e]);
                        }
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < 8; g++) {
                        const float4 l4 = lse4[g], d4 = dlt4[g];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int qi = q0 + c0 + g * 4 + e;
                            const bool vis = k_ok && kj <= qi && qi < p.tokens;
                            const float pe = vis ? fast_exp2(fmaf(__uint_as_float(sv[g * 4 + e]), p.scale_log2, bias2 - ls[e])) : 0.0f;
                            pr[g * 4 + e] = pe;
                            ds[g * 4 + e] = pe * (__uint_as_float(dv[g * 4 + e]) - dd[e]);
                        }
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(&s_empty[sb]);
                // P^T and dS^T wait in registers until the tensor core has consumed the previous sub-block's tile
                if (i >= 1) ok = mbar_wait(p_empty, (i - 1) & 1);
                if (!ok) continue;
                store_tile_chunk(sPT, r, c0, pr);
                store_tile_chunk(sDST, r, c0, ds);
                fence_proxy_async();
                mbar_arrive(p_full);
            }
            it0 += niter;
            if (ok) ok = mbar_wait(acc_full, tcount & 1);
            tcount++;
            if (ok) {
                tcgen05_fence_after();
                __half* dvrow = p.dv + (int64_t)(row_base + kj) * p.ld_g + col;
                __half* dkrow = p.dk + (int64_t)(row_base + kj) * p.ld_g + col;
#pragma unroll 1
                for (int d0 = half * (D / 2); d0 < (half + 1) * (D / 2); d0 += 32) {
                    uint32_t a[32], c[32];
                    tmem_ld_32x32b_x32(lane_addr + 256 + d0, a);
                    tmem_ld_32x32b_x32(lane_addr + 256 + D + d0, c);
                    tmem_ld_wait();
                    if (kj < p.tokens) {
#pragma unroll
                        for (int g = 0; g < 4; g++) {
                            Vec<__half> o1, o2;
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                o1.v[e] = __uint_as_float(a[g * 8 + e]);
                                o2.v[e] = __uint_as_float(c[g * 8 + e]) * p.scale;
                            }
                            o1.store(dvrow + d0 + g * 8);
                            o2.store(dkrow + d0 + g * 8);
                        }
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(acc_empty);           // the accumulators may take the next item's first products
            }
        }
        if (!ok && lane == 0) atomicExch(&g_attn_error, 13);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D>
__global__ void __launch_bounds__(AT_BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k64,
                   const __grid_constant__ CUtensorMap tmap_v64, const __grid_constant__ CUtensorMap tmap_do, AttnBwdParams p) {
    constexpr uint32_t Q_BYTES = 128 * D * 2;             // this block's Q and dO tiles
    constexpr uint32_t SUB_BYTES = AT_SUB * D * 2;        // a 64-key tile of K or V
    constexpr uint32_t DS_BYTES = 128 * AT_SUB * 2;       // dS tile: 128 queries x 64 keys
    constexpr uint32_t SUB_ATOM = AT_SUB * 128;
    constexpr uint32_t TMEM_COLS = 512;   // S x2 [0,128)  dP x2 [128,256)  dQ [256,256+D)
    constexpr uint32_t IDESC_S = make_idesc_f16_f32(128, AT_SUB, 0, 0);
    constexpr uint32_t IDESC_DQ = make_idesc_f16_f32(128, D, 0, 1);
    constexpr int KS = 4;                                 // stages of the K / V ring

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;
    unsigned char* sDO = sQ + Q_BYTES;
    unsigned char* sK = sDO + Q_BYTES;                    // KS tiles: a ring deep enough to cover the latency of the loads
    unsigned char* sV = sK + KS * SUB_BYTES;              // KS tiles
    unsigned char* sDS = sV + KS * SUB_BYTES;             // 2 tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * DS_BYTES);
    uint64_t* qdo_full = bars;
    uint64_t* qdo_empty = bars + 1;
    uint64_t* kv_full = bars + 2;      // KS
    uint64_t* kv_empty = bars + 6;     // KS
    uint64_t* s_full = bars + 10;      // 2
    uint64_t* s_empty = bars + 12;     // 2
    uint64_t* ds_full = bars + 14;     // 2
    uint64_t* ds_empty = bars + 16;    // 2
    uint64_t* acc_full = bars + 18;
    uint64_t* acc_empty = bars + 19;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 20);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qblk = (p.tokens + AT_BQ - 1) / AT_BQ;

    if (threadIdx.x == 0) {
        mbar_init(qdo_full, 1);
        mbar_init(qdo_empty, 1);
        for (int i = 0; i < KS; i++) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 256);
            mbar_init(&ds_full[i], 256);
            mbar_init(&ds_empty[i], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 256);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    // persistent CTA over the items (128-query block, head, batch), late query blocks first
    auto steps_of = [&](const AttnTile& t) {
        const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
        const int key_end = min(t.blk * AT_BQ + AT_BQ, len);
        return key_end > 0 ? (key_end + AT_SUB - 1) / AT_SUB : 0;      // 64-key sub-blocks any row of the tile sees
    };

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0, tcount = 0;
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
                const int niter = steps_of(t);
                if (niter == 0) continue;
                const int row_base = t.b * p.tokens, col = t.head * D, q0 = t.blk * AT_BQ;
                ok = mbar_wait(qdo_empty, (tcount & 1) ^ 1);       // the previous item's score products no longer read Q / dO
                if (!ok) break;
                mbar_arrive_expect_tx(qdo_full, 2 * Q_BYTES);
#pragma unroll
                for (int a = 0; a < D / 64; a++) {
                    tma_load_2d(sQ + a * 16384, &tmap_q, qdo_full, col + a * 64, row_base + q0);
                    tma_load_2d(sDO + a * 16384, &tmap_do, qdo_full, col + a * 64, row_base + q0);
                }
                for (int li = 0; li < niter && ok; li++, it++) {
                    const int ks = it % KS;
                    ok = mbar_wait(&kv_empty[ks], ((it / KS) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&kv_full[ks], 2 * SUB_BYTES);
#pragma unroll
                    for (int a = 0; a < D / 64; a++) {
                        tma_load_2d(sK + ks * SUB_BYTES + a * SUB_ATOM, &tmap_k64, &kv_full[ks], col + a * 64, row_base + li * AT_SUB);
                        tma_load_2d(sV + ks * SUB_BYTES + a * SUB_ATOM, &tmap_v64, &kv_full[ks], col + a * 64, row_base + li * AT_SUB);
                    }
                }
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 21);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
            uint32_t it0 = 0, tcount = 0;
            AttnTile t;
            for (int round = 0; ok && attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
                const int niter = steps_of(t);
                if (niter == 0) continue;
                ok = mbar_wait(qdo_full, tcount & 1);
                for (int li = 0; li <= niter && ok; li++) {
                    if (li < niter) {
                        const uint32_t i = it0 + li;
                        const int sb = i & 1, ks = i % KS;
                        ok = mbar_wait(&kv_full[ks], (i / KS) & 1) && mbar_wait(&s_empty[sb], ((i >> 1) & 1) ^ 1);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t k_addr = smem_u32(sK + ks * SUB_BYTES), v_addr = smem_u32(sV + ks * SUB_BYTES);
#pragma unroll
                        for (int kk = 0; kk < D / 16; kk++)      // S = Q K^T : [128 queries x 64 keys]
                            umma_f16_ss(tmem_base + sb * AT_SUB, make_smem_desc_sw128(q_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                                        make_smem_desc_sw128(k_addr + (kk >> 2) * SUB_ATOM + (kk & 3) * 32, 16, 1024), IDESC_S, kk != 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 0; kk < D / 16; kk++)      // dP = dO V^T
                            umma_f16_ss(tmem_base + 128 + sb * AT_SUB, make_smem_desc_sw128(do_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                                        make_smem_desc_sw128(v_addr + (kk >> 2) * SUB_ATOM + (kk & 3) * 32, 16, 1024), IDESC_S, kk != 0 ? 1u : 0u);
                        umma_commit(&s_full[sb]);
                        if (li == niter - 1) umma_commit(qdo_empty);     // last products of the item that read Q / dO
                    }
                    if (li >= 1) {
                        const int j = li - 1;
                        const uint32_t i = it0 + j;
                        const int sb = i & 1, ks = i % KS;
                        ok = mbar_wait(&ds_full[sb], (i >> 1) & 1);
                        if (ok && j == 0) ok = mbar_wait(acc_empty, (tcount & 1) ^ 1);      // the previous item's dQ has been read
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t k_addr = smem_u32(sK + ks * SUB_BYTES), ds_addr = smem_u32(sDS + sb * DS_BYTES);
#pragma unroll
                        for (int kk = 0; kk < AT_SUB / 16; kk++)      // dQ += dS K : A = dS [q x 64 keys] K-major, B = K [64 keys x d], d contiguous
                            umma_f16_ss(tmem_base + 256, make_smem_desc_sw128(ds_addr + kk * 32, 16, 1024),
                                        make_smem_desc_sw128(k_addr + kk * 2048, SUB_ATOM, 1024), IDESC_DQ, (j | kk) != 0 ? 1u : 0u);
                        umma_commit(&kv_empty[ks]);
                        umma_commit(&ds_empty[sb]);
                    }
                }
                if (ok) umma_commit(acc_full);
                it0 += niter;
                tcount++;
            }
            if (!ok) atomicExch(&g_attn_error, 22);
        }
    } else {
        // two threads per query row, 32 of the 64 key columns each
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int c0 = half * 32;
        bool ok = true;
        uint32_t it0 = 0, tcount = 0;
        AttnTile t;
        for (int round = 0; ok && attn_tile(round, n_qblk, p.heads, p.batch, t); round++) {
            const int len = p.lens ? min(max(p.lens[t.b], 0), p.tokens) : p.tokens;
            const int niter = steps_of(t);
            const int q0 = t.blk * AT_BQ;
            const int qi = q0 + r;
            const bool q_ok = qi < p.tokens;
            const int row_base = t.b * p.tokens, col = t.head * D;
            if (niter == 0) {
                if (half == 0 && q_ok) {
                    __half* dqrow = p.dq + (int64_t)(row_base + qi) * p.ld_g + col;
                    const uint4 z = make_uint4(0, 0, 0, 0);
                    for (int e = 0; e < D; e += 8) *reinterpret_cast<uint4*>(dqrow + e) = z;
                }
                continue;
            }
            const float slope2 = p.slopes ? p.slopes[t.head] * 1.4426950408889634f : 0.0f;
            const int64_t stat_base = ((int64_t)t.b * p.heads + t.head) * p.tokens;
            const float lse2 = q_ok ? p.lse[stat_base + qi] * 1.4426950408889634f : 0.0f;
            const float dlt = q_ok ? p.delta[stat_base + qi] : 0.0f;
            const int klimit = q_ok ? min(qi + 1, len) : 0;
            for (int li = 0; li < niter && ok; li++) {
                const uint32_t i = it0 + li;
                const int sb = i & 1;
                ok = mbar_wait(&s_full[sb], (i >> 1) & 1);
                if (!ok) break;
                if (i >= 2) ok = mbar_wait(&ds_empty[sb], ((i - 2) >> 1) & 1);
                if (!ok) break;
                tcgen05_fence_after();
                uint32_t sv[32], dv[32];
                tmem_ld_32x32b_x32(lane_addr + sb * AT_SUB + c0, sv);
                tmem_ld_32x32b_x32(lane_addr + 128 + sb * AT_SUB + c0, dv);
                tmem_ld_wait();
                float ds[32];
                const int kbase = li * AT_SUB + c0;
                // ALiBi + log-sum-exp term of key kbase + e as one fused multiply-add on constants (no int -> float per element)
                const float base2 = fmaf(slope2, (float)kbase, -lse2);
                const bool plain = __all_sync(0xffffffffu, kbase + 32 <= klimit);      // every key of the chunk visible to every row
                if (plain) {
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        const float pe = fast_exp2(fmaf(__uint_as_float(sv[e]), p.scale_log2, fmaf(slope2, (float)e, base2)));
                        ds[e] = pe * (__uint_as_float(dv[e]) - dlt);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        const float pe = kbase + e < klimit ? fast_exp2(fmaf(__uint_as_float(sv[e]), p.scale_log2, fmaf(slope2, (float)e, base2))) : 0.0f;
                        ds[e] = pe * (__uint_as_float(dv[e]) - dlt);
                    }
                }
                store_tile_chunk(sDS + sb * DS_BYTES, r, c0, ds);
                tcgen05_fence_before();
                mbar_arrive(&s_empty[sb]);
                fence_proxy_async();
                mbar_arrive(&ds_full[sb]);
            }
            it0 += niter;
            if (ok) ok = mbar_wait(acc_full, tcount & 1);
            tcount++;
            if (ok) {
                tcgen05_fence_after();
                __half* dqrow = p.dq + (int64_t)(row_base + qi) * p.ld_g + col;
#pragma unroll 1
                for (int d0 = half * (D / 2); d0 < (half + 1) * (D / 2); d0 += 32) {
                    uint32_t a[32];
                    tmem_ld_32x32b_x32(lane_addr + 256 + d0, a);
                    tmem_ld_wait();
                    if (q_ok) {
#pragma unroll
                        for (int g = 0; g < 4; g++) {
                            Vec<__half> o;
#pragma unroll
                            for (int e = 0; e < 8; e++) o.v[e] = __uint_as_float(a[g * 8 + e]) * p.scale;
                            o.store(dqrow + d0 + g * 8);
                        }
                    }
                }
                tcgen05_fence_before();
                mbar_arrive(acc_empty);
            }
        }
        if (!ok && lane == 0) atomicExch(&g_attn_error, 23);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                           const CUtensorMap& tq64, const CUtensorMap& tk64, const CUtensorMap& tv64, const CUtensorMap& tdo64,
                           const AttnBwdParams& p, cudaStream_t st) {
    // K, V + four 64-row tiles each of Q, dO + one tile each of P^T, dS^T + the lse / delta staging;
    // Q, dO + four 64-row tiles each of K, V + two dS tiles
    constexpr size_t smem_dkv = 1024 + (size_t)2 * 128 * D * 2 + 8 * (size_t)AT_SUB * D * 2 + 2 * (size_t)128 * AT_SUB * 2 + 1024 + 256;
    constexpr size_t smem_dq = 1024 + (size_t)2 * 128 * D * 2 + 8 * (size_t)AT_SUB * D * 2 + 2 * (size_t)128 * AT_SUB * 2 + 256;
    static_assert(smem_dkv <= 232448 && smem_dq <= 232448, "the backward attention tile sets must fit the 227 KB a CTA can have");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "attn_bwd smem attribute");
        return BRK_CUDA_ERROR;
    }
    const int64_t items = (int64_t)((p.tokens + AT_BQ - 1) / AT_BQ) * p.heads * p.batch;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());       // persistent: one CTA per SM walks the items
    attn_bwd_dkv_kernel<D><<<grid, AT_BWD_THREADS, smem_dkv, st>>>(tq64, tk, tv, tdo64, p);
    int rc = launch_status("attn_bwd_dkv_kernel");
    if (rc) return rc;
    attn_bwd_dq_kernel<D><<<grid, AT_BWD_THREADS, smem_dq, st>>>(tq, tk64, tv64, tdo, p);
    return launch_status("attn_bwd_dq_kernel");
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

extern "C" size_t brk_flash_attn_bwd_workspace_bytes(int batch, int tokens, int heads) {
    if (batch <= 0 || tokens <= 0 || heads <= 0) return 0;
    return (size_t)batch * tokens * heads * sizeof(float);
}

extern "C" int brk_flash_attn_bwd(const void* q, const void* k, const void* v, int64_t ld_qkv, const void* out, const void* d_out,
                                  int64_t ld_out, const float* lse, void* dq, void* dk, void* dv, int64_t ld_g,
                                  const int32_t* lens, const float* slopes, int batch, int tokens, int heads, int head_dim,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    using namespace brk;
    if (!q || !k || !v || !out || !d_out || !lse) return BRK_INPUT_ERROR;
    if (!dq || !dk || !dv) return BRK_OUTPUT_ERROR;
    if (batch < 0 || tokens < 0 || heads <= 0 || (head_dim != 64 && head_dim != 128)) return BRK_ATTR_ERROR;
    const int64_t hd = (int64_t)heads * head_dim;
    if (ld_qkv % 8 != 0 || ld_out % 8 != 0 || ld_g % 8 != 0 || ld_qkv < hd || ld_out < hd || ld_g < hd) return BRK_ATTR_ERROR;
    if ((reinterpret_cast<uintptr_t>(dq) & 15) || (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15)) return BRK_ATTR_ERROR;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(d_out) & 15)) return BRK_ATTR_ERROR;
    if (batch == 0 || tokens == 0) return BRK_OK;
    if ((int64_t)batch * tokens > 0x7fffffff || heads > 65535 || batch > 65535) return BRK_ATTR_ERROR;
    if (!workspace || workspace_bytes < brk_flash_attn_bwd_workspace_bytes(batch, tokens, heads)) return BRK_ATTR_ERROR;
    cudaStream_t st = (cudaStream_t)stream;
    float* delta = (float*)workspace;
    {
        int64_t threads = (int64_t)batch * tokens * heads * (head_dim / 8);
        unsigned blocks = (unsigned)((threads + 255) / 256);
        attn_delta_kernel<<<blocks, 256, 0, st>>>((const __half*)out, (const __half*)d_out, ld_out, delta, batch, tokens, heads, head_dim);
        int rc = launch_status("attn_delta_kernel");
        if (rc) return rc;
    }
    const uint64_t rows = (uint64_t)batch * tokens, cols = (uint64_t)hd;
    CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;      // boxes of 128 rows for the owned block, of 64 rows for the walked operand
    if (!make_tmap_2d_f16(&tq, q, rows, cols, (uint64_t)ld_qkv, 64, 128) || !make_tmap_2d_f16(&tk, k, rows, cols, (uint64_t)ld_qkv, 64, 128) ||
        !make_tmap_2d_f16(&tv, v, rows, cols, (uint64_t)ld_qkv, 64, 128) || !make_tmap_2d_f16(&tdo, d_out, rows, cols, (uint64_t)ld_out, 64, 128) ||
        !make_tmap_2d_f16(&tq64, q, rows, cols, (uint64_t)ld_qkv, 64, AT_SUB) || !make_tmap_2d_f16(&tk64, k, rows, cols, (uint64_t)ld_qkv, 64, AT_SUB) ||
        !make_tmap_2d_f16(&tv64, v, rows, cols, (uint64_t)ld_qkv, 64, AT_SUB) || !make_tmap_2d_f16(&tdo64, d_out, rows, cols, (uint64_t)ld_out, 64, AT_SUB)) {
        set_error_message("brk_flash_attn_bwd: could not encode a tensor map (pointers must be 16-byte aligned)");
        return BRK_CUDA_ERROR;
    }
    AttnBwdParams p;
    p.lse = lse;
    p.delta = delta;
    p.lens = lens;
    p.slopes = slopes;
    p.dq = (__half*)dq;
    p.dk = (__half*)dk;
    p.dv = (__half*)dv;
    p.ld_g = ld_g;
    p.batch = batch;
    p.tokens = tokens;
    p.heads = heads;
    p.scale = (float)(1.0 / sqrt((double)head_dim));
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)head_dim));
    if (head_dim == 128) return launch_attn_bwd<128>(tq, tk, tv, tdo, tq64, tk64, tv64, tdo64, p, st);
    return launch_attn_bwd<64>(tq, tk, tv, tdo, tq64, tk64, tv64, tdo64, p, st);
}
