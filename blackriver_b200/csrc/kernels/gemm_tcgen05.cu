// fp16 GEMM on the 5th-generation tensor cores: C[m,n] = op(A) op(B) (+bias) (+residual) (+C),
// fp32 accumulation in tensor memory, optional second output gelu(C).
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: streams 128 x 64 (A) and BN x 64 (B) fp16 tiles, 128-byte swizzled,
//               into a 4-stage shared-memory ring (plain cp.async.bulk.tensor, no multicast);
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16, four per stage) into
//               one of two TMEM accumulators and commits completion to mbarriers;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (32 lanes x 32 columns per load),
//               apply bias / residual / accumulate / GELU, convert to fp16 and store, while the
//               issuer already fills the other accumulator with the next tile.
// Operands may be K-major or MN-major in memory (all four transposition cases of the backward
// pass); the shared-memory descriptors and the instruction descriptor carry the difference.
// Tails in m, n, k are handled by TMA zero fill on loads and predication on stores.
#include <cstring>
#include <mutex>

#include "brk_common.cuh"
#include "brk_ptx.cuh"

namespace brk {

using namespace ptx;

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 192;

// set when a bounded wait gives up; read by brk_gemm_f16_status()
__device__ int g_tc_error = 0;

struct TcParams {
    __half* c;
    const __half* bias;
    const __half* residual;
    __half* gelu_out;
    int64_t ldc, ldr, ldg;
    int m, n, k;
    int accumulate;
    int tiles_m, tiles_n;
    int splits;      // CTA-pair kernel, staged epilogue only: each tile's k range is cut into this many work items
};

__device__ __forceinline__ float tc_gelu(float x) {
    float e = __expf(2.0f * 0.79788456f * x * (1.0f + 0.044715f * x * x));
    float t = 1.0f - __fdividef(2.0f, e + 1.0f);
    return x * 0.5f * (1.0f + t);
}

// Epilogue of one accumulator chunk: 32 consecutive columns of one output row held by this thread.
__device__ __forceinline__ void tc_store_chunk(const TcParams& p, const uint32_t (&v)[32], int row, bool row_ok, int col0, bool vec_ok) {
    if (!(row_ok && col0 < p.n)) return;
    __half* crow = p.c + (int64_t)row * p.ldc + col0;
    const __half* rrow = p.residual ? p.residual + (int64_t)row * p.ldr + col0 : nullptr;
    __half* grow = p.gelu_out ? p.gelu_out + (int64_t)row * p.ldg + col0 : nullptr;
    if (vec_ok && col0 + 32 <= p.n) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; e++) f[e] = __uint_as_float(v[q * 8 + e]);
            if (p.bias) {
                Vec<__half> b;
                b.load(p.bias + col0 + q * 8);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] += b.v[e];
            }
            if (rrow) {
                Vec<__half> r;
                r.load(rrow + q * 8);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] += r.v[e];
            }
            if (p.accumulate) {
                Vec<__half> o;
                o.load(crow + q * 8);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] += o.v[e];
            }
            Vec<__half> out;
#pragma unroll
            for (int e = 0; e < 8; e++) out.v[e] = f[e];
            out.store(crow + q * 8);
            if (grow) {
#pragma unroll
                for (int e = 0; e < 8; e++) out.v[e] = tc_gelu(f[e]);
                out.store(grow + q * 8);
            }
        }
    } else {
#pragma unroll
        for (int e = 0; e < 32; e++) {       // fully unrolled so that v stays in registers
            if (col0 + e >= p.n) break;
            float f = __uint_as_float(v[e]);
            if (p.bias) f += __half2float(p.bias[col0 + e]);
            if (rrow) f += __half2float(rrow[e]);
            if (p.accumulate) f += __half2float(crow[e]);
            crow[e] = __float2half_rn(f);
            if (grow) grow[e] = __float2half_rn(tc_gelu(f));
        }
    }
}

__device__ __forceinline__ bool tc_vec_ok(const TcParams& p) {
    return (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) &&
           (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) &&
           (!p.residual || ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0))) &&
           (!p.gelu_out || ((p.ldg % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.gelu_out) & 15) == 0)));
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, TcParams p) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators; 256 or 512 columns
    constexpr uint32_t IDESC = make_idesc_f16_f32(TC_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + TC_STAGES;
    uint64_t* tmem_full = empty_bar + TC_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.k + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
        }
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                for (int kb = 0; kb < kblocks && ok; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(&empty_bar[s], ((it / TC_STAGES) & 1) ^ 1);
                    if (!ok) break;
                    unsigned char* sa = tiles + s * STAGE_BYTES;
                    unsigned char* sb = sa + A_BYTES;
                    mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
                    if (!A_MN) {
                        tma_load_2d(sa, &tmap_a, &full_bar[s], kb * TC_BK, tm * TC_BM);
                    } else {
#pragma unroll
                        for (int j = 0; j < TC_BM / 64; j++)
                            tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[s], tm * TC_BM + j * 64, kb * TC_BK);
                    }
                    if (!B_MN) {
                        tma_load_2d(sb, &tmap_b, &full_bar[s], kb * TC_BK, tn * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; j++)
                            tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[s], tn * BN + j * 64, kb * TC_BK);
                    }
                }
            }
            if (!ok) atomicExch(&g_tc_error, 1);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
                const int buf = tcount & 1;
                ok = mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks && ok; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(&full_bar[s], (it / TC_STAGES) & 1);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(tiles + s * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        // K-major: 16 elements = 32 bytes further inside the 128-byte swizzle row;
                        // MN-major: 16 k-rows of 128 bytes further, 64-element groups 8 KB apart
                        const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                                 : make_smem_desc_sw128(sa + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                                 : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
                        umma_f16_ss(d_tmem, da, db, IDESC, (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(&tmem_full[buf]);
            }
            if (!ok) atomicExch(&g_tc_error, 2);
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32*quarter .. +31
        uint32_t tcount = 0;
        bool ok = true;
        const bool vec_ok = tc_vec_ok(p);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int buf = tcount & 1;
            ok = mbar_wait(&tmem_full[buf], (tcount >> 1) & 1);
            if (!ok) break;
            tcgen05_fence_after();
            const int row = tm * TC_BM + quarter * 32 + lane;
            const bool row_ok = row < p.m;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, v);
                tmem_ld_wait();
                tc_store_chunk(p, v, row, row_ok, tn * BN + c0, vec_ok);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        if (!ok && lane == 0) atomicExch(&g_tc_error, 3);
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs owns a 256 x 256 output tile.  Each CTA stages its own
// 128 rows of A and its own 128 of the 256 B rows (so a stage is 32 KB and six stages fit), the
// leader's single thread issues tcgen05.mma.cta_group::2 with M = 256, which reads both CTAs'
// shared memory and writes 128 accumulator rows into each CTA's tensor memory.  Per FLOP the pair
// moves two thirds of the operand bytes of the single-CTA kernel through L2 and shared memory.
// Barrier protocol: every TMA load credits the LEADER's full barrier (the leader's producer posts
// the expected byte count of both CTAs); tcgen05.commit multicasts stage-free and accumulator-ready
// arrivals to both CTAs; both CTAs' epilogue warps release the accumulator on the leader's barrier.
// ------------------------------------------------------------------------------------------
constexpr int TC2_STAGES = 6;
constexpr uint32_t TC2_OUT_BOX_BYTES = 32 * 64 * 2;      // one staged output box: 32 rows x 64 fp16 columns
constexpr uint32_t TC2_OUT_BYTES = 4 * 2 * TC2_OUT_BOX_BYTES;   // two boxes for each of the four epilogue warps

// Staged epilogue (STAGED = true; outputs without residual / GELU side output and a TMA-compatible C):
// every epilogue warp converts 32 rows x 64 columns of its accumulator quarter to fp16 (+ bias), writes
// them into a 128-byte-swizzled box of shared memory and hands the box to the TMA unit, as a tiled
// store, or -- when the GEMM accumulates into C (weight gradients over micro-batches) -- as a tiled
// reduction that adds the box to global memory at the memory side.  The SM therefore never reads C,
// writes leave as full 128-byte rows, and tensor memory is released as soon as the accumulator has
// been read, before the stores drain.
template <bool A_MN, bool B_MN, bool STAGED>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, TcParams p) {
    constexpr int BN = 256;                              // pair tile: 256 (M) x 256 (N)
    constexpr uint32_t A_BYTES = 128 * TC_BK * 2;        // this CTA's 128 rows of A
    constexpr uint32_t B_BYTES = 128 * TC_BK * 2;        // this CTA's 128 of the 256 B rows
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 512;                  // two accumulators of 256 columns
    constexpr uint32_t IDESC = make_idesc_f16_f32(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* out_boxes = tiles + TC2_STAGES * STAGE_BYTES;     // 1024-byte aligned: the swizzle pattern follows the address
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(out_boxes + (STAGED ? TC2_OUT_BYTES : 0));
    uint64_t* empty_bar = full_bar + TC2_STAGES;
    uint64_t* tmem_full = empty_bar + TC2_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();             // 0 = leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_m * p.tiles_n;         // pair tiles
    const int kblocks = (p.k + TC_BK - 1) / TC_BK;
    // Work items: item = split * num_tiles + tile; split s of a tile covers k-blocks [kblocks * s / splits,
    // kblocks * (s + 1) / splits) and adds its partial product into C (all splits reduce; C was cleared by the host).
    const int num_items = num_tiles * p.splits;
    auto kb_first = [&](int item) { return (int)((int64_t)kblocks * (item / num_tiles) / p.splits); };
    auto kb_last = [&](int item) { return (int)((int64_t)kblocks * (item / num_tiles + 1) / p.splits); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC2_STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 8);                // four epilogue warps in each CTA of the pair
        }
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        if (STAGED) prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_smem, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int item = pair; item < num_items && ok; item += npairs) {
                const int tile = item % num_tiles;
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int row_a = tm * 256 + (int)rank * 128;
                const int row_b = tn * BN + (int)rank * 128;
                const int kb1 = kb_last(item);
                for (int kb = kb_first(item); kb < kb1 && ok; kb++, it++) {
                    const int s = it % TC2_STAGES;
                    ok = mbar_wait(&empty_bar[s], ((it / TC2_STAGES) & 1) ^ 1);
                    if (!ok) break;
                    unsigned char* sa = tiles + s * STAGE_BYTES;
                    unsigned char* sb = sa + A_BYTES;
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                    if (!A_MN) {
                        tma_load_2d_pair(sa, &tmap_a, &full_bar[s], kb * TC_BK, row_a);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; j++) tma_load_2d_pair(sa + j * 8192, &tmap_a, &full_bar[s], row_a + j * 64, kb * TC_BK);
                    }
                    if (!B_MN) {
                        tma_load_2d_pair(sb, &tmap_b, &full_bar[s], kb * TC_BK, row_b);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; j++) tma_load_2d_pair(sb + j * 8192, &tmap_b, &full_bar[s], row_b + j * 64, kb * TC_BK);
                    }
                }
            }
            if (!ok) atomicExch(&g_tc_error, 4);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int item = pair; item < num_items && ok; item += npairs, tcount++) {
                const int buf = tcount & 1;
                ok = mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int kb0 = kb_first(item), kb1 = kb_last(item);
                for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                    const int s = it % TC2_STAGES;
                    ok = mbar_wait(&full_bar[s], (it / TC2_STAGES) & 1);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(tiles + s * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                                 : make_smem_desc_sw128(sa + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                                 : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
                        umma_f16_ss_pair(d_tmem, da, db, IDESC, (kb != kb0 || kk != 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[s], 3);      // frees the stage in both CTAs
                }
                if (ok) umma_commit_pair(&tmem_full[buf], 3);
            }
            if (!ok) atomicExch(&g_tc_error, 5);
        }
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const int quarter = warp & 3;
        uint32_t tcount = 0;
        bool ok = true;
        if constexpr (!STAGED) {
            const bool vec_ok = tc_vec_ok(p);
            for (int tile = pair; tile < num_tiles && ok; tile += npairs, tcount++) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int buf = tcount & 1;
                ok = mbar_wait(&tmem_full[buf], (tcount >> 1) & 1);
                if (!ok) break;
                tcgen05_fence_after();
                const int row = tm * 256 + (int)rank * 128 + quarter * 32 + lane;
                const bool row_ok = row < p.m;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, v);
                    tmem_ld_wait();
                    tc_store_chunk(p, v, row, row_ok, tn * BN + c0, vec_ok);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);
            }
        } else {
            unsigned char* my_boxes = out_boxes + quarter * (2 * TC2_OUT_BOX_BYTES);
            const bool bias_vec = p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
            uint32_t nbox = 0;                       // boxes handed to the TMA unit so far by this warp
            const bool reduce = p.accumulate != 0 || p.splits > 1;
            for (int item = pair; item < num_items && ok; item += npairs, tcount++) {
                const int tile = item % num_tiles;
                const bool add_bias = p.bias != nullptr && item < num_tiles;      // the first split of a tile carries the bias
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int buf = tcount & 1;
                ok = mbar_wait(&tmem_full[buf], (tcount >> 1) & 1);
                if (!ok) break;
                tcgen05_fence_after();
                const int row0 = tm * 256 + (int)rank * 128 + quarter * 32;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
                for (int g = 0; g < BN / 64; g++) {
                    uint32_t v[64];
                    tmem_ld_32x32b_x32(taddr + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
                    tmem_ld_32x32b_x32(taddr + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
                    tmem_ld_wait();
                    if (g == BN / 64 - 1) {          // the accumulator is in registers: the issuer may refill it
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);
                    }
                    const int col0 = tn * BN + g * 64;
                    if (row0 >= p.m || col0 >= p.n) continue;          // box entirely outside C (uniform over the warp)
                    unsigned char* box = my_boxes + (nbox & 1) * TC2_OUT_BOX_BYTES;
                    if (nbox >= 2) {                 // the box used two stores ago must have been read out
                        if (lane == 0) bulk_wait_read<1>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) f[e] = __uint_as_float(v[q * 8 + e]);
                        if (add_bias) {
                            const int c = col0 + q * 8;
                            if (bias_vec && c + 8 <= p.n) {
                                Vec<__half> b;
                                b.load(p.bias + c);
#pragma unroll
                                for (int e = 0; e < 8; e++) f[e] += b.v[e];
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; e++)
                                    if (c + e < p.n) f[e] += __half2float(p.bias[c + e]);
                            }
                        }
                        Vec<__half> o;
#pragma unroll
                        for (int e = 0; e < 8; e++) o.v[e] = f[e];
                        // 128-byte swizzle: 16-byte chunk q of row r lives at chunk q ^ (r & 7)
                        *reinterpret_cast<uint4*>(box + lane * 128 + ((q ^ (lane & 7)) << 4)) = o.pack();
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (reduce) tma_reduce_add_2d(&tmap_c, box, col0, row0);
                        else tma_store_2d(&tmap_c, box, col0, row0);
                        bulk_commit();
                    }
                    nbox++;
                }
            }
            if (lane == 0) bulk_wait_all();
        }
        if (!ok && lane == 0) atomicExch(&g_tc_error, 6);
    }

    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool make_tmap_2d_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p, cudaStream_t st) {
    constexpr size_t smem = 1024 + (size_t)TC_STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 256;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "gemm_tc smem attribute");
        return BRK_CUDA_ERROR;
    }
    int tiles = p.tiles_m * p.tiles_n;
    int grid = tiles < sm_count() ? tiles : sm_count();
    gemm_tc_kernel<BN, A_MN, B_MN><<<grid, TC_THREADS, smem, st>>>(ta, tb, p);
    return launch_status("gemm_tc_kernel");
}

template <int BN>
static int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p, cudaStream_t st) {
    if (!a_mn && !b_mn) return launch_tc<BN, false, false>(ta, tb, p, st);
    if (!a_mn && b_mn) return launch_tc<BN, false, true>(ta, tb, p, st);
    if (a_mn && !b_mn) return launch_tc<BN, true, false>(ta, tb, p, st);
    return launch_tc<BN, true, true>(ta, tb, p, st);
}

template <bool A_MN, bool B_MN, bool STAGED>
static int launch_tc_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const TcParams& p, cudaStream_t st) {
    constexpr size_t smem = 1024 + (size_t)TC2_STAGES * (2 * 128 * TC_BK * 2) + (STAGED ? TC2_OUT_BYTES : 0) + 256;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_pair_kernel<A_MN, B_MN, STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (attr_err != cudaSuccess) {
        set_cuda_error(attr_err, "gemm_tc_pair smem attribute");
        return BRK_CUDA_ERROR;
    }
    int tiles = p.tiles_m * p.tiles_n * p.splits;      // work items
    int pairs = sm_count() / 2;
    if (tiles < pairs) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pairs * 2));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<A_MN, B_MN, STAGED>, ta, tb, tc, p);
    if (e != cudaSuccess) {
        set_cuda_error(e, "gemm_tc_pair_kernel launch");
        return BRK_CUDA_ERROR;
    }
    return launch_status("gemm_tc_pair_kernel");
}

template <bool STAGED>
static int dispatch_pair(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const TcParams& p,
                         cudaStream_t st) {
    if (!a_mn && !b_mn) return launch_tc_pair<false, false, STAGED>(ta, tb, tc, p, st);
    if (!a_mn && b_mn) return launch_tc_pair<false, true, STAGED>(ta, tb, tc, p, st);
    if (a_mn && !b_mn) return launch_tc_pair<true, false, STAGED>(ta, tb, tc, p, st);
    return launch_tc_pair<true, true, STAGED>(ta, tb, tc, p, st);
}

// 0 = choose by shape, 1 = always the single-CTA kernel, 2 = the CTA-pair kernel whenever it applies
static int g_tc_mode = 0;
// 0 = staged (TMA store / reduce) epilogue where it applies, 1 = always the direct register epilogue
static int g_tc_epilogue = 0;
// 0 = cut the k range of the tiles into several work items where that fills the last wave of CTA pairs, 1 = never
static int g_tc_split_k = 0;

// Work items per tile for the CTA-pair kernel with the staged epilogue.  `tiles` pair tiles on `pairs` CTA pairs run in
// ceil(tiles / pairs) waves; with 128 tiles on 74 pairs the second wave is 73 % full.  Cutting every tile's k range
// into s items (each adds its partial product into C through the TMA reduction) changes the fill of the last wave; s
// is taken only if it raises the fill by a tenth and leaves at least 32 k-blocks per item (below that the epilogue of
// an item is no longer hidden behind the next item's products).
static int choose_splits(int tiles, int pairs, int kblocks) {
    if (g_tc_split_k != 0) return 1;
    auto fill = [&](int s) {
        const long items = (long)tiles * s;
        const long waves = (items + pairs - 1) / pairs;
        return (double)items / (double)(waves * pairs);
    };
    int best = 1;
    double best_fill = fill(1);
    for (int s = 2; s <= 4; s++) {
        if (kblocks / s < 32) break;
        const double f = fill(s);
        if (f > best_fill + 0.1) {
            best = s;
            best_fill = f;
        }
    }
    return best;
}

}  // namespace brk

extern "C" void brk_gemm_f16_set_mode(int mode) { brk::g_tc_mode = mode; }
extern "C" void brk_gemm_f16_set_epilogue(int mode) { brk::g_tc_epilogue = mode; }
extern "C" void brk_gemm_f16_set_split_k(int mode) { brk::g_tc_split_k = mode; }
extern "C" int brk_gemm_f16_split_items(int tiles, int pairs, int kblocks) {
    if (tiles <= 0 || pairs <= 0 || kblocks <= 0) return 1;
    return brk::choose_splits(tiles, pairs, kblocks);
}

extern "C" int brk_gemm_f16_supported(int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int64_t lda, int64_t ldb,
                                      const void* a, const void* b) {
    if (m <= 0 || n <= 0 || k <= 0 || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return 0;
    if (lda % 8 != 0 || ldb % 8 != 0) return 0;
    if ((reinterpret_cast<uintptr_t>(a) & 15) != 0 || (reinterpret_cast<uintptr_t>(b) & 15) != 0) return 0;
    (void)trans_a;
    (void)trans_b;
    return 1;
}

extern "C" int brk_gemm_f16(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                            int64_t lda, int64_t ldb, int64_t ldc, const void* bias, const void* residual, int64_t ldr,
                            void* gelu_out, int64_t ldg, int accumulate, void* stream) {
    using namespace brk;
    if (!a || !b) return BRK_INPUT_ERROR;
    if (!c) return BRK_OUTPUT_ERROR;
    if (m < 0 || n < 0 || k <= 0) return BRK_ATTR_ERROR;
    if (m == 0 || n == 0) return BRK_OK;
    if (!brk_gemm_f16_supported(m, n, k, trans_a, trans_b, lda, ldb, a, b)) return BRK_ATTR_ERROR;
    const bool a_mn = trans_a != 0;   // A stored [k, m]
    const bool b_mn = trans_b == 0;   // B stored [k, n]
    const bool use_pair = g_tc_mode != 1 && m > 128 && n > 128;
    const int bn = n > 128 ? 256 : 128;
    const uint32_t box_b_rows = use_pair ? 128u : (uint32_t)bn;
    CUtensorMap ta, tb;
    bool ok;
    if (!a_mn) ok = make_tmap_2d_f16(&ta, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda, TC_BK, TC_BM);
    else ok = make_tmap_2d_f16(&ta, a, (uint64_t)k, (uint64_t)m, (uint64_t)lda, 64, TC_BK);
    if (ok) {
        if (!b_mn) ok = make_tmap_2d_f16(&tb, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb, TC_BK, box_b_rows);
        else ok = make_tmap_2d_f16(&tb, b, (uint64_t)k, (uint64_t)n, (uint64_t)ldb, 64, TC_BK);
    }
    if (!ok) {
        set_error_message("brk_gemm_f16: could not encode a tensor map (driver entry point missing or layout not TMA-compatible)");
        return BRK_CUDA_ERROR;
    }
    TcParams p;
    p.c = (__half*)c;
    p.bias = (const __half*)bias;
    p.residual = (const __half*)residual;
    p.gelu_out = (__half*)gelu_out;
    p.ldc = ldc;
    p.ldr = ldr;
    p.ldg = ldg;
    p.m = (int)m;
    p.n = (int)n;
    p.k = (int)k;
    p.accumulate = accumulate;
    p.tiles_m = (int)((m + TC_BM - 1) / TC_BM);
    p.tiles_n = (int)((n + bn - 1) / bn);
    p.splits = 1;
    cudaStream_t st = (cudaStream_t)stream;
    if (use_pair) {
        p.tiles_m = (int)((m + 255) / 256);
        // outputs that are plain, biased or accumulated leave through shared memory and the TMA unit when C's
        // layout allows a tensor map; residual / GELU epilogues keep the direct register path
        CUtensorMap tc;
        const bool staged = g_tc_epilogue != 1 && !residual && !gelu_out &&
                            make_tmap_2d_f16(&tc, c, (uint64_t)m, (uint64_t)n, (uint64_t)ldc, 64, 32);
        if (staged) {
            p.splits = choose_splits(p.tiles_m * p.tiles_n, sm_count() / 2, (int)((k + TC_BK - 1) / TC_BK));
            if (p.splits > 1 && !accumulate) {
                // every item adds into C: clear it first (the bias rides on the first item of each tile)
                cudaError_t e = cudaMemset2DAsync(c, (size_t)ldc * 2, 0, (size_t)n * 2, (size_t)m, st);
                if (e != cudaSuccess) {
                    set_cuda_error(e, "brk_gemm_f16: clearing C for the split-k items");
                    return BRK_CUDA_ERROR;
                }
            }
            return dispatch_pair<true>(a_mn, b_mn, ta, tb, tc, p, st);
        }
        std::memset(&tc, 0, sizeof(tc));
        return dispatch_pair<false>(a_mn, b_mn, ta, tb, tc, p, st);
    }
    if (bn == 256) return dispatch_major<256>(a_mn, b_mn, ta, tb, p, st);
    return dispatch_major<128>(a_mn, b_mn, ta, tb, p, st);
}

// Synchronous: reads (and clears) the flag the kernels raise when a bounded wait gave up.
// 0 = healthy; 1 = producer, 2 = MMA issuer, 3 = epilogue timed out.
extern "C" int brk_gemm_f16_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, brk::g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(brk::g_tc_error, &zero, sizeof(int));
    return v;
}
