// Dense GEMM C[M,N] = A[M,K] * B[N,K]^T on the 5th-generation tensor cores:
// TMA -> shared-memory ring -> tcgen05.mma accumulating in tensor memory ->
// tcgen05.ld epilogue. A and B are K-major (row-major with K contiguous), which is the
// x [tokens, in] / weight [out, in] layout of every linear layer on the hot path.
//
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      tensor-memory owner and MMA issuer (one elected lane)
//   warps 2..5  epilogue: tensor memory -> registers -> bf16 -> global
// The accumulator is double buffered in tensor memory, so the epilogue of tile i
// overlaps the main loop of tile i+1. Every wait is bounded (rt_tc.cuh).
#include <algorithm>

#include "rt_tc.cuh"

namespace rt {
namespace tc {

constexpr int kBM = 128;         // tile rows (one UMMA M)
constexpr int kBK = 64;          // K elements per stage for 16-bit types (128-byte rows)
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;      // m-tiles walked before moving to the next n-tile

template <int BN>
struct GemmCfg {
    static constexpr int kStages = (BN == 256) ? 4 : 6;
    static constexpr uint32_t kABytes = kBM * kBK * 2;
    static constexpr uint32_t kBBytes = BN * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kBarOffset = kStages * kStageBytes;
    // full[S], empty[S], tmem_full[2], tmem_empty[2], tmem slot, abort flag
    static constexpr uint32_t kSmemBytes = kBarOffset + (2 * kStages + 4) * 8 + 16 + 1024;
    static constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512: powers of two
    // instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N, M = 128
    static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       (static_cast<uint32_t>(BN >> 3) << 17) |
                                       (static_cast<uint32_t>(kBM >> 4) << 24);
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& tm, int& tn) {
    const int per_group = kGroupM * num_n;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int rows = min(kGroupM, num_m - first_m);
    const int local = tile - group * per_group;
    tm = first_m + local % rows;
    tn = local / rows;
}

// F32OUT: c is fp32 (the router logits), otherwise bf16.
// SPLITK (with F32OUT): the K blocks of a tile are cut into k_splits ranges, one work item each,
// and item (tile, split) STORES its partial product into slab `split` of an fp32 workspace
// [k_splits][M][ldc] (slabs split_stride elements apart); splitk_reduce_kernel then adds the
// slabs in split order, so the result does not depend on which SM finished first. A projection
// of a few dozen decode tokens has too few output tiles to occupy the GPU, while its weight
// matrix is what has to be streamed.
// BATCHED: `batch` independent products of the same shape in one launch (the per-head absorbed
// projections of MLA: q_nope . W_UK and latent . W_UV, racetrack/models/deepseek.py:799,810): the
// tensor maps are 3-D {K, rows, batch}, a work item is (batch, m-tile, n-tile) and c advances
// by c_batch_stride elements per batch.
template <int BN, bool F32OUT, bool SPLITK = false, bool BATCHED = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_bf16_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    void* __restrict__ c_out, int M, int N, int K, int64_t ldc, int k_splits_arg = 1,
    int64_t split_stride = 0, int batch = 1, int64_t c_batch_stride = 0) {
    static_assert(!SPLITK || F32OUT, "split-K accumulates into an fp32 output");
    static_assert(!(SPLITK && BATCHED), "one or the other");
    using Cfg = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + Cfg::kBarOffset;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (Cfg::kStages + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + 2 + a); };
    const uint32_t slot = bars + 8u * (2 * Cfg::kStages + 4);
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + Cfg::kBarOffset + 8 * (2 * Cfg::kStages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_m = (M + kBM - 1) / kBM, num_n = (N + BN - 1) / BN;
    const int k_splits = SPLITK ? k_splits_arg : 1;
    const int tiles_per_batch = num_m * num_n;
    const int num_tiles = tiles_per_batch * k_splits * (BATCHED ? batch : 1);         // work items
    const int num_kb_all = (K + kBK - 1) / kBK;
    const int kb_per = (num_kb_all + k_splits - 1) / k_splits;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 128);
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                const int bidx = BATCHED ? tile / tiles_per_batch : 0;
                tile_coords(BATCHED ? tile % tiles_per_batch : tile / k_splits, num_m, num_n, tm, tn);
                const int kb0 = (tile % k_splits) * kb_per, kb1 = min(num_kb_all, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 1))) break;
                    const uint32_t sa = base + stage * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    if constexpr (BATCHED) {
                        tma_load_3d(sa, &tmap_a, kb * kBK, tm * kBM, bidx, full_bar(stage));
                        tma_load_3d(sa + Cfg::kABytes, &tmap_b, kb * kBK, tn * BN, bidx, full_bar(stage));
                    } else {
                        tma_load_2d(sa, &tmap_a, kb * kBK, tm * kBM, full_bar(stage));
                        tma_load_2d(sa + Cfg::kABytes, &tmap_b, kb * kBK, tn * BN, full_bar(stage));
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!(ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, 2))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                const int kb0 = (tile % k_splits) * kb_per, kb1 = min(num_kb_all, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * Cfg::kStageBytes;
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // 16 bf16 = 32 bytes along K: +2 in the 16-byte-unit address field
                        mma_f16(d_tmem, adesc + 2u * k, bdesc + 2u * k, Cfg::kIdesc,
                                ((kb - kb0) | k) != 0 ? 1u : 0u);
                    }
                    mma_commit(empty_bar(stage));  // frees the stage when these MMAs retire
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit(tfull_bar(acc));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;  // the TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            int tm, tn;
            const int bidx = BATCHED ? tile / tiles_per_batch : 0;
            tile_coords(BATCHED ? tile % tiles_per_batch : tile / k_splits, num_m, num_n, tm, tn);
            if (!(ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4))) break;
            tc_fence_after();
            const int row = tm * kBM + quad * 32 + lane;
            const int64_t c_off = static_cast<int64_t>(row) * ldc + static_cast<int64_t>(bidx) * c_batch_stride;
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(c_out) + c_off;
            float* crow_f = static_cast<float*>(c_out) + c_off +
                            (SPLITK ? static_cast<int64_t>(tile % k_splits) * split_stride : 0);
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(acc * BN + chunk * 32);
                tmem_ld_32x32(taddr, r);
                tmem_ld_wait(r);
                if (row < M) {
                    const int col0 = tn * BN + chunk * 32;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const int col = col0 + v * 8;
                        if (col < N) {  // N % 8 == 0, so a started vector is complete
                            if constexpr (F32OUT) {
                                *reinterpret_cast<uint4*>(crow_f + col) =
                                    make_uint4(r[8 * v], r[8 * v + 1], r[8 * v + 2], r[8 * v + 3]);
                                *reinterpret_cast<uint4*>(crow_f + col + 4) =
                                    make_uint4(r[8 * v + 4], r[8 * v + 5], r[8 * v + 6], r[8 * v + 7]);
                                continue;
                            }
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                            *reinterpret_cast<uint4*>(crow + col) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M, N] = A[M, K] * B[N, K]^T
// ---------------------------------------------------------------------------
// A pair of CTAs computes a 256 x 256 tile: each CTA supplies 128 rows of A and 128 rows of B
// (the tensor core reads B across the pair) and keeps the 128 x 256 accumulator of its A rows.
// Per 64 elements of K a CTA brings in 32 KB instead of the 48 KB of the single-CTA 128 x 256
// tile, and operand bytes per SM are what bounds these kernels. Every TMA load covers two K
// blocks (3-D maps {64 elements, rows, K blocks}, box {64, 128, 2}), because an SM retires only
// about one tiled load per 500 cycles whatever its size. 3 stages of 64 KB; two accumulators
// of 256 columns fill tensor memory, so the epilogue of a tile overlaps the next tile's MMAs.
// Warps (both CTAs): 0 producer (one elected thread), 1 tensor-memory owner and MMA issuer
// (leader, cluster rank 0) or relay (peer: forwards "my operands have landed"), 2-9 epilogue
// (lane quarter w % 4, column half (w - 2) / 4).
// Requires K % 64 == 0.
constexpr int kBPStages = 3;
constexpr int kBPThreads = 320;
constexpr uint32_t kBPABytes = 2 * 128 * 128;
constexpr uint32_t kBPBBytes = 2 * 128 * 128;
constexpr uint32_t kBPStageBytes = kBPABytes + kBPBBytes;
constexpr uint32_t kBPBarOffset = kBPStages * kBPStageBytes;
constexpr uint32_t kBPSmemBytes = kBPBarOffset + (2 * kBPStages + 4) * 8 + 16 + 1024;
// fp32 accumulate, bf16 x bf16, both K-major, N = 256, M = 256 over the pair
constexpr uint32_t kBPIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (32u << 17) | (16u << 24);

template <bool F32OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kBPThreads, 1) gemm_bf16_pair_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    void* __restrict__ c_out, int M, int N, int K, int64_t ldc) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kBPBarOffset;
    auto cfull_bar = [&](int d) { return bars + 8u * d; };
    auto cempty_bar = [&](int d) { return bars + 8u * (kBPStages + d); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kBPStages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kBPStages + 2 + a); };
    const uint32_t slot = bars + 8u * (2 * kBPStages + 4);
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kBPBarOffset + 8 * (2 * kBPStages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_m = (M + 255) / 256, num_n = (N + 255) / 256;
    const int num_tiles = num_m * num_n;
    const int num_kb = K / 64;
    const int num_ds = (num_kb + 1) / 2;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int d = 0; d < kBPStages; ++d) {
            mbar_init(cfull_bar(d), rank == 0 ? 2 : 1);   // own producer (+ the peer's relay)
            mbar_init(cempty_bar(d), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 16);    // 8 epilogue warps in each CTA of the pair
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                          // the peer's barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                int tm, tn;
                tile_coords(tile, num_m, num_n, tm, tn);
                const int a_row = tm * 256 + static_cast<int>(rank) * 128;
                const int b_row = tn * 256 + static_cast<int>(rank) * 128;
                for (int ds = 0; ds < num_ds; ++ds) {
                    if (!(ok = mbar_wait(cempty_bar(stage), phase ^ 1u, abort_flag, 31))) break;
                    const uint32_t sa = base + stage * kBPStageBytes;
                    mbar_arrive_expect_tx(cfull_bar(stage), kBPStageBytes);
                    tma_load_3d(sa, &tmap_a, 0, a_row, 2 * ds, cfull_bar(stage));
                    tma_load_3d(sa + kBPABytes, &tmap_b, 0, b_row, 2 * ds, cfull_bar(stage));
                    if (++stage == kBPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0 && lane == 0) {
            const uint32_t peer_cempty0 = map_to_cta(cempty_bar(0), 1);
            const uint32_t peer_tfull0 = map_to_cta(tfull_bar(0), 1);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                if (!(ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, 32))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
                for (int ds = 0; ds < num_ds; ++ds) {
                    if (!(ok = mbar_wait(cfull_bar(stage), phase, abort_flag, 33))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * kBPStageBytes;
                    const int halves = min(2, num_kb - 2 * ds);
                    for (int h = 0; h < halves; ++h) {
                        const uint64_t adesc = smem_desc_sw128(sa + h * (kBPABytes / 2));
                        const uint64_t bdesc =
                            smem_desc_sw128(sa + kBPABytes + h * (kBPBBytes / 2));
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // 16 bf16 = 32 bytes along K: +2 in the 16-byte-unit address field
                            mma_f16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, kBPIdesc,
                                         (ds | h | k) != 0 ? 1u : 0u);
                        }
                    }
                    mma_commit_pair(cempty_bar(stage));
                    mma_commit_pair(peer_cempty0 + 8u * stage);
                    if (++stage == kBPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit_pair(tfull_bar(acc));
                mma_commit_pair(peer_tfull0 + 8u * acc);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        } else if (rank == 1 && lane == 0) {
            const uint32_t leader_cfull0 = map_to_cta(cfull_bar(0), 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                for (int ds = 0; ds < num_ds; ++ds) {
                    if (!(ok = mbar_wait(cfull_bar(stage), phase, abort_flag, 34))) break;
                    mbar_arrive_cluster(leader_cfull0 + 8u * stage);
                    if (++stage == kBPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;  // the TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;
        const uint32_t tempty_leader0 = map_to_cta(tempty_bar(0), 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
            int tm, tn;
            tile_coords(tile, num_m, num_n, tm, tn);
            if (!(ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 35))) break;
            tc_fence_after();
            const int row = tm * 256 + static_cast<int>(rank) * 128 + quad * 32 + lane;
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(c_out) + static_cast<int64_t>(row) * ldc;
            float* crow_f = static_cast<float*>(c_out) + static_cast<int64_t>(row) * ldc;
#pragma unroll 1
            for (int chunk = 4 * half; chunk < 4 * half + 4; ++chunk) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(acc * 256 + chunk * 32);
                tmem_ld_32x32(taddr, r);
                tmem_ld_wait(r);
                if (row < M) {
                    const int col0 = tn * 256 + chunk * 32;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const int col = col0 + v * 8;
                        if (col < N) {  // N % 8 == 0, so a started vector is complete
                            if constexpr (F32OUT) {
                                *reinterpret_cast<uint4*>(crow_f + col) =
                                    make_uint4(r[8 * v], r[8 * v + 1], r[8 * v + 2], r[8 * v + 3]);
                                *reinterpret_cast<uint4*>(crow_f + col + 4) =
                                    make_uint4(r[8 * v + 4], r[8 * v + 5], r[8 * v + 6], r[8 * v + 7]);
                                continue;
                            }
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                            *reinterpret_cast<uint4*>(crow + col) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8u * acc);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();     // no CTA leaves, or frees tensor memory, while its peer may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------
// Block-scaled NVFP4 grouped GEMM
// ---------------------------------------------------------------------------
// C[rows of group g, N] = alpha_g * (A_fp4 (x) sfa) * (B_g fp4 (x) sfb_g)^T
//   A      e2m1 codes [total_rows, K/2] bytes (two per byte, even element in the low nibble),
//          rows grouped by expert; sfa: e4m3 scales, one per 16 elements, in 128-row x 4-block
//          tiles of 512 bytes; the row-tile index of a group's m-tile comes from the tile map,
//          so every group starts on a scale-tile boundary although the code rows are compact.
//   B_g    codes [N, K/2] per group, groups stacked along rows; sfb_g tiled the same way.
//   alpha  a_gs[0] * b_gs[g]: the two fp32 global scales.
// Work list: tile_map[t] = {group, first row, valid rows, scale row-tile}, t < tile_count[0],
// built on the device (moe_tile_map_kernel), so no host synchronisation is needed between the
// routing kernels and this one.
// Stage = 256 elements of K: 128-byte rows for A and B (128-byte swizzle) plus 4 scale tiles
// each. tcgen05.mma kind::mxf4nvf4 consumes 64 elements of K per instruction and reads its
// scale factors from tensor memory. Four extra warps (one per 32-lane quarter of tensor memory)
// move each stage's scale tiles shared memory -> registers -> tensor memory with one
// tcgen05.st per warp and stage; every smem stage owns 32 scale columns, so the copy of stage
// s+1 runs while the MMAs of stage s execute. (Issuing the eight tcgen05.cp per stage from the
// MMA thread instead serialised with the MMAs and cost a third of the kernel time.)
// Warps: 0 TMA producer, 1 MMA issuer, 2-5 epilogue, 6-9 scale loaders.
constexpr int kFBN = 128;                          // tile columns
constexpr int kFBK = 256;                          // K elements per stage
constexpr int kFStages = 6;
constexpr int kFThreads = 320;
constexpr uint32_t kFTileBytes = 128 * 128;        // A or B codes of a stage
constexpr uint32_t kFSfBytes = 4 * 512;            // scale tiles of a stage, per operand
constexpr uint32_t kFStageBytes = 2 * kFTileBytes + 2 * kFSfBytes;
constexpr uint32_t kFBarOffset = kFStages * kFStageBytes;
constexpr uint32_t kFSmemBytes = kFBarOffset + (3 * kFStages + 4) * 8 + 16 + 1024;
constexpr uint32_t kFTmemCols = 512;               // 2 x 128 accumulator + 6 x 32 scale columns
constexpr uint32_t kFTmemSf = 256;                 // first scale column
// block-scaled instruction descriptor: e2m1 x e2m1, e4m3 scales, K-major, N = 128, M = 128
constexpr uint32_t kFIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kFBN >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);

__global__ void __launch_bounds__(kFThreads, 1) gemm_nvfp4_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
    const float* __restrict__ a_gs, const float* __restrict__ b_gs, __nv_bfloat16* __restrict__ c,
    const int4* __restrict__ tile_map, const int* __restrict__ tile_count, int N, int K,
    int64_t ldc) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kFBarOffset;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kFStages + s); };
    auto sf_bar = [&](int s) { return bars + 8u * (2 * kFStages + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (3 * kFStages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (3 * kFStages + 2 + a); };
    const uint32_t slot = bars + 8u * (3 * kFStages + 4);
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kFBarOffset + 8 * (3 * kFStages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_n = (N + kFBN - 1) / kFBN;
    const int num_m = __ldg(tile_count);
    const int num_tiles = num_m * num_n;
    const int num_kb = K / kFBK;
    const int kt = K / 64;                          // scale k-tiles per row tile
    const int n_row_tiles = (N + 127) / 128;        // scale row tiles per group of B

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kFStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(sf_bar(s), 4);     // one arrival per scale-loader warp
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 128);
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(slot, kFTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int4 tm = __ldg(tile_map + tile / num_n);
                const int tn = tile % num_n;
                const uint8_t* sfa_t = sfa + static_cast<int64_t>(tm.w) * kt * 512;
                const uint8_t* sfb_t =
                    sfb + (static_cast<int64_t>(tm.x) * n_row_tiles + tn) * kt * 512;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 11))) break;
                    const uint32_t sa = base + stage * kFStageBytes;
                    mbar_arrive_expect_tx(full_bar(stage), kFStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * 128, tm.y, full_bar(stage));
                    tma_load_2d(sa + kFTileBytes, &tmap_b, kb * 128, tm.x * N + tn * kFBN,
                                full_bar(stage));
                    bulk_load(sa + 2 * kFTileBytes, sfa_t + static_cast<int64_t>(kb) * kFSfBytes,
                              kFSfBytes, full_bar(stage));
                    bulk_load(sa + 2 * kFTileBytes + kFSfBytes,
                              sfb_t + static_cast<int64_t>(kb) * kFSfBytes, kFSfBytes,
                              full_bar(stage));
                    if (++stage == kFStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!(ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, 12))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kFBN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    // codes landed in shared memory, scales landed in tensor memory
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, 13))) break;
                    if (!(ok = mbar_wait(sf_bar(stage), phase, abort_flag, 15))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * kFStageBytes;
                    const uint32_t t_sfa = tmem_base + kFTmemSf + 32u * stage;
                    const uint32_t t_sfb = t_sfa + 16u;
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + kFTileBytes);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // 64 e2m1 = 32 bytes along K: +2 in the 16-byte-unit address field
                        mma_nvfp4(d_tmem, adesc + 2u * j, bdesc + 2u * j, kFIdesc, t_sfa + 4u * j,
                                  t_sfb + 4u * j, (kb | j) != 0 ? 1u : 0u);
                    }
                    mma_commit(empty_bar(stage));
                    if (++stage == kFStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit(tfull_bar(acc));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp >= 6) {
        // Scale loaders: warp w serves the tensor-memory lanes [32*(w%4), +32). A 512-byte scale
        // tile holds, for lane l, the 16 bytes of rows l, l+32, l+64, l+96 (4 scales each):
        // exactly the 4 columns the MMA of that 64-element K block reads at lane l.
        const int quad = warp & 3;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, 16))) break;
                const uint8_t* sf_smem = base_ptr + stage * kFStageBytes + 2 * kFTileBytes;
                uint32_t r[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {   // 4 tiles of A scales, then 4 of B scales
                    const uint4 v = *reinterpret_cast<const uint4*>(sf_smem + j * 512 + lane * 16);
                    r[4 * j] = v.x; r[4 * j + 1] = v.y; r[4 * j + 2] = v.z; r[4 * j + 3] = v.w;
                }
                tmem_st_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kFTmemSf +
                                  32u * stage, r);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sf_bar(stage));
                if (++stage == kFStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const float ags = __ldg(a_gs);
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int4 tm = __ldg(tile_map + tile / num_n);
            const int tn = tile % num_n;
            const float alpha = ags * __ldg(b_gs + tm.x);
            if (!(ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 14))) break;
            tc_fence_after();
            const int lrow = quad * 32 + lane;
            __nv_bfloat16* crow = c + static_cast<int64_t>(tm.y + lrow) * ldc;
#pragma unroll 1
            for (int chunk = 0; chunk < kFBN / 32; ++chunk) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(acc * kFBN + chunk * 32);
                tmem_ld_32x32(taddr, r);
                tmem_ld_wait(r);
                if (lrow < tm.z) {
                    const int col0 = tn * kFBN + chunk * 32;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const int col = col0 + v * 8;
                        if (col < N) {
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * v + i]) * alpha;
                            *reinterpret_cast<uint4*>(crow + col) = pack_bf16x8(f);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kFTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Block-scaled NVFP4 grouped GEMM on CTA pairs (tcgen05 cta_group::2)
// ---------------------------------------------------------------------------
// Same contract as gemm_nvfp4_kernel, other schedule:
//   * the WEIGHTS are the MMA's A operand: a pair of CTAs covers 256 weight rows, 128 each;
//   * the TOKENS are the B operand: up to 256 rows of one group ("wide tile"); N is the
//     power of two (16 ... 256) that covers them, so a group with few rows costs a narrow MMA
//     instead of a padded 128-row tile; each CTA fetches half of the token rows and the tensor
//     core reads both halves across the pair, which halves the token bytes per SM;
//   * per 256 elements of K and CTA: 16 KB weights + <= 16 KB tokens for 2 * 128 * N * 256 flop.
// What sets the pace of such a kernel on this part is not bytes but TMA INSTRUCTIONS: one SM
// retires about one tiled load per 500 cycles whether its box holds 8 KB or 64 KB (measured:
// 492 cycles per box of 8, 16 or 32 KB, 530 for 64 KB), while the MMAs of one 256-element K
// block take about 540 cycles. So every load covers TWO K blocks (3-D tensor maps {128 bytes,
// rows, K blocks}, box {128, rows, 2}): two instructions per 512 elements of K, and the
// scale factors do not use the TMA unit at all (16-byte cp.async copies by one warp).
// Shared memory: 3 operand stages of 64 KB (weights [2][128 rows][128 B], tokens
// [2][N/2 rows][128 B], 128-byte swizzle) and a ring of 5 scale slots of 6 KB.
// Tensor memory: the accumulator D[weight row, token] takes 256 columns (one buffer), 192 more
// hold the scales of two operand stages (per K block 16 columns of weight scales and 32 of
// token scales); the epilogue drains the accumulator into registers, releases it, and only
// then writes: lane = weight row = output column, so one warp store covers 64 contiguous bytes
// of one token's output row.
// What the issuing thread does per operand stage is the pace of this kernel once the operands
// arrive in time: a tcgen05.mma costs it about 65 cycles, a commit as much and a barrier wait
// 100 - 250, whatever the MMA's shape (trace of the first version: two waits, four MMAs and two
// commits per K block, 800 cycles for 540 cycles of tensor work, the same for 16-token tiles).
// So a stage is ONE wait, eight MMAs and ONE commit: the scale loaders arrive on the same
// "stage full" barrier as the operands, and one multicast commit per stage tells both CTAs
// that the stage's shared memory AND its scale columns are free.
// Warps (both CTAs): 0 operand producer (one elected thread), 1 tensor-memory owner and MMA
// issuer (leader CTA, cluster rank 0) or relay (peer: tells the leader that its operands have
// landed), 2-5 scale loaders (shared -> tensor memory), 6-13 epilogue (lane quarter w % 4,
// token half (w - 6) / 4), 14 scale producer.
// Barriers per CTA: cfull[d] (in the leader: operands of stage d landed in both CTAs and its
// scales stored in the tensor memory of both, 2 + 8 arrivals; in the peer: its own operands),
// sdone[d] (MMAs of stage d done: the producer may refill it, the scale loaders may overwrite
// the scale columns it used), sfull[s] / sfree[s] (scale slot s of shared memory filled /
// copied out), tfull (accumulator complete); in the leader: tempty (accumulator drained by the
// 16 epilogue warps of the pair). The leader commits sdone and tfull to both CTAs.
constexpr int kPStages = 3;                        // operand stages of two K blocks each
constexpr int kPSlots = 5;                         // scale slots (shared and tensor memory)
constexpr int kPThreads = 480;
constexpr uint32_t kPWBytes = 2 * 128 * 128;       // weight rows of a stage (two K blocks)
constexpr uint32_t kPXBytes = 2 * 128 * 128;       // token rows of a stage (this CTA's half)
constexpr uint32_t kPStageBytes = kPWBytes + kPXBytes;
constexpr uint32_t kPSfwBytes = 4 * 512;           // scale tiles of the weight rows, one K block
constexpr uint32_t kPSfxBytes = 2 * 4 * 512;       // scale tiles of up to 256 token rows
constexpr uint32_t kPSlotBytes = kPSfwBytes + kPSfxBytes;
constexpr uint32_t kPSfOffset = kPStages * kPStageBytes;
constexpr uint32_t kPBarOffset = kPSfOffset + kPSlots * kPSlotBytes;
constexpr int kPBarriers = 2 * kPStages + 2 * kPSlots + 2;
constexpr uint32_t kPSmemBytes = kPBarOffset + kPBarriers * 8 + 16 + 1024;
constexpr uint32_t kPTmemCols = 512;
constexpr uint32_t kPTmemSf = 256;                 // first scale column
constexpr uint32_t kPSfCols = 48;                  // per K block: 16 weight + 32 token scale columns
constexpr uint32_t kPSfStageCols = 2 * kPSfCols;   // per operand stage (two K blocks); two stages resident
static_assert(kPStageBytes % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
static_assert(kPTmemSf + 2 * kPSfStageCols <= kPTmemCols, "tensor memory budget");
static_assert(kPSmemBytes <= 232448, "shared memory budget");

struct TokenMaps {
    CUtensorMap box[5];     // the token operand with boxes of 8, 16, 32, 64 and 128 rows
};

// Optional pipeline trace (never compiled into the library): with -DRT_PAIR_TRACE the leader
// CTA of pair 0 stamps clock64() at eight points of its first 128 K blocks.
#ifdef RT_PAIR_TRACE
__device__ long long g_pair_trace[8 * 128];
#define RT_TRACE(ev, it) \
    do { if (blockIdx.x == 0 && (it) < 128) g_pair_trace[(ev) * 128 + (it)] = clock64(); } while (0)
// per pair and tile: nanosecond clock when the accumulator became free, when the last MMA of
// the tile had been issued, and the tile's MMA width
__device__ long long g_pair_tiles[74 * 128 * 3];
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define RT_TILE_TRACE(pair, i, ev, val) \
    do { if ((pair) < 74 && (i) < 128) g_pair_tiles[((pair) * 128 + (i)) * 3 + (ev)] = (val); } while (0)
// MMA thread of pair 0, per K block: before / after the operand wait, after the scale wait,
// after the four MMAs, after the scale-slot commits, after the stage commits
__device__ long long g_pair_mma[6 * 128];
#define RT_MMA_TRACE(ev, it) \
    do { if (blockIdx.x == 0 && (it) < 128) g_pair_mma[(ev) * 128 + (it)] = clock64(); } while (0)
#else
#define RT_MMA_TRACE(ev, it) do { } while (0)
#define RT_TRACE(ev, it) do { } while (0)
#define RT_TILE_TRACE(pair, i, ev, val) do { } while (0)
#endif

// Token rows one CTA of the pair fetches for a wide tile of `valid` rows: the power of two
// (>= 8) that covers half of them.
__device__ __forceinline__ int pair_half_rows(int valid) {
    int nh = 8;
    while (2 * nh < valid) nh <<= 1;
    return nh;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1) gemm_nvfp4_pair_kernel(
    const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ TokenMaps tmaps_x,
    const uint8_t* __restrict__ sfx, const uint8_t* __restrict__ sfw,
    const float* __restrict__ x_gs, const float* __restrict__ w_gs, __nv_bfloat16* __restrict__ c,
    const int4* __restrict__ wide_map, const int* __restrict__ wide_count, int N, int K,
    int64_t ldc) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kPBarOffset;
    auto cfull_bar = [&](int d) { return bars + 8u * d; };
    auto sdone_bar = [&](int d) { return bars + 8u * (kPStages + d); };
    auto sfull_bar = [&](int s) { return bars + 8u * (2 * kPStages + s); };
    auto sfree_bar = [&](int s) { return bars + 8u * (2 * kPStages + kPSlots + s); };
    const uint32_t tfull_bar = bars + 8u * (2 * kPStages + 2 * kPSlots);
    const uint32_t tempty_bar = tfull_bar + 8u;
    const uint32_t slot_addr = tfull_bar + 16u;
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kPBarOffset + 8 * kPBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_w = (N + 255) / 256;              // weight tiles of 256 rows
    const int num_tiles = __ldg(wide_count) * num_w;
    const int num_kb = K / 256;                     // K blocks of 256 elements
    const int num_ds = (num_kb + 1) / 2;            // operand stages per tile
    const int kt = K / 64;                          // scale k-tiles per row tile
    const int n_row_tiles = (N + 127) / 128;        // scale row tiles per group of weights

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int d = 0; d < kPStages; ++d) {
            // own producer; in the leader also the peer's relay and the 4 scale-loader warps of each CTA
            mbar_init(cfull_bar(d), rank == 0 ? 10 : 1);
            mbar_init(sdone_bar(d), 1);
        }
        for (int s = 0; s < kPSlots; ++s) {
            mbar_init(sfull_bar(s), 32);     // 32 scale-copy lanes
            mbar_init(sfree_bar(s), 4);      // 4 scale-loader warps
        }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, 16);           // 8 epilogue warps in each CTA of the pair
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
#pragma unroll
        for (int b = 0; b < 5; ++b) tma_prefetch_desc(&tmaps_x.box[b]);
    }
    if (warp == 1) {
        tmem_alloc_pair(slot_addr, kPTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                          // the peer's barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        // Operand producer: per stage one load of this CTA's 128 weight rows and one of its
        // half of the token rows, two K blocks each.
        if (lane == 0) {
            int stage = 0, it = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto weight_row = [&](int tile) {
                return __ldg(wide_map + tile / num_w).x * N + (tile % num_w) * 256 + static_cast<int>(rank) * 128;
            };
            // (Requesting the weight boxes into L2 a few stages ahead was measured slower both
            // ways: with cp.async.bulk.prefetch, 1234 - 1295 us against 1195 - 1210 per w13 launch,
            // and with one prefetch.global.L2 per 128-byte line from the scale producer's warp, 3, 6
            // or 12 K blocks ahead, 1250 - 1277 against 1178 - 1186. DRAM latency is not what the
            // operand stages wait for; the extra requests only compete with the loads.)
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                const int4 tm = __ldg(wide_map + tile / num_w);
                const int nh = pair_half_rows(tm.z);
                const int x_row = tm.y + static_cast<int>(rank) * nh;
                const int w_row = weight_row(tile);
                const int xb = 31 - __clz(nh) - 3;           // index of the box with nh rows
                const uint32_t bytes = kPWBytes + static_cast<uint32_t>(nh) * 256u;
                for (int ds = 0; ds < num_ds; ++ds, ++it) {
                    if (!(ok = mbar_wait(sdone_bar(stage), phase ^ 1u, abort_flag, 21))) break;
                    const uint32_t sa = base + stage * kPStageBytes;
                    RT_TRACE(0, it);
                    mbar_arrive_expect_tx(cfull_bar(stage), bytes);
                    tma_load_3d(sa, &tmap_w, 0, w_row, 2 * ds, cfull_bar(stage));
                    RT_TRACE(1, it);
                    tma_load_3d(sa + kPWBytes, &tmaps_x.box[xb], 0, x_row, 2 * ds,
                                cfull_bar(stage));
                    RT_TRACE(6, it);
                    if (++stage == kPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0 && lane == 0) {
            int stage = 0, it = 0;
            uint32_t phase = 0, acc_phase = 0, sf_par = 0;     // sf_par: which two-stage scale slot
            bool ok = true;
#ifdef RT_PAIR_TRACE
            int tile_i = 0;
#endif
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                const int4 tm = __ldg(wide_map + tile / num_w);
                const uint32_t nh = static_cast<uint32_t>(pair_half_rows(tm.z));
                const uint32_t n_mma = 2u * nh;
                // e2m1 x e2m1, e4m3 scales, K-major, M = 256 over the pair, N = n_mma
                const uint32_t idesc = (1u << 7) | (1u << 10) | ((n_mma >> 3) << 17) | (16u << 24);
                if (!(ok = mbar_wait(tempty_bar, acc_phase ^ 1u, abort_flag, 22))) break;
                tc_fence_after();
                RT_TILE_TRACE(pair, tile_i, 0, global_ns());
                RT_TILE_TRACE(pair, tile_i, 2, static_cast<long long>(n_mma));
                for (int ds = 0; ok && ds < num_ds; ++ds) {
                    RT_MMA_TRACE(0, it);
                    // operands of both CTAs landed AND the stage's scales stored in tensor memory
                    if (!(ok = mbar_wait(cfull_bar(stage), phase, abort_flag, 23))) break;
                    RT_MMA_TRACE(1, it);
                    tc_fence_after();
                    const uint32_t sa = base + stage * kPStageBytes;
                    const int halves = min(2, num_kb - 2 * ds);
                    for (int h = 0; h < halves; ++h, ++it) {
                        RT_TRACE(4, it);
                        RT_MMA_TRACE(2, it);
                        const uint32_t t_sfw = tmem_base + kPTmemSf + kPSfStageCols * sf_par + kPSfCols * h;
                        const uint32_t t_sfx = t_sfw + 16u;
                        const uint64_t adesc = smem_desc_sw128(sa + h * (kPWBytes / 2));
                        const uint64_t bdesc = smem_desc_sw128(sa + kPWBytes + h * nh * 128u);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            mma_nvfp4_pair(tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc,
                                           t_sfw + 4u * j, t_sfx + 8u * j,
                                           (ds | h | j) != 0 ? 1u : 0u);
                        }
                        RT_MMA_TRACE(3, it);
                        RT_TRACE(5, it);
                        RT_MMA_TRACE(4, it);
                    }
                    mma_commit_pair_both(sdone_bar(stage));
                    RT_MMA_TRACE(5, it - 1);
                    sf_par ^= 1u;
                    if (++stage == kPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit_pair_both(tfull_bar);
                acc_phase ^= 1u;
#ifdef RT_PAIR_TRACE
                RT_TILE_TRACE(pair, tile_i, 1, global_ns());
                ++tile_i;
#endif
            }
        } else if (rank == 1 && lane == 0) {
            // Relay: tells the leader that this CTA's operands of a stage have landed.
            const uint32_t leader_cfull0 = map_to_cta(cfull_bar(0), 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                for (int ds = 0; ds < num_ds; ++ds) {
                    if (!(ok = mbar_wait(cfull_bar(stage), phase, abort_flag, 26))) break;
                    mbar_arrive_cluster(leader_cfull0 + 8u * stage);
                    if (++stage == kPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // Scale loaders: warp w serves the tensor-memory lanes [32 * (w % 4), +32) of its own CTA.
        // Tensor memory holds the scales of two operand stages; per K block 16 columns of weight
        // scales (4 per 64-element K step), then 32 columns of token scales (per K step: 4 for
        // token rows 0-127, 4 for 128-255). The columns of stage g are those of stage g - 2, free
        // once that stage's MMAs are done; a stage's last store is followed by one arrival per warp
        // on the leader's "stage full" barrier.
        const int quad = warp & 3;
        const uint32_t cfull_leader = map_to_cta(cfull_bar(0), 0);
        int sf_slot = 0, it = 0, stage = 0, g = 0;       // g: operand stages handled so far
        int done_stage = 0;                              // stage g - 2 (from g = 2 on): its ring index ...
        uint32_t sf_phase = 0, done_phase = 0;           // ... and the parity of its completion
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
            const int4 tm = __ldg(wide_map + tile / num_w);
            const bool two = tm.z > 128;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int h = kb & 1;
                if (!(ok = mbar_wait(sfull_bar(sf_slot), sf_phase, abort_flag, 24))) break;
                if (warp == 2 && lane == 0) RT_TRACE(2, it);
                const uint8_t* sf_smem = base_ptr + kPSfOffset + sf_slot * kPSlotBytes;
                uint32_t rw[16], rx[32];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 v = *reinterpret_cast<const uint4*>(sf_smem + j * 512 + lane * 16);
                    rw[4 * j] = v.x; rw[4 * j + 1] = v.y; rw[4 * j + 2] = v.z; rw[4 * j + 3] = v.w;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(sf_smem + kPSfwBytes +
                                                                     j * 512 + lane * 16);
                    uint4 x1 = make_uint4(0u, 0u, 0u, 0u);
                    if (two)
                        x1 = *reinterpret_cast<const uint4*>(sf_smem + kPSfwBytes + 2048 + j * 512 +
                                                             lane * 16);
                    rx[8 * j] = x0.x; rx[8 * j + 1] = x0.y; rx[8 * j + 2] = x0.z; rx[8 * j + 3] = x0.w;
                    rx[8 * j + 4] = x1.x; rx[8 * j + 5] = x1.y; rx[8 * j + 6] = x1.z; rx[8 * j + 7] = x1.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sfree_bar(sf_slot));      // the shared slot may refill
                if (h == 0 && g >= 2) {
                    // the MMAs of stage g - 2, which read these columns of tensor memory, are done
                    if (!(ok = mbar_wait(sdone_bar(done_stage), done_phase, abort_flag, 30))) break;
                    tc_fence_after();
                }
                const uint32_t t_slot = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kPTmemSf +
                                        kPSfStageCols * static_cast<uint32_t>(g & 1) +
                                        kPSfCols * static_cast<uint32_t>(h);
                tmem_st_32x16(t_slot, rw);
                tmem_st_32x32(t_slot + 16u, rx);
                if (h == 1 || kb == num_kb - 1) {
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(cfull_leader + 8u * stage);
                    if (++stage == kPStages) stage = 0;
                    if (++g > 2 && ++done_stage == kPStages) {
                        done_stage = 0;
                        done_phase ^= 1u;
                    }
                }
                if (warp == 2 && lane == 0) RT_TRACE(3, it);
                if (++sf_slot == kPSlots) {
                    sf_slot = 0;
                    sf_phase ^= 1u;
                }
            }
        }
    } else if (warp == 14) {
        // Scale producer: the scale tiles of a K block (2 KB for this CTA's weight rows, 2 or 4 KB
        // for all token rows of the tile) come in 16-byte cp.async copies, 4 per lane and tile
        // set, through the load/store unit: the TMA unit is the bottleneck and stays free of
        // them.
        int sf_slot = 0, it = 0;
        uint32_t sf_phase = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
            const int4 tm = __ldg(wide_map + tile / num_w);
            const int wn = tile % num_w;
            int w_rt = wn * 2 + static_cast<int>(rank);
            if (w_rt >= n_row_tiles) w_rt = n_row_tiles - 1;   // rows past N: results unused
            const uint8_t* sfw_t =
                sfw + (static_cast<int64_t>(tm.x) * n_row_tiles + w_rt) * kt * 512 + lane * 16;
            const uint8_t* sfx_t = sfx + static_cast<int64_t>(tm.w) * kt * 512 + lane * 16;
            const bool two = tm.z > 128;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                if (!(ok = mbar_wait(sfree_bar(sf_slot), sf_phase ^ 1u, abort_flag, 27))) break;
                const uint32_t ssf = base + kPSfOffset + sf_slot * kPSlotBytes + lane * 16;
                const int64_t o = static_cast<int64_t>(kb) * 2048;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    cp_async16(ssf + j * 512, sfw_t + o + j * 512);
                    cp_async16(ssf + kPSfwBytes + j * 512, sfx_t + o + j * 512);
                    if (two)
                        cp_async16(ssf + kPSfwBytes + 2048 + j * 512,
                                   sfx_t + static_cast<int64_t>(kt) * 512 + o + j * 512);
                }
                cp_async_arrive(sfull_bar(sf_slot));
                if (lane == 0) RT_TRACE(7, it);
                if (++sf_slot == kPSlots) {
                    sf_slot = 0;
                    sf_phase ^= 1u;
                }
            }
        }
    } else if (warp >= 6 && warp < 14) {
        const int quad = warp & 3, half = (warp - 6) >> 2;
        const uint32_t tempty_leader = map_to_cta(tempty_bar, 0);
        uint32_t tphase = 0;
        bool ok = true;
        const float xgs = __ldg(x_gs);
        for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
            const int4 tm = __ldg(wide_map + tile / num_w);
            const int wn = tile % num_w;
            const int n_mma = 2 * pair_half_rows(tm.z);
            const float alpha = xgs * __ldg(w_gs + tm.x);
            if (!(ok = mbar_wait(tfull_bar, tphase, abort_flag, 25))) break;
            tc_fence_after();
            __nv_bfloat162 packed[64];
            // two 32-column loads per wait: the accumulator is single-buffered, so the latency
            // of its drain (a few hundred cycles per tensor-memory load) is on the critical path
#pragma unroll
            for (int chunk = 0; chunk < 4; chunk += 2) {
                const int col0 = half * 128 + chunk * 32;
                if (col0 < n_mma) {
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                           static_cast<uint32_t>(col0);
                    const bool second = col0 + 32 < n_mma;       // warp-uniform
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(taddr, r0);
                    if (second) tmem_ld_32x32(taddr + 32, r1);
                    tmem_ld_wait(r0);
                    if (second) tmem_ld_wait(r1);
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        packed[16 * chunk + i] =
                            __floats2bfloat162_rn(__uint_as_float(r0[2 * i]) * alpha,
                                                  __uint_as_float(r0[2 * i + 1]) * alpha);
                    if (second) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            packed[16 * chunk + 16 + i] =
                                __floats2bfloat162_rn(__uint_as_float(r1[2 * i]) * alpha,
                                                      __uint_as_float(r1[2 * i + 1]) * alpha);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader);
            // the accumulator is free again; write this thread's output column
            const int f = wn * 256 + static_cast<int>(rank) * 128 + quad * 32 + lane;
            if (f < N) {
#pragma unroll
                for (int chunk = 0; chunk < 4; ++chunk) {
                    const int col0 = half * 128 + chunk * 32;
                    if (col0 < tm.z) {
                        __nv_bfloat16* cp = c + static_cast<int64_t>(tm.y + col0) * ldc + f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (col0 + 2 * i < tm.z) cp[0] = packed[16 * chunk + i].x;
                            if (col0 + 2 * i + 1 < tm.z) cp[ldc] = packed[16 * chunk + i].y;
                            cp += 2 * ldc;
                        }
                    }
                }
            }
            tphase ^= 1u;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();     // no CTA leaves, or frees tensor memory, while its peer may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kPTmemCols);
    }
}

// Builds the work lists of the grouped GEMMs from the per-expert row offsets of the sorted
// (token, slot) pairs. One CTA. For groups g in [g_begin, g_end):
//   tile_map[t] = {g - g_begin, first row, valid rows (<= 128), scale row-tile index}
//   tile_base[g - g_begin] = index of the group's first tile (= its first scale row tile),
//   tile_base[g_end - g_begin] = tile_count[0] = number of tiles;
// and, in the second half of tile_map, the same rows cut into "wide" tiles of up to 256 rows
// (two scale row tiles) for the CTA-pair kernel:
//   tile_map[max_tiles + u] = {g - g_begin, first row, valid rows (<= 256), scale row-tile
//   index of its first 128 rows}, u < tile_count[1].
// Both prefix sums ride in one 64-bit scan (128-row tiles in the low word, wide tiles in the
// high word).
__global__ void __launch_bounds__(1024) moe_tile_map_kernel(const int32_t* __restrict__ offsets,
                                                            int g_begin, int g_end,
                                                            int4* __restrict__ tile_map,
                                                            int32_t* __restrict__ tile_base,
                                                            int32_t* __restrict__ tile_count,
                                                            int max_tiles) {
    __shared__ long long warp_tot[32];
    __shared__ long long carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int groups = g_end - g_begin;
    for (int b = 0; b < groups; b += blockDim.x) {
        const int g = b + threadIdx.x;
        int rows = 0, row0 = 0;
        if (g < groups) {
            row0 = offsets[g_begin + g];
            rows = offsets[g_begin + g + 1] - row0;
        }
        const int ntile = (rows + 127) >> 7, nwide = (rows + 255) >> 8;
        const long long mine = static_cast<long long>(ntile) | (static_cast<long long>(nwide) << 32);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const long long w = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
            long long wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long v = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += v;
            }
            warp_tot[lane] = wi - w;
        }
        __syncthreads();
        const long long excl = carry_s + warp_tot[warp] + incl - mine;
        const int first = static_cast<int>(excl & 0xffffffffLL);
        const int wfirst = static_cast<int>(excl >> 32);
        if (g < groups) {
            tile_base[g] = first;
            for (int t = 0; t < ntile; ++t) {
                if (first + t < max_tiles)
                    tile_map[first + t] =
                        make_int4(g, row0 + t * 128, min(128, rows - t * 128), first + t);
            }
            for (int t = 0; t < nwide; ++t) {
                if (wfirst + t < max_tiles)
                    tile_map[max_tiles + wfirst + t] =
                        make_int4(g, row0 + t * 256, min(256, rows - t * 256), first + 2 * t);
            }
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_s = excl + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int total = static_cast<int>(carry_s & 0xffffffffLL);
        tile_base[groups] = total;
        tile_count[0] = min(total, max_tiles);
        tile_count[1] = min(static_cast<int>(carry_s >> 32), max_tiles);
    }
}

// ---------------------------------------------------------------------------
// FP8 e4m3 GEMM with DeepSeek block scales
// ---------------------------------------------------------------------------
// C[m, n] = sum over 128-wide K blocks kb of
//           (A_fp8[m, kb] . B_fp8[n, kb]) * a_s[m, kb] * b_s[n / 128, kb]         -> bf16
// (activation scales per row and K block, weight scales per 128 x 128 block). The scales are
// arbitrary fp32 numbers, so they cannot ride along inside the MMA: every K block is
// multiplied on its own into a fresh tensor-memory buffer (4 x tcgen05.mma kind::f8f6f4,
// K = 32 each) and eight epilogue warps fold it, scaled, into fp32 register accumulators while
// the tensor core works on the next K block (two 256-column buffers alternate).
// Tile 128 x 256, stage = one K block: 16 KB of A + 32 KB of B, 4 stages.
// Warps: 0 TMA producer, 1 MMA issuer, 2-9 epilogue (warp w: lane quarter w % 4, column half
// (w - 2) / 4).
// What holds it at about 975 cycles per K block (1.8-1.9 PFLOP/s; the four MMAs of a K block
// take 512): the round trip of a buffer. Measured in isolation on this part: an e4m3
// 128 x 256 x 32 MMA takes 128 cycles back to back (twice the bf16 flops per cycle); tensor-memory
// loads and MMAs do not slow each other down (the fold alone, eight warps, 386 cycles per
// 128 x 256 block, with or without MMAs running); one hop through an mbarrier (arrive or commit
// -> the parked waiter runs again) costs 145-175 cycles; and four MMAs issued into an IDLE
// tensor pipe are seen complete by a waiter 977 cycles after the first issue (about 260 cycles
// from issue to execution, 512 of execution, the hop). With two buffers a buffer comes back after
// issue + execution + hop + loads + hop + the issuing thread's own wait, about 1900 cycles, and
// two K blocks fit into that. Tried and measured no faster, because none of them shortens that
// loop: a CTA-pair variant (256 x 256 tiles, two thirds of the operand bytes per K block, one
// wait and one multicast commit per K block), a second issuing thread (one per buffer), one
// arrival per warp instead of per thread, polling instead of parked waits, and the issuing thread
// looking at the next K block's barriers before its last MMA. A third buffer does not fit (512
// tensor-memory columns), narrower buffers make the issuing thread the limit (eight MMAs per K
// block), and 16 fold warps or a register copy of the whole buffer before the fold do not fit
// the register file (128 accumulators per thread).
constexpr int kQBN = 256;
constexpr int kQBK = 128;
constexpr int kQStages = 4;
constexpr int kQThreads = 320;
constexpr uint32_t kQABytes = kBM * kQBK;
constexpr uint32_t kQBBytes = kQBN * kQBK;
constexpr uint32_t kQStageBytes = kQABytes + kQBBytes;
constexpr uint32_t kQBarOffset = kQStages * kQStageBytes;
constexpr uint32_t kQSmemBytes = kQBarOffset + (2 * kQStages + 4) * 8 + 16 + 1024;
constexpr uint32_t kQTmemCols = 512;
// fp32 accumulate, e4m3 x e4m3 (format code 0), K-major, N = 256, M = 128
constexpr uint32_t kQIdesc = (1u << 4) | (static_cast<uint32_t>(kQBN >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);

__global__ void __launch_bounds__(kQThreads, 1) gemm_fp8_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const float* __restrict__ a_s, const float* __restrict__ b_s, __nv_bfloat16* __restrict__ c,
    int M, int N, int K, int64_t ldc) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kQBarOffset;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kQStages + s); };
    auto pfull_bar = [&](int a) { return bars + 8u * (2 * kQStages + a); };
    auto pempty_bar = [&](int a) { return bars + 8u * (2 * kQStages + 2 + a); };
    const uint32_t slot = bars + 8u * (2 * kQStages + 4);
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kQBarOffset + 8 * (2 * kQStages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_m = (M + kBM - 1) / kBM, num_n = (N + kQBN - 1) / kQBN;
    const int num_tiles = num_m * num_n;
    const int num_kb = K / kQBK;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kQStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(pfull_bar(a), 1);
            mbar_init(pempty_bar(a), 256);
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(slot, kQTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, num_m, num_n, tm, tn);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 21))) break;
                    const uint32_t sa = base + stage * kQStageBytes;
                    mbar_arrive_expect_tx(full_bar(stage), kQStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kQBK, tm * kBM, full_bar(stage));
                    tma_load_2d(sa + kQABytes, &tmap_b, kb * kQBK, tn * kQBN, full_bar(stage));
                    if (++stage == kQStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t buf_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(pempty_bar(buf), buf_phase ^ 1u, abort_flag, 22))) break;
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, 23))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * kQStageBytes;
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kQBN);
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + kQABytes);
#pragma unroll
                    for (int j = 0; j < kQBK / 32; ++j) {
                        // 32 e4m3 = 32 bytes along K: +2 in the 16-byte-unit address field
                        mma_f8f6f4(d_tmem, adesc + 2u * j, bdesc + 2u * j, kQIdesc, j != 0 ? 1u : 0u);
                    }
                    mma_commit(empty_bar(stage));   // smem stage reusable
                    mma_commit(pfull_bar(buf));     // partial product of this K block complete
                    if (++stage == kQStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    if (++buf == 2) {
                        buf = 0;
                        buf_phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;       // which 128 columns of the tile
        const int kbs = num_kb;                 // scales per row of A / per block row of B
        int buf = 0;
        uint32_t buf_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            int tm, tn;
            tile_coords(tile, num_m, num_n, tm, tn);
            const int row = tm * kBM + quad * 32 + lane;
            const int col_base = tn * kQBN + half * 128;
            const bool live = col_base < N;                       // whole half outside the matrix?
            const float* as_row = a_s + static_cast<int64_t>(row < M ? row : 0) * kbs;
            const float* bs_row = b_s + static_cast<int64_t>(live ? col_base >> 7 : 0) * kbs;
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;
            for (int kb = 0; kb < num_kb; ++kb) {
                const float scale = __ldg(as_row + kb) * __ldg(bs_row + kb);
                if (!(ok = mbar_wait(pfull_bar(buf), buf_phase, abort_flag, 24))) break;
                tc_fence_after();
                // 64 columns per wait: the latency of a tensor-memory load (a few hundred cycles)
                // is paid twice per K block, not four times
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(buf * kQBN + half * 128);
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(taddr, r0);
                tmem_ld_32x32(taddr + 32, r1);
                tmem_ld_wait(r0);
                tmem_ld_wait(r1);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(__uint_as_float(r0[i]), scale, acc[i]);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(__uint_as_float(r1[i]), scale, acc[32 + i]);
                tmem_ld_32x32(taddr + 64, r0);
                tmem_ld_32x32(taddr + 96, r1);
                tmem_ld_wait(r0);
                tmem_ld_wait(r1);
                // every column of the buffer has been read: hand it back before the last fold
                tc_fence_before();
                mbar_arrive(pempty_bar(buf));
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(__uint_as_float(r0[i]), scale, acc[64 + i]);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(__uint_as_float(r1[i]), scale, acc[96 + i]);
                if (++buf == 2) {
                    buf = 0;
                    buf_phase ^= 1u;
                }
            }
            if (!ok) break;
            if (row < M && live) {
                __nv_bfloat16* crow = c + static_cast<int64_t>(row) * ldc + col_base;
#pragma unroll
                for (int v = 0; v < 16; ++v) {
                    if (col_base + v * 8 < N) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = acc[v * 8 + i];
                        *reinterpret_cast<uint4*>(crow + v * 8) = pack_bf16x8(f);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kQTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Index scores of the sparse-attention indexer (FP8 x FP8, tcgen05)
// ---------------------------------------------------------------------------
//   score[m, n] = k_s[n] * sum_h w[m, h] * relu(q[m, h, :] . k[n, :])        (dim = 128)
// The KEYS are the MMA's M (128 per tile, so an epilogue thread owns one key), the (query, head)
// pairs its N (256 per tile = 256 / heads queries): the sum over heads is then a loop over the
// thread's own accumulator columns, no cross-lane traffic, and for one query a warp stores 32
// consecutive keys' scores. One K block (128 e4m3) per MMA group, so each key tile costs one TMA
// load; the query block (32 KB) is loaded once per work item and reused for a chunk of key tiles.
// Work item = (query block, chunk of up to kIdxChunk key tiles); persistent CTAs.
// Warps: 0 producer, 1 MMA issuer, then EW epilogue warps (lane quarter w % 4, column slice
// (w - 2) / 4 of 256 / (EW / 4) columns). EW = 16 (64 columns each: four warps per scheduler hide
// the tensor-memory load latency, which 8 warps do not) whenever a query's heads fit into 64
// columns, EW = 8 for 128 heads.
// Barriers: kfull/kempty[4] (key tiles), qfull/qempty[2] (query blocks), pfull/pempty[2]
// (accumulator buffers of 256 columns).
constexpr int kIdxStages = 4;
constexpr int kIdxChunk = 16;
constexpr uint32_t kIdxKBytes = 128 * 128;
constexpr uint32_t kIdxQBytes = 256 * 128;
constexpr uint32_t kIdxQOffset = kIdxStages * kIdxKBytes;
constexpr uint32_t kIdxWOffset = kIdxQOffset + 2 * kIdxQBytes;      // 2 x 256 fp32 head weights
constexpr uint32_t kIdxBarOffset = kIdxWOffset + 2 * 256 * 4;
constexpr int kIdxBarriers = 2 * kIdxStages + 4 + 4;
constexpr uint32_t kIdxSmemBytes = kIdxBarOffset + kIdxBarriers * 8 + 16 + 1024;
// fp32 accumulate, e4m3 x e4m3, K-major, N = 256, M = 128
constexpr uint32_t kIdxIdesc = (1u << 4) | (32u << 17) | (8u << 24);

template <int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1) index_score_kernel(
    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
    const float* __restrict__ weights, const float* __restrict__ k_scale,
    float* __restrict__ scores, int queries, int heads, int keys, int64_t ld,
    int64_t causal_offset, int batch, int64_t ks_batch_stride, int64_t score_batch_stride) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    float* wsm = reinterpret_cast<float*>(base_ptr + kIdxWOffset);
    const uint32_t bars = base + kIdxBarOffset;
    auto kfull_bar = [&](int s) { return bars + 8u * s; };
    auto kempty_bar = [&](int s) { return bars + 8u * (kIdxStages + s); };
    auto qfull_bar = [&](int s) { return bars + 8u * (2 * kIdxStages + s); };
    auto qempty_bar = [&](int s) { return bars + 8u * (2 * kIdxStages + 2 + s); };
    auto pfull_bar = [&](int a) { return bars + 8u * (2 * kIdxStages + 4 + a); };
    auto pempty_bar = [&](int a) { return bars + 8u * (2 * kIdxStages + 6 + a); };
    const uint32_t slot = bars + 8u * kIdxBarriers;
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kIdxBarOffset + 8 * kIdxBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_rows = queries * heads;
    const int num_qb = (q_rows + 255) / 256;
    const int num_kt = (keys + 127) / 128;
    const int num_kc = (num_kt + kIdxChunk - 1) / kIdxChunk;
    const int per_seq = num_qb * num_kc;            // work items of one sequence
    const int num_items = batch * per_seq;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kIdxStages; ++s) {
            mbar_init(kfull_bar(s), 1);
            mbar_init(kempty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(qfull_bar(a), 1);
            mbar_init(qempty_bar(a), 1);
            mbar_init(pfull_bar(a), 1);
            mbar_init(pempty_bar(a), EW);    // one arrival per epilogue warp
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_q);
    }
    if (warp == 1) {
        tmem_alloc(slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0, qs = 0;
            uint32_t phase = 0, qphase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                const int bi = item / per_seq, rem = item % per_seq;
                const int qb = rem / num_kc, kc = rem % num_kc;
                if (!(ok = mbar_wait(qempty_bar(qs), qphase ^ 1u, abort_flag, 51))) break;
                mbar_arrive_expect_tx(qfull_bar(qs), kIdxQBytes);
                tma_load_3d(base + kIdxQOffset + qs * kIdxQBytes, &tmap_q, 0, qb * 256, bi,
                            qfull_bar(qs));
                const int kt_end = min(num_kt, (kc + 1) * kIdxChunk);
                for (int kt = kc * kIdxChunk; kt < kt_end; ++kt) {
                    if (!(ok = mbar_wait(kempty_bar(stage), phase ^ 1u, abort_flag, 52))) break;
                    mbar_arrive_expect_tx(kfull_bar(stage), kIdxKBytes);
                    tma_load_3d(base + stage * kIdxKBytes, &tmap_k, 0, kt * 128, bi, kfull_bar(stage));
                    if (++stage == kIdxStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (++qs == 2) {
                    qs = 0;
                    qphase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0, qs = 0, buf = 0;
            uint32_t phase = 0, qphase = 0, buf_phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                const int kc = (item % per_seq) % num_kc;
                if (!(ok = mbar_wait(qfull_bar(qs), qphase, abort_flag, 53))) break;
                const uint64_t bdesc = smem_desc_sw128(base + kIdxQOffset + qs * kIdxQBytes);
                const int kt_end = min(num_kt, (kc + 1) * kIdxChunk);
                for (int kt = kc * kIdxChunk; kt < kt_end; ++kt) {
                    if (!(ok = mbar_wait(pempty_bar(buf), buf_phase ^ 1u, abort_flag, 54))) break;
                    if (!(ok = mbar_wait(kfull_bar(stage), phase, abort_flag, 55))) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * 256);
                    const uint64_t adesc = smem_desc_sw128(base + stage * kIdxKBytes);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma_f8f6f4(d_tmem, adesc + 2u * j, bdesc + 2u * j, kIdxIdesc, j != 0 ? 1u : 0u);
                    mma_commit(kempty_bar(stage));
                    mma_commit(pfull_bar(buf));
                    if (++stage == kIdxStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    if (++buf == 2) {
                        buf = 0;
                        buf_phase ^= 1u;
                    }
                }
                if (!ok) break;
                mma_commit(qempty_bar(qs));      // the query block is free when these MMAs retire
                if (++qs == 2) {
                    qs = 0;
                    qphase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        constexpr int kCols = 256 / (EW / 4);   // accumulator columns per epilogue warp
        const int quad = warp & 3;
        const int slice = (warp - 2) >> 2;      // which kCols (query, head) columns of the tile
        const int et = threadIdx.x - 64;        // index among the epilogue threads
        const int q_per_slice = kCols / heads;
        int buf = 0, parity = 0;
        uint32_t buf_phase = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x, parity ^= 1) {
            const int bi = item / per_seq, rem = item % per_seq;
            const int qb = rem / num_kc, kc = rem % num_kc;
            const float* ks_b = k_scale + bi * ks_batch_stride;
            float* scores_b = scores + bi * score_batch_stride;
            // head weights of the block's 256 (query, head) rows; the named barrier also says
            // that every epilogue thread has left the item that used this half of wsm before
            if (et < 256) {
                const int qrow = qb * 256 + et;
                wsm[parity * 256 + et] =
                    qrow < q_rows ? __ldg(weights + static_cast<int64_t>(bi) * q_rows + qrow) : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
            const float4* wv = reinterpret_cast<const float4*>(wsm + parity * 256 + slice * kCols);
            const int m0 = (qb * 256 + slice * kCols) / heads;      // first query of this slice
            const int kt_end = min(num_kt, (kc + 1) * kIdxChunk);
            for (int kt = kc * kIdxChunk; kt < kt_end; ++kt) {
                const int n = kt * 128 + quad * 32 + lane;
                const float ks = n < keys ? __ldg(ks_b + n) : 0.f;
                if (!(ok = mbar_wait(pfull_bar(buf), buf_phase, abort_flag, 56))) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(buf * 256 + slice * kCols);
                float sums[kCols / 16];          // 16-column partial sums
#pragma unroll
                for (int j = 0; j < kCols / 16; ++j) sums[j] = 0.f;
#pragma unroll
                for (int pairi = 0; pairi < kCols / 64; ++pairi) {
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(taddr + pairi * 64, r0);
                    tmem_ld_32x32(taddr + pairi * 64 + 32, r1);
                    tmem_ld_wait(r0);
                    tmem_ld_wait(r1);
                    if (pairi == kCols / 64 - 1) {
                        // every column of the slice has been read: hand the buffer back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(pempty_bar(buf));
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 w0 = wv[(pairi * 64 + i) >> 2];
                        const float4 w1 = wv[(pairi * 64 + 32 + i) >> 2];
                        float& s0 = sums[(pairi * 64 + i) / 16];
                        float& s1 = sums[(pairi * 64 + 32 + i) / 16];
                        s0 = fmaf(fmaxf(__uint_as_float(r0[i]), 0.f), w0.x, s0);
                        s0 = fmaf(fmaxf(__uint_as_float(r0[i + 1]), 0.f), w0.y, s0);
                        s0 = fmaf(fmaxf(__uint_as_float(r0[i + 2]), 0.f), w0.z, s0);
                        s0 = fmaf(fmaxf(__uint_as_float(r0[i + 3]), 0.f), w0.w, s0);
                        s1 = fmaf(fmaxf(__uint_as_float(r1[i]), 0.f), w1.x, s1);
                        s1 = fmaf(fmaxf(__uint_as_float(r1[i + 1]), 0.f), w1.y, s1);
                        s1 = fmaf(fmaxf(__uint_as_float(r1[i + 2]), 0.f), w1.z, s1);
                        s1 = fmaf(fmaxf(__uint_as_float(r1[i + 3]), 0.f), w1.w, s1);
                    }
                }
                // a query owns heads / 16 of the partial sums
                if (n < keys) {
                    const int per_q = heads / 16;
                    for (int j = 0; j < q_per_slice; ++j) {
                        float s = 0.f;
                        for (int t = 0; t < per_q; ++t) s += sums[j * per_q + t];
                        const int m = m0 + j;
                        if (m < queries) {
                            const bool visible = causal_offset < 0 || n <= m + causal_offset;
                            scores_b[static_cast<int64_t>(m) * ld + n] =
                                visible ? s * ks : __int_as_float(0xff800000);
                        }
                    }
                }
                if (++buf == 2) {
                    buf = 0;
                    buf_phase ^= 1u;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D K-major tensor map: dims {k_elems, rows}, row pitch in bytes, box {box_k, box_rows},
// 128-byte swizzle, zero fill outside the tensor.
int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t k_elems,
                 uint64_t rows, uint64_t pitch_bytes, uint32_t box_k, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {k_elems, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_k, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

// 3-D K-major tensor map over a byte matrix [rows, k_bytes] (row pitch pitch_bytes) whose rows
// are cut into K blocks of 128 bytes: dims {128, rows, k_bytes / 128}, box {128, box_rows,
// box_kblocks}. One load brings box_kblocks swizzled K-major tiles, stored one after the
// other; K blocks past the end of a row read as zeros.
int make_tmap_kblocks(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t k_bytes,
                      uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_kblocks) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {128, rows, k_bytes / 128};
    const cuuint64_t strides[2] = {pitch_bytes, 128};
    const cuuint32_t box[3] = {128, box_rows, box_kblocks};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

// 3-D map over `batch` K-major matrices of 128-byte rows: dims {128 bytes, rows, batch}, box
// {128, box_rows, 1}; the batch stride is in bytes (a multiple of 16).
int make_tmap_rows128_batched(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t batch,
                              uint64_t batch_stride_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {128, rows, batch};
    const cuuint64_t strides[2] = {128, batch_stride_bytes};
    const cuuint32_t box[3] = {128, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

// 4-D bf16 tensor map with the 128-byte swizzle for the attention kernels (rt_attn.cu): dims and
// box are given fastest dimension first, strides in bytes for dimensions 1..3.
int make_tmap_bf16_4d(CUtensorMap* map, const void* ptr, const uint64_t dims_in[4],
                      const uint64_t strides_in[3], const uint32_t box_in[4]) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {dims_in[0], dims_in[1], dims_in[2], dims_in[3]};
    const cuuint64_t strides[3] = {strides_in[0], strides_in[1], strides_in[2]};
    const cuuint32_t box[4] = {box_in[0], box_in[1], box_in[2], box_in[3]};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <int BN, bool F32OUT>
static int launch_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t st) {
    using Cfg = GemmCfg<BN>;
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, K, M, lda * 2, kBK, kBM))
        return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, K, N, ldb * 2, kBK, BN))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_bf16_kernel<BN, F32OUT>),
                                     static_cast<int>(Cfg::kSmemBytes), "rt_gemm_bf16"))
        return rc;
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_bf16_kernel<BN, F32OUT><<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(
        ta, tb, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_bf16_kernel");
}

// out[m, n] = part[0][m, n] + part[1][m, n] + ... in split order (fp32), rounded to bf16 or kept.
template <bool F32OUT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part,
                                                            void* __restrict__ out, int64_t total4,
                                                            int n4, int64_t ld4, int64_t ldo,
                                                            int64_t slab4, int splits) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total4;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = i / n4;
        const int c4 = static_cast<int>(i - row * n4);
        const float4* src = reinterpret_cast<const float4*>(part) + row * ld4 + c4;
        float4 acc = __ldg(src);
        for (int sidx = 1; sidx < splits; ++sidx) {
            const float4 v = __ldg(src + sidx * slab4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if constexpr (F32OUT) {
            *reinterpret_cast<float4*>(static_cast<float*>(out) + row * ldo + 4 * c4) = acc;
        } else {
            uint2 o;
            o.x = pack_bf16x2(acc.x, acc.y);
            o.y = pack_bf16x2(acc.z, acc.w);
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + row * ldo + 4 * c4) = o;
        }
    }
}

// 3-D bf16 operand {K, rows, batch} with box {64, box_rows, 1}.
static int make_tmap_bf16_batched(CUtensorMap* map, const void* ptr, uint64_t k, uint64_t rows, uint64_t batch,
                                  uint64_t pitch_bytes, uint64_t batch_pitch_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {k, rows, batch};
    const cuuint64_t strides[2] = {pitch_bytes, batch_pitch_bytes};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(kBK), box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled (batched) failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

static int launch_bf16_batched(const void* a, const void* b, void* c, int64_t batch, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t a_bs, int64_t ldb, int64_t b_bs, int64_t ldc,
                               int64_t c_bs, cudaStream_t st) {
    using Cfg = GemmCfg<128>;
    CUtensorMap ta, tb;
    if (int rc = make_tmap_bf16_batched(&ta, a, K, M, batch, lda * 2, a_bs * 2, kBM)) return rc;
    if (int rc = make_tmap_bf16_batched(&tb, b, K, N, batch, ldb * 2, b_bs * 2, 128)) return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_bf16_kernel<128, false, false, true>),
                                     static_cast<int>(Cfg::kSmemBytes), "rt_gemm_bf16_batched"))
        return rc;
    const int64_t items = ((M + kBM - 1) / kBM) * ((N + 127) / 128) * batch;
    const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
    gemm_bf16_kernel<128, false, false, true><<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(
        ta, tb, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc, 1, 0,
        static_cast<int>(batch), c_bs);
    count_launch();
    return check_launch("gemm_bf16_kernel<batched>");
}

// Split-K launch of the 128 x 128 tiling: partial products into the workspace slabs, then the
// ordered sum into `out`.
static int launch_bf16_splitk(const void* a, const void* b, float* c, void* out, int out_dtype,
                              int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                              int64_t ldo, int splits, cudaStream_t st) {
    using Cfg = GemmCfg<128>;
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, K, M, lda * 2, kBK, kBM))
        return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, K, N, ldb * 2, kBK, 128))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_bf16_kernel<128, true, true>),
                                     static_cast<int>(Cfg::kSmemBytes), "rt_gemm_bf16_splitk"))
        return rc;
    const int64_t items = ((M + kBM - 1) / kBM) * ((N + 127) / 128) * splits;
    const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
    gemm_bf16_kernel<128, true, true><<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(
        ta, tb, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc, splits, M * ldc);
    count_launch();
    if (int rc = check_launch("gemm_bf16_kernel<split-K>")) return rc;
    const int64_t total4 = M * (N / 4);
    const int blocks = static_cast<int>(std::min<int64_t>((total4 + 255) / 256, 8 * sm_count()));
    auto reduce = out_dtype == RT_F32 ? splitk_reduce_kernel<true> : splitk_reduce_kernel<false>;
    reduce<<<blocks, 256, 0, st>>>(c, out, total4, static_cast<int>(N / 4), ldc / 4, ldo, M * ldc / 4,
                                   splits);
    count_launch();
    return check_launch("splitk_reduce_kernel");
}

// bf16 operand as 64-element K blocks: dims {64, rows, K / 64}, box {64, 128, 2}.
static int make_tmap_bf16_kblocks(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t k,
                                  uint64_t pitch_bytes) {
    EncodeTiledFn fn = encode_fn();
    RT_REQUIRE(fn, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {64, rows, k / 64};
    const cuuint64_t strides[2] = {pitch_bytes, 128};
    const cuuint32_t box[3] = {64, 128, 2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
               static_cast<int>(r));
    return RT_OK;
}

// Schedule of the bf16 GEMM: 0 = by size, 1 = single-CTA tiles, 2 = CTA pairs (needs K % 64 == 0).
static int g_bf16_schedule = 0;

template <bool F32OUT>
static int launch_bf16_pair(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t st) {
    CUtensorMap ta, tb;
    if (int rc = make_tmap_bf16_kblocks(&ta, a, M, K, lda * 2)) return rc;
    if (int rc = make_tmap_bf16_kblocks(&tb, b, N, K, ldb * 2)) return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_bf16_pair_kernel<F32OUT>),
                                     static_cast<int>(kBPSmemBytes), "rt_gemm_bf16"))
        return rc;
    const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t max_pairs = sm_count() / 2;
    const int grid = 2 * static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    gemm_bf16_pair_kernel<F32OUT><<<grid, kBPThreads, kBPSmemBytes, st>>>(
        ta, tb, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_bf16_pair_kernel");
}

static int launch_index_score(const void* q, const float* weights, const void* k,
                              const float* k_scale, float* scores, int64_t batch, int64_t queries,
                              int64_t heads, int64_t keys, int64_t ld, int64_t causal_offset,
                              int64_t k_batch_stride, int64_t ks_batch_stride,
                              int64_t score_batch_stride, cudaStream_t st) {
    CUtensorMap tk, tq;
    const uint64_t kbs = batch > 1 ? static_cast<uint64_t>(k_batch_stride) * 128u : static_cast<uint64_t>(keys) * 128u;
    if (int rc = make_tmap_rows128_batched(&tk, k, keys, batch, kbs, 128)) return rc;
    if (int rc = make_tmap_rows128_batched(&tq, q, queries * heads, batch,
                                           static_cast<uint64_t>(queries * heads) * 128u, 256))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&index_score_kernel<16>),
                                     static_cast<int>(kIdxSmemBytes), "rt_fp8_index"))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&index_score_kernel<8>),
                                     static_cast<int>(kIdxSmemBytes), "rt_fp8_index"))
        return rc;
    const int64_t num_qb = (queries * heads + 255) / 256;
    const int64_t num_kt = (keys + 127) / 128;
    const int64_t items = batch * num_qb * ((num_kt + kIdxChunk - 1) / kIdxChunk);
    const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
    if (heads <= 64)
        index_score_kernel<16><<<grid, 64 + 32 * 16, kIdxSmemBytes, st>>>(
            tk, tq, weights, k_scale, scores, static_cast<int>(queries), static_cast<int>(heads),
            static_cast<int>(keys), ld, causal_offset, static_cast<int>(batch), ks_batch_stride,
            score_batch_stride);
    else
        index_score_kernel<8><<<grid, 64 + 32 * 8, kIdxSmemBytes, st>>>(
            tk, tq, weights, k_scale, scores, static_cast<int>(queries), static_cast<int>(heads),
            static_cast<int>(keys), ld, causal_offset, static_cast<int>(batch), ks_batch_stride,
            score_batch_stride);
    count_launch();
    return check_launch("index_score_kernel");
}

static int launch_fp8(const void* a, const float* a_s, const void* b, const float* b_s, void* c,
                      int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                      cudaStream_t st) {
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, a, K, M, lda, kQBK, kBM)) return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, b, K, N, ldb, kQBK, kQBN)) return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_fp8_kernel),
                                     static_cast<int>(kQSmemBytes), "rt_gemm_fp8"))
        return rc;
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kQBN - 1) / kQBN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_fp8_kernel<<<grid, kQThreads, kQSmemBytes, st>>>(
        ta, tb, a_s, b_s, static_cast<__nv_bfloat16*>(c), static_cast<int>(M), static_cast<int>(N),
        static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_fp8_kernel");
}

// Schedule of the NVFP4 GEMM: 0 = by size (CTA pairs unless the work list is too short to
// occupy them or the groups average fewer than 128 rows), 1 = single-CTA 128 x 128 tiles,
// 2 = CTA pairs. Process-wide; meant for A/B
// measurements and tests.
static int g_nvfp4_schedule = 0;

static int launch_nvfp4_single(const void* a_codes, const void* a_sf, const float* a_gs,
                               const void* b_codes, const void* b_sf, const float* b_gs, void* c,
                               const int32_t* tile_map, const int32_t* tile_count,
                               int64_t max_m_tiles, int64_t total_rows, int64_t groups, int64_t N,
                               int64_t K, int64_t ldc, cudaStream_t st) {
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, K / 2, total_rows,
                              K / 2, 128, kBM))
        return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_codes, K / 2, groups * N, K / 2,
                              128, kFBN))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_nvfp4_kernel),
                                     static_cast<int>(kFSmemBytes), "rt_gemm_nvfp4_grouped"))
        return rc;
    const int64_t tiles = max_m_tiles * ((N + kFBN - 1) / kFBN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_nvfp4_kernel<<<grid, kFThreads, kFSmemBytes, st>>>(
        ta, tb, static_cast<const uint8_t*>(a_sf), static_cast<const uint8_t*>(b_sf), a_gs, b_gs,
        static_cast<__nv_bfloat16*>(c), reinterpret_cast<const int4*>(tile_map), tile_count,
        static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_nvfp4_kernel");
}

static int launch_nvfp4_pair(const void* a_codes, const void* a_sf, const float* a_gs,
                             const void* b_codes, const void* b_sf, const float* b_gs, void* c,
                             const int32_t* tile_map, const int32_t* tile_count,
                             int64_t max_m_tiles, int64_t total_rows, int64_t groups, int64_t N,
                             int64_t K, int64_t ldc, cudaStream_t st) {
    CUtensorMap tw;
    TokenMaps tx;
    if (int rc = make_tmap_kblocks(&tw, b_codes, groups * N, K / 2, K / 2, 128, 2)) return rc;
    for (int b = 0; b < 5; ++b) {
        if (int rc = make_tmap_kblocks(&tx.box[b], a_codes, total_rows, K / 2, K / 2, 8u << b, 2)) return rc;
    }
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_nvfp4_pair_kernel),
                                     static_cast<int>(kPSmemBytes), "rt_gemm_nvfp4_grouped"))
        return rc;
    // wide tiles: never more than 128-row tiles, so max_m_tiles bounds them as well
    const int64_t tiles = max_m_tiles * ((N + 255) / 256);
    const int64_t max_pairs = sm_count() / 2;
    const int grid = 2 * static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    gemm_nvfp4_pair_kernel<<<grid, kPThreads, kPSmemBytes, st>>>(
        tw, tx, static_cast<const uint8_t*>(a_sf), static_cast<const uint8_t*>(b_sf), a_gs, b_gs,
        static_cast<__nv_bfloat16*>(c), reinterpret_cast<const int4*>(tile_map) + max_m_tiles,
        tile_count + 1, static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_nvfp4_pair_kernel");
}

}  // namespace tc
}  // namespace rt

using namespace rt;

extern "C" int rt_gemm_fp8(const void* a, const float* a_scales, const void* b,
                           const float* b_scales, void* c, int64_t m, int64_t n, int64_t k,
                           int64_t lda, int64_t ldb, int64_t ldc, void* stream) {
    RT_REQUIRE(m >= 0 && n > 0 && k > 0, RT_ERR_BAD_ARG, "rt_gemm_fp8: bad shape");
    if (m == 0) return RT_OK;
    RT_REQUIRE(a && a_scales && b && b_scales && c, RT_ERR_BAD_ARG, "rt_gemm_fp8: null pointer");
    RT_REQUIRE(k % 128 == 0, RT_ERR_UNSUPPORTED, "rt_gemm_fp8: k must be a multiple of 128");
    RT_REQUIRE(n % 8 == 0 && lda % 16 == 0 && ldb % 16 == 0 && ldc % 8 == 0, RT_ERR_UNSUPPORTED,
               "rt_gemm_fp8: n %% 8, lda/ldb %% 16 and ldc %% 8 are required");
    RT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c), RT_ERR_UNSUPPORTED,
               "rt_gemm_fp8: pointers must be 16-byte aligned");
    RT_REQUIRE(m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_gemm_fp8: dimension too large");
    return tc::launch_fp8(a, a_scales, b, b_scales, c, m, n, k, lda, ldb, ldc, as_stream(stream));
}

static int fp8_index_checked(const void* q, const float* weights, const void* k,
                             const float* k_scale, float* scores, int64_t batch, int64_t queries,
                             int64_t heads, int64_t keys, int64_t dim, int64_t score_stride,
                             int64_t causal_offset, int64_t k_batch_stride,
                             int64_t ks_batch_stride, int64_t score_batch_stride, void* stream) {
    RT_REQUIRE(batch >= 0 && queries >= 0 && heads > 0 && keys > 0, RT_ERR_BAD_ARG,
               "rt_fp8_index: bad shape");
    if (queries == 0 || batch == 0) return RT_OK;
    RT_REQUIRE(q && weights && k && k_scale && scores, RT_ERR_BAD_ARG, "rt_fp8_index: null pointer");
    RT_REQUIRE(dim == 128, RT_ERR_UNSUPPORTED, "rt_fp8_index: the index head dimension must be 128");
    RT_REQUIRE(heads % 16 == 0 && 128 % heads == 0, RT_ERR_UNSUPPORTED,
               "rt_fp8_index: heads must be 16, 32, 64 or 128");
    RT_REQUIRE(aligned16(q) && aligned16(k), RT_ERR_UNSUPPORTED,
               "rt_fp8_index: q and k must be 16-byte aligned");
    RT_REQUIRE(score_stride >= keys, RT_ERR_BAD_ARG, "rt_fp8_index: score stride below keys");
    RT_REQUIRE(queries * heads < (1LL << 31) && keys < (1LL << 31) && batch < (1LL << 20) &&
                   batch * queries * heads < (1LL << 31),
               RT_ERR_UNSUPPORTED, "rt_fp8_index: dimension too large");
    RT_REQUIRE(batch == 1 || (k_batch_stride >= keys && ks_batch_stride >= keys &&
                              score_batch_stride >= queries * score_stride),
               RT_ERR_BAD_ARG, "rt_fp8_index: a batch stride is below the extent of one sequence");
    return tc::launch_index_score(q, weights, k, k_scale, scores, batch, queries, heads, keys,
                                  score_stride, causal_offset, k_batch_stride, ks_batch_stride,
                                  score_batch_stride, as_stream(stream));
}

extern "C" int rt_fp8_index(const void* q, const float* weights, const void* k, const float* k_scale,
                            float* scores, int64_t queries, int64_t heads, int64_t keys,
                            int64_t dim, int64_t score_stride, int64_t causal_offset,
                            void* stream) {
    return fp8_index_checked(q, weights, k, k_scale, scores, 1, queries, heads, keys, dim,
                             score_stride, causal_offset, 0, 0, 0, stream);
}

extern "C" int rt_fp8_index_batched(const void* q, const float* weights, const void* k,
                                    const float* k_scale, float* scores, int64_t batch,
                                    int64_t queries, int64_t heads, int64_t keys, int64_t dim,
                                    int64_t score_stride, int64_t causal_offset,
                                    int64_t k_batch_stride, int64_t ks_batch_stride,
                                    int64_t score_batch_stride, void* stream) {
    return fp8_index_checked(q, weights, k, k_scale, scores, batch, queries, heads, keys, dim,
                             score_stride, causal_offset, k_batch_stride, ks_batch_stride,
                             score_batch_stride, stream);
}

extern "C" int rt_moe_tile_map(const int32_t* offsets, int64_t g_begin, int64_t g_end,
                               int32_t* tile_map, int32_t* tile_base, int32_t* tile_count,
                               int64_t max_tiles, void* stream) {
    RT_REQUIRE(offsets && tile_map && tile_base && tile_count, RT_ERR_BAD_ARG,
               "rt_moe_tile_map: null pointer");
    RT_REQUIRE(g_begin >= 0 && g_end > g_begin && max_tiles > 0, RT_ERR_BAD_ARG,
               "rt_moe_tile_map: bad group range or tile bound");
    RT_REQUIRE(aligned16(tile_map), RT_ERR_UNSUPPORTED, "rt_moe_tile_map: tile_map must be 16-byte aligned");
    int threads = static_cast<int>((g_end - g_begin + 31) / 32 * 32);
    if (threads > 1024) threads = 1024;
    tc::moe_tile_map_kernel<<<1, threads, 0, as_stream(stream)>>>(
        offsets, static_cast<int>(g_begin), static_cast<int>(g_end),
        reinterpret_cast<int4*>(tile_map), tile_base, tile_count, static_cast<int>(max_tiles));
    count_launch();
    return check_launch("moe_tile_map_kernel");
}

extern "C" int rt_gemm_nvfp4_grouped(const void* a_codes, const void* a_sf, const float* a_gs,
                                     const void* b_codes, const void* b_sf, const float* b_gs,
                                     void* c, const int32_t* tile_map, const int32_t* tile_count,
                                     int64_t max_m_tiles, int64_t total_rows, int64_t groups,
                                     int64_t n, int64_t k, int64_t ldc, void* stream) {
    RT_REQUIRE(total_rows >= 0 && groups > 0 && n > 0 && k > 0 && max_m_tiles >= 0, RT_ERR_BAD_ARG,
               "rt_gemm_nvfp4_grouped: bad shape");
    if (total_rows == 0 || max_m_tiles == 0) return RT_OK;
    RT_REQUIRE(a_codes && a_sf && a_gs && b_codes && b_sf && b_gs && c && tile_map && tile_count,
               RT_ERR_BAD_ARG, "rt_gemm_nvfp4_grouped: null pointer");
    RT_REQUIRE(k % 256 == 0, RT_ERR_UNSUPPORTED, "rt_gemm_nvfp4_grouped: k must be a multiple of 256");
    RT_REQUIRE(n % 8 == 0 && ldc % 8 == 0, RT_ERR_UNSUPPORTED,
               "rt_gemm_nvfp4_grouped: n and ldc must be multiples of 8");
    RT_REQUIRE(groups == 1 || n % 128 == 0, RT_ERR_UNSUPPORTED,
               "rt_gemm_nvfp4_grouped: with several groups n must be a multiple of 128");
    RT_REQUIRE(aligned16(a_codes) && aligned16(b_codes) && aligned16(a_sf) && aligned16(b_sf) &&
                   aligned16(c) && aligned16(tile_map),
               RT_ERR_UNSUPPORTED, "rt_gemm_nvfp4_grouped: pointers must be 16-byte aligned");
    RT_REQUIRE(total_rows < (1LL << 31) && groups * n < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_gemm_nvfp4_grouped: dimension too large");
    // Pairs pay off when the tensor cores are the bottleneck: at least 128 rows per group on
    // average and 2 x 74 CTAs' worth of 256-row weight tiles. With fewer rows the launch streams
    // the weights once from HBM and the single-CTA tiles, which keep more loads in flight, were
    // 4-7 % faster from 8 to 1024 tokens of a 256-expert layer.
    const bool few_tiles = max_m_tiles * ((n + 255) / 256) < tc::sm_count();
    const bool few_rows = total_rows < 128 * groups;
    if (tc::g_nvfp4_schedule == 1 || (tc::g_nvfp4_schedule == 0 && (few_tiles || few_rows)))
        return tc::launch_nvfp4_single(a_codes, a_sf, a_gs, b_codes, b_sf, b_gs, c, tile_map,
                                       tile_count, max_m_tiles, total_rows, groups, n, k, ldc,
                                       as_stream(stream));
    return tc::launch_nvfp4_pair(a_codes, a_sf, a_gs, b_codes, b_sf, b_gs, c, tile_map, tile_count,
                                 max_m_tiles, total_rows, groups, n, k, ldc, as_stream(stream));
}

#ifdef RT_PAIR_TRACE
extern "C" int rt_pair_trace_read(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, tc::g_pair_trace, sizeof(long long) * 8 * 128) == cudaSuccess
               ? RT_OK : RT_ERR_CUDA;
}
extern "C" int rt_pair_mma_read(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, tc::g_pair_mma, sizeof(long long) * 6 * 128) == cudaSuccess
               ? RT_OK : RT_ERR_CUDA;
}
extern "C" int rt_pair_tiles_read(long long* host_out, int clear) {
    if (clear) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, tc::g_pair_tiles) != cudaSuccess) return RT_ERR_CUDA;
        return cudaMemset(p, 0, sizeof(long long) * 74 * 128 * 3) == cudaSuccess ? RT_OK : RT_ERR_CUDA;
    }
    return cudaMemcpyFromSymbol(host_out, tc::g_pair_tiles, sizeof(long long) * 74 * 128 * 3) ==
                   cudaSuccess ? RT_OK : RT_ERR_CUDA;
}
#endif

extern "C" int rt_gemm_bf16_schedule(int schedule) {
    const int previous = tc::g_bf16_schedule;
    if (schedule >= 0 && schedule <= 2) tc::g_bf16_schedule = schedule;
    return previous;
}

extern "C" int rt_gemm_nvfp4_schedule(int schedule) {
    const int previous = tc::g_nvfp4_schedule;
    if (schedule >= 0 && schedule <= 2) tc::g_nvfp4_schedule = schedule;
    return previous;
}

extern "C" int rt_gemm_bf16(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                            int64_t lda, int64_t ldb, int64_t ldc, int out_dtype, void* stream) {
    RT_REQUIRE(out_dtype == RT_BF16 || out_dtype == RT_F32, RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16: output dtype must be bf16 or f32");
    RT_REQUIRE(m >= 0 && n > 0 && k > 0, RT_ERR_BAD_ARG, "rt_gemm_bf16: bad shape");
    if (m == 0) return RT_OK;
    RT_REQUIRE(a && b && c, RT_ERR_BAD_ARG, "rt_gemm_bf16: null pointer");
    RT_REQUIRE(k % 8 == 0 && n % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0,
               RT_ERR_UNSUPPORTED, "rt_gemm_bf16: k, n and the leading dimensions must be multiples of 8");
    RT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c), RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16: pointers must be 16-byte aligned");
    RT_REQUIRE(m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16: dimension too large");
    cudaStream_t st = as_stream(stream);
    // CTA pairs (256 x 256 tiles) once they fill the machine; they need whole 64-element K blocks
    const bool pair_ok = k % 64 == 0;
    const bool pair_pays = ((m + 255) / 256) * ((n + 255) / 256) >= tc::sm_count() / 2;
    if (pair_ok && (tc::g_bf16_schedule == 2 || (tc::g_bf16_schedule == 0 && pair_pays))) {
        if (out_dtype == RT_F32) return tc::launch_bf16_pair<true>(a, b, c, m, n, k, lda, ldb, ldc, st);
        return tc::launch_bf16_pair<false>(a, b, c, m, n, k, lda, ldb, ldc, st);
    }
    if (out_dtype == RT_F32) {
        if (n <= 128) return tc::launch_bf16<128, true>(a, b, c, m, n, k, lda, ldb, ldc, st);
        return tc::launch_bf16<256, true>(a, b, c, m, n, k, lda, ldb, ldc, st);
    }
    if (n <= 128) return tc::launch_bf16<128, false>(a, b, c, m, n, k, lda, ldb, ldc, st);
    return tc::launch_bf16<256, false>(a, b, c, m, n, k, lda, ldb, ldc, st);
}

extern "C" int rt_gemm_bf16_batched(const void* a, const void* b, void* c, int64_t batch, int64_t m,
                                    int64_t n, int64_t k, int64_t lda, int64_t a_batch_stride, int64_t ldb,
                                    int64_t b_batch_stride, int64_t ldc, int64_t c_batch_stride, void* stream) {
    RT_REQUIRE(batch >= 0 && m >= 0 && n > 0 && k > 0, RT_ERR_BAD_ARG, "rt_gemm_bf16_batched: bad shape");
    if (batch == 0 || m == 0) return RT_OK;
    RT_REQUIRE(a && b && c, RT_ERR_BAD_ARG, "rt_gemm_bf16_batched: null pointer");
    RT_REQUIRE(k % 8 == 0 && n % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0 &&
                   a_batch_stride % 8 == 0 && b_batch_stride % 8 == 0 && c_batch_stride % 8 == 0,
               RT_ERR_UNSUPPORTED, "rt_gemm_bf16_batched: k, n and every stride must be multiples of 8");
    RT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c), RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16_batched: pointers must be 16-byte aligned");
    RT_REQUIRE(m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31) && batch < (1LL << 20) &&
                   ((m + 127) / 128) * ((n + 127) / 128) * batch < (1LL << 31),
               RT_ERR_UNSUPPORTED, "rt_gemm_bf16_batched: dimension too large");
    return tc::launch_bf16_batched(a, b, c, batch, m, n, k, lda, a_batch_stride, ldb, b_batch_stride, ldc,
                                   c_batch_stride, as_stream(stream));
}

extern "C" int64_t rt_gemm_bf16_splitk_splits(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k <= 0) return 1;
    const int64_t tiles = ((m + 127) / 128) * ((n + 127) / 128);
    const int64_t num_kb = (k + 63) / 64;
    // enough work items for two per SM, at least 4 K blocks each
    int64_t splits = (2 * tc::sm_count() + tiles - 1) / tiles;
    if (splits > num_kb / 4) splits = num_kb / 4;
    if (splits < 1) splits = 1;
    const int64_t per = (num_kb + splits - 1) / splits;
    return (num_kb + per - 1) / per;          // no split is empty
}

extern "C" int rt_gemm_bf16_splitk(const void* a, const void* b, float* workspace, void* out,
                                   int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                   int64_t ldw, int64_t ldo, int64_t splits, int out_dtype,
                                   void* stream) {
    float* c = workspace;
    const int64_t ldc = ldw;
    RT_REQUIRE(m >= 0 && n > 0 && k > 0, RT_ERR_BAD_ARG, "rt_gemm_bf16_splitk: bad shape");
    if (m == 0) return RT_OK;
    RT_REQUIRE(a && b && c && out, RT_ERR_BAD_ARG, "rt_gemm_bf16_splitk: null pointer");
    RT_REQUIRE(out_dtype == RT_BF16 || out_dtype == RT_F32, RT_ERR_BAD_ARG,
               "rt_gemm_bf16_splitk: out_dtype must be RT_BF16 or RT_F32");
    RT_REQUIRE(k % 8 == 0 && n % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldc % 4 == 0 && ldo % 4 == 0,
               RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16_splitk: k, n, lda, ldb must be multiples of 8, ldw and ldo of 4");
    RT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c) && aligned16(out), RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16_splitk: pointers must be 16-byte aligned");
    RT_REQUIRE(m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_gemm_bf16_splitk: dimension too large");
    const int64_t num_kb = (k + 63) / 64;
    RT_REQUIRE(splits >= 1 && splits <= num_kb, RT_ERR_BAD_ARG, "rt_gemm_bf16_splitk: bad split count");
    const int64_t per = (num_kb + splits - 1) / splits;
    RT_REQUIRE((num_kb + per - 1) / per == splits, RT_ERR_BAD_ARG,
               "rt_gemm_bf16_splitk: a split would be empty (use rt_gemm_bf16_splitk_splits)");
    return tc::launch_bf16_splitk(a, b, c, out, out_dtype, m, n, k, lda, ldb, ldc, ldo,
                                  static_cast<int>(splits), as_stream(stream));
}

namespace rt { namespace tc { int attn_error_take(); } }   // the flag of the attention kernels (rt_attn.cu)

extern "C" int rt_tc_error_state(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_tc_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_tc_error_state: cannot read the device flag");
    }
    const int va = tc::attn_error_take();
    if (va < 0) return fail(RT_ERR_CUDA, "rt_tc_error_state: cannot read the device flag");
    if (v == 0 && va > 0)
        return fail(RT_ERR_TIMEOUT, "a tensor-core kernel abandoned wait #%d (bounded spin expired)", va);
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc::g_tc_error, &zero, sizeof(int));
        return fail(RT_ERR_TIMEOUT, "a tensor-core kernel abandoned wait #%d (bounded spin expired)", v);
    }
    return RT_OK;
}
