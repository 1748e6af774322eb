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
template <int BN, bool F32OUT>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_bf16_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    void* __restrict__ c_out, int M, int N, int K, int64_t ldc) {
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
    const int num_tiles = num_m * num_n;
    const int num_kb = (K + kBK - 1) / kBK;

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
                tile_coords(tile, num_m, num_n, tm, tn);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 1))) break;
                    const uint32_t sa = base + stage * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kBK, tm * kBM, full_bar(stage));
                    tma_load_2d(sa + Cfg::kABytes, &tmap_b, kb * kBK, tn * BN, full_bar(stage));
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
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * Cfg::kStageBytes;
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // 16 bf16 = 32 bytes along K: +2 in the 16-byte-unit address field
                        mma_f16(d_tmem, adesc + 2u * k, bdesc + 2u * k, Cfg::kIdesc,
                                (kb | k) != 0 ? 1u : 0u);
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
            tile_coords(tile, num_m, num_n, tm, tn);
            if (!(ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4))) break;
            tc_fence_after();
            const int row = tm * kBM + quad * 32 + lane;
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(c_out) + static_cast<int64_t>(row) * ldc;
            float* crow_f = static_cast<float*>(c_out) + static_cast<int64_t>(row) * ldc;
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

// Builds the work list of the grouped GEMM from the per-expert row offsets of the sorted
// (token, slot) pairs. One CTA. For groups g in [g_begin, g_end):
//   tile_map[t] = {g - g_begin, first row, valid rows (<= 128), scale row-tile index}
//   tile_base[g - g_begin] = index of the group's first tile (= its first scale row tile),
//   tile_base[g_end - g_begin] = tile_count[0] = number of tiles.
__global__ void __launch_bounds__(1024) moe_tile_map_kernel(const int32_t* __restrict__ offsets,
                                                            int g_begin, int g_end,
                                                            int4* __restrict__ tile_map,
                                                            int32_t* __restrict__ tile_base,
                                                            int32_t* __restrict__ tile_count,
                                                            int max_tiles) {
    __shared__ int warp_tot[32];
    __shared__ int carry_s;
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
        const int ntile = (rows + 127) >> 7;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        int incl = ntile;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int w = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += v;
            }
            warp_tot[lane] = wi - w;
        }
        __syncthreads();
        const int first = carry_s + warp_tot[warp] + incl - ntile;
        if (g < groups) {
            tile_base[g] = first;
            for (int t = 0; t < ntile; ++t) {
                if (first + t < max_tiles)
                    tile_map[first + t] =
                        make_int4(g, row0 + t * 128, min(128, rows - t * 128), first + t);
            }
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_s = first + ntile;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        tile_base[groups] = carry_s;
        tile_count[0] = min(carry_s, max_tiles);
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
                // two register buffers: the load of chunk c+1 is in flight while chunk c is folded in
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(buf * kQBN + half * 128);
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(taddr, r0);
                tmem_ld_wait(r0);
                tmem_ld_32x32(taddr + 32, r1);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(__uint_as_float(r0[i]), scale, acc[i]);
                tmem_ld_wait(r1);
                tmem_ld_32x32(taddr + 64, r0);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(__uint_as_float(r1[i]), scale, acc[32 + i]);
                tmem_ld_wait(r0);
                tmem_ld_32x32(taddr + 96, r1);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(__uint_as_float(r0[i]), scale, acc[64 + i]);
                tmem_ld_wait(r1);
                // every column of the buffer has been read: hand it back before the last fold
                tc_fence_before();
                mbar_arrive(pempty_bar(buf));
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
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, F32OUT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(Cfg::kSmemBytes));
        RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_gemm_bf16: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_bf16_kernel<BN, F32OUT><<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(
        ta, tb, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_bf16_kernel");
}

static int launch_fp8(const void* a, const float* a_s, const void* b, const float* b_s, void* c,
                      int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                      cudaStream_t st) {
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, a, K, M, lda, kQBK, kBM)) return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, b, K, N, ldb, kQBK, kQBN)) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kQSmemBytes));
        RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_gemm_fp8: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kQBN - 1) / kQBN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_fp8_kernel<<<grid, kQThreads, kQSmemBytes, st>>>(
        ta, tb, a_s, b_s, static_cast<__nv_bfloat16*>(c), static_cast<int>(M), static_cast<int>(N),
        static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_fp8_kernel");
}

static int launch_nvfp4(const void* a_codes, const void* a_sf, const float* a_gs,
                        const void* b_codes, const void* b_sf, const float* b_gs, void* c,
                        const int32_t* tile_map, const int32_t* tile_count, int64_t max_m_tiles,
                        int64_t total_rows, int64_t groups, int64_t N, int64_t K, int64_t ldc,
                        cudaStream_t st) {
    CUtensorMap ta, tb;
    if (int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, K / 2, total_rows,
                              K / 2, 128, kBM))
        return rc;
    if (int rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_codes, K / 2, groups * N, K / 2,
                              128, kFBN))
        return rc;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kFSmemBytes));
        RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_gemm_nvfp4_grouped: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    const int64_t tiles = max_m_tiles * ((N + kFBN - 1) / kFBN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_nvfp4_kernel<<<grid, kFThreads, kFSmemBytes, st>>>(
        ta, tb, static_cast<const uint8_t*>(a_sf), static_cast<const uint8_t*>(b_sf), a_gs, b_gs,
        static_cast<__nv_bfloat16*>(c), reinterpret_cast<const int4*>(tile_map), tile_count,
        static_cast<int>(N), static_cast<int>(K), ldc);
    count_launch();
    return check_launch("gemm_nvfp4_kernel");
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
    return tc::launch_nvfp4(a_codes, a_sf, a_gs, b_codes, b_sf, b_gs, c, tile_map, tile_count,
                            max_m_tiles, total_rows, groups, n, k, ldc, as_stream(stream));
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
    if (out_dtype == RT_F32) {
        if (n <= 128) return tc::launch_bf16<128, true>(a, b, c, m, n, k, lda, ldb, ldc, st);
        return tc::launch_bf16<256, true>(a, b, c, m, n, k, lda, ldb, ldc, st);
    }
    if (n <= 128) return tc::launch_bf16<128, false>(a, b, c, m, n, k, lda, ldb, ldc, st);
    return tc::launch_bf16<256, false>(a, b, c, m, n, k, lda, ldb, ldc, st);
}

extern "C" int rt_tc_error_state(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_tc_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_tc_error_state: cannot read the device flag");
    }
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc::g_tc_error, &zero, sizeof(int));
        return fail(RT_ERR_TIMEOUT, "a tensor-core kernel abandoned wait #%d (bounded spin expired)", v);
    }
    return RT_OK;
}
