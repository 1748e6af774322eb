// Sparse multi-query attention of the MLA decode step on the 5th-generation tensor cores.
//
//   out[b, h, :] = softmax_j( scale * (q_abs[b, h, :] . kv[b, idx_j, :] + q_pe[b, h, :] . pe[b, idx_j, :]) )
//                  . kv[b, idx_j, :]                                   j over the selected keys
//
// which is the decode branch of racetrack/models/deepseek.py:799-810 (MLA.forward) with the
// indexer's -inf mask applied by visiting only the selected cache rows: q_abs is q_nope already
// multiplied by the key half of wkv_b (512 wide, the "absorbed" query), kv the latent cache
// [batch, keys, 512], pe the rope cache [batch, keys, 64]; the value half of wkv_b is applied to
// `out` by the caller.
//
// Work item = (sequence b, split of the selected keys, group of G <= 32 heads, half of the 512
// output dims); one CTA each. Per tile of 64 selected keys:
//   loaders   gather the 64 cache rows (1152 bytes each: 1024 latent + 128 rope) with 16-byte
//             cp.async copies into nine 64-dim column blocks [64 keys][128 B], 128-byte swizzle;
//   S = Q K^T 36 tcgen05.mma (M = 128 head rows of which G are real, N = 64 keys, K = 16 dims),
//             the tile read as a K-major B operand;
//   softmax   one thread per head row: tcgen05.ld of its 64 scores, running maximum with a lazy
//             rescale (the accumulator is only rescaled when the maximum grows by more than 2^8),
//             P = exp2(s - m) as bf16 into shared memory (K-major A operand);
//   O += P V  4 tcgen05.mma (N = 256 dims, K = 16 keys) reading THE SAME shared-memory tile as an
//             MN-major B operand (dims contiguous): the gathered rows are staged once.
// Tensor memory: O in columns [0, 256), two S buffers of 64 columns behind it; QK^T of tile t + 1
// is issued before P V of tile t, so the tensor core computes scores while the softmax runs.
// Each CTA leaves an unnormalised fp32 partial (O, running maximum, denominator); a second kernel
// merges the splits. Every wait is bounded (rt_tc.cuh).
#include "rt_tc.cuh"

namespace rt {
namespace tc {

constexpr int kATile = 64;                          // keys per tile
constexpr int kABlocks = 9;                         // 64-dim column blocks of a cache row (8 latent + 1 rope)
constexpr int kAMaxG = 32;                          // head rows staged per CTA
constexpr uint32_t kAPBytes = 128 * 128;            // P: 128 rows x 64 keys bf16
constexpr uint32_t kAQBytes = kABlocks * kAMaxG * 128;
constexpr uint32_t kAKBytes = kABlocks * kATile * 128;
constexpr uint32_t kAQOffset = kAPBytes;
constexpr uint32_t kAKOffset = kAQOffset + kAQBytes;
constexpr uint32_t kABarOffset = kAKOffset + 2 * kAKBytes;
constexpr int kABarriers = 9;                       // qfull, kfull[2], kfree[2], sfull[2], pfull, pfree
constexpr uint32_t kASmemBytes = kABarOffset + kABarriers * 8 + 16 + 1024;
constexpr int kAThreads = 512;
constexpr int kALoaders = 256;                      // warps 8..15
constexpr uint32_t kATmemCols = 512;
constexpr uint32_t kATmemS = 256;                   // first score column
// fp32 accumulate, bf16 x bf16, M = 128; S: both K-major, N = 64; O: B MN-major, N = 256
constexpr uint32_t kASIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (8u << 17) | (8u << 24);
constexpr uint32_t kAOIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (32u << 17) | (8u << 24);
static_assert(kAKOffset % 1024 == 0 && kAKBytes % 1024 == 0, "swizzle atoms are 1024-byte aligned");
static_assert(kASmemBytes <= 232448, "shared memory budget");

// Shared-memory descriptor of an MN-major operand stored with the 128-byte swizzle: a 128-byte
// line holds 64 consecutive MN elements of one K index, 8 lines (K indices) form a 1024-byte
// atom; `lbo` = bytes between 64-element MN blocks, stride byte offset = bytes between groups
// of 8 K indices (1024).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(lbo >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct AttnArgs {
    const __nv_bfloat16* q_abs;   // [batch, heads, 512]
    const __nv_bfloat16* q_pe;    // [batch, heads, 64]
    const __nv_bfloat16* kv;      // [batch, keys, 512]
    const __nv_bfloat16* pe;      // [batch, keys, 64]
    const int32_t* indices;       // [batch, n_sel] or null (all keys in order)
    float* part_o;                // [batch, splits, heads, 512]
    float* part_ml;               // [batch, splits, heads, 2]
    int64_t qa_bs, qa_hs, qp_bs, qp_hs, kv_bs, kv_rs, pe_bs, pe_rs, idx_bs;
    int heads, keys, n_sel, splits, tiles_per_split, group;   // group = G
    float scale_log2;
};

__global__ void __launch_bounds__(kAThreads, 1) mla_sparse_decode_kernel(const AttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kABarOffset;
    const uint32_t qfull = bars;
    auto kfull = [&](int s) { return bars + 8u * (1 + s); };
    auto kfree = [&](int s) { return bars + 8u * (3 + s); };
    auto sfull = [&](int s) { return bars + 8u * (5 + s); };
    const uint32_t pfull = bars + 8u * 7, pfree = bars + 8u * 8;
    const uint32_t slot = bars + 8u * kABarriers;
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kABarOffset + 8 * kABarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x;
    const int half = blockIdx.y & 1, hg = blockIdx.y >> 1;
    const int b = blockIdx.z;
    const int G = a.group;
    const int total_tiles = (a.n_sel + kATile - 1) / kATile;
    const int tile0 = split * a.tiles_per_split;
    const int n_tiles = min(a.tiles_per_split, total_tiles - tile0);
    const int32_t* idx_row = a.indices ? a.indices + b * a.idx_bs : nullptr;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(qfull, kALoaders);
        for (int s = 0; s < 2; ++s) {
            mbar_init(kfull(s), kALoaders);
            mbar_init(kfree(s), 1);
            mbar_init(sfull(s), 1);
        }
        mbar_init(pfull, 4);
        mbar_init(pfree, 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(slot, kATmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            bool ok = mbar_wait(qfull, 0, abort_flag, 61);
            auto issue_qk = [&](int t) {
                const uint32_t kb = base + kAKOffset + (t & 1) * kAKBytes;
                const uint32_t d = tmem_base + kATmemS + static_cast<uint32_t>(t & 1) * 64u;
#pragma unroll
                for (int cb = 0; cb < kABlocks; ++cb) {
                    const uint64_t adesc = smem_desc_sw128(base + kAQOffset + cb * G * 128);
                    const uint64_t bdesc = smem_desc_sw128(kb + cb * (kATile * 128));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma_f16(d, adesc + 2u * j, bdesc + 2u * j, kASIdesc, (cb | j) != 0 ? 1u : 0u);
                }
                mma_commit(sfull(t & 1));
            };
            if (ok && (ok = mbar_wait(kfull(0), 0, abort_flag, 62))) {
                tc_fence_after();
                issue_qk(0);
            }
            for (int t = 0; ok && t < n_tiles; ++t) {
                if (t + 1 < n_tiles) {
                    if (!(ok = mbar_wait(kfull((t + 1) & 1), ((t + 1) >> 1) & 1, abort_flag, 63))) break;
                    tc_fence_after();
                    issue_qk(t + 1);
                }
                if (!(ok = mbar_wait(pfull, t & 1, abort_flag, 64))) break;
                tc_fence_after();
                const uint32_t kb = base + kAKOffset + (t & 1) * kAKBytes + half * 4 * (kATile * 128);
                const uint64_t adesc = smem_desc_sw128(base);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint64_t bdesc = smem_desc_sw128_mn(kb + j * 2048, kATile * 128);
                    mma_f16(tmem_base, adesc + 2u * j, bdesc, kAOIdesc, (t | j) != 0 ? 1u : 0u);
                }
                mma_commit(kfree(t & 1));
                mma_commit(pfree);
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // softmax: thread = head row
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const bool live = row < G && hg * G + row < a.heads;
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        float m_ref = __int_as_float(0xff800000), l = 0.f;
        bool ok = n_tiles > 0;
        for (int t = 0; ok && t < n_tiles; ++t) {
            // which of the tile's 64 slots hold a key
            const int j0 = (tile0 + t) * kATile + lane, j1 = j0 + 32;
            bool v0 = j0 < a.n_sel, v1 = j1 < a.n_sel;
            if (idx_row) {
                if (v0) { const int k = __ldg(idx_row + j0); v0 = k >= 0 && k < a.keys; }
                if (v1) { const int k = __ldg(idx_row + j1); v1 = k >= 0 && k < a.keys; }
            }
            const uint32_t mask0 = __ballot_sync(0xffffffffu, v0), mask1 = __ballot_sync(0xffffffffu, v1);
            if (!(ok = mbar_wait(sfull(t & 1), (t >> 1) & 1, abort_flag, 65))) break;
            tc_fence_after();
            uint32_t r0[32], r1[32];
            const uint32_t taddr = tmem_base + lane_base + kATmemS + static_cast<uint32_t>(t & 1) * 64u;
            tmem_ld_32x32(taddr, r0);
            tmem_ld_32x32(taddr + 32, r1);
            tmem_ld_wait(r0);
            tmem_ld_wait(r1);
            const float ninf = __int_as_float(0xff800000);
            float mt = ninf;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float s0 = (live && ((mask0 >> i) & 1u)) ? __uint_as_float(r0[i]) * a.scale_log2 : ninf;
                const float s1 = (live && ((mask1 >> i) & 1u)) ? __uint_as_float(r1[i]) * a.scale_log2 : ninf;
                r0[i] = __float_as_uint(s0);
                r1[i] = __float_as_uint(s1);
                mt = fmaxf(mt, fmaxf(s0, s1));
            }
            const bool grow = mt > m_ref + 8.f;          // false while mt is -inf
            const float m_new = grow ? mt : m_ref;
            const float alpha = grow ? exp2f(m_ref - m_new) : 1.f;     // exp2f(-inf) = 0 on the first tile
            const float m_use = m_new == ninf ? 0.f : m_new;
            float sum = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float p0 = exp2f(__uint_as_float(r0[2 * i]) - m_use);
                const float p1 = exp2f(__uint_as_float(r0[2 * i + 1]) - m_use);
                const float p2 = exp2f(__uint_as_float(r1[2 * i]) - m_use);
                const float p3 = exp2f(__uint_as_float(r1[2 * i + 1]) - m_use);
                sum += (p0 + p1) + (p2 + p3);
                __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
                packed[i] = *reinterpret_cast<uint32_t*>(&lo);
                packed[16 + i] = *reinterpret_cast<uint32_t*>(&hi);
            }
            l = l * alpha + sum;
            m_ref = m_new;
            if (t > 0) {
                // P V of the previous tile has retired: P may be overwritten, O is at rest
                if (!(ok = mbar_wait(pfree, (t - 1) & 1, abort_flag, 66))) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(tmem_base + lane_base + c * 32, o);
                        tmem_ld_wait(o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(tmem_base + lane_base + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            // P row: 64 bf16 = 8 chunks of 16 bytes, 128-byte swizzle
            uint8_t* prow = base_ptr + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pfull);
        }
        if (ok && n_tiles > 0 && (ok = mbar_wait(pfree, (n_tiles - 1) & 1, abort_flag, 67))) {
            tc_fence_after();
            const int head = hg * G + row;
            const int64_t prt = (static_cast<int64_t>(b) * a.splits + split) * a.heads + head;
            float* po = a.part_o + prt * 512 + half * 256;
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(tmem_base + lane_base + c * 32, o);
                tmem_ld_wait(o);
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(po + c * 32 + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                }
            }
            if (live && half == 0) {
                a.part_ml[prt * 2] = m_ref;
                a.part_ml[prt * 2 + 1] = l;
            }
        }
    } else if (warp >= 8) {
        // loaders
        const int lt = threadIdx.x - 256;
        // the head rows of this group: G x 72 chunks
        {
            const __nv_bfloat16* qa = a.q_abs + b * a.qa_bs;
            const __nv_bfloat16* qp = a.q_pe + b * a.qp_bs;
            for (int c = lt; c < G * 72; c += kALoaders) {
                const int r = c / 72, ch = c % 72, cb = ch >> 3, j = ch & 7;
                const int head = min(hg * G + r, a.heads - 1);
                const void* src = cb < 8 ? static_cast<const void*>(qa + head * a.qa_hs + ch * 8)
                                         : static_cast<const void*>(qp + head * a.qp_hs + j * 8);
                cp_async16(base + kAQOffset + cb * G * 128 + r * 128 + ((j ^ (r & 7)) << 4), src);
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async();
            mbar_arrive(qfull);
        }
        const __nv_bfloat16* kvb = a.kv + b * a.kv_bs;
        const __nv_bfloat16* peb = a.pe + b * a.pe_bs;
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            if (t > 0) {
                // tile t - 1 has landed: publish it BEFORE waiting for a free buffer, because the
                // buffer is freed by an MMA that is issued behind the scores of tile t - 1
                cp_async_wait<0>();
                fence_proxy_async();
                mbar_arrive(kfull((t - 1) & 1));
            }
            if (!(ok = mbar_wait(kfree(t & 1), ((t >> 1) & 1) ^ 1u, abort_flag, 68))) break;
            const uint32_t kb = base + kAKOffset + (t & 1) * kAKBytes;
#pragma unroll 2
            for (int c = lt; c < kATile * 72; c += kALoaders) {
                const int r = c / 72, ch = c % 72, cb = ch >> 3, j = ch & 7;
                const int slot_j = (tile0 + t) * kATile + r;
                int key = -1;
                if (slot_j < a.n_sel) key = idx_row ? __ldg(idx_row + slot_j) : slot_j;
                const bool valid = key >= 0 && key < a.keys;
                const int64_t kk = valid ? key : 0;
                const void* src = cb < 8 ? static_cast<const void*>(kvb + kk * a.kv_rs + ch * 8)
                                         : static_cast<const void*>(peb + kk * a.pe_rs + j * 8);
                cp_async16_zfill(kb + cb * (kATile * 128) + r * 128 + ((j ^ (r & 7)) << 4), src,
                                 valid ? 16u : 0u);
            }
            cp_async_commit();
        }
        cp_async_wait<0>();
        if (ok && n_tiles > 0) {
            fence_proxy_async();
            mbar_arrive(kfull((n_tiles - 1) & 1));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kATmemCols);
    }
}

// out[b, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M): one CTA of 128 threads per
// (sequence, head), 4 dims per thread.
__global__ void __launch_bounds__(128) mla_merge_kernel(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_ml,
                                                        __nv_bfloat16* __restrict__ out, int heads,
                                                        int splits) {
    const int head = blockIdx.x, b = blockIdx.y;
    const float ninf = __int_as_float(0xff800000);
    float m = ninf;
    for (int s = 0; s < splits; ++s)
        m = fmaxf(m, __ldg(part_ml + ((static_cast<int64_t>(b) * splits + s) * heads + head) * 2));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (int s = 0; s < splits; ++s) {
        const int64_t prt = (static_cast<int64_t>(b) * splits + s) * heads + head;
        const float ms = __ldg(part_ml + prt * 2), ls = __ldg(part_ml + prt * 2 + 1);
        if (ms == ninf) continue;
        const float w = exp2f(ms - m);
        const float4 o = __ldg(reinterpret_cast<const float4*>(part_o + prt * 512) + threadIdx.x);
        acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
        den += ls * w;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(out + (static_cast<int64_t>(b) * heads + head) * 512 + threadIdx.x * 4) = v;
}

int attn_error_take() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    }
    return v;
}

}  // namespace tc
}  // namespace rt

using namespace rt;

extern "C" int64_t rt_mla_sparse_decode_splits(int64_t batch, int64_t heads, int64_t n_sel) {
    if (batch <= 0 || heads <= 0 || n_sel <= 0) return 1;
    const int64_t group = heads < tc::kAMaxG ? heads : tc::kAMaxG;
    const int64_t per_split = batch * 2 * ((heads + group - 1) / group);
    const int64_t tiles = (n_sel + tc::kATile - 1) / tc::kATile;
    int64_t splits = (2 * 148 + per_split - 1) / per_split;
    if (splits > tiles) splits = tiles;
    if (splits < 1) splits = 1;
    const int64_t tps = (tiles + splits - 1) / splits;
    return (tiles + tps - 1) / tps;          // every split owns at least one tile
}

extern "C" int rt_mla_sparse_decode(const void* q_abs, const void* q_pe, const void* kv, const void* pe,
                                    const int32_t* indices, void* out, float* part_o, float* part_ml,
                                    int64_t batch, int64_t heads, int64_t keys, int64_t n_sel,
                                    int64_t qa_batch_stride, int64_t qa_head_stride,
                                    int64_t qp_batch_stride, int64_t qp_head_stride,
                                    int64_t kv_batch_stride, int64_t kv_row_stride,
                                    int64_t pe_batch_stride, int64_t pe_row_stride,
                                    int64_t idx_batch_stride, int64_t splits, float softmax_scale,
                                    void* stream) {
    RT_REQUIRE(batch >= 0 && heads > 0 && keys > 0 && n_sel > 0, RT_ERR_BAD_ARG,
               "rt_mla_sparse_decode: bad shape");
    if (batch == 0) return RT_OK;
    RT_REQUIRE(q_abs && q_pe && kv && pe && out && part_o && part_ml, RT_ERR_BAD_ARG,
               "rt_mla_sparse_decode: null pointer");
    RT_REQUIRE(heads % 8 == 0 && (heads <= tc::kAMaxG || heads % tc::kAMaxG == 0), RT_ERR_UNSUPPORTED,
               "rt_mla_sparse_decode: heads must be 8, 16, 24, 32 or a multiple of 32");
    RT_REQUIRE(aligned16(q_abs) && aligned16(q_pe) && aligned16(kv) && aligned16(pe) && aligned16(part_o),
               RT_ERR_BAD_ARG, "rt_mla_sparse_decode: pointers must be 16-byte aligned");
    RT_REQUIRE(qa_batch_stride % 8 == 0 && qa_head_stride % 8 == 0 && qp_batch_stride % 8 == 0 &&
                   qp_head_stride % 8 == 0 && kv_batch_stride % 8 == 0 && kv_row_stride % 8 == 0 &&
                   pe_batch_stride % 8 == 0 && pe_row_stride % 8 == 0,
               RT_ERR_BAD_ARG, "rt_mla_sparse_decode: strides must be multiples of 8 elements");
    RT_REQUIRE(keys < (1ll << 31) && n_sel < (1ll << 31) && batch < 65536, RT_ERR_UNSUPPORTED,
               "rt_mla_sparse_decode: dimension too large");
    RT_REQUIRE(indices || n_sel == keys, RT_ERR_BAD_ARG,
               "rt_mla_sparse_decode: without indices n_sel must equal keys");
    const int64_t tiles = (n_sel + tc::kATile - 1) / tc::kATile;
    RT_REQUIRE(splits >= 1 && splits <= tiles, RT_ERR_BAD_ARG, "rt_mla_sparse_decode: bad split count");
    const int64_t tps = (tiles + splits - 1) / splits;
    RT_REQUIRE((tiles + tps - 1) / tps == splits, RT_ERR_BAD_ARG,
               "rt_mla_sparse_decode: a split would own no tile (use rt_mla_sparse_decode_splits)");
    cudaStream_t st = as_stream(stream);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&tc::mla_sparse_decode_kernel),
                                     static_cast<int>(tc::kASmemBytes), "rt_mla_sparse_decode"))
        return rc;
    tc::AttnArgs a;
    a.q_abs = static_cast<const __nv_bfloat16*>(q_abs);
    a.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
    a.kv = static_cast<const __nv_bfloat16*>(kv);
    a.pe = static_cast<const __nv_bfloat16*>(pe);
    a.indices = indices;
    a.part_o = part_o;
    a.part_ml = part_ml;
    a.qa_bs = qa_batch_stride; a.qa_hs = qa_head_stride;
    a.qp_bs = qp_batch_stride; a.qp_hs = qp_head_stride;
    a.kv_bs = kv_batch_stride; a.kv_rs = kv_row_stride;
    a.pe_bs = pe_batch_stride; a.pe_rs = pe_row_stride;
    a.idx_bs = idx_batch_stride;
    a.heads = static_cast<int>(heads);
    a.keys = static_cast<int>(keys);
    a.n_sel = static_cast<int>(n_sel);
    a.splits = static_cast<int>(splits);
    a.tiles_per_split = static_cast<int>(tps);
    a.group = static_cast<int>(heads < tc::kAMaxG ? heads : tc::kAMaxG);
    a.scale_log2 = softmax_scale * 1.4426950408889634f;
    const int groups = static_cast<int>((heads + a.group - 1) / a.group);
    dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(2 * groups), static_cast<unsigned>(batch));
    tc::mla_sparse_decode_kernel<<<grid, tc::kAThreads, tc::kASmemBytes, st>>>(a);
    count_launch();
    if (int rc = check_launch("mla_sparse_decode_kernel")) return rc;
    dim3 mgrid(static_cast<unsigned>(heads), static_cast<unsigned>(batch));
    tc::mla_merge_kernel<<<mgrid, 128, 0, st>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out),
                                                 static_cast<int>(heads), static_cast<int>(splits));
    count_launch();
    return check_launch("mla_merge_kernel");
}
