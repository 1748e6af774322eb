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
// Work item = (sequence b, split of the selected keys, group of G <= 64 heads); one CTA each.
// Per tile of 32 selected keys:
//   loaders   gather the 32 cache rows (1152 bytes each: 1024 latent + 128 rope) with 16-byte
//             cp.async copies into nine 64-dim column blocks [32 keys][128 B], 128-byte swizzle,
//             a ring of 4 tiles (3 when G > 32). What bounds this kernel is the gather: the
//             load/store path of one SM sustains about 12 B/clk for it (measured; it keeps about
//             8 KB in flight), so the ring only has to keep that path busy all the time;
//   S = Q K^T 36 tcgen05.mma (M = 128 head rows of which G are real, N = 32 keys, K = 16 dims),
//             the tile read as a K-major B operand;
//   softmax   one thread per head row: tcgen05.ld of its 32 scores, running maximum with a lazy
//             rescale (the accumulator is only rescaled when the maximum grows by more than 2^8),
//             P = exp2(s - m) as bf16 into shared memory (K-major A operand);
//   O += P V  tcgen05.mma (N = 256 dims, K = 16 keys) reading THE SAME shared-memory tile as an
//             MN-major B operand (dims contiguous): the gathered rows are staged once. The 512
//             output dims would fill all of tensor memory as columns, so they are folded into the
//             LANES instead: P occupies 64 rows with a block of 64 zero rows before and behind
//             it; the MMA whose A operand starts at P writes dims [0, 256) of head r to lane r
//             (and adds zeros to lanes 64-127), the MMA whose A operand starts at the zero block
//             before P writes dims [256, 512) to lane 64 + r, both into the same 256 columns.
// Tensor memory: O in columns [0, 256), two S buffers of 32 columns behind it. One thread issues
// all MMAs and takes whichever is ready first, the scores of the next landed tile or P V of the
// tile whose probabilities are written, so the tensor core computes scores while the softmax runs.
// Each CTA leaves an unnormalised fp32 partial (O, running maximum, denominator); a second kernel
// merges the splits. Every wait is bounded (rt_tc.cuh).
#include "rt_tc.cuh"

namespace rt {
namespace tc {

constexpr int kATile = 32;                          // keys per tile
constexpr int kABlocks = 9;                         // 64-dim column blocks of a cache row (8 latent + 1 rope)
constexpr int kAMaxG = 64;                          // head rows staged per CTA
constexpr int kAMaxStages = 4;
constexpr uint32_t kAPOffset = 64 * 128;            // 64 zero rows | P: 64 rows of 128 bytes | 64 zero rows
constexpr uint32_t kAKBytes = kABlocks * kATile * 128;
constexpr uint32_t kAQOffset = 3 * 64 * 128;
// the tile ring follows the G staged head rows: 4 tiles for G <= 32, 3 for G = 64
constexpr uint32_t kABarOffset = kAQOffset + kABlocks * 32 * 128 + kAMaxStages * kAKBytes;
constexpr int kABarriers = 1 + 2 * kAMaxStages + 2 + 2 + 2;   // qfull, kfull[4], kfree[4], sfull[2], pfull, pfree, afull[2]
constexpr uint32_t kAAlphaOffset = kABarOffset + kABarriers * 8 + 16;   // rescale factors [2][64] + flags [2][2]
constexpr uint32_t kASmemBytes = kAAlphaOffset + 2 * 64 * 4 + 16 + 1024;
constexpr int kAThreads = 512;
constexpr int kALoaders = 256;                      // warps 8..15
constexpr uint32_t kATmemCols = 512;
constexpr uint32_t kATmemS = 256;                   // first score column
// fp32 accumulate, bf16 x bf16, M = 128; S: both K-major, N = 32; O: B MN-major, N = 256
constexpr uint32_t kASIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kATile >> 3) << 17) | (8u << 24);
constexpr uint32_t kAOIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (32u << 17) | (8u << 24);
static_assert(kAKBytes % 1024 == 0 && kAQOffset % 1024 == 0, "swizzle atoms are 1024-byte aligned");
static_assert(kAQOffset + kABlocks * 64 * 128 + 3 * kAKBytes <= kABarOffset, "G = 64 leaves room for 3 tiles");
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

// Optional pipeline trace (never compiled into the library): with -DRT_ATTN_TRACE the CTA
// (0, 0, 0) stamps clock64() at eight points of its first 64 tiles.
#ifdef RT_ATTN_TRACE
__device__ long long g_attn_trace[8 * 64];
#define RT_ATRACE(ev, it) \
    do { if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0 && (it) < 64) g_attn_trace[(ev) * 64 + (it)] = clock64(); } while (0)
#else
#define RT_ATRACE(ev, it) do { } while (0)
#endif

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
    auto kfree = [&](int s) { return bars + 8u * (1 + kAMaxStages + s); };
    auto sfull = [&](int s) { return bars + 8u * (1 + 2 * kAMaxStages + s); };
    const uint32_t pfull = bars + 8u * (3 + 2 * kAMaxStages), pfree = pfull + 8u;
    auto afull = [&](int s) { return pfree + 8u * (1 + s); };
    const uint32_t slot = bars + 8u * kABarriers;
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(base_ptr + kABarOffset + 8 * kABarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x;
    const int hg = blockIdx.y;
    const int b = blockIdx.z;
    const int G = a.group;
    const int stages = G > 32 ? 3 : kAMaxStages;
    const uint32_t k_off = kAQOffset + static_cast<uint32_t>(kABlocks * (G > 32 ? 64 : 32) * 128);
    const int total_tiles = (a.n_sel + kATile - 1) / kATile;
    const int tile0 = split * a.tiles_per_split;
    const int n_tiles = min(a.tiles_per_split, total_tiles - tile0);
    const int32_t* idx_row = a.indices ? a.indices + b * a.idx_bs : nullptr;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(qfull, kALoaders);
        for (int s = 0; s < kAMaxStages; ++s) {
            mbar_init(kfull(s), kALoaders);
            mbar_init(kfree(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(sfull(s), 1);
            mbar_init(afull(s), 2);          // lane 0 of the two softmax warps
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
            // Scores of tile q are issued as soon as its rows have landed and a score buffer is
            // free (q - v < 2), P V of tile v as soon as its probabilities are written: whichever
            // comes first, so neither the gather nor the softmax waits behind the other.
            int q = 0, v = 0, qs = 0, vs = 0;          // tile counters and their ring slots
            uint32_t qphase = 0;
            long long t0 = 0;
            uint32_t spins = 0;
            while (ok && v < n_tiles) {
                bool progressed = false;
                if (q < n_tiles && q - v < 2 && mbar_try_wait(kfull(qs), qphase)) {
                    tc_fence_after();
                    RT_ATRACE(0, q);
                    const uint32_t kb = base + k_off + qs * kAKBytes;
                    const uint32_t d = tmem_base + kATmemS + static_cast<uint32_t>(q & 1) * kATile;
#pragma unroll
                    for (int cb = 0; cb < kABlocks; ++cb) {
                        const uint64_t adesc = smem_desc_sw128(base + kAQOffset + cb * G * 128);
                        const uint64_t bdesc = smem_desc_sw128(kb + cb * (kATile * 128));
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            mma_f16(d, adesc + 2u * j, bdesc + 2u * j, kASIdesc, (cb | j) != 0 ? 1u : 0u);
                    }
                    mma_commit(sfull(q & 1));
                    ++q;
                    if (++qs == stages) {
                        qs = 0;
                        qphase ^= 1u;
                    }
                    progressed = true;
                }
                if (v < q && mbar_try_wait(pfull, v & 1)) {
                    RT_ATRACE(1, v);
                    tc_fence_after();
                    const uint32_t kb = base + k_off + vs * kAKBytes;
                    const uint64_t a_lo = smem_desc_sw128(base + kAPOffset);      // [P; zeros]
                    const uint64_t a_hi = smem_desc_sw128(base);                  // [zeros; P]
#pragma unroll
                    for (int j = 0; j < kATile / 16; ++j) {
                        const uint64_t b_lo = smem_desc_sw128_mn(kb + j * 2048, kATile * 128);
                        const uint64_t b_hi = smem_desc_sw128_mn(kb + 4 * (kATile * 128) + j * 2048, kATile * 128);
                        mma_f16(tmem_base, a_lo + 2u * j, b_lo, kAOIdesc, (v | j) != 0 ? 1u : 0u);
                        mma_f16(tmem_base, a_hi + 2u * j, b_hi, kAOIdesc, 1u);
                    }
                    mma_commit(kfree(vs));
                    mma_commit(pfree);
                    RT_ATRACE(2, v);
                    ++v;
                    if (++vs == stages) vs = 0;
                    progressed = true;
                }
                if (progressed) {
                    spins = 0;
                } else if ((++spins & 63u) == 0) {
                    // bounded like mbar_wait: give up after the cycle budget or when another
                    // thread of the CTA already has
                    if (spins == 64) t0 = clock64();
                    if (*abort_flag) ok = false;
                    else if (clock64() - t0 > kWaitCycles) {
                        *abort_flag = 63;
                        atomicCAS(&g_tc_error, 0, 63);
                        ok = false;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // Softmax (warps 4, 5: thread = head row, lanes 0-63 of tensor memory) and the keepers of
        // lanes 64-127 (warps 6, 7: the upper 256 dims of the same heads), which only take part
        // in rescaling and in the final read-out.
        const int quad = warp & 3;
        const int row = (quad & 1) * 32 + lane;            // head row within the group
        const bool upper = quad >= 2;
        const bool live = row < G && hg * G + row < a.heads;
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const float ninf = __int_as_float(0xff800000);
        float* alpha_s = reinterpret_cast<float*>(base_ptr + kAAlphaOffset);       // [2][64]
        volatile int* grow_s = reinterpret_cast<volatile int*>(alpha_s + 128);     // [2][2]
        float m_ref = ninf, l = 0.f;
        bool ok = n_tiles > 0;
        for (int t = 0; ok && t < n_tiles; ++t) {
            float alpha = 1.f;
            uint32_t packed[16];
            if (!upper) {
                // which of the tile's 32 slots hold a key
                const int j0 = (tile0 + t) * kATile + lane;
                bool v0 = j0 < a.n_sel;
                if (idx_row && v0) {
                    const int k = __ldg(idx_row + j0);
                    v0 = k >= 0 && k < a.keys;
                }
                const uint32_t mask0 = __ballot_sync(0xffffffffu, v0);
                if (!(ok = mbar_wait(sfull(t & 1), (t >> 1) & 1, abort_flag, 65))) break;
                if (threadIdx.x == 128) RT_ATRACE(3, t);
                tc_fence_after();
                uint32_t r0[32];
                tmem_ld_32x32(tmem_base + lane_base + kATmemS + static_cast<uint32_t>(t & 1) * kATile, r0);
                tmem_ld_wait(r0);
                float mt = ninf;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float s0 = (live && ((mask0 >> i) & 1u)) ? __uint_as_float(r0[i]) * a.scale_log2 : ninf;
                    r0[i] = __float_as_uint(s0);
                    mt = fmaxf(mt, s0);
                }
                const bool grow = mt > m_ref + 8.f;          // false while mt is -inf
                const float m_new = grow ? mt : m_ref;
                alpha = grow ? exp2f(m_ref - m_new) : 1.f;   // exp2f(-inf) = 0 on the first tile
                const float m_use = m_new == ninf ? 0.f : m_new;
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = exp2f(__uint_as_float(r0[2 * i]) - m_use);
                    const float p1 = exp2f(__uint_as_float(r0[2 * i + 1]) - m_use);
                    sum += p0 + p1;
                    __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    packed[i] = *reinterpret_cast<uint32_t*>(&pk);
                }
                l = l * alpha + sum;
                m_ref = m_new;
                alpha_s[(t & 1) * 64 + row] = alpha;
                const bool any = __any_sync(0xffffffffu, grow);
                if (lane == 0) grow_s[(t & 1) * 2 + quad] = any ? 1 : 0;
                __syncwarp();
                if (lane == 0) mbar_arrive(afull(t & 1));
            }
            // rescale factors and flags of this tile are visible to all four warps
            if (!(ok = mbar_wait(afull(t & 1), (t >> 1) & 1, abort_flag, 69))) break;
            if (t > 0) {
                // P V of the previous tile has retired: P may be overwritten, O is at rest
                if (!(ok = mbar_wait(pfree, (t - 1) & 1, abort_flag, 66))) break;
                tc_fence_after();
                if (grow_s[(t & 1) * 2] | grow_s[(t & 1) * 2 + 1]) {
                    const float al = alpha_s[(t & 1) * 64 + row];
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(tmem_base + lane_base + c * 32, o);
                        tmem_ld_wait(o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * al);
                        tmem_st_32x32(tmem_base + lane_base + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            if (!upper) {
                // P row: 32 bf16 = 4 chunks of 16 bytes in a 128-byte swizzled row
                uint8_t* prow = base_ptr + kAPOffset + row * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                fence_proxy_async();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pfull);
            if (threadIdx.x == 128) RT_ATRACE(4, t);
        }
        if (ok && n_tiles > 0 && (ok = mbar_wait(pfree, (n_tiles - 1) & 1, abort_flag, 67))) {
            tc_fence_after();
            const int head = hg * G + row;
            const int64_t prt = (static_cast<int64_t>(b) * a.splits + split) * a.heads + head;
            float* po = a.part_o + prt * 512 + (upper ? 256 : 0);
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
            if (live && !upper) {
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
            // the zero rows before and behind P
            for (int c = lt; c < 2 * 64 * 8; c += kALoaders) {
                const int blk = c >> 9, off = (c & 511) << 4;
                *reinterpret_cast<uint4*>(base_ptr + (blk ? 2 * kAPOffset : 0) + off) = make_uint4(0u, 0u, 0u, 0u);
            }
            cp_async_wait<0>();
            fence_proxy_async();
            mbar_arrive(qfull);
        }
        const __nv_bfloat16* kvb = a.kv + b * a.kv_bs;
        const __nv_bfloat16* peb = a.pe + b * a.pe_bs;
        // Tile t goes into ring slot t % stages once P V of tile t - stages has retired. Its copies
        // are committed as one group and tile t - 1 is published when ITS group has landed, so
        // two tiles are in flight; a tile that is waited for never depends on a later one (the
        // MMA thread takes scores and P V in whichever order they become ready).
        bool ok = true;
        int ls = 0;
        uint32_t lphase = 0;
        for (int t = 0; t < n_tiles; ++t) {
            if (!(ok = mbar_wait(kfree(ls), lphase ^ 1u, abort_flag, 68))) break;
            if (lt == 0) RT_ATRACE(5, t);
            const uint32_t kb = base + k_off + ls * kAKBytes;
#pragma unroll 3
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
            if (lt == 0) RT_ATRACE(6, t);
            if (t > 0) {
                cp_async_wait<1>();
                fence_proxy_async();
                mbar_arrive(kfull(ls == 0 ? stages - 1 : ls - 1));
                if (lt == 0) RT_ATRACE(7, t - 1);
            }
            if (++ls == stages) {
                ls = 0;
                lphase ^= 1u;
            }
        }
        cp_async_wait<0>();
        if (ok && n_tiles > 0) {
            fence_proxy_async();
            mbar_arrive(kfull(ls == 0 ? stages - 1 : ls - 1));
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
// (sequence, head), 4 dims per thread; the partials of eight splits are loaded before any of
// them is used, so a merge of many splits is not a chain of dependent loads.
__global__ void __launch_bounds__(128) mla_merge_kernel(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_ml,
                                                        __nv_bfloat16* __restrict__ out, int heads,
                                                        int splits) {
    const int head = blockIdx.x, b = blockIdx.y;
    const float ninf = __int_as_float(0xff800000);
    const int64_t prt0 = static_cast<int64_t>(b) * splits * heads + head;      // + s * heads
    __shared__ float w_s[64], red_s[2];
    // weights of the splits: lane s of the first two warps owns split s (splits <= 64)
    if (threadIdx.x < 64) {
        const int s = threadIdx.x;
        const float ms = s < splits ? __ldg(part_ml + (prt0 + static_cast<int64_t>(s) * heads) * 2) : ninf;
        const float ls = s < splits ? __ldg(part_ml + (prt0 + static_cast<int64_t>(s) * heads) * 2 + 1) : 0.f;
        float m = ms;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = m;
        asm volatile("bar.sync 1, 64;" ::: "memory");
        m = fmaxf(red_s[0], red_s[1]);
        const float w = ms == ninf ? 0.f : exp2f(ms - m);
        w_s[s] = w;
        float den = ls * w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        asm volatile("bar.sync 1, 64;" ::: "memory");      // both maxima have been read
        if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = den;
    }
    __syncthreads();
    const float den = red_s[0] + red_s[1];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 8) {
        float4 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s = min(s0 + i, splits - 1);
            o[i] = __ldg(reinterpret_cast<const float4*>(part_o + (prt0 + static_cast<int64_t>(s) * heads) * 512) +
                         threadIdx.x);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float w = s0 + i < splits ? w_s[s0 + i] : 0.f;
            acc.x += o[i].x * w; acc.y += o[i].y * w; acc.z += o[i].z * w; acc.w += o[i].w * w;
        }
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

#ifdef RT_ATTN_TRACE
extern "C" int rt_attn_trace_read(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, tc::g_attn_trace, sizeof(long long) * 8 * 64) == cudaSuccess
               ? RT_OK : RT_ERR_CUDA;
}
#endif

extern "C" int64_t rt_mla_sparse_decode_splits(int64_t batch, int64_t heads, int64_t n_sel) {
    if (batch <= 0 || heads <= 0 || n_sel <= 0) return 1;
    const int64_t group = heads < tc::kAMaxG ? heads : tc::kAMaxG;
    const int64_t per_split = batch * ((heads + group - 1) / group);
    const int64_t tiles = (n_sel + tc::kATile - 1) / tc::kATile;
    // One CTA per SM at a time: the launch takes (waves of CTAs) x (tiles per CTA + the CTA's
    // fixed cost: query rows, tensor-memory allocation, fp32 partials; about a tile and a half).
    // Pick the split count that minimises it; every split owns at least one tile.
    const int64_t sms = 148;
    int64_t best = 1;
    double best_cost = 1e30;
    for (int64_t s = 1; s <= tiles && s <= 64; ++s) {
        const int64_t tps = (tiles + s - 1) / s;
        const int64_t eff = (tiles + tps - 1) / tps;
        const int64_t waves = (per_split * eff + sms - 1) / sms;
        const double cost = static_cast<double>(waves) * (static_cast<double>(tps) + 1.5) + 0.02 * eff;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = eff;
        }
    }
    return best;
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
               "rt_mla_sparse_decode: heads must be a multiple of 8 up to 64, or a multiple of 64");
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
    RT_REQUIRE(splits >= 1 && splits <= tiles && splits <= 64, RT_ERR_BAD_ARG,
               "rt_mla_sparse_decode: the split count must lie in [1, min(tiles, 64)]");
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
    dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(groups), static_cast<unsigned>(batch));
    tc::mla_sparse_decode_kernel<<<grid, tc::kAThreads, tc::kASmemBytes, st>>>(a);
    count_launch();
    if (int rc = check_launch("mla_sparse_decode_kernel")) return rc;
    dim3 mgrid(static_cast<unsigned>(heads), static_cast<unsigned>(batch));
    tc::mla_merge_kernel<<<mgrid, 128, 0, st>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out),
                                                 static_cast<int>(heads), static_cast<int>(splits));
    count_launch();
    return check_launch("mla_merge_kernel");
}
