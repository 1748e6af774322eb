// Attention kernels on the 5th-generation tensor cores: the sparse multi-query attention of the
// MLA decode step (first part of this file) and the causal attention of the prefill stack
// (attn_prefill_kernel, second part).
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


// ---------------------------------------------------------------------------
// Causal attention of the prefill stack (racetrack/runtime/torch_ops.py:97-110,
// racetrack/realistic_bench.py:304-313): out[t, h] = softmax_j<=t(scale q[t, h] . k[j, h]) v[j, h]
// ---------------------------------------------------------------------------
// The key of head h is [k_nope[j, h] | k_pe[j]]: the rope part may be one row per token shared by
// all heads (MLA), so it is a separate operand and is never broadcast in memory.
//
// One CTA per (block of 256 query rows, head): two query tiles of 128 rows, processed in
// ping-pong against key tiles of 128 keys, so that the tensor core works on one tile while the
// other tile's softmax runs. Per key tile j and query tile t:
//   S_t = Q_t K_j^T    tcgen05.mma, both operands K-major in shared memory (64-dim chunks of
//                      [128 rows][128 B], 128-byte swizzle), 128 x 128 fp32 scores in tensor memory;
//   softmax            two threads per query row (8 warps per tile: the special-function unit
//                      evaluates 16 exponentials per clock and SM, so a tile's 16384 take 1024
//                      clocks whoever issues them; two warps per scheduler keep it busy), each
//                      with 64 of the row's scores in registers after one tcgen05.ld pass: causal
//                      mask on the diagonal tile, the two half-row maxima exchanged through shared
//                      memory (as bf16, so both threads use the same value), running maximum with a
//                      lazy rescale (the accumulator is rescaled only when the maximum grows by
//                      more than 2^8), P = exp2(s - m) written back as bf16 INTO THE SCORE COLUMNS
//                      (two per column);
//   O_t += P_t V_j     tcgen05.mma with A = P read from tensor memory and B = V read from shared
//                      memory MN-major (the value dims contiguous), so P never touches shared memory.
// Tensor memory (512 columns): S_0 | S_1 | O_0 | O_1, 128 columns each. Shared memory: the two
// query tiles (96 KB), two stages of key tiles (96 KB), one value tile (32 KB). MMAs issued by
// one thread execute in order, which is what lets P alias S: S_t(j + 1) is issued after
// O_t += P_t(j) V_j. Warps: 0 TMA producer, 1 tensor-memory owner and MMA issuer, 2-9 softmax and
// epilogue of tile 0, 10-17 of tile 1 (within a tile the first four warps take key columns
// 0-63, the other four 64-127; a warp touches the tensor-memory lanes of quarter warp % 4).
// Every wait is bounded (rt_tc.cuh).
// CTAs are launched heaviest first (the last query block of a head attends to the most keys)
// and head-major, so the CTAs in flight share few heads' keys and values in L2.
constexpr int kFThreads = 576;                             // 2 + 2 tiles x 8 softmax warps
constexpr uint32_t kFChunk = 128 * 128;                    // [128 rows][64 bf16]
constexpr uint32_t kFQOff = 0;                             // 2 tiles x 3 chunks
constexpr uint32_t kFKOff = 6 * kFChunk;                   // 2 stages x 3 chunks
constexpr uint32_t kFVOff = 12 * kFChunk;                  // 2 chunks
constexpr uint32_t kFBarOff = 14 * kFChunk;
constexpr int kFBars = 12;     // q_full[2] k_full[2] k_empty[2] v_full v_empty s_full[2] p_full[2] + o_full[2] below
constexpr uint32_t kFXmOff = kFBarOff + (kFBars + 2) * 8 + 16;        // row maxima exchanged as bf16 [2][128][2]
constexpr uint32_t kFSmemBytes = kFXmOff + 2 * 128 * 2 * 2 + 1024;
static_assert(kFSmemBytes <= 232448, "shared memory budget");

// Optional pipeline trace (never compiled into the library): with -DRT_FA_TRACE the CTA of the
// heaviest query block of head 0 stamps clock64() at ten points of its first 64 key tiles.
#ifdef RT_FA_TRACE
__device__ long long g_fa_trace[10 * 64];
#define RT_FTRACE(ev, it) \
    do { if ((blockIdx.x | blockIdx.y) == 0 && (it) < 64) g_fa_trace[(ev) * 64 + (it)] = clock64(); } while (0)
#else
#define RT_FTRACE(ev, it) do { } while (0)
#endif

// 0: by shape and length, 1: the single-CTA kernel, 2: CTA pairs wherever the head shape allows
// (rt_attn_prefill_schedule; for A/B measurements and tests).
static int g_attn_schedule = 0;

struct PrefillArgs {
    __nv_bfloat16* out;          // [tokens, heads, v_dim] with strides o_ts / o_hs (elements)
    int64_t o_ts, o_hs;
    int tokens, heads;
    int cn, cp, cv;              // 64-dim chunks of the nope part, the rope part, the values
    int v_dim;
    int one_op;                  // bit i set: operand i (q_nope, q_pe, k_nope, k_pe, v) arrives as ONE box
    int pe_shared;               // k_pe has one row per token for all heads
    float scale_log2;
    // optional (pair schedule, v_dim 128): the output as act_quant leaves it, FP8 e4m3 codes
    // [tokens, heads * 128] and one fp32 scale per token and head (= per 128-wide group)
    uint8_t* out_codes;
    float* out_scales;
};

// Two fp32 -> two e4m3 (RNE, saturating), `lo` in the low byte.
__device__ __forceinline__ uint32_t attn_cvt_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for x <= 8 on the FMA pipe (the special-function unit evaluates only 4 exponentials per
// clock and scheduler, which would bound the softmax): x = n + f with n = round(x), |f| <= 1/2,
// 2^f by a degree-4 polynomial (relative error 4e-6, far below the bf16 rounding of P), 2^n by
// adding n to the exponent field. Inputs below -125 give 0 like ex2.approx.ftz.
__device__ __forceinline__ float ex2_poly(float x) {
    x = fmaxf(x, -125.f);
    const float t = x + 12582912.f;                       // 1.5 * 2^23: the integer part lands in the low bits
    const float f = x - (t - 12582912.f);
    float p = fmaf(f, 9.6181291e-3f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.0f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}

// 32 scores of one row -> 32 probabilities as 16 bf16 pairs, and their fp32 sum. One pair in
// kFPolyEvery takes the polynomial route, the rest the special-function unit (0: none).
#ifndef RT_FA_POLY_EVERY
#define RT_FA_POLY_EVERY 0
#endif
#ifndef RT_FA_PAIR_POLY_EVERY
#define RT_FA_PAIR_POLY_EVERY 0
#endif
template <int kFPolyEvery>
__device__ __forceinline__ void softmax_chunk(const uint32_t (&r)[32], uint32_t (&pk)[16], float scale,
                                              float m, float& sum) {
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float x0 = fmaf(__uint_as_float(r[2 * i]), scale, -m);
        const float x1 = fmaf(__uint_as_float(r[2 * i + 1]), scale, -m);
        float p0, p1;
        if (kFPolyEvery > 0 && (i % (kFPolyEvery > 0 ? kFPolyEvery : 1)) == kFPolyEvery - 1) {
            p0 = ex2_poly(x0);
            p1 = ex2_poly(x1);
        } else {
            p0 = ex2_approx(x0);
            p1 = ex2_approx(x1);
        }
#if defined(RT_FA_DIAG) && RT_FA_DIAG == 2      // diagnostic build only: no exponentials
        p0 = x0;
        p1 = x1;
#endif
        acc0 += p0;
        acc1 += p1;
        pk[i] = pack_bf16x2(p0, p1);
    }
    sum += acc0 + acc1;
}

__global__ void __launch_bounds__(kFThreads, 1) attn_prefill_kernel(
    const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp,
    const __grid_constant__ CUtensorMap tm_kn, const __grid_constant__ CUtensorMap tm_kp,
    const __grid_constant__ CUtensorMap tm_v, const PrefillArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kFBarOff;
    auto q_full = [&](int t) { return bars + 8u * t; };
    auto k_full = [&](int st) { return bars + 8u * (2 + st); };
    auto k_empty = [&](int st) { return bars + 8u * (4 + st); };
    const uint32_t v_full = bars + 8u * 6, v_empty = bars + 8u * 7;
    auto s_full = [&](int t) { return bars + 8u * (8 + t); };
    auto p_full = [&](int t) { return bars + 8u * (10 + t); };
    auto o_full = [&](int t) { return bars + 8u * (12 + t); };
    const uint32_t slot = bars + 8u * (kFBars + 2);
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + kFBarOff + 8 * (kFBars + 2));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // heaviest first
    const int h = blockIdx.y;
    const int q0 = qb * 256;
    const int n0 = q0 / 128 + 1;                        // key tiles of query tile 0 (the last one is diagonal)
    const bool has1 = q0 + 128 < a.tokens;
    const int n1 = has1 ? n0 + 1 : 0;
    const int n_max = has1 ? n1 : n0;
    const int nk = a.cn + a.cp;                         // 64-dim chunks of a query / key row

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full(i), 1);
            mbar_init(k_full(i), 1);
            mbar_init(k_empty(i), 1);
            mbar_init(s_full(i), 1);
            mbar_init(p_full(i), 8);                    // lane 0 of the tile's eight softmax warps
            mbar_init(o_full(i), 1);
        }
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        fence_mbar_init();
        tma_prefetch_desc(&tm_qn);
        tma_prefetch_desc(&tm_kn);
        tma_prefetch_desc(&tm_v);
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
            // one operand: `chunks` 64-dim blocks of 128 rows starting at `row`, as one box or one per chunk
            auto load = [&](const CUtensorMap* m, bool one, int chunks, uint32_t dst, int row, int head,
                            uint32_t bar) {
                if (one) {
                    tma_load_4d(dst, m, 0, row, 0, head, bar);
                } else {
                    for (int c = 0; c < chunks; ++c) tma_load_4d(dst + c * kFChunk, m, 64 * c, row, 0, head, bar);
                }
            };
            const int pe_head = a.pe_shared ? 0 : h;
            for (int t = 0; t < (has1 ? 2 : 1); ++t) {
                const uint32_t dst = base + kFQOff + t * 3 * kFChunk;
                mbar_arrive_expect_tx(q_full(t), nk * kFChunk);
                load(&tm_qn, a.one_op & 1, a.cn, dst, q0 + 128 * t, h, q_full(t));
                if (a.cp) load(&tm_qp, a.one_op & 2, a.cp, dst + a.cn * kFChunk, q0 + 128 * t, h, q_full(t));
            }
            bool ok = true;
            auto load_k = [&](int j) {
                const int st = j & 1;
                if (!(ok = mbar_wait(k_empty(st), ((j >> 1) & 1) ^ 1u, abort_flag, 71))) return;
                const uint32_t dst = base + kFKOff + st * 3 * kFChunk;
                mbar_arrive_expect_tx(k_full(st), nk * kFChunk);
                load(&tm_kn, a.one_op & 4, a.cn, dst, 128 * j, h, k_full(st));
                if (a.cp) load(&tm_kp, a.one_op & 8, a.cp, dst + a.cn * kFChunk, 128 * j, pe_head, k_full(st));
            };
            auto load_v = [&](int j) {
                if (!(ok = mbar_wait(v_empty, (j & 1) ^ 1u, abort_flag, 72))) return;
                mbar_arrive_expect_tx(v_full, a.cv * kFChunk);
                load(&tm_v, a.one_op & 16, a.cv, base + kFVOff, 128 * j, h, v_full);
            };
            // in the order the buffers become free: K_0 V_0 K_1, then K_(j+2) V_(j+1)
            load_k(0);
            if (ok) load_v(0);
            if (ok && n_max > 1) load_k(1);
            for (int j = 0; ok && j < n_max; ++j) {
                if (j + 2 < n_max) load_k(j + 2);
                if (ok && j + 1 < n_max) load_v(j + 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // fp32 accumulate, bf16 x bf16, M = 128; S: both K-major, N = 128; O: B MN-major, N = 64 * cv
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (16u << 17) | (8u << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                     (static_cast<uint32_t>(8 * a.cv) << 17) | (8u << 24);
            auto t_s = [&](int t) { return tmem_base + static_cast<uint32_t>(128 * t); };
            auto t_o = [&](int t) { return tmem_base + static_cast<uint32_t>(256 + 128 * t); };
            auto issue_s = [&](int t, int j) {
                const uint32_t qa = base + kFQOff + t * 3 * kFChunk, kb = base + kFKOff + (j & 1) * 3 * kFChunk;
                for (int c = 0; c < nk; ++c) {
                    const uint64_t adesc = smem_desc_sw128(qa + c * kFChunk);
                    const uint64_t bdesc = smem_desc_sw128(kb + c * kFChunk);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_f16(t_s(t), adesc + 2u * k, bdesc + 2u * k, idesc_s, (c | k) != 0 ? 1u : 0u);
                }
                mma_commit(s_full(t));
            };
            auto issue_pv = [&](int t, int j) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t bdesc = smem_desc_sw128_mn(base + kFVOff + k * 2048, kFChunk);
                    mma_f16_ts(t_o(t), t_s(t) + 8u * k, bdesc, idesc_o, (j | k) != 0 ? 1u : 0u);
                }
            };
            bool ok = mbar_wait(q_full(0), 0, abort_flag, 73) && mbar_wait(k_full(0), 0, abort_flag, 74);
            if (ok) {
                tc_fence_after();
                issue_s(0, 0);
                if (has1 && (ok = mbar_wait(q_full(1), 0, abort_flag, 73))) {
                    tc_fence_after();
                    issue_s(1, 0);
                }
                if (ok) mma_commit(k_empty(0));
            }
            for (int j = 0; ok && j < n_max; ++j) {
                const uint32_t vpar = j & 1, kpar = ((j + 1) >> 1) & 1;
                if (j < n0) {
                    RT_FTRACE(0, j);
                    if (!(ok = mbar_wait(p_full(0), j & 1, abort_flag, 75))) break;
                    RT_FTRACE(1, j);
                    if (!(ok = mbar_wait(v_full, vpar, abort_flag, 76))) break;
                    RT_FTRACE(2, j);
                    tc_fence_after();
                    issue_pv(0, j);
                    if (j == n0 - 1) mma_commit(o_full(0));
                }
                if (j + 1 < n0) {
                    if (!(ok = mbar_wait(k_full((j + 1) & 1), kpar, abort_flag, 74))) break;
                    tc_fence_after();
                    issue_s(0, j + 1);
                }
                if (j < n1) {
                    RT_FTRACE(3, j);
                    if (!(ok = mbar_wait(p_full(1), j & 1, abort_flag, 75))) break;
                    RT_FTRACE(4, j);
                    if (!(ok = mbar_wait(v_full, vpar, abort_flag, 76))) break;
                    tc_fence_after();
                    issue_pv(1, j);
                    if (j == n1 - 1) mma_commit(o_full(1));
                }
                mma_commit(v_empty);
                if (j + 1 < n1) {
                    if (!(ok = mbar_wait(k_full((j + 1) & 1), kpar, abort_flag, 74))) break;
                    tc_fence_after();
                    issue_s(1, j + 1);
                    RT_FTRACE(5, j);
                }
                if (j + 1 < n_max) mma_commit(k_empty((j + 1) & 1));
            }
        }
        __syncwarp();
    } else {
        const int t = (warp - 2) >> 3;                        // query tile of this warp
        const int hh = ((warp - 2) >> 2) & 1;                 // which 64 key columns of the tile
        const int quad = warp & 3;                            // the tensor-memory lane quarter it may touch
        const int row = quad * 32 + lane;                     // query row within the tile
        const int n_t = t == 0 ? n0 : n1;
        const int pair_bar = 1 + 4 * t + quad;                // named barrier of the two warps of these rows
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t ts = tmem_base + lane_base + static_cast<uint32_t>(128 * t);
        const uint32_t to = tmem_base + lane_base + static_cast<uint32_t>(256 + 128 * t);
        const float ninf = __int_as_float(0xff800000);
        const int o_half = a.cv;                              // 32-column accumulator chunks per thread
        __nv_bfloat16* xm = reinterpret_cast<__nv_bfloat16*>(base_ptr + kFXmOff) + (t * 128 + row) * 2;
        float m_ref = ninf, l = 0.f;
        bool ok = n_t > 0;
        for (int j = 0; ok && j < n_t; ++j) {
            if (!(ok = mbar_wait(s_full(t), j & 1, abort_flag, 77))) break;
            if (threadIdx.x == 64) RT_FTRACE(6, j);
            tc_fence_after();
#if defined(RT_FA_DIAG) && RT_FA_DIAG == 1      // diagnostic build only: the pipeline without any softmax
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t));
            continue;
#endif
            // this thread's 64 scores in registers: one pass over tensor memory
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(ts + 64u * hh, r0);
            tmem_ld_32x32(ts + 64u * hh + 32u, r1);
            tmem_ld_wait(r0);
            tmem_ld_wait(r1);
            if (threadIdx.x == 64) RT_FTRACE(7, j);
            if (j == n_t - 1) {                               // diagonal tile: keys beyond the row's own are masked
                const int c0 = 64 * hh;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (c0 + i > row) r0[i] = 0xff800000u;
                    if (c0 + 32 + i > row) r1[i] = 0xff800000u;
                }
            }
            float mx0 = ninf, mx1 = ninf, mx2 = ninf, mx3 = ninf;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(r0[i]));
                mx1 = fmaxf(mx1, __uint_as_float(r0[16 + i]));
                mx2 = fmaxf(mx2, __uint_as_float(r1[i]));
                mx3 = fmaxf(mx3, __uint_as_float(r1[16 + i]));
            }
            // both threads of a row round both half maxima to bf16, so they agree on the maximum
            const __nv_bfloat16 mine = __float2bfloat16_rn(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2);
            xm[hh] = mine;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            const float mt = fmaxf(__bfloat162float(mine), __bfloat162float(xm[hh ^ 1]));
            const bool grow = mt > m_ref + 8.f;
            const float m_new = grow ? mt : m_ref;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // O_t is at rest: the scores of this tile were committed after O_t += P V of the last one
                const float alpha = grow ? ex2_approx(m_ref - m_new) : 1.f;
                l *= alpha;
#pragma unroll 1
                for (int c = 4 * o_half * hh; c < 4 * o_half * (hh + 1); ++c) {      // 8 columns at a time
                    uint32_t o[8];
                    tmem_ld_32x8(to + 8u * c, o);
                    tmem_ld_wait(o);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x8(to + 8u * c, o);
                }
            }
            m_ref = m_new;
            // P = exp2(s * scale - m) as bf16 pairs into columns [32 hh, 32 hh + 32) of S_t
            float s0 = 0.f, s1 = 0.f;
            uint32_t pk[16];
            softmax_chunk<RT_FA_POLY_EVERY>(r0, pk, a.scale_log2, m_new, s0);
            tmem_st_32x16(ts + 32u * hh, pk);
            softmax_chunk<RT_FA_POLY_EVERY>(r1, pk, a.scale_log2, m_new, s1);
            tmem_st_32x16(ts + 32u * hh + 16u, pk);
            l += s0 + s1;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            // (the partner reads this step's maximum before it arrives here, and the next scores
            // only exist once both warps have arrived: the slot is free to overwrite by then)
            if (lane == 0) mbar_arrive(p_full(t));
            if (threadIdx.x == 64) RT_FTRACE(8, j);
            if (threadIdx.x == 320) RT_FTRACE(9, j);
        }
        if (ok && n_t > 0 && (ok = mbar_wait(o_full(t), 0, abort_flag, 78))) {
            tc_fence_after();
            // the row's denominator is the sum of its two threads' partial sums: exchanged through
            // the query tile's shared memory, which no MMA reads any more
            float* xl = reinterpret_cast<float*>(base_ptr + kFQOff) + (t * 128 + row) * 2;
            xl[hh] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            const float inv = 1.f / (l + xl[hh ^ 1]);
            const int token = q0 + 128 * t + row;
            __nv_bfloat16* orow = a.out + static_cast<int64_t>(token) * a.o_ts + static_cast<int64_t>(h) * a.o_hs;
#pragma unroll 1
            for (int c = o_half * hh; c < o_half * (hh + 1); ++c) {
                uint32_t o[32];
                tmem_ld_32x32(to + 32u * c, o);
                tmem_ld_wait(o);
                if (token < a.tokens) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const int d = 32 * c + 8 * v;
                        if (d < a.v_dim) {                  // v_dim % 8 == 0: a started vector is complete
                            uint4 w;
                            w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                            w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                            w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                            w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                            *reinterpret_cast<uint4*>(orow + d) = w;
                        }
                    }
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
// The same attention on CTA PAIRS (tcgen05 cta_group::2) with key tiles of 256 keys, for the
// MLA head shape (128 nope + 64 rope dims, values of 128)
// ---------------------------------------------------------------------------
// What paces the kernel above is the thread that issues its MMAs: every tcgen05.mma costs that
// thread about 65 cycles, every commit as much and every barrier wait about 100, whatever the
// shape of the MMA, and a 128 x 128 x 16 MMA keeps the tensor core busy for just 64. So this
// schedule issues larger MMAs: a pair of CTAs covers 256 query rows of one head (128 per CTA)
// and walks key tiles of 256 keys,
//   S = Q K^T     12 MMAs of 256 x 256 x 16 (each CTA brings its own 128 query rows as A and 128
//                 of the tile's keys as B), 128 cycles of tensor core each;
//   O += P V      16 MMAs of 256 x 128 x 16 (A = P from tensor memory, B = the values MN-major,
//                 each CTA bringing 64 of the 128 value dims for all 256 keys), 64 cycles each;
// 28 MMAs, two commits and four waits (about 2400 cycles of the issuing thread) for 2560 cycles
// of tensor-core work per key tile, where the single-CTA schedule spends 40 MMAs on the same
// work. Tensor memory per CTA: S 256 columns | P 128 (bf16 pairs) | O 128. P has its own columns,
// so S(j + 1) is issued as soon as the softmax threads hold the scores of tile j in registers
// and runs under their exponentials; O += P(j) V(j) follows when P(j) is complete. Softmax: 16
// warps, four threads per query row with 64 scores each; the four partial maxima of a row meet
// in shared memory as bf16. A thread writes P(j) only after O += P(j - 1) V(j - 1) has completed
// (the same barrier tells it that O is at rest for a rescale). Shared memory per CTA: Q 48 KB,
// two stages of its 128 keys (96 KB), two stages of its 64 value dims of 256 keys (64 KB).
// One thread of the leader CTA (cluster rank 0) issues every MMA and commits to the barriers of
// both CTAs; the peer's warp 1 relays "my tiles have landed" to the leader; the softmax warps of
// both CTAs arrive on the leader's s_free and p_full. Loads never use multicast.
constexpr uint32_t kGQOff = 0;                              // [3 chunks][128 rows][128 B]
constexpr uint32_t kGKOff = 3 * kFChunk;                    // key stages: 2 x 3 chunks of this CTA's 128 keys
constexpr uint32_t kGKStage = 3 * kFChunk;
constexpr uint32_t kGVOff = kGKOff + 2 * kGKStage;          // value stages: 2 x [256 keys][64 dims]
constexpr uint32_t kGVStage = 2 * kFChunk;
constexpr uint32_t kGBarOff = kGVOff + 2 * kGVStage;
constexpr int kGBars = 15;     // q_full k_full[2] v_full[2] s_done[2] pv_done[2] s_free p_full row_sync[4]
constexpr uint32_t kGXmOff = kGBarOff + kGBars * 8 + 16;    // row maxima as bf16 [2 steps][128 rows][4]
constexpr uint32_t kGSmemBytes = kGXmOff + 2 * 128 * 4 * 2 + 1024;
constexpr uint32_t kGTmemP = 256, kGTmemO = 384;            // first column of P and of O
static_assert(kGSmemBytes <= 232448, "shared memory budget");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFThreads, 1) attn_prefill_pair_kernel(
    const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp,
    const __grid_constant__ CUtensorMap tm_kn, const __grid_constant__ CUtensorMap tm_kp,
    const __grid_constant__ CUtensorMap tm_v, const PrefillArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kGBarOff;
    const uint32_t q_full = bars;
    auto k_full = [&](int st) { return bars + 8u * (1 + st); };
    auto v_full = [&](int st) { return bars + 8u * (3 + st); };
    auto s_done = [&](int st) { return bars + 8u * (5 + st); };     // S of a key tile complete: scores
                                                                    // readable, its key stage free
    auto pv_done = [&](int st) { return bars + 8u * (7 + st); };    // O += P V of a key tile complete: its
                                                                    // value stage and P free, O at rest
    const uint32_t s_free = bars + 8u * 9, p_full = bars + 8u * 10; // used in the leader only
    auto row_sync = [&](int quad) { return bars + 8u * (11 + quad); };  // the four warps that share query rows
    const uint32_t slot = bars + 8u * kGBars;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + kGBarOff + 8 * kGBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_ptr + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());
    const int qb = static_cast<int>(gridDim.x >> 1) - 1 - static_cast<int>(blockIdx.x >> 1);   // heaviest first
    const int h = blockIdx.y;
    const int q0 = qb * 256;                 // first query row of the pair
    const int n = qb + 1;                    // key tiles 0 .. qb of 256 keys; the last one is diagonal

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        const uint32_t landed = rank == 0 ? 2 : 1;          // own producer (+ the peer's relay)
        mbar_init(q_full, landed);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full(i), landed);
            mbar_init(v_full(i), landed);
            mbar_init(s_done(i), 1);
            mbar_init(pv_done(i), 1);
        }
        mbar_init(s_free, 32);                              // lane 0 of the 16 softmax warps of both CTAs
        mbar_init(p_full, 32);
        for (int i = 0; i < 4; ++i) mbar_init(row_sync(i), 4);
        fence_mbar_init();
        // The queries and the first two key tiles are requested here, by the thread that has just
        // initialised the barriers they complete on (this CTA's own), so that their latency runs
        // under the tensor-memory allocation and the cluster-wide synchronisation below instead
        // of after them: a work item lasts some tens of microseconds and there are thousands.
        const int pe_head0 = a.pe_shared ? 0 : h;
        mbar_arrive_expect_tx(q_full, 3 * kFChunk);
        tma_load_4d(base + kGQOff, &tm_qn, 0, q0 + 128 * rank, 0, h, q_full);
        tma_load_4d(base + kGQOff + 2 * kFChunk, &tm_qp, 0, q0 + 128 * rank, 0, h, q_full);
        for (int j = 0; j < 2 && j < n; ++j) {
            const uint32_t dst = base + kGKOff + j * kGKStage;
            mbar_arrive_expect_tx(k_full(j), kGKStage);
            tma_load_4d(dst, &tm_kn, 0, 256 * j + 128 * rank, 0, h, k_full(j));
            tma_load_4d(dst + 2 * kFChunk, &tm_kp, 0, 256 * j + 128 * rank, 0, pe_head0, k_full(j));
        }
        tma_prefetch_desc(&tm_v);
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

    // The u-th use of a two-stage barrier (key tile 2 u + st) completes its phase u.
    if (warp == 0) {
        if (lane == 0) {
            const int pe_head = a.pe_shared ? 0 : h;
            bool ok = true;
            auto load_k = [&](int j) {                         // this CTA's 128 keys of key tile j
                const int st = j & 1;
                if (j >= 2 && !(ok = mbar_wait(s_done(st), ((j >> 1) & 1) ^ 1u, abort_flag, 81))) return;
                const uint32_t dst = base + kGKOff + st * kGKStage;
                const int row = 256 * j + 128 * rank;
                mbar_arrive_expect_tx(k_full(st), kGKStage);
                tma_load_4d(dst, &tm_kn, 0, row, 0, h, k_full(st));
                tma_load_4d(dst + 2 * kFChunk, &tm_kp, 0, row, 0, pe_head, k_full(st));
            };
            auto load_v = [&](int j) {                         // this CTA's 64 value dims of key tile j
                const int st = j & 1;
                if (j >= 2 && !(ok = mbar_wait(pv_done(st), ((j >> 1) & 1) ^ 1u, abort_flag, 82))) return;
                mbar_arrive_expect_tx(v_full(st), kGVStage);
                tma_load_4d(base + kGVOff + st * kGVStage, &tm_v, 0, 256 * j, rank, h, v_full(st));
            };
            // in the order the stages become free: S(j) completes after O += P(j - 2) V(j - 2)
            // (the queries and key tiles 0 and 1 were requested before the cluster-wide set-up)
            for (int j = 0; ok && j < n; ++j) {
                load_v(j);
                if (ok && j + 2 < n) load_k(j + 2);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0 && lane == 0) {
            // fp32 accumulate, bf16 x bf16, M = 256 over the pair; S: N = 256, both K-major; O: N = 128, B MN-major
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (32u << 17) | (16u << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (16u << 17) | (16u << 24);
            auto issue_s = [&](int j) {
                const uint32_t kb = base + kGKOff + (j & 1) * kGKStage;
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    const uint64_t adesc = smem_desc_sw128(base + kGQOff + c * kFChunk);
                    const uint64_t bdesc = smem_desc_sw128(kb + c * kFChunk);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_f16_pair(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc_s, (c | k) != 0 ? 1u : 0u);
                }
                mma_commit_pair_both(s_done(j & 1));
            };
            auto issue_pv = [&](int j) {
                const uint32_t vb = base + kGVOff + (j & 1) * kGVStage;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
#if defined(RT_FA_DIAG) && RT_FA_DIAG == 3      // diagnostic build only (wrong results): B read K-major
                    mma_f16_ts_pair(tmem_base + kGTmemO, tmem_base + kGTmemP + 8u * k,
                                    smem_desc_sw128(vb + (k >> 2) * 8192) + 2u * (k & 3), idesc_o & ~(1u << 16),
                                    (j | k) != 0 ? 1u : 0u);
#elif defined(RT_FA_DIAG) && RT_FA_DIAG == 4    // diagnostic build only (wrong results): A read from shared memory
                    mma_f16_pair(tmem_base + kGTmemO, smem_desc_sw128(base + kGQOff) + 2u * (k & 3),
                                 smem_desc_sw128_mn(vb + k * 2048, kGVStage), idesc_o, (j | k) != 0 ? 1u : 0u);
#else
                    mma_f16_ts_pair(tmem_base + kGTmemO, tmem_base + kGTmemP + 8u * k,
                                    smem_desc_sw128_mn(vb + k * 2048, kGVStage), idesc_o, (j | k) != 0 ? 1u : 0u);
#endif
                }
                mma_commit_pair_both(pv_done(j & 1));
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, 83) && mbar_wait(k_full(0), 0, abort_flag, 84);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; ok && j < n; ++j) {
                if (j + 1 < n) {
                    RT_FTRACE(0, j);
                    if (!(ok = mbar_wait(s_free, j & 1, abort_flag, 85))) break;
                    if (!(ok = mbar_wait(k_full((j + 1) & 1), ((j + 1) >> 1) & 1, abort_flag, 84))) break;
                    RT_FTRACE(1, j);
                    tc_fence_after();
                    issue_s(j + 1);
                    RT_FTRACE(2, j);
                }
                if (!(ok = mbar_wait(p_full, j & 1, abort_flag, 86))) break;
                RT_FTRACE(3, j);
                if (!(ok = mbar_wait(v_full(j & 1), (j >> 1) & 1, abort_flag, 87))) break;
                RT_FTRACE(4, j);
                tc_fence_after();
                issue_pv(j);
                RT_FTRACE(5, j);
            }
        } else if (rank == 1 && lane == 0) {
            // Relay: tells the leader that this CTA's tiles have landed, in the producer's order.
            bool ok = mbar_wait(q_full, 0, abort_flag, 88);
            if (ok) mbar_arrive_cluster(map_to_cta(q_full, 0));
            auto relay = [&](uint32_t bar, int j) {
                if ((ok = mbar_wait(bar, (j >> 1) & 1, abort_flag, 89))) mbar_arrive_cluster(map_to_cta(bar, 0));
            };
            if (ok) relay(k_full(0), 0);
            if (ok && n > 1) relay(k_full(1), 1);
            for (int j = 0; ok && j < n; ++j) {
                relay(v_full(j & 1), j);
                if (ok && j + 2 < n) relay(k_full(j & 1), j + 2);
            }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;                            // the tensor-memory lane quarter it may touch
        const int cq = (warp - 2) >> 2;                       // which 64 key columns of the tile
        const int row = quad * 32 + lane;                     // query row within this CTA's tile
        const int prow = 128 * rank + row;                    // query row within the pair's 256
        const uint32_t row_bar = row_sync(quad);              // barrier of the four warps of these rows (a
                                                              // bounded wait, unlike a named barrier)
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t ts = tmem_base + lane_base + static_cast<uint32_t>(64 * cq);
        const uint32_t tp = tmem_base + lane_base + kGTmemP + static_cast<uint32_t>(32 * cq);
        const uint32_t to = tmem_base + lane_base + kGTmemO + static_cast<uint32_t>(32 * cq);
        const uint32_t s_free_leader = map_to_cta(s_free, 0), p_leader = map_to_cta(p_full, 0);
        const float ninf = __int_as_float(0xff800000);
        __nv_bfloat16* xm_base = reinterpret_cast<__nv_bfloat16*>(base_ptr + kGXmOff) + row * 4;
        float m_ref = ninf, l = 0.f;
        bool ok = true;
        for (int j = 0; ok && j < n; ++j) {
            if (!(ok = mbar_wait(s_done(j & 1), (j >> 1) & 1, abort_flag, 90))) break;
            if (threadIdx.x == 64) RT_FTRACE(6, j);
            tc_fence_after();
            // this thread's 64 scores in registers; then the score columns are free for the next tile
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(ts, r0);
            tmem_ld_32x32(ts + 32u, r1);
            tmem_ld_wait(r0);
            tmem_ld_wait(r1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(s_free_leader);
            if (threadIdx.x == 64) RT_FTRACE(7, j);
            if (j == n - 1) {                                 // diagonal tile: keys beyond the row's own are masked
                const int c0 = 64 * cq;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (c0 + i > prow) r0[i] = 0xff800000u;
                    if (c0 + 32 + i > prow) r1[i] = 0xff800000u;
                }
            }
            float mx0 = ninf, mx1 = ninf, mx2 = ninf, mx3 = ninf;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(r0[i]));
                mx1 = fmaxf(mx1, __uint_as_float(r0[16 + i]));
                mx2 = fmaxf(mx2, __uint_as_float(r1[i]));
                mx3 = fmaxf(mx3, __uint_as_float(r1[16 + i]));
            }
            // the four threads of a row exchange their maxima as bf16, so all use the same value;
            // the slots alternate with the step, so a fast warp cannot overwrite one still being read
            __nv_bfloat16* xm = xm_base + (j & 1) * 512;
            xm[cq] = __float2bfloat16_rn(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2);
            __syncwarp();
            if (lane == 0) mbar_arrive(row_bar);
            if (!(ok = mbar_wait(row_bar, j & 1, abort_flag, 93))) break;
            const uint2 all = *reinterpret_cast<const uint2*>(xm_base + (j & 1) * 512);
            const __nv_bfloat162 p01 = *reinterpret_cast<const __nv_bfloat162*>(&all.x);
            const __nv_bfloat162 p23 = *reinterpret_cast<const __nv_bfloat162*>(&all.y);
            const float mt = fmaxf(fmaxf(__low2float(p01), __high2float(p01)),
                                   fmaxf(__low2float(p23), __high2float(p23)));
            const bool grow = mt > m_ref + 8.f;
            const float m_new = grow ? mt : m_ref;
            // the probabilities first, in registers: P(j - 1) still occupies the P columns
            float s0 = 0.f, s1 = 0.f;
            uint32_t pk0[16], pk1[16];
#if defined(RT_FA_DIAG) && RT_FA_DIAG == 1      // diagnostic build only (wrong results): no exponentials
#pragma unroll
            for (int i = 0; i < 16; ++i) { pk0[i] = r0[i]; pk1[i] = r1[i]; }
#else
            softmax_chunk<RT_FA_PAIR_POLY_EVERY>(r0, pk0, a.scale_log2, m_new, s0);
            softmax_chunk<RT_FA_PAIR_POLY_EVERY>(r1, pk1, a.scale_log2, m_new, s1);
#endif
            if (threadIdx.x == 64) RT_FTRACE(8, j);
            // P(j - 1) has been consumed and O is at rest once O += P(j - 1) V(j - 1) has completed
            if (j > 0) {
                if (!(ok = mbar_wait(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag, 91))) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? ex2_approx(m_ref - m_new) : 1.f;
                    l *= alpha;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {             // this thread's 32 output columns, 8 at a time
                        uint32_t o[8];
                        tmem_ld_32x8(to + 8u * c, o);
                        tmem_ld_wait(o);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x8(to + 8u * c, o);
                    }
                }
            }
            m_ref = m_new;
            tmem_st_32x16(tp, pk0);
            tmem_st_32x16(tp + 16u, pk1);
            l += s0 + s1;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(p_leader);
            if (threadIdx.x == 64) RT_FTRACE(9, j);
        }
        if (ok && (ok = mbar_wait(pv_done((n - 1) & 1), ((n - 1) >> 1) & 1, abort_flag, 92))) {
            tc_fence_after();
            // the row's denominator is the sum of its four threads' partial sums: exchanged through
            // the query tile's shared memory, which no MMA reads any more
            float* xl = reinterpret_cast<float*>(base_ptr + kGQOff) + row * 4;
            xl[cq] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(row_bar);
            ok = mbar_wait(row_bar, n & 1, abort_flag, 93);
            const float4 ls = *reinterpret_cast<const float4*>(xl);
            const float inv = 1.f / ((ls.x + ls.y) + (ls.z + ls.w));
            const int token = q0 + prow;
            uint32_t o[32];
            tmem_ld_32x32(to, o);
            tmem_ld_wait(o);
            if (a.out_codes != nullptr) {
                // act_quant of the bf16 output (racetrack/models/deepseek.py:85-107) without writing
                // it: the 128 values of this row and head are one quantisation group; its amax is
                // the maximum of the four threads' 32 values, rounded to bf16 as the tensor would be
                float xb[32];
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    xb[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(o[i]) * inv));
                    amax = fmaxf(amax, fabsf(xb[i]));
                }
                float* xa = xl + 512;                         // [128 rows][4], behind the denominators
                xa[cq] = amax;
                __syncwarp();
                if (lane == 0) mbar_arrive(row_bar);
                ok = ok && mbar_wait(row_bar, (n + 1) & 1, abort_flag, 93);
                const float4 am = *reinterpret_cast<const float4*>(xa);
                amax = fmaxf(fmaxf(fmaxf(am.x, am.y), fmaxf(am.z, am.w)), 1.0e-4f);
                const float scale = __fdiv_rn(amax, 448.0f);
                const float rscale = __frcp_rn(scale);
                if (ok && token < a.tokens) {
                    uint32_t w[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        w[k] = attn_cvt_e4m3x2(div_shared(xb[4 * k], scale, rscale),
                                               div_shared(xb[4 * k + 1], scale, rscale)) |
                               (attn_cvt_e4m3x2(div_shared(xb[4 * k + 2], scale, rscale),
                                                div_shared(xb[4 * k + 3], scale, rscale)) << 16);
                    uint8_t* crow = a.out_codes + (static_cast<int64_t>(token) * a.heads + h) * 128 + 32 * cq;
                    *reinterpret_cast<uint4*>(crow) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(crow + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                    if (cq == 0) a.out_scales[static_cast<int64_t>(token) * a.heads + h] = scale;
                }
            } else if (ok && token < a.tokens) {
                __nv_bfloat16* orow = a.out + static_cast<int64_t>(token) * a.o_ts +
                                      static_cast<int64_t>(h) * a.o_hs + 32 * cq;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                    w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                    w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                    w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + 8 * v) = w;
                }
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

int make_tmap_bf16_4d(CUtensorMap* map, const void* ptr, const uint64_t dims[4], const uint64_t strides[3],
                      const uint32_t box[4]);      // rt_gemm.cu

// Tensor map of one attention operand x[token, head, dim] (element strides ts / hs): when dim is
// a multiple of 64 its 64-dim chunks are a dimension of their own, so one box brings all of them
// (an SM retires about one tiled load per 500 cycles whatever its size); otherwise the row is
// the fastest dimension and one box per chunk is issued, the part beyond dim reading as zero.
static int make_attn_tmap(CUtensorMap* map, const void* ptr, int64_t dim, int64_t tokens, int64_t heads,
                          int64_t ts, int64_t hs, bool* one_op, uint32_t box_rows = 128, uint32_t box_chunks = 0) {
    *one_op = dim % 64 == 0;
    if (*one_op) {
        const uint64_t dims[4] = {64, static_cast<uint64_t>(tokens), static_cast<uint64_t>(dim / 64),
                                  static_cast<uint64_t>(heads)};
        const uint64_t strides[3] = {static_cast<uint64_t>(ts) * 2, 128, static_cast<uint64_t>(hs) * 2};
        const uint32_t box[4] = {64, box_rows, box_chunks ? box_chunks : static_cast<uint32_t>(dim / 64), 1};
        return make_tmap_bf16_4d(map, ptr, dims, strides, box);
    }
    const uint64_t dims[4] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(tokens), 1,
                              static_cast<uint64_t>(heads)};
    const uint64_t strides[3] = {static_cast<uint64_t>(ts) * 2, static_cast<uint64_t>(ts) * 2,
                                 static_cast<uint64_t>(hs) * 2};
    const uint32_t box[4] = {64, 128, 1, 1};
    return make_tmap_bf16_4d(map, ptr, dims, strides, box);
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

#ifdef RT_FA_TRACE
extern "C" int rt_fa_trace_read(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, tc::g_fa_trace, sizeof(long long) * 10 * 64) == cudaSuccess
               ? RT_OK : RT_ERR_CUDA;
}
#endif

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

extern "C" int rt_attn_prefill_schedule(int schedule) {
    const int prev = tc::g_attn_schedule;
    if (schedule >= 0 && schedule <= 2) tc::g_attn_schedule = schedule;
    return prev;
}

static int attn_causal_prefill(const void* q, const void* k_nope, const void* k_pe, const void* v,
                               void* out, void* out_codes, float* out_scales, int64_t tokens,
                               int64_t heads, int64_t nope_dim, int64_t rope_dim, int64_t v_dim,
                               int64_t q_token_stride, int64_t q_head_stride, int64_t kn_token_stride,
                               int64_t kn_head_stride, int64_t kp_token_stride, int64_t kp_head_stride,
                               int64_t v_token_stride, int64_t v_head_stride, int64_t o_token_stride,
                               int64_t o_head_stride, float softmax_scale, void* stream);

extern "C" int rt_attn_causal_prefill(const void* q, const void* k_nope, const void* k_pe, const void* v,
                                      void* out, int64_t tokens, int64_t heads, int64_t nope_dim,
                                      int64_t rope_dim, int64_t v_dim, int64_t q_token_stride,
                                      int64_t q_head_stride, int64_t kn_token_stride,
                                      int64_t kn_head_stride, int64_t kp_token_stride,
                                      int64_t kp_head_stride, int64_t v_token_stride,
                                      int64_t v_head_stride, int64_t o_token_stride,
                                      int64_t o_head_stride, float softmax_scale, void* stream) {
    RT_REQUIRE(out, RT_ERR_BAD_ARG, "rt_attn_causal_prefill: null pointer");
    return attn_causal_prefill(q, k_nope, k_pe, v, out, nullptr, nullptr, tokens, heads, nope_dim, rope_dim,
                               v_dim, q_token_stride, q_head_stride, kn_token_stride, kn_head_stride,
                               kp_token_stride, kp_head_stride, v_token_stride, v_head_stride,
                               o_token_stride, o_head_stride, softmax_scale, stream);
}

extern "C" int rt_attn_causal_prefill_fp8(const void* q, const void* k_nope, const void* k_pe, const void* v,
                                          void* out_codes, float* out_scales, int64_t tokens,
                                          int64_t heads, int64_t nope_dim, int64_t rope_dim,
                                          int64_t v_dim, int64_t q_token_stride, int64_t q_head_stride,
                                          int64_t kn_token_stride, int64_t kn_head_stride,
                                          int64_t kp_token_stride, int64_t kp_head_stride,
                                          int64_t v_token_stride, int64_t v_head_stride,
                                          float softmax_scale, void* stream) {
    RT_REQUIRE(out_codes && out_scales, RT_ERR_BAD_ARG, "rt_attn_causal_prefill_fp8: null pointer");
    RT_REQUIRE(nope_dim == 128 && rope_dim == 64 && v_dim == 128, RT_ERR_UNSUPPORTED,
               "rt_attn_causal_prefill_fp8: the FP8 epilogue exists for the 128 + 64 / 128 head shape");
    RT_REQUIRE(aligned16(out_codes), RT_ERR_BAD_ARG, "rt_attn_causal_prefill_fp8: codes must be 16-byte aligned");
    return attn_causal_prefill(q, k_nope, k_pe, v, nullptr, out_codes, out_scales, tokens, heads, nope_dim,
                               rope_dim, v_dim, q_token_stride, q_head_stride, kn_token_stride, kn_head_stride,
                               kp_token_stride, kp_head_stride, v_token_stride, v_head_stride, 8, 8,
                               softmax_scale, stream);
}

static int attn_causal_prefill(const void* q, const void* k_nope, const void* k_pe, const void* v,
                               void* out, void* out_codes, float* out_scales, int64_t tokens, int64_t heads, int64_t nope_dim,
                                      int64_t rope_dim, int64_t v_dim, int64_t q_token_stride,
                                      int64_t q_head_stride, int64_t kn_token_stride,
                                      int64_t kn_head_stride, int64_t kp_token_stride,
                                      int64_t kp_head_stride, int64_t v_token_stride,
                                      int64_t v_head_stride, int64_t o_token_stride,
                                      int64_t o_head_stride, float softmax_scale, void* stream) {
    RT_REQUIRE(tokens >= 0 && heads > 0, RT_ERR_BAD_ARG, "rt_attn_causal_prefill: bad shape");
    if (tokens == 0) return RT_OK;
    RT_REQUIRE(q && k_nope && v && (out || out_codes) && (k_pe || rope_dim == 0), RT_ERR_BAD_ARG,
               "rt_attn_causal_prefill: null pointer");
    RT_REQUIRE(nope_dim > 0 && nope_dim <= 128 && rope_dim >= 0 && rope_dim <= 64 && v_dim > 0 && v_dim <= 128 &&
                   nope_dim % 8 == 0 && rope_dim % 8 == 0 && v_dim % 8 == 0,
               RT_ERR_UNSUPPORTED,
               "rt_attn_causal_prefill: dims must be multiples of 8 with nope <= 128, rope <= 64, v <= 128");
    const int64_t strides[] = {q_token_stride, q_head_stride, kn_token_stride, kn_head_stride, kp_token_stride,
                               kp_head_stride, v_token_stride, v_head_stride, o_token_stride, o_head_stride};
    for (int64_t st : strides)
        RT_REQUIRE(st >= 0 && st % 8 == 0, RT_ERR_BAD_ARG,
                   "rt_attn_causal_prefill: strides must be non-negative multiples of 8 elements");
    RT_REQUIRE(aligned16(q) && aligned16(k_nope) && aligned16(v) && (!out || aligned16(out)) && (!k_pe || aligned16(k_pe)),
               RT_ERR_BAD_ARG, "rt_attn_causal_prefill: pointers must be 16-byte aligned");
    RT_REQUIRE(tokens < (1ll << 31) - 256 && heads < 65536, RT_ERR_UNSUPPORTED,
               "rt_attn_causal_prefill: dimension too large");
    const bool pe_shared = rope_dim > 0 && kp_head_stride == 0;
    tc::PrefillArgs a;
    a.out = static_cast<__nv_bfloat16*>(out);
    a.o_ts = o_token_stride;
    a.o_hs = o_head_stride;
    a.tokens = static_cast<int>(tokens);
    a.heads = static_cast<int>(heads);
    a.cn = static_cast<int>((nope_dim + 63) / 64);
    a.cp = static_cast<int>((rope_dim + 63) / 64);
    a.cv = static_cast<int>((v_dim + 63) / 64);
    a.v_dim = static_cast<int>(v_dim);
    a.pe_shared = pe_shared ? 1 : 0;
    a.scale_log2 = softmax_scale * 1.4426950408889634f;
    a.out_codes = static_cast<uint8_t*>(out_codes);
    a.out_scales = out_scales;
    CUtensorMap tm_qn, tm_qp, tm_kn, tm_kp, tm_v;
    bool one[5] = {false, false, false, false, false};
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
    if (int rc = tc::make_attn_tmap(&tm_qn, qb, nope_dim, tokens, heads, q_token_stride, q_head_stride, &one[0]))
        return rc;
    if (int rc = tc::make_attn_tmap(&tm_kn, k_nope, nope_dim, tokens, heads, kn_token_stride, kn_head_stride, &one[2]))
        return rc;
    if (int rc = tc::make_attn_tmap(&tm_v, v, v_dim, tokens, heads, v_token_stride, v_head_stride, &one[4]))
        return rc;
    if (rope_dim > 0) {
        if (int rc = tc::make_attn_tmap(&tm_qp, qb + nope_dim, rope_dim, tokens, heads, q_token_stride,
                                        q_head_stride, &one[1]))
            return rc;
        // a shared rope key has no head dimension: one "head" whose stride is never used
        if (int rc = tc::make_attn_tmap(&tm_kp, k_pe, rope_dim, tokens, pe_shared ? 1 : heads, kp_token_stride,
                                        pe_shared ? kp_token_stride : kp_head_stride, &one[3]))
            return rc;
    } else {
        tm_qp = tm_qn;
        tm_kp = tm_kn;
    }
    a.one_op = (one[0] ? 1 : 0) | (one[1] ? 2 : 0) | (one[2] ? 4 : 0) | (one[3] ? 8 : 0) | (one[4] ? 16 : 0);
    const bool mla_shape = nope_dim == 128 && rope_dim == 64 && v_dim == 128;
    if (mla_shape && (out_codes || tc::g_attn_schedule == 2 || (tc::g_attn_schedule == 0 && tokens >= 1024))) {
        // the MLA head shape on CTA pairs with key tiles of 256 keys: a CTA brings 128 keys of a
        // tile (the boxes above) and 64 of the value dims for all of its 256 keys
        bool ignore;
        if (int rc = tc::make_attn_tmap(&tm_v, v, v_dim, tokens, heads, v_token_stride, v_head_stride, &ignore,
                                        256, 1))
            return rc;
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&tc::attn_prefill_pair_kernel),
                                         static_cast<int>(tc::kGSmemBytes), "rt_attn_causal_prefill"))
            return rc;
        dim3 pgrid(static_cast<unsigned>(2 * ((tokens + 255) / 256)), static_cast<unsigned>(heads));
        tc::attn_prefill_pair_kernel<<<pgrid, tc::kFThreads, tc::kGSmemBytes, as_stream(stream)>>>(
            tm_qn, tm_qp, tm_kn, tm_kp, tm_v, a);
        count_launch();
        return check_launch("attn_prefill_pair_kernel");
    }
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&tc::attn_prefill_kernel),
                                     static_cast<int>(tc::kFSmemBytes), "rt_attn_causal_prefill"))
        return rc;
    dim3 grid(static_cast<unsigned>((tokens + 255) / 256), static_cast<unsigned>(heads));
    tc::attn_prefill_kernel<<<grid, tc::kFThreads, tc::kFSmemBytes, as_stream(stream)>>>(
        tm_qn, tm_qp, tm_kn, tm_kp, tm_v, a);
    count_launch();
    return check_launch("attn_prefill_kernel");
}
