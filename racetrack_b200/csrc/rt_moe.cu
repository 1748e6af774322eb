// MoE routing (grouped top-k on router logits), stable token permutation by
// expert, row gather and weighted combine.
//
// Routing: one warp per token, the expert scores live in registers (n_experts/32
// per lane), every selection step is a warp collective (redux / ballot / shuffle),
// nothing touches shared memory. Algorithmic bytes per token: 4*n_experts read,
// 12*topk written.
// Permutation: counting sort in three small launches (per-block histograms,
// scan, stable scatter); positions are a pure function of the indices, so the
// result is deterministic and equal to what a per-expert torch.where loop yields.
#include <mutex>

#include "rt_common.cuh"

namespace rt {

constexpr int kRouteWarps = 8;
constexpr int kPermThreads = 1024;

__device__ __forceinline__ uint32_t orderable(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// EPL experts per lane; lane l owns experts [l*EPL, (l+1)*EPL).
template <int EPL>
__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias,
    float* __restrict__ weights_out, int64_t* __restrict__ indices_out, int64_t tokens,
    int n_experts, int64_t lstride, int n_groups, int topk_groups, int topk, float route_scale,
    int score_func) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRouteWarps + (threadIdx.x >> 5);
    if (t >= tokens) return;  // whole warp leaves together
    const float* row = logits + t * lstride;
    const float ninf = -INFINITY;

    float s[EPL];  // unbiased scores
    float b[EPL];  // selection scores (biased, masked)
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane * EPL + j;
        s[j] = (e < n_experts) ? __ldg(row + e) : ninf;
    }
    if (score_func == RT_SCORE_SOFTMAX) {
        float m = ninf;
#pragma unroll
        for (int j = 0; j < EPL; ++j) m = fmaxf(m, s[j]);
        m = warp_max(m);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            s[j] = (lane * EPL + j < n_experts) ? expf(s[j] - m) : 0.f;
            sum += s[j];
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int j = 0; j < EPL; ++j) s[j] = __fdiv_rn(s[j], sum);
    } else if (score_func == RT_SCORE_TOPK_SOFTMAX) {
        // selection happens on the raw logits; the softmax comes after it
    } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) s[j] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-s[j])));
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane * EPL + j;
        b[j] = (e < n_experts) ? (bias ? __fadd_rn(s[j], __ldg(bias + e)) : s[j]) : ninf;
    }

    if (n_groups > 1) {
        // a group covers `lpg` whole consecutive lanes (checked on the host)
        const int lpg = (n_experts / n_groups) / EPL;
        float m1 = ninf, m2 = ninf;  // two largest selection scores of the lane
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const float v = b[j];
            m2 = fmaxf(m2, fminf(m1, v));
            m1 = fmaxf(m1, v);
        }
        for (int o = 1; o < lpg; o <<= 1) {
            const float o1 = __shfl_xor_sync(0xffffffffu, m1, o);
            const float o2 = __shfl_xor_sync(0xffffffffu, m2, o);
            m2 = fmaxf(fmaxf(m2, o2), fminf(m1, o1));
            m1 = fmaxf(m1, o1);
        }
        const float gscore = bias ? __fadd_rn(m1, m2) : m1;
        const int my_group = lane / lpg;
        int rank = 0;
        for (int g = 0; g < n_groups; ++g) {
            const float og = __shfl_sync(0xffffffffu, gscore, g * lpg);
            rank += (og > gscore) || (og == gscore && g < my_group);
        }
        const bool keep = (my_group < n_groups) && (rank < topk_groups);
        if (!keep) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) b[j] = ninf;
        }
    }

    float my_w = 0.f;
    int my_idx = 0;
    for (int k = 0; k < topk; ++k) {
        float best = ninf;
        int bj = 0;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            if (b[j] > best) {
                best = b[j];
                bj = j;
            }
        }
        const uint32_t key = orderable(best);
        const uint32_t top = __reduce_max_sync(0xffffffffu, key);
        const int owner = __ffs(__ballot_sync(0xffffffffu, key == top)) - 1;
        float sv = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            if (j == bj) sv = s[j];
        }
        const float w = __shfl_sync(0xffffffffu, sv, owner);
        const int idx = __shfl_sync(0xffffffffu, lane * EPL + bj, owner);
        if (lane == owner) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                if (j == bj) b[j] = ninf;
            }
        }
        if (lane == k) {
            my_w = w;
            my_idx = idx;
        }
    }
    if (score_func == RT_SCORE_SIGMOID) {
        const float sum = warp_sum(lane < topk ? my_w : 0.f);
        my_w = __fdiv_rn(my_w, sum);
    } else if (score_func == RT_SCORE_TOPK_SOFTMAX) {
        // softmax over the selected logits, rounded to bf16 like the activations it scales
        const float m = warp_max(lane < topk ? my_w : ninf);
        const float e = lane < topk ? expf(my_w - m) : 0.f;
        const float sum = warp_sum(e);
        my_w = round_bf16(__fdiv_rn(e, sum));
    }
    my_w = __fmul_rn(my_w, route_scale);
    if (lane < topk) {
        weights_out[t * topk + lane] = my_w;
        indices_out[t * topk + lane] = my_idx;
    }
}

// ---------------------------------------------------------------------------
// Stable permutation by expert
// ---------------------------------------------------------------------------

// Pass 1: per-block histogram of expert ids. counts[b * n_experts + e].
__global__ void __launch_bounds__(kPermThreads) moe_count_kernel(
    const int64_t* __restrict__ indices, int32_t* __restrict__ counts, int n_pairs,
    int n_experts) {
    extern __shared__ int hist[];
    for (int e = threadIdx.x; e < n_experts; e += kPermThreads) hist[e] = 0;
    __syncthreads();
    const int p = blockIdx.x * kPermThreads + threadIdx.x;
    if (p < n_pairs) {
        const int e = static_cast<int>(indices[p]);
        if (e >= 0 && e < n_experts) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += kPermThreads)
        counts[blockIdx.x * n_experts + e] = hist[e];
}

// Pass 2 (one CTA): turns per-block counts into per-block bases (exclusive over
// blocks) and writes the exclusive scan of expert totals to expert_offsets.
__global__ void __launch_bounds__(1024) moe_scan_kernel(int32_t* __restrict__ counts,
                                                        int32_t* __restrict__ expert_offsets,
                                                        int n_blocks, int n_experts) {
    __shared__ int warp_tot[32];
    __shared__ int carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n_experts; base += blockDim.x) {
        const int e = base + threadIdx.x;
        int total = 0;
        if (e < n_experts) {
            for (int b = 0; b < n_blocks; ++b) {
                const int c = counts[b * n_experts + e];
                counts[b * n_experts + e] = total;
                total += c;
            }
        }
        // block-wide exclusive scan of `total`
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        int incl = total;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += v;
            }
            warp_tot[lane] = wi - w;  // exclusive warp offsets
        }
        __syncthreads();
        const int carry = carry_s;
        const int excl = carry + warp_tot[warp] + incl - total;
        if (e < n_experts) expert_offsets[e] = excl;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_s = excl + total;
        __syncthreads();
    }
    if (threadIdx.x == 0) expert_offsets[n_experts] = carry_s;
}

// Pass 3: stable scatter. Within a block, pairs of one expert keep ascending
// pair id: rank inside the warp by match_any, warps ordered by a scan in shared memory.
__global__ void __launch_bounds__(kPermThreads) moe_scatter_kernel(
    const int64_t* __restrict__ indices, const int32_t* __restrict__ block_base,
    const int32_t* __restrict__ expert_offsets, int32_t* __restrict__ sorted_pairs,
    int32_t* __restrict__ pair_pos, int n_pairs, int n_experts) {
    extern __shared__ unsigned short wc[];  // [32][n_experts]
    for (int i = threadIdx.x; i < 32 * n_experts; i += kPermThreads) wc[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.x * kPermThreads + threadIdx.x;
    int e = -1;
    if (p < n_pairs) {
        e = static_cast<int>(indices[p]);
        if (e < 0 || e >= n_experts) e = -1;
    }
    // invalid lanes get unique keys so they match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e >= 0 ? e : n_experts + lane);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wc[warp * n_experts + e] = static_cast<unsigned short>(__popc(peers));
    __syncthreads();
    for (int x = threadIdx.x; x < n_experts; x += kPermThreads) {
        unsigned run = 0;
        for (int w = 0; w < 32; ++w) {
            const unsigned c = wc[w * n_experts + x];
            wc[w * n_experts + x] = static_cast<unsigned short>(run);
            run += c;
        }
    }
    __syncthreads();
    if (e >= 0) {
        const int dest = expert_offsets[e] + block_base[blockIdx.x * n_experts + e] +
                         wc[warp * n_experts + e] + rank;
        sorted_pairs[dest] = p;
        pair_pos[p] = dest;
    }
}

// ---------------------------------------------------------------------------
// Gather / combine
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_gather_kernel(
    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ sorted_pairs,
    __nv_bfloat16* __restrict__ out, int64_t n_items, int nvec, int topk, int64_t xstride) {
    const int64_t id = blockIdx.x * 256LL + threadIdx.x;
    if (id >= n_items) return;
    const int64_t r = id / nvec;
    const int v = static_cast<int>(id - r * nvec);
    const int64_t tok = __ldg(sorted_pairs + r) / topk;
    const uint4 d = ld_cached16(reinterpret_cast<const uint4*>(x + tok * xstride) + v);
    st_stream16(reinterpret_cast<uint4*>(out) + r * nvec + v, d);
}

template <bool F32OUT>
__global__ void __launch_bounds__(256) moe_combine_kernel(
    const __nv_bfloat16* __restrict__ expert_out, const int32_t* __restrict__ pair_pos,
    const float* __restrict__ weights, const __nv_bfloat16* __restrict__ shared,
    void* __restrict__ y, int nvec, int topk, int pos_begin, int pos_end,
    const int32_t* __restrict__ pos_begin_ptr, const int32_t* __restrict__ pos_end_ptr) {
    const int64_t t = blockIdx.x;
    // a window given in device memory (expert offsets of this rank) overrides the host values
    if (pos_begin_ptr) pos_begin = __ldg(pos_begin_ptr);
    if (pos_end_ptr) pos_end = __ldg(pos_end_ptr);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        for (int s = 0; s < topk; ++s) {
            const int pos = __ldg(pair_pos + t * topk + s);
            if (pos < pos_begin || pos >= pos_end) continue;
            const float w = __ldg(weights + t * topk + s);
            float f[8];
            unpack_bf16x8(
                ld_stream16(reinterpret_cast<const uint4*>(expert_out) + (int64_t)pos * nvec + v), f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = __fadd_rn(acc[k], __fmul_rn(f[k], w));
        }
        if (shared) {
            float f[8];
            unpack_bf16x8(ld_stream16(reinterpret_cast<const uint4*>(shared) + t * nvec + v), f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = __fadd_rn(acc[k], f[k]);
        }
        if constexpr (F32OUT) {
            // the fp32 sums themselves (an expert-parallel rank all-reduces them before the cast)
            uint4* dst = reinterpret_cast<uint4*>(y) + (t * nvec + v) * 2;
            st_stream16(dst, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]),
                                        __float_as_uint(acc[2]), __float_as_uint(acc[3])));
            st_stream16(dst + 1, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]),
                                            __float_as_uint(acc[6]), __float_as_uint(acc[7])));
        } else {
            st_stream16(reinterpret_cast<uint4*>(y) + t * nvec + v, pack_bf16x8(acc));
        }
    }
}


// ---------------------------------------------------------------------------
// Top-k selection of the sparse indexer: the k largest scores of every query row
// ---------------------------------------------------------------------------
// One CTA per row. fp32 scores become order-preserving 32-bit keys; four 8-bit radix passes
// (shared-memory histograms, most significant digit first) find the k-th largest key exactly
// and how many elements equal to it still belong to the selection; a last pass writes the
// indices of all larger keys and of the first of the equal ones, in ascending index order
// (ballot-based ordered compaction, 1024 elements per sweep).
constexpr int kTopkThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
    uint32_t u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0u;                           // -0.0 compares equal to +0.0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);      // larger float <=> larger key
}

__global__ void __launch_bounds__(kTopkThreads) index_topk_kernel(
    const float* __restrict__ scores, int32_t* __restrict__ indices, int keys, int64_t ld,
    int topk) {
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_remaining;
    __shared__ int warp_count[kTopkThreads / 32];
    __shared__ int s_base, s_eq_base;
    const float* row = scores + static_cast<int64_t>(blockIdx.x) * ld;
    int32_t* out = indices + static_cast<int64_t>(blockIdx.x) * topk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        s_prefix = 0u;
        s_remaining = topk;          // elements still to take among those matching the prefix
    }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask_hi = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int i = tid; i < keys; i += kTopkThreads) {
            const uint32_t key = order_key(row[i]);
            if ((key & mask_hi) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int remaining = s_remaining, bin = 255;
            for (; bin > 0; --bin) {
                if (hist[bin] >= remaining) break;
                remaining -= hist[bin];
            }
            s_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
            s_remaining = remaining;
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;       // key of the k-th largest element
    const int take_eq = s_remaining;     // how many elements equal to it are selected
    if (tid == 0) {
        s_base = 0;
        s_eq_base = 0;
    }
    __syncthreads();
    for (int start = 0; start < keys; start += kTopkThreads) {
        const int i = start + tid;
        uint32_t key = 0u;
        if (i < keys) key = order_key(row[i]);
        const bool gt = i < keys && key > kth;
        const bool eq = i < keys && key == kth;
        // rank of this element among the equal ones of the row, in index order
        const uint32_t eq_ballot = __ballot_sync(0xffffffffu, eq);
        const int eq_before_in_warp = __popc(eq_ballot & ((1u << lane) - 1u));
        if (lane == 0) warp_count[warp] = __popc(eq_ballot);
        __syncthreads();
        int eq_before = s_eq_base + eq_before_in_warp;
        for (int w = 0; w < warp; ++w) eq_before += warp_count[w];
        const bool sel = gt || (eq && eq_before < take_eq);
        __syncthreads();
        if (tid == kTopkThreads - 1) s_eq_base = eq_before + (eq ? 1 : 0);
        const uint32_t sel_ballot = __ballot_sync(0xffffffffu, sel);
        const int sel_before_in_warp = __popc(sel_ballot & ((1u << lane) - 1u));
        if (lane == 0) warp_count[warp] = __popc(sel_ballot);
        __syncthreads();
        int pos = s_base + sel_before_in_warp;
        for (int w = 0; w < warp; ++w) pos += warp_count[w];
        if (sel && pos < topk) out[pos] = i;
        __syncthreads();
        if (tid == kTopkThreads - 1) s_base = pos + (sel ? 1 : 0);
        __syncthreads();
    }
}

}  // namespace rt

using namespace rt;

extern "C" int rt_moe_route(const float* logits, const float* bias, float* weights_out,
                            int64_t* indices_out, int64_t tokens, int64_t n_experts,
                            int64_t logits_stride, int64_t n_groups, int64_t topk_groups,
                            int64_t topk, float route_scale, int score_func, void* stream) {
    RT_REQUIRE(logits && weights_out && indices_out, RT_ERR_BAD_ARG, "rt_moe_route: null pointer");
    RT_REQUIRE(tokens >= 0 && n_experts > 0 && topk > 0 && n_groups > 0, RT_ERR_BAD_ARG,
               "rt_moe_route: bad shape");
    RT_REQUIRE(score_func == RT_SCORE_SIGMOID || score_func == RT_SCORE_SOFTMAX ||
                   score_func == RT_SCORE_TOPK_SOFTMAX,
               RT_ERR_BAD_ARG, "rt_moe_route: bad score_func %d", score_func);
    RT_REQUIRE(n_experts <= 512 && topk <= 32 && topk <= n_experts, RT_ERR_UNSUPPORTED,
               "rt_moe_route: needs n_experts <= 512 and topk <= min(32, n_experts)");
    RT_REQUIRE(n_experts % n_groups == 0, RT_ERR_BAD_ARG,
               "rt_moe_route: n_experts must be divisible by n_groups");
    int epl = 1;
    while (32 * epl < n_experts) epl <<= 1;
    if (n_groups > 1) {
        RT_REQUIRE(topk_groups > 0 && topk_groups <= n_groups, RT_ERR_BAD_ARG,
                   "rt_moe_route: bad topk_groups");
        const int64_t gsize = n_experts / n_groups;
        const int64_t lpg = gsize / epl;
        RT_REQUIRE(gsize % epl == 0 && lpg >= 1 && (lpg & (lpg - 1)) == 0 && lpg * n_groups <= 32,
                   RT_ERR_UNSUPPORTED,
                   "rt_moe_route: a group must cover a power-of-two number of whole lanes "
                   "(n_experts=%lld n_groups=%lld)",
                   (long long)n_experts, (long long)n_groups);
        RT_REQUIRE(topk <= topk_groups * gsize, RT_ERR_BAD_ARG,
                   "rt_moe_route: topk exceeds the experts left after group selection");
    }
    if (tokens == 0) return RT_OK;
    const unsigned grid = static_cast<unsigned>((tokens + kRouteWarps - 1) / kRouteWarps);
    cudaStream_t st = as_stream(stream);
#define RT_LAUNCH_ROUTE(E)                                                                       \
    moe_route_kernel<E><<<grid, kRouteWarps * 32, 0, st>>>(                                      \
        logits, bias, weights_out, indices_out, tokens, (int)n_experts, logits_stride,           \
        (int)n_groups, (int)topk_groups, (int)topk, route_scale, score_func)
    switch (epl) {
        case 1: RT_LAUNCH_ROUTE(1); break;
        case 2: RT_LAUNCH_ROUTE(2); break;
        case 4: RT_LAUNCH_ROUTE(4); break;
        case 8: RT_LAUNCH_ROUTE(8); break;
        default: RT_LAUNCH_ROUTE(16); break;
    }
#undef RT_LAUNCH_ROUTE
    count_launch();
    return check_launch("moe_route_kernel");
}

extern "C" int64_t rt_moe_permute_workspace_bytes(int64_t tokens, int64_t topk,
                                                  int64_t n_experts) {
    if (tokens < 0 || topk <= 0 || n_experts <= 0) return 0;
    const int64_t blocks = (tokens * topk + kPermThreads - 1) / kPermThreads;
    return (blocks > 0 ? blocks : 1) * n_experts * static_cast<int64_t>(sizeof(int32_t));
}

extern "C" int rt_moe_permute(const int64_t* indices, int32_t* expert_offsets,
                              int32_t* sorted_pairs, int32_t* pair_pos, void* workspace,
                              int64_t tokens, int64_t topk, int64_t n_experts, void* stream) {
    RT_REQUIRE(indices && expert_offsets && sorted_pairs && pair_pos && workspace, RT_ERR_BAD_ARG,
               "rt_moe_permute: null pointer");
    RT_REQUIRE(tokens >= 0 && topk > 0 && n_experts > 0, RT_ERR_BAD_ARG,
               "rt_moe_permute: bad shape");
    RT_REQUIRE(n_experts <= 1024, RT_ERR_UNSUPPORTED, "rt_moe_permute: n_experts above 1024");
    const int64_t n_pairs = tokens * topk;
    RT_REQUIRE(n_pairs < (1LL << 30), RT_ERR_UNSUPPORTED, "rt_moe_permute: too many pairs");
    const int blocks = static_cast<int>((n_pairs + kPermThreads - 1) / kPermThreads);
    cudaStream_t st = as_stream(stream);
    int32_t* counts = static_cast<int32_t*>(workspace);
    const int ne = static_cast<int>(n_experts);
    if (blocks > 0) {
        moe_count_kernel<<<blocks, kPermThreads, ne * sizeof(int), st>>>(indices, counts,
                                                                         (int)n_pairs, ne);
        count_launch();
        if (int rc = check_launch("moe_count_kernel")) return rc;
    }
    int scan_threads = (ne + 31) / 32 * 32;
    if (scan_threads > 1024) scan_threads = 1024;
    moe_scan_kernel<<<1, scan_threads, 0, st>>>(counts, expert_offsets, blocks, ne);
    count_launch();
    if (int rc = check_launch("moe_scan_kernel")) return rc;
    if (blocks > 0) {
        const size_t smem = 32u * ne * sizeof(unsigned short);
        if (smem > 48u * 1024u) {
            cudaError_t e = cudaFuncSetAttribute(
                moe_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_moe_permute: %s", cudaGetErrorString(e));
        }
        moe_scatter_kernel<<<blocks, kPermThreads, smem, st>>>(
            indices, counts, expert_offsets, sorted_pairs, pair_pos, (int)n_pairs, ne);
        count_launch();
        if (int rc = check_launch("moe_scatter_kernel")) return rc;
    }
    return RT_OK;
}

// ---------------------------------------------------------------------------
// rt_moe_permute without a caller-provided workspace
// ---------------------------------------------------------------------------
// Some hosts cannot give this library scratch memory: an inference runtime that carved all
// device memory into a fixed arena at start-up and offers plugins no allocator, or a
// caller bound to a fixed operator signature that carries inputs and outputs only. For them
// the per-block histogram of the counting sort lives in a fixed array inside the library
// image. Every GPU that loads the library holds these 256 KiB until the process exits.
constexpr int64_t kStaticScratchInts = 65536;  // ceil(pairs / 1024) * n_experts must fit
static __device__ __align__(256) int32_t g_permute_scratch[kStaticScratchInts];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
int32_t* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_permute_scratch on the current device. In host code the array's name
// only stands for the symbol; the address a kernel can use has to be asked for, once per
// device, with that device current.
int static_scratch(int32_t** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_moe_permute_static: cudaGetDevice: %s",
               cudaGetErrorString(e));
    RT_REQUIRE(dev >= 0 && dev < kMaxDevices, RT_ERR_UNSUPPORTED,
               "rt_moe_permute_static: device index %d above the supported %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_permute_scratch);
        RT_REQUIRE(e == cudaSuccess && p != nullptr, RT_ERR_CUDA,
                   "rt_moe_permute_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = static_cast<int32_t*>(p);
    }
    *out = g_scratch_ptr[dev];
    return RT_OK;
}
}  // namespace

extern "C" int64_t rt_moe_permute_static_max_ints(void) { return kStaticScratchInts; }

extern "C" int rt_moe_permute_static(const int64_t* indices, int32_t* expert_offsets,
                                     int32_t* sorted_pairs, int32_t* pair_pos, int64_t tokens,
                                     int64_t topk, int64_t n_experts, void* stream) {
    RT_REQUIRE(indices && expert_offsets && sorted_pairs && pair_pos, RT_ERR_BAD_ARG,
               "rt_moe_permute_static: null pointer");
    RT_REQUIRE(tokens >= 0 && topk > 0 && n_experts > 0, RT_ERR_BAD_ARG,
               "rt_moe_permute_static: bad shape");
    RT_REQUIRE(n_experts <= 1024, RT_ERR_UNSUPPORTED, "rt_moe_permute_static: n_experts above 1024");
    const int64_t n_pairs = tokens * topk;
    const int64_t blocks64 = (n_pairs + kPermThreads - 1) / kPermThreads;
    RT_REQUIRE(blocks64 * n_experts <= kStaticScratchInts, RT_ERR_UNSUPPORTED,
               "rt_moe_permute_static: %lld pairs x %lld experts need %lld scratch entries, the "
               "built-in array holds %lld; use rt_moe_permute with a caller workspace",
               (long long)n_pairs, (long long)n_experts, (long long)(blocks64 * n_experts),
               (long long)kStaticScratchInts);
    int32_t* counts = nullptr;
    if (int rc = static_scratch(&counts)) return rc;
    const int blocks = static_cast<int>(blocks64);
    const int ne = static_cast<int>(n_experts);
    cudaStream_t st = as_stream(stream);
    // Nothing in the array has to start at zero: the count kernel writes every entry of the
    // blocks x n_experts region before the scan and scatter kernels read it.
    if (blocks > 0) {
        moe_count_kernel<<<blocks, kPermThreads, ne * sizeof(int), st>>>(indices, counts,
                                                                         (int)n_pairs, ne);
        count_launch();
        if (int rc = check_launch("moe_count_kernel")) return rc;
    }
    int scan_threads = (ne + 31) / 32 * 32;
    if (scan_threads > 1024) scan_threads = 1024;
    moe_scan_kernel<<<1, scan_threads, 0, st>>>(counts, expert_offsets, blocks, ne);
    count_launch();
    if (int rc = check_launch("moe_scan_kernel")) return rc;
    if (blocks > 0) {
        const size_t smem = 32u * ne * sizeof(unsigned short);
        if (smem > 48u * 1024u) {
            cudaError_t e = cudaFuncSetAttribute(
                moe_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            RT_REQUIRE(e == cudaSuccess, RT_ERR_CUDA, "rt_moe_permute_static: %s",
                       cudaGetErrorString(e));
        }
        moe_scatter_kernel<<<blocks, kPermThreads, smem, st>>>(
            indices, counts, expert_offsets, sorted_pairs, pair_pos, (int)n_pairs, ne);
        count_launch();
        if (int rc = check_launch("moe_scatter_kernel")) return rc;
    }
    return RT_OK;
}

extern "C" int rt_index_topk(const float* scores, int32_t* indices, int64_t queries, int64_t keys,
                             int64_t score_stride, int64_t topk, void* stream) {
    RT_REQUIRE(queries >= 0 && keys > 0 && topk > 0, RT_ERR_BAD_ARG, "rt_index_topk: bad shape");
    if (queries == 0) return RT_OK;
    RT_REQUIRE(scores && indices, RT_ERR_BAD_ARG, "rt_index_topk: null pointer");
    RT_REQUIRE(topk <= keys, RT_ERR_BAD_ARG, "rt_index_topk: topk (%lld) exceeds keys (%lld)",
               (long long)topk, (long long)keys);
    RT_REQUIRE(keys < (1LL << 31) && queries < (1LL << 31) && score_stride >= keys,
               RT_ERR_UNSUPPORTED, "rt_index_topk: dimension too large or stride below keys");
    index_topk_kernel<<<static_cast<unsigned>(queries), kTopkThreads, 0, as_stream(stream)>>>(
        scores, indices, static_cast<int>(keys), score_stride, static_cast<int>(topk));
    count_launch();
    return check_launch("index_topk_kernel");
}

extern "C" int rt_moe_gather(const void* x, const int32_t* sorted_pairs, void* out,
                             int64_t n_pairs, int64_t topk, int64_t cols, int64_t x_stride,
                             int dtype, void* stream) {
    RT_REQUIRE(x && sorted_pairs && out, RT_ERR_BAD_ARG, "rt_moe_gather: null pointer");
    RT_REQUIRE(n_pairs >= 0 && topk > 0 && cols > 0, RT_ERR_BAD_ARG, "rt_moe_gather: bad shape");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_moe_gather: only bf16");
    RT_REQUIRE(cols % 8 == 0 && x_stride % 8 == 0 && aligned16(x) && aligned16(out),
               RT_ERR_UNSUPPORTED, "rt_moe_gather: cols/stride %% 8 and 16-byte alignment needed");
    if (n_pairs == 0) return RT_OK;
    const int64_t nvec = cols / 8, items = n_pairs * nvec;
    RT_REQUIRE(items / 256 < 0x7fffffffLL, RT_ERR_UNSUPPORTED, "rt_moe_gather: too large");
    moe_gather_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, as_stream(stream)>>>(
        (const __nv_bfloat16*)x, sorted_pairs, (__nv_bfloat16*)out, items, (int)nvec, (int)topk,
        x_stride);
    count_launch();
    return check_launch("moe_gather_kernel");
}

extern "C" int rt_moe_combine(const void* expert_out, const int32_t* pair_pos,
                              const float* weights, const void* shared, void* y, int64_t tokens,
                              int64_t topk, int64_t cols, int64_t pos_begin, int64_t pos_end,
                              const int32_t* pos_begin_ptr, const int32_t* pos_end_ptr,
                              int dtype, void* stream) {
    RT_REQUIRE(expert_out && pair_pos && weights && y, RT_ERR_BAD_ARG,
               "rt_moe_combine: null pointer");
    RT_REQUIRE(tokens >= 0 && topk > 0 && cols > 0, RT_ERR_BAD_ARG, "rt_moe_combine: bad shape");
    RT_REQUIRE(dtype == RT_BF16 || dtype == RT_F32, RT_ERR_UNSUPPORTED,
               "rt_moe_combine: y must be bf16 or fp32");
    RT_REQUIRE(cols % 8 == 0 && aligned16(expert_out) && aligned16(y) &&
                   (!shared || aligned16(shared)),
               RT_ERR_UNSUPPORTED, "rt_moe_combine: cols %% 8 and 16-byte alignment needed");
    RT_REQUIRE(tokens <= 0x7fffffffLL && pos_end < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_moe_combine: too large");
    if (tokens == 0) return RT_OK;
    const int nvec = static_cast<int>(cols / 8);
    int threads = (nvec + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    auto kernel = dtype == RT_F32 ? moe_combine_kernel<true> : moe_combine_kernel<false>;
    kernel<<<static_cast<unsigned>(tokens), threads, 0, as_stream(stream)>>>(
        (const __nv_bfloat16*)expert_out, pair_pos, weights, (const __nv_bfloat16*)shared, y, nvec,
        (int)topk, (int)pos_begin, (int)pos_end, pos_begin_ptr, pos_end_ptr);
    count_launch();
    return check_launch("moe_combine_kernel");
}
