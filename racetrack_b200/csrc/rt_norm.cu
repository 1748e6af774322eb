// Residual-add + RMSNorm, RMSNorm, the fused q_a/kv_a RMSNorm + k_pe RoPE
// prologue and the standalone RoPE of the MLA block.
//
// All kernels are HBM-bound row kernels: one CTA per row (or token), the row
// lives in registers as 16-byte vectors, every input byte is read once with a
// streaming load and every output byte written once with a streaming store.
// Algorithmic bytes per row of C columns (bf16, fp32 weight):
//   residual_norm: 4 * C * 2 (+ the weight vector, served from L2)
//   rms_norm:      2 * C * 2
//   rope:          2 * heads * rope_dim * 2
#include "rt_common.cuh"

namespace rt {

// ---------------------------------------------------------------------------
// residual add + RMSNorm
// ---------------------------------------------------------------------------
// VPT = 16-byte vectors per thread. blockDim.x * VPT >= cols / 8.
template <int VPT, bool W_BF16>
__global__ void __launch_bounds__(512) residual_norm_kernel(
    const __nv_bfloat16* __restrict__ update, const __nv_bfloat16* __restrict__ residual,
    const void* __restrict__ weight, __nv_bfloat16* __restrict__ normed,
    __nv_bfloat16* __restrict__ hidden, int nvec, int64_t ustride, int64_t rstride, float cols_f,
    float eps) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const uint4* u = reinterpret_cast<const uint4*>(update + row * ustride);
    const uint4* r = reinterpret_cast<const uint4*>(residual + row * rstride);
    uint4* hrow = reinterpret_cast<uint4*>(hidden) + row * nvec;
    uint4* nrow = reinterpret_cast<uint4*>(normed) + row * nvec;

    uint4 uv[VPT], rv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            uv[i] = ld_stream16(u + v);
            rv[i] = ld_stream16(r + v);
        }
    }
    float h[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            float a[8], b[8];
            unpack_bf16x8(uv[i], a);
            unpack_bf16x8(rv[i], b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                h[i][k] = a[k] + b[k];
                ss += h[i][k] * h[i][k];
            }
            st_stream16(hrow + v, pack_bf16x8(h[i]));
        }
    }
    ss = block_sum(ss, scratch);
    const float rs = rsqrtf(ss / cols_f + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            float w[8], o[8];
            load_weight8<W_BF16>(weight, v, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = w[k] * (h[i][k] * rs);
            st_stream16(nrow + v, pack_bf16x8(o));
        }
    }
}

// ---------------------------------------------------------------------------
// RMSNorm
// ---------------------------------------------------------------------------
template <int VPT, bool W_BF16>
__global__ void __launch_bounds__(512) rms_norm_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const void* __restrict__ weight,
                                                       __nv_bfloat16* __restrict__ out, int nvec,
                                                       int64_t xstride, int64_t ostride,
                                                       float cols_f, float eps) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * xstride);
    uint4* orow = reinterpret_cast<uint4*>(out + row * ostride);
    // The row stays in registers in its packed bf16 form (4 registers per vector instead of
    // 8) and is widened twice; the smaller footprint keeps more rows in flight per SM, which
    // is what a kernel with a single load stream per thread needs.
    uint4 raw[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) raw[i] = ld_stream16(xr + v);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            float h[8];
            unpack_bf16x8(raw[i], h);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += h[k] * h[k];
        }
    }
    ss = block_sum(ss, scratch);
    const float rs = rsqrtf(ss / cols_f + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            float h[8], w[8], o[8];
            unpack_bf16x8(raw[i], h);
            load_weight8<W_BF16>(weight, v, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = (h[k] * rs) * w[k];
            st_stream16(orow + v, pack_bf16x8(o));
        }
    }
}

// ---------------------------------------------------------------------------
// RoPE helpers
// ---------------------------------------------------------------------------

// Row of the rotary table for a caller-given position: positions must lie in [0, table_rows);
// anything else is clamped to the nearest row so that no load leaves the table (the rotation is
// then meaningless, but memory-safe). table_rows == 0 means the caller did not state the size.
__device__ __forceinline__ int64_t table_row(int64_t pos, int64_t table_rows) {
    if (table_rows <= 0) return pos;
    return pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);
}

// Fills cs[0..half) = cos, cs[half..2*half) = sin for one token.
// HALF mode rounds both to bf16 (the reference casts the tables to x.dtype).
__device__ __forceinline__ void fill_cos_sin(float* cs, int half, int64_t token,
                                             const int64_t* positions, const float* table,
                                             int64_t table_rows, int mode) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c, s;
        if (mode == RT_ROPE_HALF) {
            const float pos = static_cast<float>(positions[token]);
            const float ang = __fmul_rn(pos, __ldg(table + i));
            c = round_bf16(cosf(ang));
            s = round_bf16(sinf(ang));
        } else {
            const int64_t trow = positions ? table_row(positions[token], table_rows) : (token % table_rows);
            const float2 f = __ldg(reinterpret_cast<const float2*>(table) + trow * half + i);
            c = f.x;
            s = f.y;
        }
        cs[i] = c;
        cs[half + i] = s;
    }
}

// Half-split rotation of one element pair with torch-eager bf16 rounding
// after every product and after the sum.
__device__ __forceinline__ void rot_half(float x1, float x2, float c, float s, float& o1,
                                         float& o2) {
    o1 = round_bf16(__fsub_rn(round_bf16(__fmul_rn(x1, c)), round_bf16(__fmul_rn(x2, s))));
    o2 = round_bf16(__fadd_rn(round_bf16(__fmul_rn(x2, c)), round_bf16(__fmul_rn(x1, s))));
}

// Interleaved rotation: (x0 + i x1) * (c + i s) in fp32, no intermediate rounding.
__device__ __forceinline__ void rot_pair(float x0, float x1, float c, float s, float& o0,
                                         float& o1) {
    o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// ---------------------------------------------------------------------------
// q_a / kv_a RMSNorm + k_pe RoPE, one CTA per token
// ---------------------------------------------------------------------------
template <int VPT, bool W_BF16>
__global__ void __launch_bounds__(512) norm_rope_kernel(
    const __nv_bfloat16* __restrict__ q_c, const void* __restrict__ q_w,
    const __nv_bfloat16* __restrict__ kv_c, const void* __restrict__ kv_w,
    const __nv_bfloat16* __restrict__ k_pe, const int64_t* __restrict__ positions,
    const float* __restrict__ table, int64_t table_rows, __nv_bfloat16* __restrict__ q_out,
    __nv_bfloat16* __restrict__ kv_out, __nv_bfloat16* __restrict__ k_out, int nq, int nkv,
    int rope_dim, int64_t q_stride, int64_t kv_stride, int64_t k_stride, float q_cols_f,
    float kv_cols_f, float eps, int mode) {
    __shared__ float scratch[64];
    extern __shared__ float cs[];  // [2 * rope_dim/2]
    const int64_t t = blockIdx.x;
    const int half = rope_dim >> 1;
    fill_cos_sin(cs, half, t, positions, table, table_rows, mode);

    const uint4* qr = reinterpret_cast<const uint4*>(q_c + t * q_stride);
    const uint4* kvr = reinterpret_cast<const uint4*>(kv_c + t * kv_stride);
    const int ntot = nq + nkv;
    float h[VPT][8];
    float sq = 0.f, skv = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < ntot) {
            const bool is_q = v < nq;
            unpack_bf16x8(ld_stream16(is_q ? (qr + v) : (kvr + (v - nq))), h[i]);
            float s = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) s += h[i][k] * h[i][k];
            if (is_q) sq += s; else skv += s;
        }
    }
    block_sum2(sq, skv, scratch);  // contains the __syncthreads that publishes cs[]
    const float rq = rsqrtf(sq / q_cols_f + eps);
    const float rkv = rsqrtf(skv / kv_cols_f + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < ntot) {
            const bool is_q = v < nq;
            float w[8], o[8];
            if (is_q) load_weight8<W_BF16>(q_w, v, w); else load_weight8<W_BF16>(kv_w, v - nq, w);
            const float rs = is_q ? rq : rkv;
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = (h[i][k] * rs) * w[k];
            uint4* dst = is_q ? (reinterpret_cast<uint4*>(q_out) + t * nq + v)
                              : (reinterpret_cast<uint4*>(kv_out) + t * nkv + (v - nq));
            st_stream16(dst, pack_bf16x8(o));
        }
    }
    // k_pe rotation: rope_dim elements per token, scalar accesses are enough.
    const __nv_bfloat16* kin = k_pe + t * k_stride;
    __nv_bfloat16* kout = k_out + t * rope_dim;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float c = cs[i], s = cs[half + i];
        float o1, o2;
        if (mode == RT_ROPE_HALF) {
            rot_half(__bfloat162float(kin[i]), __bfloat162float(kin[half + i]), c, s, o1, o2);
            kout[i] = __float2bfloat16_rn(o1);
            kout[half + i] = __float2bfloat16_rn(o2);
        } else {
            rot_pair(__bfloat162float(kin[2 * i]), __bfloat162float(kin[2 * i + 1]), c, s, o1, o2);
            kout[2 * i] = __float2bfloat16_rn(o1);
            kout[2 * i + 1] = __float2bfloat16_rn(o2);
        }
    }
}

// Same operation, one WARP per token (8 tokens per CTA): for the MLA widths (1536 + 512 + 64
// columns = 4 KB per token) a CTA per token spends its life in block-barrier and launch
// latency. Here a lane keeps up to 8 + 4 packed vectors, the two sums of squares are warp
// shuffles, cos/sin are evaluated by the lane that rotates the pair; no shared memory, no
// block barrier, 12 independent 16-byte loads in flight per lane.
constexpr int kNrWarps = 8;
constexpr int kNrQMax = 8;    // q_cols  <= 8 * 32 * 8 = 2048
constexpr int kNrKvMax = 4;   // kv_cols <= 4 * 32 * 8 = 1024

template <bool W_BF16>
__global__ void __launch_bounds__(kNrWarps * 32) norm_rope_warp_kernel(
    const __nv_bfloat16* __restrict__ q_c, const void* __restrict__ q_w,
    const __nv_bfloat16* __restrict__ kv_c, const void* __restrict__ kv_w,
    const __nv_bfloat16* __restrict__ k_pe, const int64_t* __restrict__ positions,
    const float* __restrict__ table, int64_t table_rows, __nv_bfloat16* __restrict__ q_out,
    __nv_bfloat16* __restrict__ kv_out, __nv_bfloat16* __restrict__ k_out, int64_t tokens, int nq,
    int nkv, int rope_dim, int64_t q_stride, int64_t kv_stride, int64_t k_stride, float q_cols_f,
    float kv_cols_f, float eps, int mode) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kNrWarps + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const uint4* qr = reinterpret_cast<const uint4*>(q_c + t * q_stride);
    const uint4* kvr = reinterpret_cast<const uint4*>(kv_c + t * kv_stride);
    uint4 qv[kNrQMax], kvv[kNrKvMax];
#pragma unroll
    for (int i = 0; i < kNrQMax; ++i)
        if (lane + 32 * i < nq) qv[i] = ld_stream16(qr + lane + 32 * i);
#pragma unroll
    for (int i = 0; i < kNrKvMax; ++i)
        if (lane + 32 * i < nkv) kvv[i] = ld_stream16(kvr + lane + 32 * i);
    float sq = 0.f, skv = 0.f;
#pragma unroll
    for (int i = 0; i < kNrQMax; ++i)
        if (lane + 32 * i < nq) {
            float h[8];
            unpack_bf16x8(qv[i], h);
#pragma unroll
            for (int k = 0; k < 8; ++k) sq += h[k] * h[k];
        }
#pragma unroll
    for (int i = 0; i < kNrKvMax; ++i)
        if (lane + 32 * i < nkv) {
            float h[8];
            unpack_bf16x8(kvv[i], h);
#pragma unroll
            for (int k = 0; k < 8; ++k) skv += h[k] * h[k];
        }
    sq = warp_sum(sq);
    skv = warp_sum(skv);
    const float rq = rsqrtf(sq / q_cols_f + eps);
    const float rkv = rsqrtf(skv / kv_cols_f + eps);
    uint4* qo = reinterpret_cast<uint4*>(q_out) + t * nq;
    uint4* kvo = reinterpret_cast<uint4*>(kv_out) + t * nkv;
#pragma unroll
    for (int i = 0; i < kNrQMax; ++i)
        if (lane + 32 * i < nq) {
            float h[8], w[8], o[8];
            unpack_bf16x8(qv[i], h);
            load_weight8<W_BF16>(q_w, lane + 32 * i, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = (h[k] * rq) * w[k];
            st_stream16(qo + lane + 32 * i, pack_bf16x8(o));
        }
#pragma unroll
    for (int i = 0; i < kNrKvMax; ++i)
        if (lane + 32 * i < nkv) {
            float h[8], w[8], o[8];
            unpack_bf16x8(kvv[i], h);
            load_weight8<W_BF16>(kv_w, lane + 32 * i, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = (h[k] * rkv) * w[k];
            st_stream16(kvo + lane + 32 * i, pack_bf16x8(o));
        }
    const int half = rope_dim >> 1;
    const __nv_bfloat16* kin = k_pe + t * k_stride;
    __nv_bfloat16* kout = k_out + t * rope_dim;
    for (int i = lane; i < half; i += 32) {
        float c, s, o1, o2;
        if (mode == RT_ROPE_HALF) {
            const float ang = __fmul_rn(static_cast<float>(positions[t]), __ldg(table + i));
            c = round_bf16(cosf(ang));
            s = round_bf16(sinf(ang));
            rot_half(__bfloat162float(kin[i]), __bfloat162float(kin[half + i]), c, s, o1, o2);
            kout[i] = __float2bfloat16_rn(o1);
            kout[half + i] = __float2bfloat16_rn(o2);
        } else {
            const int64_t trow = positions ? table_row(positions[t], table_rows) : (t % table_rows);
            const float2 f = __ldg(reinterpret_cast<const float2*>(table) + trow * half + i);
            rot_pair(__bfloat162float(kin[2 * i]), __bfloat162float(kin[2 * i + 1]), f.x, f.y, o1, o2);
            kout[2 * i] = __float2bfloat16_rn(o1);
            kout[2 * i + 1] = __float2bfloat16_rn(o2);
        }
    }
}

// ---------------------------------------------------------------------------
// RoPE over [tokens, heads, rope_dim]; one CTA per token
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(
    const __nv_bfloat16* __restrict__ x, const int64_t* __restrict__ positions,
    const float* __restrict__ table, int64_t table_rows, __nv_bfloat16* __restrict__ out,
    int heads, int rope_dim, int64_t tstride, int64_t hstride, int64_t otstride, int64_t ohstride,
    int mode) {
    extern __shared__ float cs[];
    const int64_t t = blockIdx.x;
    const int half = rope_dim >> 1;
    fill_cos_sin(cs, half, t, positions, table, table_rows, mode);
    __syncthreads();
    const __nv_bfloat16* xin = x + t * tstride;
    __nv_bfloat16* xout = out + t * otstride;
    if (mode == RT_ROPE_HALF) {
        // work item = (head, j): vectors j and j + half/8 of that head
        const int per_head = rope_dim >> 4;
        const int items = heads * per_head;
        for (int it = threadIdx.x; it < items; it += blockDim.x) {
            const int hd = it / per_head, j = it - hd * per_head;
            const uint4* src = reinterpret_cast<const uint4*>(xin + hd * hstride);
            uint4* dst = reinterpret_cast<uint4*>(xout + hd * ohstride);
            float a[8], b[8], oa[8], ob[8];
            unpack_bf16x8(ld_once16(src + j), a);
            unpack_bf16x8(ld_once16(src + j + per_head), b);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                rot_half(a[k], b[k], cs[8 * j + k], cs[half + 8 * j + k], oa[k], ob[k]);
            st_stream16(dst + j, pack_bf16x8(oa));
            st_stream16(dst + j + per_head, pack_bf16x8(ob));
        }
    } else {
        const int per_head = rope_dim >> 3;
        const int items = heads * per_head;
        for (int it = threadIdx.x; it < items; it += blockDim.x) {
            const int hd = it / per_head, j = it - hd * per_head;
            const uint4* src = reinterpret_cast<const uint4*>(xin + hd * hstride);
            uint4* dst = reinterpret_cast<uint4*>(xout + hd * ohstride);
            float a[8], o[8];
            unpack_bf16x8(ld_once16(src + j), a);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                rot_pair(a[2 * k], a[2 * k + 1], cs[4 * j + k], cs[half + 4 * j + k], o[2 * k],
                         o[2 * k + 1]);
            st_stream16(dst + j, pack_bf16x8(o));
        }
    }
}

// ---------------------------------------------------------------------------
// Launch helpers
// ---------------------------------------------------------------------------

// Picks vectors-per-thread and a block size (multiple of 32) for `nvec` vectors.
static bool pick_block(int64_t nvec, int& vpt, int& threads) {
    for (int cand : {1, 2, 4, 8}) {
        const int64_t th = ((nvec + cand - 1) / cand + 31) / 32 * 32;
        if (th <= 256 || (cand == 8 && th <= 512)) {
            vpt = cand;
            threads = static_cast<int>(th < 32 ? 32 : th);
            return true;
        }
    }
    return false;
}

}  // namespace rt

using namespace rt;

extern "C" int rt_residual_norm(const void* update, const void* residual, const void* weight,
                                int weight_dtype, void* normed, void* hidden, int64_t rows,
                                int64_t cols, int64_t update_stride, int64_t residual_stride,
                                float eps, int dtype, void* stream) {
    RT_REQUIRE(rows >= 0 && cols > 0, RT_ERR_BAD_ARG, "rt_residual_norm: bad shape %lld x %lld",
               (long long)rows, (long long)cols);
    if (rows == 0) return RT_OK;
    RT_REQUIRE(update && residual && weight && normed && hidden, RT_ERR_BAD_ARG,
               "rt_residual_norm: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_residual_norm: only bf16 activations");
    RT_REQUIRE(weight_dtype == RT_BF16 || weight_dtype == RT_F32, RT_ERR_UNSUPPORTED,
               "rt_residual_norm: weight dtype must be bf16 or f32");
    RT_REQUIRE(cols % 8 == 0 && update_stride % 8 == 0 && residual_stride % 8 == 0,
               RT_ERR_UNSUPPORTED, "rt_residual_norm: cols and strides must be multiples of 8");
    RT_REQUIRE(aligned16(update) && aligned16(residual) && aligned16(weight) && aligned16(normed) &&
                   aligned16(hidden),
               RT_ERR_UNSUPPORTED, "rt_residual_norm: pointers must be 16-byte aligned");
    RT_REQUIRE(rows <= 0x7fffffffLL, RT_ERR_UNSUPPORTED, "rt_residual_norm: too many rows");
    if (rows == 0) return RT_OK;
    int vpt, threads;
    RT_REQUIRE(pick_block(cols / 8, vpt, threads), RT_ERR_UNSUPPORTED,
               "rt_residual_norm: cols %lld above the 32768 limit", (long long)cols);
    const auto* u = static_cast<const __nv_bfloat16*>(update);
    const auto* r = static_cast<const __nv_bfloat16*>(residual);
    auto* n = static_cast<__nv_bfloat16*>(normed);
    auto* h = static_cast<__nv_bfloat16*>(hidden);
    const int nvec = static_cast<int>(cols / 8);
    const dim3 grid(static_cast<unsigned>(rows));
    cudaStream_t st = as_stream(stream);
    const bool wb = weight_dtype == RT_BF16;
#define RT_LAUNCH_RN(V)                                                                          \
    if (wb)                                                                                      \
        residual_norm_kernel<V, true><<<grid, threads, 0, st>>>(                                 \
            u, r, weight, n, h, nvec, update_stride, residual_stride, (float)cols, eps);         \
    else                                                                                         \
        residual_norm_kernel<V, false><<<grid, threads, 0, st>>>(                                \
            u, r, weight, n, h, nvec, update_stride, residual_stride, (float)cols, eps);
    switch (vpt) {
        case 1: RT_LAUNCH_RN(1) break;
        case 2: RT_LAUNCH_RN(2) break;
        case 4: RT_LAUNCH_RN(4) break;
        default: RT_LAUNCH_RN(8) break;
    }
#undef RT_LAUNCH_RN
    count_launch();
    return check_launch("residual_norm_kernel");
}

extern "C" int rt_rms_norm(const void* x, const void* weight, int weight_dtype, void* out,
                           int64_t rows, int64_t cols, int64_t x_stride, int64_t out_stride,
                           float eps, int dtype, void* stream) {
    RT_REQUIRE(rows >= 0 && cols > 0, RT_ERR_BAD_ARG, "rt_rms_norm: bad shape");
    if (rows == 0) return RT_OK;
    RT_REQUIRE(x && weight && out, RT_ERR_BAD_ARG, "rt_rms_norm: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_rms_norm: only bf16 activations");
    RT_REQUIRE(weight_dtype == RT_BF16 || weight_dtype == RT_F32, RT_ERR_UNSUPPORTED,
               "rt_rms_norm: weight dtype must be bf16 or f32");
    RT_REQUIRE(cols % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0, RT_ERR_UNSUPPORTED,
               "rt_rms_norm: cols and strides must be multiples of 8");
    RT_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out), RT_ERR_UNSUPPORTED,
               "rt_rms_norm: pointers must be 16-byte aligned");
    RT_REQUIRE(rows <= 0x7fffffffLL, RT_ERR_UNSUPPORTED, "rt_rms_norm: too many rows");
    if (rows == 0) return RT_OK;
    int vpt, threads;
    RT_REQUIRE(pick_block(cols / 8, vpt, threads), RT_ERR_UNSUPPORTED,
               "rt_rms_norm: cols %lld above the 32768 limit", (long long)cols);
    const auto* xi = static_cast<const __nv_bfloat16*>(x);
    auto* o = static_cast<__nv_bfloat16*>(out);
    const int nvec = static_cast<int>(cols / 8);
    const dim3 grid(static_cast<unsigned>(rows));
    cudaStream_t st = as_stream(stream);
    const bool wb = weight_dtype == RT_BF16;
#define RT_LAUNCH_N(V)                                                                           \
    if (wb)                                                                                      \
        rms_norm_kernel<V, true><<<grid, threads, 0, st>>>(xi, weight, o, nvec, x_stride,        \
                                                           out_stride, (float)cols, eps);        \
    else                                                                                         \
        rms_norm_kernel<V, false><<<grid, threads, 0, st>>>(xi, weight, o, nvec, x_stride,       \
                                                            out_stride, (float)cols, eps);
    switch (vpt) {
        case 1: RT_LAUNCH_N(1) break;
        case 2: RT_LAUNCH_N(2) break;
        case 4: RT_LAUNCH_N(4) break;
        default: RT_LAUNCH_N(8) break;
    }
#undef RT_LAUNCH_N
    count_launch();
    return check_launch("rms_norm_kernel");
}

static int check_rope_args(const char* who, const int64_t* positions, const float* table,
                           int64_t table_rows, int64_t rope_dim, int rope_mode) {
    RT_REQUIRE(table, RT_ERR_BAD_ARG, "%s: null rope table", who);
    RT_REQUIRE(rope_mode == RT_ROPE_HALF || rope_mode == RT_ROPE_INTERLEAVED, RT_ERR_BAD_ARG,
               "%s: bad rope_mode %d", who, rope_mode);
    RT_REQUIRE(rope_dim > 0 && rope_dim % 2 == 0 && rope_dim <= 512, RT_ERR_UNSUPPORTED,
               "%s: rope_dim %lld must be even and <= 512", who, (long long)rope_dim);
    if (rope_mode == RT_ROPE_HALF)
        RT_REQUIRE(positions, RT_ERR_BAD_ARG, "%s: half-split RoPE needs positions", who);
    else
        RT_REQUIRE(positions || table_rows > 0, RT_ERR_BAD_ARG,
                   "%s: interleaved RoPE needs positions or table_rows", who);
    return RT_OK;
}

extern "C" int rt_norm_rope(const void* q_c, const void* q_weight, const void* kv_c,
                            const void* kv_weight, int weight_dtype, const void* k_pe,
                            const int64_t* positions, const float* table, int64_t table_rows,
                            void* q_out, void* kv_out, void* k_out, int64_t tokens, int64_t q_cols,
                            int64_t kv_cols, int64_t rope_dim, int64_t q_stride, int64_t kv_stride,
                            int64_t k_stride, float eps, int rope_mode, int dtype, void* stream) {
    RT_REQUIRE(tokens >= 0 && q_cols > 0 && kv_cols > 0, RT_ERR_BAD_ARG, "rt_norm_rope: bad shape");
    if (tokens == 0) return RT_OK;
    RT_REQUIRE(q_c && q_weight && kv_c && kv_weight && k_pe && q_out && kv_out && k_out,
               RT_ERR_BAD_ARG, "rt_norm_rope: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_norm_rope: only bf16 activations");
    RT_REQUIRE(weight_dtype == RT_BF16 || weight_dtype == RT_F32, RT_ERR_UNSUPPORTED,
               "rt_norm_rope: weight dtype must be bf16 or f32");
    if (int rc = check_rope_args("rt_norm_rope", positions, table, table_rows, rope_dim, rope_mode))
        return rc;
    RT_REQUIRE(q_cols % 8 == 0 && kv_cols % 8 == 0 && q_stride % 8 == 0 && kv_stride % 8 == 0,
               RT_ERR_UNSUPPORTED, "rt_norm_rope: q/kv cols and strides must be multiples of 8");
    RT_REQUIRE(aligned16(q_c) && aligned16(kv_c) && aligned16(q_weight) && aligned16(kv_weight) &&
                   aligned16(q_out) && aligned16(kv_out),
               RT_ERR_UNSUPPORTED, "rt_norm_rope: pointers must be 16-byte aligned");
    RT_REQUIRE(tokens <= 0x7fffffffLL, RT_ERR_UNSUPPORTED, "rt_norm_rope: too many tokens");
    if (tokens == 0) return RT_OK;
    int vpt, threads;
    RT_REQUIRE(pick_block((q_cols + kv_cols) / 8, vpt, threads), RT_ERR_UNSUPPORTED,
               "rt_norm_rope: q_cols + kv_cols above the 32768 limit");
    const int nq = static_cast<int>(q_cols / 8), nkv = static_cast<int>(kv_cols / 8);
    const size_t smem = static_cast<size_t>(rope_dim) * sizeof(float);
    const dim3 grid(static_cast<unsigned>(tokens));
    cudaStream_t st = as_stream(stream);
    const bool wb = weight_dtype == RT_BF16;
    if (nq <= kNrQMax * 32 && nkv <= kNrKvMax * 32) {   // the MLA widths: one warp per token
        const unsigned wgrid = static_cast<unsigned>((tokens + kNrWarps - 1) / kNrWarps);
        if (wb)
            norm_rope_warp_kernel<true><<<wgrid, kNrWarps * 32, 0, st>>>(
                (const __nv_bfloat16*)q_c, q_weight, (const __nv_bfloat16*)kv_c, kv_weight,
                (const __nv_bfloat16*)k_pe, positions, table, table_rows, (__nv_bfloat16*)q_out,
                (__nv_bfloat16*)kv_out, (__nv_bfloat16*)k_out, tokens, nq, nkv, (int)rope_dim,
                q_stride, kv_stride, k_stride, (float)q_cols, (float)kv_cols, eps, rope_mode);
        else
            norm_rope_warp_kernel<false><<<wgrid, kNrWarps * 32, 0, st>>>(
                (const __nv_bfloat16*)q_c, q_weight, (const __nv_bfloat16*)kv_c, kv_weight,
                (const __nv_bfloat16*)k_pe, positions, table, table_rows, (__nv_bfloat16*)q_out,
                (__nv_bfloat16*)kv_out, (__nv_bfloat16*)k_out, tokens, nq, nkv, (int)rope_dim,
                q_stride, kv_stride, k_stride, (float)q_cols, (float)kv_cols, eps, rope_mode);
        count_launch();
        return check_launch("norm_rope_warp_kernel");
    }
#define RT_LAUNCH_NR(V)                                                                         \
    if (wb)                                                                                      \
        norm_rope_kernel<V, true><<<grid, threads, smem, st>>>(                                  \
            (const __nv_bfloat16*)q_c, q_weight, (const __nv_bfloat16*)kv_c, kv_weight,          \
            (const __nv_bfloat16*)k_pe, positions, table, table_rows, (__nv_bfloat16*)q_out,     \
            (__nv_bfloat16*)kv_out, (__nv_bfloat16*)k_out, nq, nkv, (int)rope_dim, q_stride,     \
            kv_stride, k_stride, (float)q_cols, (float)kv_cols, eps, rope_mode);                 \
    else                                                                                         \
        norm_rope_kernel<V, false><<<grid, threads, smem, st>>>(                                 \
            (const __nv_bfloat16*)q_c, q_weight, (const __nv_bfloat16*)kv_c, kv_weight,          \
            (const __nv_bfloat16*)k_pe, positions, table, table_rows, (__nv_bfloat16*)q_out,     \
            (__nv_bfloat16*)kv_out, (__nv_bfloat16*)k_out, nq, nkv, (int)rope_dim, q_stride,     \
            kv_stride, k_stride, (float)q_cols, (float)kv_cols, eps, rope_mode);
    switch (vpt) {
        case 1: RT_LAUNCH_NR(1) break;
        case 2: RT_LAUNCH_NR(2) break;
        case 4: RT_LAUNCH_NR(4) break;
        default: RT_LAUNCH_NR(8) break;
    }
#undef RT_LAUNCH_NR
    count_launch();
    return check_launch("norm_rope_kernel");
}

extern "C" int rt_rope(const void* x, const int64_t* positions, const float* table,
                       int64_t table_rows, void* out, int64_t tokens, int64_t heads,
                       int64_t rope_dim, int64_t token_stride, int64_t head_stride,
                       int64_t out_token_stride, int64_t out_head_stride, int rope_mode, int dtype,
                       void* stream) {
    RT_REQUIRE(tokens >= 0 && heads > 0, RT_ERR_BAD_ARG, "rt_rope: bad shape");
    if (tokens == 0) return RT_OK;
    RT_REQUIRE(x && out, RT_ERR_BAD_ARG, "rt_rope: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_rope: only bf16 activations");
    if (int rc = check_rope_args("rt_rope", positions, table, table_rows, rope_dim, rope_mode))
        return rc;
    RT_REQUIRE(rope_dim % 16 == 0, RT_ERR_UNSUPPORTED, "rt_rope: rope_dim must be a multiple of 16");
    RT_REQUIRE(token_stride % 8 == 0 && head_stride % 8 == 0 && out_token_stride % 8 == 0 &&
                   out_head_stride % 8 == 0 && aligned16(x) && aligned16(out),
               RT_ERR_UNSUPPORTED, "rt_rope: strides must be multiples of 8, pointers 16-byte aligned");
    RT_REQUIRE(tokens <= 0x7fffffffLL && heads <= (1 << 20), RT_ERR_UNSUPPORTED,
               "rt_rope: shape too large");
    if (tokens == 0) return RT_OK;
    const int64_t items = heads * (rope_mode == RT_ROPE_HALF ? rope_dim / 16 : rope_dim / 8);
    int threads = static_cast<int>((items + 31) / 32 * 32);
    if (threads > 256) threads = 256;
    const size_t smem = static_cast<size_t>(rope_dim) * sizeof(float);
    rope_kernel<<<static_cast<unsigned>(tokens), threads, smem, as_stream(stream)>>>(
        (const __nv_bfloat16*)x, positions, table, table_rows, (__nv_bfloat16*)out, (int)heads,
        (int)rope_dim, token_stride, head_stride, out_token_stride, out_head_stride, rope_mode);
    count_launch();
    return check_launch("rope_kernel");
}

namespace rt {
// dst[t, h, 0:dim] = src[t, 0:dim] for every head h: the rotated k_pe row of a token copied
// next to each head's k_nope, so that K = [k_nope | k_pe] exists without a concatenation.
__global__ void __launch_bounds__(256) head_broadcast_kernel(
    const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int heads, int nvec,
    int64_t sstride, int64_t tstride, int64_t hstride) {
    const int64_t t = blockIdx.x;
    const uint4* s = reinterpret_cast<const uint4*>(src + t * sstride);
    for (int it = threadIdx.x; it < heads * nvec; it += blockDim.x) {
        const int h = it / nvec, v = it - h * nvec;
        reinterpret_cast<uint4*>(dst + t * tstride + h * hstride)[v] = __ldg(s + v);
    }
}
}  // namespace rt

extern "C" int rt_head_broadcast(const void* src, void* dst, int64_t tokens, int64_t heads,
                                 int64_t dim, int64_t src_stride, int64_t dst_token_stride,
                                 int64_t dst_head_stride, int dtype, void* stream) {
    RT_REQUIRE(tokens >= 0 && heads > 0 && dim > 0, RT_ERR_BAD_ARG, "rt_head_broadcast: bad shape");
    if (tokens == 0) return RT_OK;
    RT_REQUIRE(src && dst, RT_ERR_BAD_ARG, "rt_head_broadcast: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_head_broadcast: only bf16");
    RT_REQUIRE(dim % 8 == 0 && src_stride % 8 == 0 && dst_token_stride % 8 == 0 &&
                   dst_head_stride % 8 == 0 && aligned16(src) && aligned16(dst),
               RT_ERR_UNSUPPORTED, "rt_head_broadcast: dim/strides %% 8 and 16-byte alignment needed");
    RT_REQUIRE(tokens <= 0x7fffffffLL && heads * dim < (1LL << 30), RT_ERR_UNSUPPORTED,
               "rt_head_broadcast: shape too large");
    rt::head_broadcast_kernel<<<static_cast<unsigned>(tokens), 256, 0, as_stream(stream)>>>(
        (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, (int)heads, (int)(dim / 8), src_stride,
        dst_token_stride, dst_head_stride);
    count_launch();
    return check_launch("head_broadcast_kernel");
}
