// SwiGLU and activation quantisation (FP8 e4m3 per-128 group, NVFP4 per-16 block).
//
// Streaming kernels over a [rows, cols] matrix, flattened into work items of 16
// consecutive columns of one row: two 16-byte loads per input per thread, one
// 16-byte (fp8) or 8-byte (fp4) store of codes. Items of one row are contiguous
// in the thread index, so a 128-column FP8 group is 8 neighbouring lanes and its
// amax needs three shuffles. Algorithmic bytes per element (bf16 input):
//   swiglu            2 + 2 read, 2 written
//   act_quant_fp8     2 read, 1 + 4/128 written
//   swiglu_quant_fp8  4 read, 1 + 4/128 written
//   nvfp4_quant       2 (or 4 with swiglu) read, 1/2 + 1/16 written
//   absmax            2 (or 4) read
#include "rt_common.cuh"

namespace rt {

constexpr int kItem = 16;         // columns per work item
constexpr int kActThreads = 256;  // threads per CTA for the streaming kernels

// Loads the 16 values of one work item. With UP, the values are
// bf16(silu(gate) * up), i.e. what the unfused torch path would hand to the quantiser.
template <bool UP>
__device__ __forceinline__ void load_item(const __nv_bfloat16* __restrict__ x,
                                          const __nv_bfloat16* __restrict__ up, int64_t row,
                                          int64_t col, int64_t xstride, int64_t ustride,
                                          float (&v)[16]) {
    const uint4* px = reinterpret_cast<const uint4*>(x + row * xstride + col);
    const uint4 a0 = ld_stream16(px), a1 = ld_stream16(px + 1);
    float lo[8], hi[8];
    unpack_bf16x8(a0, lo);
    unpack_bf16x8(a1, hi);
    if constexpr (UP) {
        const uint4* pu = reinterpret_cast<const uint4*>(up + row * ustride + col);
        const uint4 b0 = ld_stream16(pu), b1 = ld_stream16(pu + 1);
        float ulo[8], uhi[8];
        unpack_bf16x8(b0, ulo);
        unpack_bf16x8(b1, uhi);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            lo[k] = round_bf16(swiglu_f32(lo[k], ulo[k]));
            hi[k] = round_bf16(swiglu_f32(hi[k], uhi[k]));
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        v[k] = lo[k];
        v[8 + k] = hi[k];
    }
}

__device__ __forceinline__ float absmax16(const float (&v)[16]) {
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) m = fmaxf(m, fabsf(v[k]));
    return m;
}

// Two fp32 -> two e4m3 (RNE, saturating), `lo` in the low byte.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}

// e4m3 byte -> fp32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(b)));
    return __half2float(__ushort_as_half(static_cast<uint16_t>(h2 & 0xffffu)));
}

// ---------------------------------------------------------------------------
// SwiGLU
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kActThreads) swiglu_kernel(
    const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
    __nv_bfloat16* __restrict__ out, uint32_t items, uint32_t items_per_row, int64_t gstride,
    int64_t ustride, int64_t cols) {
    const uint32_t id = blockIdx.x * kActThreads + threadIdx.x;
    if (id >= items) return;
    const uint32_t row = id / items_per_row;
    const int64_t col = static_cast<int64_t>(id - row * items_per_row) * 8;
    const uint4 g = ld_stream16(gate + row * gstride + col);
    const uint4 u = ld_stream16(up + row * ustride + col);
    float gf[8], uf[8], o[8];
    unpack_bf16x8(g, gf);
    unpack_bf16x8(u, uf);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = swiglu_f32(gf[k], uf[k]);
    st_stream16(out + row * cols + col, pack_bf16x8(o));
}

// ---------------------------------------------------------------------------
// FP8 e4m3 per-128-column group quantisation (optionally of swiglu(gate, up))
// ---------------------------------------------------------------------------
template <bool UP>
__global__ void __launch_bounds__(kActThreads) quant_fp8_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    uint8_t* __restrict__ codes, float* __restrict__ scales, uint32_t items,
    uint32_t items_per_row, int64_t xstride, int64_t ustride, int64_t cols) {
    const uint32_t id = blockIdx.x * kActThreads + threadIdx.x;
    // items is a multiple of 8 and CTAs start on a multiple of 8, so the eight
    // lanes of a group are either all in range or all out of range.
    if (id >= items) return;
    const uint32_t row = id / items_per_row;
    const uint32_t item = id - row * items_per_row;
    const int64_t col = static_cast<int64_t>(item) * kItem;
    float v[16];
    load_item<UP>(x, up, row, col, xstride, ustride, v);
    float amax = absmax16(v);
    // the 8 lanes of a group share one shuffle mask segment
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t gmask = 0xffu << (lane & 24u);
    amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 4));
    amax = fmaxf(amax, 1.0e-4f);
    const float scale = __fdiv_rn(amax, 448.0f);
    const float rscale = __frcp_rn(scale);
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // no explicit clamp: the saturating conversion maps |q| > 448 to +-448,
            // which is what clamp(-448, 448) followed by a cast yields
            q[j] = div_shared(v[4 * k + j], scale, rscale);
        }
        w[k] = cvt_e4m3x2(q[0], q[1]) | (cvt_e4m3x2(q[2], q[3]) << 16);
    }
    st_stream16(codes + static_cast<int64_t>(row) * cols + col, make_uint4(w[0], w[1], w[2], w[3]));
    if ((item & 7u) == 0) scales[static_cast<int64_t>(row) * (cols >> 7) + (item >> 3)] = scale;
}

// ---------------------------------------------------------------------------
// Indexer prologue: (LayerNorm) -> non-interleaved RoPE -> Hadamard rotation -> FP8 quantisation
// ---------------------------------------------------------------------------
// One warp per 128-wide row (an index head of a query, or a key), lane l owning elements
// 4l .. 4l + 3; every stage rounds to bf16 where the reference's op-by-op path does.
//   LayerNorm (keys only): fp32 mean / biased variance, (x * rstd - rstd * mean) * w + b.
//   RoPE on dims [0, 64), pairs (i, i + 32): complex product with freqs[pos][i] in fp32.
//   Hadamard: fast Walsh-Hadamard transform in natural (Sylvester) order, two butterfly stages
//   inside the lane and five across lanes, times 128^-0.5.
//   act_quant: one 128-wide group per row: scale = max(amax, 1e-4) / 448, e4m3 codes.
template <bool HAS_LN>
__global__ void __launch_bounds__(256) index_prep_kernel(
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ ln_w,
    const float* __restrict__ ln_b, const int64_t* __restrict__ positions,
    const float2* __restrict__ freqs, int table_rows, int rows_per_pos,
    uint8_t* __restrict__ codes, float* __restrict__ scales, __nv_bfloat16* __restrict__ rotated,
    int64_t rows, int64_t xstride, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint2 raw = *reinterpret_cast<const uint2*>(x + row * xstride + 4 * lane);
    float v[4];
    v[0] = __uint_as_float(raw.x << 16);
    v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16);
    v[3] = __uint_as_float(raw.y & 0xffff0000u);
    if constexpr (HAS_LN) {
        const float mean = warp_sum((v[0] + v[1]) + (v[2] + v[3])) * (1.0f / 128.0f);
        float d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) d[j] = v[j] - mean;
        const float var = warp_sum((d[0] * d[0] + d[1] * d[1]) + (d[2] * d[2] + d[3] * d[3])) *
                          (1.0f / 128.0f);
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(var + eps));
        const float shift = -(rstd * mean);
        const float4 w = *reinterpret_cast<const float4*>(ln_w + 4 * lane);
        const float4 b = *reinterpret_cast<const float4*>(ln_b + 4 * lane);
        v[0] = round_bf16((v[0] * rstd + shift) * w.x + b.x);
        v[1] = round_bf16((v[1] * rstd + shift) * w.y + b.y);
        v[2] = round_bf16((v[2] * rstd + shift) * w.z + b.z);
        v[3] = round_bf16((v[3] * rstd + shift) * w.w + b.w);
    }
    // RoPE: lanes 0-7 hold dims 0-31 (real parts), lanes 8-15 dims 32-63 (imaginary parts)
    {
        int64_t pos = positions ? positions[row / rows_per_pos] : row / rows_per_pos;
        // positions must lie in [0, table_rows); others are clamped (memory-safe, not meaningful)
        if (pos >= table_rows) pos = table_rows - 1;
        if (pos < 0) pos = 0;
        float other[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) other[j] = __shfl_xor_sync(0xffffffffu, v[j], 8);
        if (lane < 16) {
            const float2* f = freqs + pos * 32 + 4 * (lane & 7);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 cs = f[j];
                const float re = lane < 8 ? v[j] : other[j];
                const float im = lane < 8 ? other[j] : v[j];
                const float out = lane < 8 ? (re * cs.x - im * cs.y) : (re * cs.y + im * cs.x);
                v[j] = round_bf16(out);
            }
        }
    }
    // Hadamard rotation
    {
        float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
        v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = __shfl_xor_sync(0xffffffffu, v[j], m);
                v[j] = (lane & m) ? (p - v[j]) : (v[j] + p);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = round_bf16(v[j] * 0.08838834764831845f);
    }
    if (rotated) {
        uint2 o;
        o.x = pack_bf16x2(v[0], v[1]);
        o.y = pack_bf16x2(v[2], v[3]);
        *reinterpret_cast<uint2*>(rotated + row * 128 + 4 * lane) = o;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(warp_max(amax), 1.0e-4f);
    const float scale = __fdiv_rn(amax, 448.0f);
    const float rscale = __frcp_rn(scale);
    const uint32_t packed = cvt_e4m3x2(div_shared(v[0], scale, rscale), div_shared(v[1], scale, rscale)) |
                            (cvt_e4m3x2(div_shared(v[2], scale, rscale), div_shared(v[3], scale, rscale)) << 16);
    *reinterpret_cast<uint32_t*>(codes + row * 128 + 4 * lane) = packed;
    if (lane == 0) scales[row] = scale;
}

// ---------------------------------------------------------------------------
// Tensor-wide abs-max (NVFP4 global scale)
// ---------------------------------------------------------------------------
__global__ void absmax_clear_kernel(float* out) { *out = 0.f; }

// STORE: also writes the values it took the maximum of (bf16(silu(x) * up) when UP) to
// h[row, col], so that a later pass can quantise them without evaluating SwiGLU again.
template <bool UP, bool STORE>
__global__ void __launch_bounds__(kActThreads) absmax_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    float* __restrict__ out, uint32_t items, uint32_t items_per_row, int64_t xstride,
    int64_t ustride, const int32_t* __restrict__ row_begin, const int32_t* __restrict__ row_end,
    __nv_bfloat16* __restrict__ h, int64_t hstride) {
    __shared__ float scratch[32];
    float m = 0.f;
    // optional row window read from device memory (the rows an expert-parallel rank owns)
    const uint32_t r_lo = row_begin ? static_cast<uint32_t>(__ldg(row_begin)) : 0u;
    const uint32_t r_hi = row_end ? static_cast<uint32_t>(__ldg(row_end)) : 0xffffffffu;
    for (uint32_t id = blockIdx.x * kActThreads + threadIdx.x; id < items;
         id += gridDim.x * kActThreads) {
        const uint32_t row = id / items_per_row;
        if (row < r_lo || row >= r_hi) continue;
        const int64_t col = static_cast<int64_t>(id - row * items_per_row) * kItem;
        float v[16];
        load_item<UP>(x, up, row, col, xstride, ustride, v);
        m = fmaxf(m, absmax16(v));
        if constexpr (STORE) {
            float lo[8], hi[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                lo[k] = v[k];
                hi[k] = v[8 + k];
            }
            uint4* ph = reinterpret_cast<uint4*>(h + static_cast<int64_t>(row) * hstride + col);
            st_stream16(ph, pack_bf16x8(lo));
            st_stream16(ph + 1, pack_bf16x8(hi));
        }
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = (threadIdx.x < (kActThreads >> 5)) ? scratch[threadIdx.x] : 0.f;
        m = warp_max(m);
        // non-negative floats order like their bit patterns
        if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
    }
}

// ---------------------------------------------------------------------------
// NVFP4: e2m1 codes, e4m3 scale per 16-element block, fp32 global scale
// ---------------------------------------------------------------------------

// Two fp32 -> two e2m1 codes in one byte (`lo` in the low nibble): round to nearest
// even onto {0, .5, 1, 1.5, 2, 3, 4, 6}, saturating, sign kept (also for zero).
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t d;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }"
        : "=h"(d)
        : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ int64_t sf_offset(int layout, int64_t row, int64_t blk,
                                             int64_t nblk) {
    if (layout == RT_SF_ROWMAJOR) return row * nblk + blk;
    const int64_t kt = (nblk + 3) >> 2;
    return ((row >> 7) * kt + (blk >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
           (blk & 3);
}

template <bool UP>
__global__ void __launch_bounds__(kActThreads) quant_nvfp4_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    const float* __restrict__ amax_in, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
    float* __restrict__ gs_out, uint32_t items, uint32_t items_per_row, int64_t xstride,
    int64_t ustride, int64_t cols, int layout) {
    const uint32_t id = blockIdx.x * kActThreads + threadIdx.x;
    const float amax = __ldg(amax_in);
    const float gs = amax > 0.f ? __fdiv_rn(amax, 2688.0f) : 1.0f;
    if (id == 0 && gs_out) *gs_out = gs;
    if (id >= items) return;
    const uint32_t row = id / items_per_row;
    const uint32_t blk = id - row * items_per_row;
    const int64_t col = static_cast<int64_t>(blk) * kItem;
    float v[16];
    load_item<UP>(x, up, row, col, xstride, ustride, v);
    const float bmax = absmax16(v);
    const float t = fminf(__fdiv_rn(bmax, __fmul_rn(6.0f, gs)), 448.0f);
    const uint32_t bs = cvt_e4m3x2(t, 0.f) & 0xffu;
    const float denom = __fmul_rn(gs, e4m3_to_f32(bs));
    uint32_t lo = 0, hi = 0;
    if (denom > 0.f) {
        const float inv = __frcp_rn(denom);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            lo |= cvt_e2m1x2(__fmul_rn(v[2 * k], inv), __fmul_rn(v[2 * k + 1], inv)) << (8 * k);
            hi |= cvt_e2m1x2(__fmul_rn(v[8 + 2 * k], inv), __fmul_rn(v[9 + 2 * k], inv)) << (8 * k);
        }
    }
    st_stream8(codes + static_cast<int64_t>(row) * (cols >> 1) + (col >> 1), make_uint2(lo, hi));
    sf[sf_offset(layout, row, blk, items_per_row)] = static_cast<uint8_t>(bs);
}

// NVFP4 quantisation of the rows a grouped-GEMM tile map covers. Tile t = {group, first
// row, valid rows, scale row tile}: codes go to the (compact) destination row, scales to the
// tile's own 128-row scale tiles, rows of the tile beyond `valid rows` get zero scales.
// With sorted_pairs the source row of destination row r is sorted_pairs[r] / topk (the
// token gather of the MoE dispatch fused into the quantiser); otherwise source = destination.
// Grid: 16 CTAs per tile, each doing 8 rows.
template <bool UP>
__global__ void __launch_bounds__(kActThreads) quant_nvfp4_tiles_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ up,
    const int32_t* __restrict__ sorted_pairs, int topk, const float* __restrict__ amax_in,
    uint8_t* __restrict__ codes, uint8_t* __restrict__ sf, float* __restrict__ gs_out,
    const int4* __restrict__ tile_map, const int32_t* __restrict__ tile_count,
    uint32_t items_per_row, int64_t xstride, int64_t ustride, int64_t cols) {
    const int tile = blockIdx.x >> 4, sub = blockIdx.x & 15;
    const float amax = __ldg(amax_in);
    const float gs = amax > 0.f ? __fdiv_rn(amax, 2688.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0 && gs_out) *gs_out = gs;
    if (tile >= __ldg(tile_count)) return;
    const int4 tm = __ldg(tile_map + tile);
    const float six_gs = __fmul_rn(6.0f, gs);
    const uint32_t kt = items_per_row >> 2;
    uint8_t* sf_tile = sf + static_cast<int64_t>(tm.w) * kt * 512;
    for (uint32_t it = threadIdx.x; it < 8u * items_per_row; it += kActThreads) {
        const uint32_t rr = it / items_per_row;
        const uint32_t blk = it - rr * items_per_row;
        const uint32_t r_local = sub * 8u + rr;
        uint8_t* sf_dst = sf_tile + static_cast<int64_t>(blk >> 2) * 512 + (r_local & 31u) * 16u +
                          (r_local >> 5) * 4u + (blk & 3u);
        if (static_cast<int>(r_local) >= tm.z) {
            *sf_dst = 0;
            continue;
        }
        const int64_t dst_row = tm.y + r_local;
        const int64_t src_row = sorted_pairs ? (__ldg(sorted_pairs + dst_row) / topk) : dst_row;
        const int64_t col = static_cast<int64_t>(blk) * kItem;
        float v[16];
        load_item<UP>(x, up, src_row, col, xstride, ustride, v);
        const float bmax = absmax16(v);
        const float t = fminf(__fdiv_rn(bmax, six_gs), 448.0f);
        const uint32_t bs = cvt_e4m3x2(t, 0.f) & 0xffu;
        const float denom = __fmul_rn(gs, e4m3_to_f32(bs));
        uint32_t lo = 0, hi = 0;
        if (denom > 0.f) {
            const float inv = __frcp_rn(denom);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                lo |= cvt_e2m1x2(__fmul_rn(v[2 * k], inv), __fmul_rn(v[2 * k + 1], inv)) << (8 * k);
                hi |= cvt_e2m1x2(__fmul_rn(v[8 + 2 * k], inv), __fmul_rn(v[9 + 2 * k], inv)) << (8 * k);
            }
        }
        st_stream8(codes + dst_row * (cols >> 1) + (col >> 1), make_uint2(lo, hi));
        *sf_dst = static_cast<uint8_t>(bs);
    }
}

// MoE dispatch of activations that are ALREADY NVFP4: the token rows were quantised once
// (codes [tokens, cols/2], row-major scales [tokens, cols/16]); this kernel copies, for every
// 128-row tile of the tile map, the rows its sorted (token, slot) pairs name: codes to the
// compact destination rows, scales into the 128 x 4 tiled layout of the tile (zeros for the rows
// past the tile's valid rows). One CTA per tile: each warp copies 16 rows (a row's codes in 7
// coalesced 16-byte sweeps for 7168 columns) and parks their scales in shared memory (row pitch
// padded to an odd number of words so the column reads below spread over all banks); then every
// warp assembles 512-byte scale tiles: lane l packs the 4 scale bytes of rows l, l + 32, l + 64,
// l + 96 and stores 16 bytes.
constexpr int kGatherThreads = 256;

__global__ void __launch_bounds__(kGatherThreads) moe_gather_nvfp4_kernel(
    const uint8_t* __restrict__ codes_in, const uint8_t* __restrict__ sf_in,
    const int32_t* __restrict__ sorted_pairs, int topk, uint8_t* __restrict__ codes_out,
    uint8_t* __restrict__ sf_out, const int4* __restrict__ tile_map,
    const int32_t* __restrict__ tile_count, int64_t cols) {
    extern __shared__ uint32_t sf_smem[];
    const int tile = blockIdx.x;
    if (tile >= __ldg(tile_count)) return;
    const int4 tm = __ldg(tile_map + tile);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t code_bytes = cols >> 1;            // per row, a multiple of 32
    const int sf_words = static_cast<int>(cols >> 6);   // 4-byte scale groups per row (k-tiles)
    const int pitch = sf_words | 1;                  // odd word pitch
    for (int r = warp; r < 128; r += kGatherThreads / 32) {
        if (r >= tm.z) {
            for (int w = lane; w < sf_words; w += 32) sf_smem[r * pitch + w] = 0u;
            continue;
        }
        const int64_t dst_row = tm.y + r;
        const int64_t src_row = __ldg(sorted_pairs + dst_row) / topk;
        const uint4* src = reinterpret_cast<const uint4*>(codes_in + src_row * code_bytes);
        uint4* dst = reinterpret_cast<uint4*>(codes_out + dst_row * code_bytes);
        for (int64_t i = lane; i < (code_bytes >> 4); i += 32) st_stream16(dst + i, ld_cached16(src + i));
        const uint32_t* ssf = reinterpret_cast<const uint32_t*>(sf_in + src_row * (cols >> 4));
        for (int w = lane; w < sf_words; w += 32) sf_smem[r * pitch + w] = __ldg(ssf + w);
    }
    __syncthreads();
    uint8_t* sf_tile = sf_out + static_cast<int64_t>(tm.w) * sf_words * 512;
    for (int kt = warp; kt < sf_words; kt += kGatherThreads / 32) {
        uint4 v;
        v.x = sf_smem[lane * pitch + kt];
        v.y = sf_smem[(lane + 32) * pitch + kt];
        v.z = sf_smem[(lane + 64) * pitch + kt];
        v.w = sf_smem[(lane + 96) * pitch + kt];
        st_stream16(sf_tile + static_cast<int64_t>(kt) * 512 + lane * 16, v);
    }
}

// Zero-fills the padding entries of a 128x4-tiled scale buffer (rows beyond
// `rows` inside the last 128-row tile, blocks beyond nblk inside the last 4-block tile).
__global__ void sf_pad_kernel(uint8_t* __restrict__ sf, int64_t rows, int64_t nblk,
                              int64_t rows_pad, int64_t nblk_pad) {
    const int64_t total = rows_pad * nblk_pad;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / nblk_pad, b = i - r * nblk_pad;
        if (r >= rows || b >= nblk) sf[sf_offset(RT_SF_TILED128x4, r, b, nblk)] = 0;
    }
}

static int check_stream_args(const char* who, const void* x, int64_t rows, int64_t cols,
                             int64_t xstride, int64_t mult, int dtype, uint32_t& items,
                             uint32_t& per_row, int64_t item_cols) {
    RT_REQUIRE(rows >= 0 && cols > 0, RT_ERR_BAD_ARG, "%s: bad shape %lld x %lld", who,
               (long long)rows, (long long)cols);
    RT_REQUIRE(x || rows == 0, RT_ERR_BAD_ARG, "%s: null pointer", who);
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "%s: only bf16 activations", who);
    RT_REQUIRE(cols % mult == 0, RT_ERR_UNSUPPORTED, "%s: cols %lld must be a multiple of %lld",
               who, (long long)cols, (long long)mult);
    RT_REQUIRE(xstride % 8 == 0 && aligned16(x), RT_ERR_UNSUPPORTED,
               "%s: row stride must be a multiple of 8 and pointers 16-byte aligned", who);
    const int64_t pr = cols / item_cols;
    const int64_t total = rows * pr;
    RT_REQUIRE(total < (1LL << 32) - kActThreads, RT_ERR_UNSUPPORTED, "%s: tensor too large", who);
    items = static_cast<uint32_t>(total);
    per_row = static_cast<uint32_t>(pr);
    return RT_OK;
}

}  // namespace rt

using namespace rt;

extern "C" int rt_swiglu(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                         int64_t gate_stride, int64_t up_stride, int dtype, void* stream) {
    uint32_t items, per_row;
    if (int rc = check_stream_args("rt_swiglu", gate, rows, cols, gate_stride, 8, dtype, items,
                                   per_row, 8))
        return rc;
    if (items == 0) return RT_OK;
    RT_REQUIRE(up && out, RT_ERR_BAD_ARG, "rt_swiglu: null pointer");
    RT_REQUIRE(up_stride % 8 == 0 && aligned16(up) && aligned16(out), RT_ERR_UNSUPPORTED,
               "rt_swiglu: up/out must be 16-byte aligned with stride %% 8 == 0");
    if (items == 0) return RT_OK;
    const unsigned grid = (items + kActThreads - 1) / kActThreads;
    swiglu_kernel<<<grid, kActThreads, 0, as_stream(stream)>>>(
        (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)out, items, per_row,
        gate_stride, up_stride, cols);
    count_launch();
    return check_launch("swiglu_kernel");
}

static int quant_fp8_common(const char* who, const void* x, const void* up, void* codes,
                            float* scales, int64_t rows, int64_t cols, int64_t x_stride,
                            int64_t up_stride, int dtype, void* stream) {
    uint32_t items, per_row;
    if (int rc = check_stream_args(who, x, rows, cols, x_stride, 128, dtype, items, per_row, kItem))
        return rc;
    if (items == 0) return RT_OK;
    RT_REQUIRE(codes && scales, RT_ERR_BAD_ARG, "%s: null output pointer", who);
    RT_REQUIRE(aligned16(codes), RT_ERR_UNSUPPORTED, "%s: codes must be 16-byte aligned", who);
    if (up) RT_REQUIRE(up_stride % 8 == 0 && aligned16(up), RT_ERR_UNSUPPORTED,
                       "%s: up must be 16-byte aligned with stride %% 8 == 0", who);
    if (items == 0) return RT_OK;
    const unsigned grid = (items + kActThreads - 1) / kActThreads;
    if (up)
        quant_fp8_kernel<true><<<grid, kActThreads, 0, as_stream(stream)>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)up, (uint8_t*)codes, scales, items,
            per_row, x_stride, up_stride, cols);
    else
        quant_fp8_kernel<false><<<grid, kActThreads, 0, as_stream(stream)>>>(
            (const __nv_bfloat16*)x, nullptr, (uint8_t*)codes, scales, items, per_row, x_stride, 0,
            cols);
    count_launch();
    return check_launch("quant_fp8_kernel");
}

extern "C" int rt_act_quant_fp8(const void* x, void* codes, float* scales, int64_t rows,
                                int64_t cols, int64_t x_stride, int dtype, void* stream) {
    return quant_fp8_common("rt_act_quant_fp8", x, nullptr, codes, scales, rows, cols, x_stride, 0,
                            dtype, stream);
}

extern "C" int rt_swiglu_quant_fp8(const void* gate, const void* up, void* codes, float* scales,
                                   int64_t rows, int64_t cols, int64_t gate_stride,
                                   int64_t up_stride, int dtype, void* stream) {
    RT_REQUIRE(up, RT_ERR_BAD_ARG, "rt_swiglu_quant_fp8: null up pointer");
    return quant_fp8_common("rt_swiglu_quant_fp8", gate, up, codes, scales, rows, cols,
                            gate_stride, up_stride, dtype, stream);
}

static int absmax_common(const void* x, const void* up, float* amax_out, int64_t rows,
                         int64_t cols, int64_t x_stride, int64_t up_stride,
                         const int32_t* row_begin, const int32_t* row_end, int dtype,
                         void* stream, void* h = nullptr, int64_t h_stride = 0) {
    uint32_t items, per_row;
    if (int rc = check_stream_args("rt_absmax", x, rows, cols, x_stride, 16, dtype, items, per_row,
                                   kItem))
        return rc;
    RT_REQUIRE(amax_out, RT_ERR_BAD_ARG, "rt_absmax: null output pointer");
    if (up) RT_REQUIRE(up_stride % 8 == 0 && aligned16(up), RT_ERR_UNSUPPORTED,
                       "rt_absmax: up must be 16-byte aligned with stride %% 8 == 0");
    cudaStream_t st = as_stream(stream);
    absmax_clear_kernel<<<1, 1, 0, st>>>(amax_out);
    count_launch();
    if (items == 0) return check_launch("absmax_clear_kernel");
    // persistent grid: 148 SMs x 8 resident CTAs, each thread loops over items
    unsigned grid = (items + kActThreads - 1) / kActThreads;
    if (grid > 148u * 8u) grid = 148u * 8u;
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* ub = static_cast<const __nv_bfloat16*>(up);
    __nv_bfloat16* hb = static_cast<__nv_bfloat16*>(h);
    if (up && h)
        absmax_kernel<true, true><<<grid, kActThreads, 0, st>>>(
            xb, ub, amax_out, items, per_row, x_stride, up_stride, row_begin, row_end, hb, h_stride);
    else if (up)
        absmax_kernel<true, false><<<grid, kActThreads, 0, st>>>(
            xb, ub, amax_out, items, per_row, x_stride, up_stride, row_begin, row_end, nullptr, 0);
    else
        absmax_kernel<false, false><<<grid, kActThreads, 0, st>>>(
            xb, nullptr, amax_out, items, per_row, x_stride, 0, row_begin, row_end, nullptr, 0);
    count_launch();
    return check_launch("absmax_kernel");
}

extern "C" int rt_absmax(const void* x, const void* up, float* amax_out, int64_t rows,
                         int64_t cols, int64_t x_stride, int64_t up_stride, int dtype,
                         void* stream) {
    return absmax_common(x, up, amax_out, rows, cols, x_stride, up_stride, nullptr, nullptr, dtype,
                         stream);
}

extern "C" int rt_absmax_rows(const void* x, const void* up, float* amax_out, int64_t rows,
                              int64_t cols, int64_t x_stride, int64_t up_stride,
                              const int32_t* row_begin, const int32_t* row_end, int dtype,
                              void* stream) {
    return absmax_common(x, up, amax_out, rows, cols, x_stride, up_stride, row_begin, row_end,
                         dtype, stream);
}

extern "C" int rt_swiglu_absmax_rows(const void* gate, const void* up, void* h, float* amax_out,
                                     int64_t rows, int64_t cols, int64_t gate_stride,
                                     int64_t up_stride, int64_t h_stride,
                                     const int32_t* row_begin, const int32_t* row_end, int dtype,
                                     void* stream) {
    RT_REQUIRE(up && h, RT_ERR_BAD_ARG, "rt_swiglu_absmax_rows: null pointer");
    RT_REQUIRE(h_stride % 8 == 0 && aligned16(h), RT_ERR_UNSUPPORTED,
               "rt_swiglu_absmax_rows: h must be 16-byte aligned with stride %% 8 == 0");
    return absmax_common(gate, up, amax_out, rows, cols, gate_stride, up_stride, row_begin, row_end,
                         dtype, stream, h, h_stride);
}

extern "C" int rt_moe_quant_nvfp4(const void* x, const void* up, const int32_t* sorted_pairs,
                                  int64_t topk, const float* amax_in, void* codes,
                                  void* block_scales, float* global_scale_out,
                                  const int32_t* tile_map, const int32_t* tile_count,
                                  int64_t max_tiles, int64_t cols, int64_t x_stride,
                                  int64_t up_stride, int dtype, void* stream) {
    RT_REQUIRE(max_tiles >= 0 && cols > 0 && topk > 0, RT_ERR_BAD_ARG,
               "rt_moe_quant_nvfp4: bad shape");
    if (max_tiles == 0) return RT_OK;
    RT_REQUIRE(x && amax_in && codes && block_scales && tile_map && tile_count, RT_ERR_BAD_ARG,
               "rt_moe_quant_nvfp4: null pointer");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_moe_quant_nvfp4: only bf16 activations");
    RT_REQUIRE(cols % 64 == 0, RT_ERR_UNSUPPORTED,
               "rt_moe_quant_nvfp4: cols must be a multiple of 64 (whole scale tiles)");
    RT_REQUIRE(x_stride % 8 == 0 && aligned16(x) && (!up || (up_stride % 8 == 0 && aligned16(up))) &&
                   aligned16(tile_map) && (reinterpret_cast<uintptr_t>(codes) & 7u) == 0,
               RT_ERR_UNSUPPORTED, "rt_moe_quant_nvfp4: alignment (16-byte inputs, stride %% 8)");
    RT_REQUIRE(max_tiles < (1LL << 27), RT_ERR_UNSUPPORTED, "rt_moe_quant_nvfp4: too many tiles");
    const unsigned grid = static_cast<unsigned>(max_tiles * 16);
    const uint32_t per_row = static_cast<uint32_t>(cols / kItem);
    cudaStream_t st = as_stream(stream);
    if (up)
        quant_nvfp4_tiles_kernel<true><<<grid, kActThreads, 0, st>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)up, sorted_pairs, (int)topk, amax_in,
            (uint8_t*)codes, (uint8_t*)block_scales, global_scale_out, (const int4*)tile_map,
            tile_count, per_row, x_stride, up_stride, cols);
    else
        quant_nvfp4_tiles_kernel<false><<<grid, kActThreads, 0, st>>>(
            (const __nv_bfloat16*)x, nullptr, sorted_pairs, (int)topk, amax_in, (uint8_t*)codes,
            (uint8_t*)block_scales, global_scale_out, (const int4*)tile_map, tile_count, per_row,
            x_stride, 0, cols);
    count_launch();
    return check_launch("quant_nvfp4_tiles_kernel");
}

extern "C" int rt_moe_gather_nvfp4(const void* codes_in, const void* sf_in,
                                   const int32_t* sorted_pairs, int64_t topk, void* codes_out,
                                   void* sf_out, const int32_t* tile_map,
                                   const int32_t* tile_count, int64_t max_tiles, int64_t cols,
                                   void* stream) {
    RT_REQUIRE(max_tiles >= 0 && cols > 0 && topk > 0, RT_ERR_BAD_ARG,
               "rt_moe_gather_nvfp4: bad shape");
    if (max_tiles == 0) return RT_OK;
    RT_REQUIRE(codes_in && sf_in && sorted_pairs && codes_out && sf_out && tile_map && tile_count,
               RT_ERR_BAD_ARG, "rt_moe_gather_nvfp4: null pointer");
    RT_REQUIRE(cols % 64 == 0, RT_ERR_UNSUPPORTED,
               "rt_moe_gather_nvfp4: cols must be a multiple of 64 (whole scale tiles)");
    RT_REQUIRE(aligned16(codes_in) && aligned16(codes_out) && aligned16(sf_out) &&
                   aligned16(tile_map) && (reinterpret_cast<uintptr_t>(sf_in) & 3u) == 0,
               RT_ERR_UNSUPPORTED, "rt_moe_gather_nvfp4: alignment (16-byte codes and tiles, 4-byte scales)");
    const int64_t smem = 128 * ((cols >> 6) | 1) * 4;
    RT_REQUIRE(smem <= 200 * 1024, RT_ERR_UNSUPPORTED, "rt_moe_gather_nvfp4: cols too large");
    RT_REQUIRE(max_tiles < (1LL << 31), RT_ERR_UNSUPPORTED, "rt_moe_gather_nvfp4: too many tiles");
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&moe_gather_nvfp4_kernel),
                                     static_cast<int>(smem), "rt_moe_gather_nvfp4"))
        return rc;
    moe_gather_nvfp4_kernel<<<static_cast<unsigned>(max_tiles), kGatherThreads, smem,
                              as_stream(stream)>>>(
        (const uint8_t*)codes_in, (const uint8_t*)sf_in, sorted_pairs, (int)topk,
        (uint8_t*)codes_out, (uint8_t*)sf_out, (const int4*)tile_map, tile_count, cols);
    count_launch();
    return check_launch("moe_gather_nvfp4_kernel");
}

extern "C" int rt_index_prep(const void* x, const float* ln_weight, const float* ln_bias,
                             const int64_t* positions, const float* freqs, int64_t table_rows,
                             int64_t rows_per_position, void* codes, float* scales, void* rotated,
                             int64_t rows, int64_t dim, int64_t rope_dim, int64_t x_stride,
                             float eps, int dtype, void* stream) {
    RT_REQUIRE(rows >= 0 && rows_per_position > 0 && table_rows > 0, RT_ERR_BAD_ARG,
               "rt_index_prep: bad shape");
    if (rows == 0) return RT_OK;
    RT_REQUIRE(x && freqs && codes && scales, RT_ERR_BAD_ARG, "rt_index_prep: null pointer");
    RT_REQUIRE((ln_weight == nullptr) == (ln_bias == nullptr), RT_ERR_BAD_ARG,
               "rt_index_prep: LayerNorm weight and bias come together");
    RT_REQUIRE(dtype == RT_BF16, RT_ERR_UNSUPPORTED, "rt_index_prep: only bf16 activations");
    RT_REQUIRE(dim == 128 && rope_dim == 64, RT_ERR_UNSUPPORTED,
               "rt_index_prep: index head dimension 128 with a 64-wide rope slice only");
    RT_REQUIRE(x_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 7u) == 0 &&
                   (reinterpret_cast<uintptr_t>(codes) & 3u) == 0 &&
                   (!rotated || (reinterpret_cast<uintptr_t>(rotated) & 7u) == 0) &&
                   (!ln_weight || (aligned16(ln_weight) && aligned16(ln_bias))) &&
                   (reinterpret_cast<uintptr_t>(freqs) & 7u) == 0,
               RT_ERR_UNSUPPORTED, "rt_index_prep: alignment (8-byte rows, stride %% 4 == 0)");
    RT_REQUIRE(rows < (1LL << 34) && table_rows < (1LL << 31), RT_ERR_UNSUPPORTED,
               "rt_index_prep: tensor too large");
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    cudaStream_t st = as_stream(stream);
    if (ln_weight)
        index_prep_kernel<true><<<grid, 256, 0, st>>>(
            (const __nv_bfloat16*)x, ln_weight, ln_bias, positions, (const float2*)freqs,
            (int)table_rows, (int)rows_per_position, (uint8_t*)codes, scales,
            (__nv_bfloat16*)rotated, rows, x_stride, eps);
    else
        index_prep_kernel<false><<<grid, 256, 0, st>>>(
            (const __nv_bfloat16*)x, nullptr, nullptr, positions, (const float2*)freqs,
            (int)table_rows, (int)rows_per_position, (uint8_t*)codes, scales,
            (__nv_bfloat16*)rotated, rows, x_stride, eps);
    count_launch();
    return check_launch("index_prep_kernel");
}

extern "C" int rt_nvfp4_quant(const void* x, const void* up, const float* amax_in, void* codes,
                              void* block_scales, float* global_scale_out, int64_t rows,
                              int64_t cols, int64_t x_stride, int64_t up_stride, int sf_layout,
                              int dtype, void* stream) {
    uint32_t items, per_row;
    if (int rc = check_stream_args("rt_nvfp4_quant", x, rows, cols, x_stride, 16, dtype, items,
                                   per_row, kItem))
        return rc;
    if (items == 0) return RT_OK;
    RT_REQUIRE(amax_in && codes && block_scales, RT_ERR_BAD_ARG, "rt_nvfp4_quant: null pointer");
    RT_REQUIRE(sf_layout == RT_SF_ROWMAJOR || sf_layout == RT_SF_TILED128x4, RT_ERR_BAD_ARG,
               "rt_nvfp4_quant: bad sf_layout %d", sf_layout);
    RT_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 7u) == 0, RT_ERR_UNSUPPORTED,
               "rt_nvfp4_quant: codes must be 8-byte aligned");
    if (up) RT_REQUIRE(up_stride % 8 == 0 && aligned16(up), RT_ERR_UNSUPPORTED,
                       "rt_nvfp4_quant: up must be 16-byte aligned with stride %% 8 == 0");
    if (items == 0) return RT_OK;
    cudaStream_t st = as_stream(stream);
    const unsigned grid = (items + kActThreads - 1) / kActThreads;
    if (up)
        quant_nvfp4_kernel<true><<<grid, kActThreads, 0, st>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)up, amax_in, (uint8_t*)codes,
            (uint8_t*)block_scales, global_scale_out, items, per_row, x_stride, up_stride, cols,
            sf_layout);
    else
        quant_nvfp4_kernel<false><<<grid, kActThreads, 0, st>>>(
            (const __nv_bfloat16*)x, nullptr, amax_in, (uint8_t*)codes, (uint8_t*)block_scales,
            global_scale_out, items, per_row, x_stride, 0, cols, sf_layout);
    count_launch();
    if (int rc = check_launch("quant_nvfp4_kernel")) return rc;
    if (sf_layout == RT_SF_TILED128x4) {
        const int64_t rows_pad = (rows + 127) / 128 * 128, nblk = cols / 16;
        const int64_t nblk_pad = (nblk + 3) / 4 * 4;
        if (rows_pad != rows || nblk_pad != nblk) {
            sf_pad_kernel<<<148, 256, 0, st>>>((uint8_t*)block_scales, rows, nblk, rows_pad,
                                               nblk_pad);
            count_launch();
            return check_launch("sf_pad_kernel");
        }
    }
    return RT_OK;
}
