/*
 * rt_b200.h - C ABI of librt_b200.so: hand-written sm_100a kernels for the
 * DeepSeek-V3.2 partition hot path of racetrack.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".
 *   - Row-major 2-D tensors; a `*_stride` argument is the distance between two
 *     consecutive rows IN ELEMENTS, so a column slice of a wider matrix (the
 *     q_c / kv_c / k_pe slices of the [T,2112] qkv_a output) needs no copy.
 *   - `dtype` / `weight_dtype` take an rt_dtype tag.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *     Nothing here synchronises, allocates or frees; every call only enqueues
 *     kernels on `stream`, so all entry points are CUDA-graph capturable unless
 *     stated otherwise.
 *   - Return value: RT_OK (0) or a negative rt_status. rt_last_error() returns
 *     a thread-local, human readable description of the last failure.
 *
 * Each entry point names the racetrack interface it stands in for as
 * `ref: <file>:<lines>` (paths inside the racetrack project).
 */
#ifndef RT_B200_H
#define RT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum rt_dtype {
    RT_BF16 = 0,
    RT_F32 = 1,
    RT_F16 = 2
} rt_dtype;

typedef enum rt_status {
    RT_OK = 0,
    RT_ERR_BAD_ARG = -1,      /* null pointer, negative size, bad enum */
    RT_ERR_UNSUPPORTED = -2,  /* shape / dtype / alignment this build does not cover */
    RT_ERR_CUDA = -3,         /* a CUDA runtime call or launch failed */
    RT_ERR_TIMEOUT = -4       /* a bounded device-side wait expired */
} rt_status;

/* Library ABI version (bumped when a signature changes). */
int rt_version(void);

/* Thread-local description of the last non-zero status returned on this thread. */
const char* rt_last_error(void);

/* Number of kernels this library has launched since load (all threads).
 * Lets a harness count launches inside a timed region. */
int64_t rt_launch_count(void);

/* ------------------------------------------------------------------------ */
/* Residual add + RMSNorm                                                     */
/* ------------------------------------------------------------------------ */

/*
 * hidden = update + residual (fp32); normed = weight * (hidden * rsqrt(mean(hidden^2) + eps)),
 * computed from the un-rounded fp32 sum; both outputs rounded to `dtype`.
 * One pass: each input element is read once, each output written once.
 * `normed` and `hidden` are contiguous [rows, cols]. cols % 8 == 0, cols <= 32768.
 * ref: racetrack/models/deepseek.py:485-495 (RMSNorm.forward fallback),
 *      partitions/dsv3_2/a1f6d7e2/kernels/cutedsl/residual_norm.py:47-147 (the op it replaces).
 */
int rt_residual_norm(const void* update, const void* residual,
                     const void* weight, int weight_dtype,
                     void* normed, void* hidden,
                     int64_t rows, int64_t cols,
                     int64_t update_stride, int64_t residual_stride,
                     float eps, int dtype, void* stream);

/*
 * out = (x * rsqrt(mean(x^2) + eps)) * weight, fp32 math, rounded to `dtype`.
 * `out` has row stride `out_stride`. cols % 8 == 0, cols <= 32768.
 * ref: partitions/_base.py:24-28 (rms_norm), racetrack/models/deepseek.py:478-483.
 */
int rt_rms_norm(const void* x, const void* weight, int weight_dtype, void* out,
                int64_t rows, int64_t cols, int64_t x_stride, int64_t out_stride,
                float eps, int dtype, void* stream);

/* ------------------------------------------------------------------------ */
/* MLA prologue: q_a / kv_a RMSNorm fused with RoPE on the k_pe slice         */
/* ------------------------------------------------------------------------ */

/* RoPE conventions */
typedef enum rt_rope_mode {
    RT_ROPE_HALF = 0,        /* [x1*c - x2*s, x2*c + x1*s], x1 = x[:d/2], x2 = x[d/2:];
                                cos/sin rounded to `dtype` and every product/sum rounded to
                                `dtype` like torch eager does on tensors of that dtype.
                                ref: partitions/dsv3_2/model.py:55-81 (apply_rope) */
    RT_ROPE_INTERLEAVED = 1  /* complex multiply of (x[2i], x[2i+1]) by (cos_i, sin_i) in fp32,
                                one rounding at the end.
                                ref: racetrack/models/deepseek.py:604-624 (apply_rotary_emb) */
} rt_rope_mode;

/*
 * One launch per token batch:
 *   q_out  = rms_norm(q_c,  q_weight)   [tokens, q_cols]   contiguous
 *   kv_out = rms_norm(kv_c, kv_weight)  [tokens, kv_cols]  contiguous
 *   k_out  = rope(k_pe)                 [tokens, rope_dim] contiguous
 * Rotation angles:
 *   RT_ROPE_HALF:        `table` = inv_freq fp32 [rope_dim/2]; the kernel forms
 *                        angle = float(positions[t]) * inv_freq[i] and evaluates cosf/sinf.
 *   RT_ROPE_INTERLEAVED: `table` = [table_rows, rope_dim/2] (cos, sin) fp32 pairs, the
 *                        memory image of the complex64 tensor precompute_freqs_cis returns;
 *                        row = positions[t], or t % table_rows when positions is NULL.
 *                        positions must lie in [0, table_rows) when table_rows > 0; values
 *                        outside are clamped to the nearest row (memory-safe, not meaningful).
 * q_cols % 8 == 0, kv_cols % 8 == 0, rope_dim % 2 == 0, rope_dim <= 512.
 * ref: partitions/dsv3_2/model.py:84-99 (fused_norm_rope), :333-344 (its call site),
 *      racetrack/models/deepseek.py:766-776 (q_norm / kv_norm / k_pe rotary in MLA.forward).
 */
int rt_norm_rope(const void* q_c, const void* q_weight,
                 const void* kv_c, const void* kv_weight, int weight_dtype,
                 const void* k_pe, const int64_t* positions,
                 const float* table, int64_t table_rows,
                 void* q_out, void* kv_out, void* k_out,
                 int64_t tokens, int64_t q_cols, int64_t kv_cols, int64_t rope_dim,
                 int64_t q_stride, int64_t kv_stride, int64_t k_stride,
                 float eps, int rope_mode, int dtype, void* stream);

/*
 * RoPE on a [tokens, heads, rope_dim] view: element (t, h, :) starts at
 * x + t*token_stride + h*head_stride (elements); `out` uses out_token_stride /
 * out_head_stride the same way (x == out is allowed: in-place on the q_pe slice of q).
 * positions / table / table_rows as in rt_norm_rope.
 * rope_dim % 16 == 0, rope_dim <= 512; all strides % 8 == 0.
 * ref: racetrack/models/deepseek.py:604-624, :771 (q_pe), racetrack/realistic_bench.py:297-302.
 */
int rt_rope(const void* x, const int64_t* positions, const float* table, int64_t table_rows,
            void* out, int64_t tokens, int64_t heads, int64_t rope_dim,
            int64_t token_stride, int64_t head_stride,
            int64_t out_token_stride, int64_t out_head_stride,
            int rope_mode, int dtype, void* stream);

/*
 * dst[t, h, 0:dim] = src[t, 0:dim] for h in [0, heads): element (t, h, 0) of dst is at
 * dst + t*dst_token_stride + h*dst_head_stride. Writes the rotated k_pe of each token next to
 * every head's k_nope inside the kv_b projection output, so K = [k_nope | k_pe] needs no
 * concatenation. dim % 8 == 0, strides % 8 == 0.
 * ref: racetrack/realistic_bench.py:311, racetrack/models/deepseek.py:785
 *      (k_pe.expand(..., n_local_heads, ...) inside torch.cat).
 */
int rt_head_broadcast(const void* src, void* dst, int64_t tokens, int64_t heads, int64_t dim,
                      int64_t src_stride, int64_t dst_token_stride, int64_t dst_head_stride,
                      int dtype, void* stream);

/* ------------------------------------------------------------------------ */
/* SwiGLU and activation quantisation                                         */
/* ------------------------------------------------------------------------ */

/*
 * out = (silu(gate.float()) * up.float()) rounded to `dtype`; out contiguous [rows, cols].
 * gate and up may be the two halves of one [rows, 2*cols] gate_up matrix (strides = 2*cols).
 * cols % 8 == 0.
 * ref: racetrack/models/deepseek.py:850-851 (MLP fallback), :958-959 (Expert fallback).
 */
int rt_swiglu(const void* gate, const void* up, void* out,
              int64_t rows, int64_t cols, int64_t gate_stride, int64_t up_stride,
              int dtype, void* stream);

/*
 * FP8 e4m3 per-row, per-128-column-group quantisation:
 *   amax = max(|x|) clamped to >= 1e-4; scale = amax / 448 (IEEE division);
 *   code = e4m3_rne(clamp(x / scale, -448, 448)).
 * codes: [rows, cols] bytes (e4m3fn), scales: [rows, cols/128] fp32, both contiguous.
 * cols % 128 == 0.
 * ref: racetrack/models/deepseek.py:85-107 (act_quant).
 */
int rt_act_quant_fp8(const void* x, void* codes, float* scales,
                     int64_t rows, int64_t cols, int64_t x_stride,
                     int dtype, void* stream);

/*
 * h = (silu(gate.float()) * up.float()) rounded to `dtype`, then the FP8 group
 * quantisation of rt_act_quant_fp8 applied to h; h is never written to memory.
 * ref: benchmarks/gsm8k/flat_decode.py:132-136 (SwiGLU -> act_quant composite),
 *      partitions/dsv3_2/3336cdbd/kernels/cutedsl/act_quant.py:96-151 (the op it replaces).
 */
int rt_swiglu_quant_fp8(const void* gate, const void* up, void* codes, float* scales,
                        int64_t rows, int64_t cols, int64_t gate_stride, int64_t up_stride,
                        int dtype, void* stream);

/*
 * Tensor-wide max(|x|) (optionally of h = swiglu(gate, up) when `up` is non-NULL,
 * `x` then being the gate). Writes one fp32 to *amax_out. The kernel clears
 * *amax_out itself (a first tiny launch), so no host memset is needed.
 * No counterpart in racetrack: NVFP4 exists there only as a model label.
 */
int rt_absmax(const void* x, const void* up, float* amax_out,
              int64_t rows, int64_t cols, int64_t x_stride, int64_t up_stride,
              int dtype, void* stream);

/*
 * rt_absmax restricted to rows [*row_begin, *row_end) (device int32 values, NULL = no bound):
 * the rows of the sorted MoE buffer that an expert-parallel rank actually wrote.
 * No counterpart in racetrack.
 */
int rt_absmax_rows(const void* x, const void* up, float* amax_out,
                   int64_t rows, int64_t cols, int64_t x_stride, int64_t up_stride,
                   const int32_t* row_begin, const int32_t* row_end, int dtype, void* stream);

/*
 * rt_absmax_rows over h = bf16(silu(gate) * up) that also WRITES h (bf16 [rows, cols], row pitch
 * h_stride; rows outside the window are left untouched): the expert MLP needs max |h| before it
 * can quantise h to NVFP4, and this way SwiGLU (an expf and an IEEE division per element) is
 * evaluated once instead of once per pass.
 * ref: racetrack/models/deepseek.py:958-959 (F.silu(w1(x)) * w3(x)).
 */
int rt_swiglu_absmax_rows(const void* gate, const void* up, void* h, float* amax_out,
                          int64_t rows, int64_t cols, int64_t gate_stride, int64_t up_stride,
                          int64_t h_stride, const int32_t* row_begin, const int32_t* row_end,
                          int dtype, void* stream);

/* Block-scale layouts for NVFP4 */
typedef enum rt_sf_layout {
    RT_SF_ROWMAJOR = 0,   /* [rows, cols/16] bytes */
    RT_SF_TILED128x4 = 1  /* the 128-row x 4-block tile the tcgen05 block-scaled MMA reads:
                             byte offset of (row r, block b) =
                             ((r/128) * ceil(nblk/4) + b/4) * 512 + (r%32)*16 + ((r%128)/32)*4 + b%4 */
} rt_sf_layout;

/*
 * NVFP4 quantisation: 16-element blocks along a row, e2m1 codes (two per byte,
 * element 2i in the low nibble), e4m3 block scale, fp32 tensor-wide global scale.
 *   gs   = amax / 2688            (2688 = 448 * 6; gs := 1 when amax == 0), read from *amax_in
 *   bs   = e4m3_rne(min(block_amax / (6 * gs), 448))
 *   code = e2m1_rne_sat(x / (gs * float(bs)))   (0 when bs == 0)
 * `amax_in` is a device fp32 (from rt_absmax or a calibrated constant).
 * When `up` is non-NULL the quantised tensor is h = bf16(silu(x) * up) (x = gate).
 * codes: [rows, cols/2] bytes contiguous; block_scales per `sf_layout`.
 * global_scale_out (device fp32, may be NULL) receives gs.
 * cols % 16 == 0 (RT_SF_TILED128x4: the scale buffer must hold
 * ceil(rows/128)*ceil(cols/64)*512 bytes; padding entries are written as 0).
 * No counterpart in racetrack (see rt_absmax).
 */
int rt_nvfp4_quant(const void* x, const void* up, const float* amax_in,
                   void* codes, void* block_scales, float* global_scale_out,
                   int64_t rows, int64_t cols, int64_t x_stride, int64_t up_stride,
                   int sf_layout, int dtype, void* stream);

/*
 * NVFP4 quantisation of the rows a grouped-GEMM tile map covers (see rt_moe_tile_map):
 * codes [*, cols/2] are written at the tiles' (compact) rows, block scales into the
 * RT_SF_TILED128x4 layout with row tile = the tile map's scale row-tile index, so each expert
 * segment starts on a scale-tile boundary; rows of a tile beyond its valid rows get zero scales.
 * With sorted_pairs != NULL the source row of destination row r is sorted_pairs[r] / topk:
 * the token gather of the MoE dispatch is fused into the quantiser (x is the un-permuted
 * [tokens, cols] activation). With up != NULL the quantised values are swiglu(x, up) and rows
 * are taken as they are. block_scales must hold max_tiles * (cols/64) * 512 bytes.
 * cols % 64 == 0. Arithmetic as rt_nvfp4_quant.
 * ref: racetrack/models/deepseek.py:1017 (x[idx] gather); NVFP4 has no counterpart in racetrack.
 */
int rt_moe_quant_nvfp4(const void* x, const void* up, const int32_t* sorted_pairs, int64_t topk,
                       const float* amax_in, void* codes, void* block_scales,
                       float* global_scale_out, const int32_t* tile_map,
                       const int32_t* tile_count, int64_t max_tiles, int64_t cols,
                       int64_t x_stride, int64_t up_stride, int dtype, void* stream);

/*
 * MoE dispatch of token rows that are already NVFP4 (quantised ONCE per token with
 * rt_nvfp4_quant, RT_SF_ROWMAJOR scales): for every 128-row tile of the tile map, copies the
 * rows its sorted (token, slot) pairs name (source row = sorted_pairs[r] / topk) -- codes
 * [tokens, cols/2] -> codes_out at the tiles' compact rows, scales [tokens, cols/16] -> sf_out
 * in the RT_SF_TILED128x4 layout with row tile = the tile map's scale row-tile index, zeros for
 * rows past a tile's valid rows. Same result as rt_moe_quant_nvfp4 with sorted_pairs (the
 * quantisation is per row), without reading the bf16 rows topk times. cols % 64 == 0;
 * sf_out must hold max_tiles * (cols/64) * 512 bytes.
 * ref: racetrack/models/deepseek.py:1017 (x[idx] gather); NVFP4 has no counterpart in racetrack.
 */
int rt_moe_gather_nvfp4(const void* codes_in, const void* sf_in, const int32_t* sorted_pairs,
                        int64_t topk, void* codes_out, void* sf_out, const int32_t* tile_map,
                        const int32_t* tile_count, int64_t max_tiles, int64_t cols, void* stream);

/* ------------------------------------------------------------------------ */
/* MoE routing and token permutation                                          */
/* ------------------------------------------------------------------------ */

typedef enum rt_score_func {
    RT_SCORE_SIGMOID = 0,
    RT_SCORE_SOFTMAX = 1,
    RT_SCORE_TOPK_SOFTMAX = 2  /* top-k on the raw logits, weights = softmax over the selected
                                  logits rounded to bf16 (no bias, no groups);
                                  ref: racetrack/realistic_bench.py:321-327 */
} rt_score_func;

/*
 * Grouped top-k routing on fp32 router logits [tokens, n_experts] (row stride
 * logits_stride): scores = sigmoid|softmax(logits); biased = scores + bias
 * (bias may be NULL); experts are split into n_groups contiguous groups, a
 * group's score is the sum of its two largest biased scores (the max when bias
 * is NULL); only the topk_groups best groups stay eligible; the topk largest
 * biased scores among them are selected, in descending order (ties: lowest
 * expert id). weights = unbiased scores of the selected experts, divided by
 * their sum when score_func is sigmoid, times route_scale.
 * weights_out: [tokens, topk] fp32; indices_out: [tokens, topk] int64.
 * n_experts <= 512, n_experts % n_groups == 0, topk <= 32.
 * ref: racetrack/models/deepseek.py:888-920 (Gate.forward, after the logits GEMM at :898).
 */
int rt_moe_route(const float* logits, const float* bias,
                 float* weights_out, int64_t* indices_out,
                 int64_t tokens, int64_t n_experts, int64_t logits_stride,
                 int64_t n_groups, int64_t topk_groups, int64_t topk,
                 float route_scale, int score_func, void* stream);

/*
 * Stable counting sort of the tokens*topk (token, slot) pairs by expert id.
 *   expert_offsets [n_experts + 1] int32: pairs of expert e occupy sorted positions
 *                   [expert_offsets[e], expert_offsets[e+1])
 *   sorted_pairs   [tokens*topk] int32: pair id p = token*topk + slot, grouped by expert,
 *                   ascending p inside an expert (the order torch.where(indices == e) yields)
 *   pair_pos       [tokens*topk] int32: inverse map, sorted position of pair p
 * workspace: caller-provided device scratch of rt_moe_permute_workspace_bytes() bytes.
 * ref: racetrack/models/deepseek.py:1011-1018 (bincount + per-expert torch.where loop).
 */
int64_t rt_moe_permute_workspace_bytes(int64_t tokens, int64_t topk, int64_t n_experts);
int rt_moe_permute(const int64_t* indices, int32_t* expert_offsets,
                   int32_t* sorted_pairs, int32_t* pair_pos, void* workspace,
                   int64_t tokens, int64_t topk, int64_t n_experts, void* stream);

/*
 * rt_moe_permute for callers that have no scratch memory to hand over and must not trigger
 * an allocation: a host that pre-sized one device arena at start-up and gives plugins no
 * allocator, or an operator signature that carries inputs and outputs only. Same inputs,
 * outputs and results as rt_moe_permute; the per-block histogram lives in a fixed 256 KiB
 * array inside the library image (every GPU that loads the library holds it until exit).
 * This entry point has no counterpart in racetrack.
 *   - Limit: ceil(tokens*topk / 1024) * n_experts <= rt_moe_permute_static_max_ints() (65536),
 *     e.g. 32 768 pairs with 256 experts. Larger problems are refused with RT_ERR_UNSUPPORTED;
 *     use rt_moe_permute with a workspace for them.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins.
 *   - All calls on a device share the one array, which keeps the previous call's contents.
 *     Nothing in it has to be cleared (each call overwrites the region it reads), but two
 *     calls whose kernels overlap on the GPU (different streams, or concurrent host threads)
 *     race on it: serialise them.
 */
int64_t rt_moe_permute_static_max_ints(void);
int rt_moe_permute_static(const int64_t* indices, int32_t* expert_offsets,
                          int32_t* sorted_pairs, int32_t* pair_pos,
                          int64_t tokens, int64_t topk, int64_t n_experts, void* stream);

/*
 * Row gather: out[i, :] = x[sorted_pairs[i] / topk, :] for i in [0, n_pairs).
 * cols % 8 == 0. Used to lay tokens out expert-by-expert for the grouped GEMM.
 * ref: racetrack/models/deepseek.py:1017 (x[idx] inside the expert loop).
 */
int rt_moe_gather(const void* x, const int32_t* sorted_pairs, void* out,
                  int64_t n_pairs, int64_t topk, int64_t cols, int64_t x_stride,
                  int dtype, void* stream);

/*
 * Weighted combine: y[t, :] = sum_s weights[t, s] * expert_out[pair_pos[t*topk + s], :]
 * (+ shared[t, :] when `shared` is non-NULL), fp32 accumulation in slot order.
 * expert_out and shared are bf16; `dtype` is the type of y: RT_BF16 (rounded once) or RT_F32
 * (the fp32 sums, which an expert-parallel rank all-reduces before the cast, as the reference
 * does with its fp32 y). Pairs whose sorted position lies outside
 * [pos_begin, pos_end) are skipped (expert-parallel ranks own a slice of the
 * sorted range); pos_begin_ptr / pos_end_ptr, when non-NULL, are device int32 values that
 * override the host ones (entries of expert_offsets, so no host read-back is needed).
 * cols % 8 == 0.
 * ref: racetrack/models/deepseek.py:1018-1022 (y[idx] += expert(x[idx]) * weights[idx, top]; y += shared).
 */
int rt_moe_combine(const void* expert_out, const int32_t* pair_pos, const float* weights,
                   const void* shared, void* y,
                   int64_t tokens, int64_t topk, int64_t cols,
                   int64_t pos_begin, int64_t pos_end,
                   const int32_t* pos_begin_ptr, const int32_t* pos_end_ptr,
                   int dtype, void* stream);

/* ------------------------------------------------------------------------ */
/* Tensor-core GEMMs (tcgen05 + TMA + tensor memory)                          */
/* ------------------------------------------------------------------------ */

/*
 * c[m, n] = a[m, k] * b[n, k]^T, bf16 inputs, fp32 accumulation in tensor memory, bf16
 * output: y = F.linear(x, weight) with x = a and weight = b. lda / ldb / ldc are row
 * pitches in elements. k, n and the pitches must be multiples of 8, pointers 16-byte aligned.
 * out_dtype RT_BF16 rounds the result to bf16; RT_F32 stores the fp32 accumulators, which is
 * how the router logits x.float() @ W.float()^T of bf16-valued operands are formed (every
 * product is exact in fp32, only the summation order differs from an fp32 GEMM).
 * ref: racetrack/models/deepseek.py:341-342 (bf16 branch of linear()), :898 (Gate logits),
 *      racetrack/realistic_bench.py:288,295,307,315,321 (F.linear of the MLA projections, router).
 */
int rt_gemm_bf16(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                 int64_t lda, int64_t ldb, int64_t ldc, int out_dtype, void* stream);

/*
 * `batch` independent products c[i] = a[i] . b[i]^T of one shape in one launch: a[i] is [m, k] at
 * a + i * a_batch_stride (row pitch lda), b[i] is [n, k] at b + i * b_batch_stride (row pitch
 * ldb), c[i] is [m, n] bf16 at c + i * c_batch_stride (row pitch ldc); all bf16, strides in
 * elements (multiples of 8), so the operands may be per-head slices of [tokens, heads, dim]
 * tensors. The per-head absorbed projections of the MLA decode branch:
 * ref: racetrack/models/deepseek.py:799 (einsum "bshd,hdc->bshc" of q_nope with wkv_b[:, :nope]),
 *      :810 (einsum "bshc,hdc->bshd" of the attention output with wkv_b[:, -v_head_dim:]).
 */
int rt_gemm_bf16_batched(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
                         int64_t k, int64_t lda, int64_t a_batch_stride, int64_t ldb,
                         int64_t b_batch_stride, int64_t ldc, int64_t c_batch_stride, void* stream);

/*
 * The same product for FEW rows (decode: m up to a few dozen tokens), where a projection has too
 * few output tiles to occupy the GPU although its whole weight matrix must be streamed: the K
 * range is cut into `splits` pieces, work item (tile, split) stores its partial product into
 * slab `split` of `workspace` (fp32 [splits, m, ldw], caller-provided scratch, no initialisation
 * needed), and a second kernel adds the slabs in split order and writes out [m, n] (row pitch
 * ldo) as RT_BF16 (one rounding of the fp32 sum, as a single-pass GEMM does) or RT_F32.
 * The summation order is fixed, so the result is bit-reproducible from run to run and equal
 * on every rank that computes it from the same operands. splits =
 * rt_gemm_bf16_splitk_splits(m, n, k).
 * ref: racetrack/models/deepseek.py:316-345 (linear with bf16 weights -> F.linear).
 */
int64_t rt_gemm_bf16_splitk_splits(int64_t m, int64_t n, int64_t k);
int rt_gemm_bf16_splitk(const void* a, const void* b, float* workspace, void* out, int64_t m,
                        int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldw, int64_t ldo,
                        int64_t splits, int out_dtype, void* stream);

/*
 * FP8 e4m3 GEMM with DeepSeek block scales, bf16 output:
 *   c[m, n] = sum_kb (a[m, kb] . b[n, kb]) * a_scales[m, kb] * b_scales[n / 128, kb]
 * a [m, k] and b [n, k] are e4m3fn bytes (row pitches lda / ldb in bytes = elements);
 * a_scales fp32 [m, k/128] (what rt_act_quant_fp8 writes), b_scales fp32 [ceil(n/128), k/128]
 * (one scale per 128 x 128 weight block). Products are summed per 128-wide K block on
 * tcgen05 (kind::f8f6f4) and folded, scaled, into fp32 accumulators.
 * k % 128 == 0, n % 8 == 0, lda / ldb % 16 == 0, ldc % 8 == 0.
 * ref: racetrack/models/deepseek.py:30-82 (_fp8_gemm_kernel), :110-145 (fp8_gemm), :316-345 (linear).
 */
int rt_gemm_fp8(const void* a, const float* a_scales, const void* b, const float* b_scales,
                void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                void* stream);

/*
 * Work lists of the grouped GEMM, built on the device from the per-expert row offsets
 * that rt_moe_permute wrote (no host synchronisation). For groups g in [g_begin, g_end),
 * rows [offsets[g], offsets[g+1]) are cut into m-tiles of 128 rows:
 *   tile_map   int32 [2 * max_tiles, 4], 16-byte aligned. Entries [0, tile_count[0]):
 *              {g - g_begin, first row, valid rows (<= 128), scale row-tile index}; the scale
 *              row-tile index equals the tile's own index, so every group starts on a 128-row
 *              scale-tile boundary. Entries [max_tiles, max_tiles + tile_count[1]): the same
 *              rows cut into tiles of up to 256 rows, {g - g_begin, first row, valid rows
 *              (<= 256), scale row-tile index of the first 128 rows}, the work list of the
 *              CTA-pair schedule of rt_gemm_nvfp4_grouped
 *   tile_base  int32 [g_end - g_begin + 1]: index of each group's first tile; last = total
 *   tile_count int32 [2]: number of 128-row tiles and of 256-row tiles written (each
 *              clamped to max_tiles)
 * max_tiles >= ceil(rows/128) + number of groups is always enough.
 * ref: racetrack/models/deepseek.py:1012-1017 (the per-expert loop bounds this replaces).
 */
int rt_moe_tile_map(const int32_t* offsets, int64_t g_begin, int64_t g_end,
                    int32_t* tile_map, int32_t* tile_base, int32_t* tile_count,
                    int64_t max_tiles, void* stream);

/*
 * Block-scaled NVFP4 grouped GEMM on tcgen05 (kind::mxf4nvf4, scale factors in tensor memory):
 *   c[rows of tile t, :] = a_gs[0] * b_gs[g] * dequant(a)[rows] * dequant(b_g)^T,  g = tile group
 * a_codes [total_rows, k/2] e2m1 pairs (even element in the low nibble), rows grouped as the
 * tile map says; a_sf: e4m3 block scales (16 elements) in the RT_SF_TILED128x4 layout, row tile
 * = the tile map's scale row-tile index; b_codes [groups * n, k/2] and b_sf (each group tiled
 * on its own, ceil(n/128) row tiles per group) hold the weights; a_gs / b_gs [groups] are the
 * fp32 global scales (device memory). c is bf16 [total_rows, n] with row pitch ldc.
 * tile_map / tile_count / max_m_tiles: as rt_moe_tile_map wrote them with max_tiles =
 * max_m_tiles (both halves of the map are needed: the schedule picks its own work list).
 * With groups == 1 and a tile map over [0, m) this is a dense NVFP4 linear layer.
 * k % 256 == 0, n % 8 == 0 (n % 128 == 0 when groups > 1).
 * Default schedule: CTA pairs (cta_group::2). 256 weight rows per pair are the MMA's M, up to
 * 256 token rows of one group its N (rounded up to 16 only), each CTA fetching half of the
 * token rows; 1.9 x the flops per byte brought into an SM of the single-CTA 128 x 128 tiling.
 * ref: racetrack/models/deepseek.py:1013-1018 (expert(x[idx]) per routed expert),
 *      racetrack/realistic_bench.py:338-346 (gathered-weight bmm it replaces). The NVFP4
 *      arithmetic itself has no counterpart in racetrack.
 */
int rt_gemm_nvfp4_grouped(const void* a_codes, const void* a_sf, const float* a_gs,
                          const void* b_codes, const void* b_sf, const float* b_gs,
                          void* c, const int32_t* tile_map, const int32_t* tile_count,
                          int64_t max_m_tiles, int64_t total_rows, int64_t groups,
                          int64_t n, int64_t k, int64_t ldc, void* stream);

/*
 * Schedule of rt_gemm_bf16 for this process: 0 = default (CTA pairs with 256 x 256 tiles when
 * k % 64 == 0 and ceil(m/256) * ceil(n/256) is at least half the SM count, else single-CTA
 * 128 x 256 tiles), 1 = single-CTA, 2 = CTA pairs wherever k % 64 == 0. Returns the previous
 * value; any other argument only queries. No counterpart in racetrack.
 */
int rt_gemm_bf16_schedule(int schedule);

/*
 * Schedule of rt_gemm_nvfp4_grouped for this process: 0 = default (CTA pairs, unless
 * max_m_tiles * ceil(n/256) is below the SM count or total_rows < 128 * groups: then
 * single-CTA tiles), 1 = single-CTA
 * 128 x 128 tiles, 2 = CTA pairs. Returns the previous value; any other argument only queries.
 * For A/B measurements and tests. No counterpart in racetrack.
 */
int rt_gemm_nvfp4_schedule(int schedule);

/*
 * Indexer prologue, one pass per 128-wide row (an index head of a query, or a key):
 *   [LayerNorm(weight, bias, eps) when ln_weight != NULL]  -> bf16
 *   RoPE on the first 64 dims, non-interleaved pairs (i, i + 32), complex product with
 *   freqs[position][i] (freqs: fp32 [table_rows, 32, 2] = view_as_real of freqs_cis)   -> bf16
 *   Hadamard rotation x . H_128 * 128^-0.5 (Sylvester order, fp32 butterflies)          -> bf16
 *   act_quant with one 128-wide group: codes e4m3 [rows, 128], scales fp32 [rows].
 * The position of row r is positions[r / rows_per_position] (positions int64, may be NULL:
 * then r / rows_per_position itself); rows_per_position = index heads for queries, 1 for keys.
 * Positions must lie in [0, table_rows); values outside are clamped to the nearest table row
 * (memory-safe, not meaningful).
 * rotated (bf16 [rows, 128], may be NULL) receives the tensor that is quantised.
 * dim == 128, rope_dim == 64.
 * ref: racetrack/models/deepseek.py:659-676 (Indexer.forward: k_norm, apply_rotary_emb(...,
 *      False), rotate_activation, act_quant), :508-520 (LayerNorm), :627-631 (rotate_activation:
 *      fast_hadamard_transform, a third-party package racetrack does not vendor).
 */
int rt_index_prep(const void* x, const float* ln_weight, const float* ln_bias,
                  const int64_t* positions, const float* freqs, int64_t table_rows,
                  int64_t rows_per_position, void* codes, float* scales, void* rotated,
                  int64_t rows, int64_t dim, int64_t rope_dim, int64_t x_stride, float eps,
                  int dtype, void* stream);

/*
 * Index scores of the sparse-attention indexer (tcgen05, FP8 x FP8, fp32 accumulate):
 *   scores[m, n] = k_scale[n] * sum_h weights[m, h] * relu(q[m, h, :] . k[n, :])
 * q e4m3 [queries, heads, dim], k e4m3 [keys, dim] (both contiguous), weights fp32 [queries,
 * heads] (per-head weight times the query's quantisation scale and the softmax scale),
 * k_scale fp32 [keys], scores fp32 [queries, keys] with row pitch score_stride.
 * causal_offset >= 0: key n is visible to query m iff n <= m + causal_offset, other scores are
 * written as -inf (the reference adds a -inf mask, deepseek.py:681-682); causal_offset < 0:
 * no mask. dim == 128; heads in {16, 32, 64, 128}.
 * ref: racetrack/models/deepseek.py:164-176 (fp8_index), :677-682 (Indexer.forward).
 */
int rt_fp8_index(const void* q, const float* weights, const void* k, const float* k_scale,
                 float* scores, int64_t queries, int64_t heads, int64_t keys, int64_t dim,
                 int64_t score_stride, int64_t causal_offset, void* stream);

/*
 * The same for `batch` sequences with caches of their own (a decode step: one query per
 * sequence): q e4m3 [batch, queries, heads, dim] contiguous, weights fp32 [batch, queries,
 * heads], k e4m3 [batch, keys, dim] with k_batch_stride ROWS between sequences (the cache may be
 * longer than `keys`), k_scale fp32 with ks_batch_stride elements between sequences, scores
 * fp32 [batch, queries, keys] with score_stride / score_batch_stride elements between rows /
 * sequences. One launch; the mask is that of rt_fp8_index within each sequence.
 * ref: racetrack/models/deepseek.py:656-686 (Indexer.forward with bsz > 1).
 */
int rt_fp8_index_batched(const void* q, const float* weights, const void* k, const float* k_scale,
                         float* scores, int64_t batch, int64_t queries, int64_t heads,
                         int64_t keys, int64_t dim, int64_t score_stride, int64_t causal_offset,
                         int64_t k_batch_stride, int64_t ks_batch_stride,
                         int64_t score_batch_stride, void* stream);

/*
 * Top-k selection of the indexer: indices [queries, topk] (int32) of the topk largest scores
 * of every row, written in ascending index order; among scores equal to the k-th largest the
 * lower indices are taken. Exact (radix select on the ordered bit patterns), -inf allowed.
 * topk <= keys. The reference consumes the indices as a set (deepseek.py:683, :757-759).
 * ref: racetrack/models/deepseek.py:683 (index_score.topk).
 */
int rt_index_topk(const float* scores, int32_t* indices, int64_t queries, int64_t keys,
                  int64_t score_stride, int64_t topk, void* stream);

/*
 * Sparse multi-query attention of the MLA decode step (tcgen05): for every sequence b and head h
 *   s_j      = softmax_scale * (q_abs[b, h, :] . kv[b, i_j, :] + q_pe[b, h, :] . pe[b, i_j, :])
 *   out[b, h] = sum_j softmax(s)_j * kv[b, i_j, :]          i_j = indices[b, j], j < n_sel
 * i.e. the decode branch of MLA.forward with the indexer's mask (0 on the selected keys, -inf
 * elsewhere) applied by visiting only the selected cache rows. q_abs is q_nope times the key
 * half of wkv_b (bf16 [batch, heads, 512], strides in elements), q_pe bf16 [batch, heads, 64],
 * kv the latent cache bf16 [batch, keys, 512], pe the rope cache bf16 [batch, keys, 64], indices
 * int32 [batch, n_sel] (entries < 0 or >= keys are skipped; NULL: all keys, n_sel == keys), out
 * bf16 [batch, heads, 512] contiguous (the caller applies the value half of wkv_b).
 * splits = rt_mla_sparse_decode_splits(batch, heads, n_sel) partial results are merged by a
 * second kernel; the caller provides part_o fp32 [batch * splits * heads * 512] and part_ml fp32
 * [batch * splits * heads * 2]. heads: a multiple of 8 up to 64, or a multiple of 64; all strides multiples
 * of 8 elements; pointers 16-byte aligned. No allocation, no host synchronisation.
 * ref: racetrack/models/deepseek.py:793-810 (MLA.forward, "MQA decode").
 */
int64_t rt_mla_sparse_decode_splits(int64_t batch, int64_t heads, int64_t n_sel);
int rt_mla_sparse_decode(const void* q_abs, const void* q_pe, const void* kv, const void* pe,
                         const int32_t* indices, void* out, float* part_o, float* part_ml,
                         int64_t batch, int64_t heads, int64_t keys, int64_t n_sel,
                         int64_t qa_batch_stride, int64_t qa_head_stride,
                         int64_t qp_batch_stride, int64_t qp_head_stride,
                         int64_t kv_batch_stride, int64_t kv_row_stride,
                         int64_t pe_batch_stride, int64_t pe_row_stride,
                         int64_t idx_batch_stride, int64_t splits, float softmax_scale,
                         void* stream);

/*
 * Causal attention of the prefill stack on the tensor cores (flash-style: scores and
 * probabilities never leave the SM):
 *   out[t, h, :] = sum_{j <= t} softmax_j(softmax_scale * q[t, h, :] . key[j, h, :]) * v[j, h, :]
 * where key[j, h] = [k_nope[j, h, :nope_dim] | k_pe[j, (h), :rope_dim]] and q[t, h] =
 * [q_nope | q_pe] with the same split. All operands bf16, strides in elements (multiples of 8),
 * so q / k_nope / v may be column slices of wider projection outputs. kp_head_stride == 0 means
 * one rope key per token shared by all heads (MLA: the k_pe broadcast of the reference's
 * torch.cat is never materialised); rope_dim == 0 means the key is k_nope alone (k_pe may be
 * NULL). fp32 scores / softmax / accumulation, probabilities rounded to bf16 before they
 * multiply v, as the reference's probs.to(v.dtype).
 * nope_dim <= 128, rope_dim <= 64, v_dim <= 128, each a multiple of 8.
 * ref: racetrack/runtime/torch_ops.py:97-110 (causal_attention),
 *      racetrack/realistic_bench.py:304-313 (q / k / v of the synthetic layer),
 *      racetrack/models/deepseek.py:780-792 (MHA prefill of MLA.forward).
 */
/* Selects the schedule of rt_attn_causal_prefill for this process and returns the previous
 * setting: 0 = by shape and length (default), 1 = one CTA per 256 query rows with key tiles of
 * 128, 2 = CTA pairs (tcgen05 cta_group::2, 256 query rows per pair, key tiles of 256) wherever
 * the head shape is 128 + 64 / 128. */
int rt_attn_prefill_schedule(int schedule);
int rt_attn_causal_prefill(const void* q, const void* k_nope, const void* k_pe, const void* v,
                           void* out, int64_t tokens, int64_t heads, int64_t nope_dim,
                           int64_t rope_dim, int64_t v_dim,
                           int64_t q_token_stride, int64_t q_head_stride,
                           int64_t kn_token_stride, int64_t kn_head_stride,
                           int64_t kp_token_stride, int64_t kp_head_stride,
                           int64_t v_token_stride, int64_t v_head_stride,
                           int64_t o_token_stride, int64_t o_head_stride,
                           float softmax_scale, void* stream);

/*
 * The same attention with the epilogue of its consumer fused in: instead of the bf16 output the
 * kernel writes act_quant(output) (racetrack/models/deepseek.py:85-107), FP8 e4m3 codes
 * out_codes [tokens, heads * 128] and fp32 scales out_scales [tokens, heads] (a 128-wide
 * quantisation group is one head's value dims), bit for bit what rt_act_quant_fp8 makes of the
 * bf16 output of rt_attn_causal_prefill: the input of an FP8 output projection
 * (racetrack/models/deepseek.py:343-345 applied to w_o) without the [tokens, heads * 128] bf16
 * round trip. Head shape 128 + 64 / 128 only (the CTA-pair schedule).
 */
int rt_attn_causal_prefill_fp8(const void* q, const void* k_nope, const void* k_pe, const void* v,
                               void* out_codes, float* out_scales, int64_t tokens, int64_t heads,
                               int64_t nope_dim, int64_t rope_dim, int64_t v_dim,
                               int64_t q_token_stride, int64_t q_head_stride, int64_t kn_token_stride,
                               int64_t kn_head_stride, int64_t kp_token_stride, int64_t kp_head_stride,
                               int64_t v_token_stride, int64_t v_head_stride, float softmax_scale,
                               void* stream);

/* ------------------------------------------------------------------------ */
/* Collective steps over NVLink peer memory (one process per GPU)              */
/* ------------------------------------------------------------------------ */

/*
 * Exchange buffers of a rank group. rt_peer_alloc: `bytes` of zeroed device memory on the
 * current device (cudaMalloc) and its 64-byte CUDA IPC handle; the handle travels to the other
 * ranks by any host channel. rt_peer_open: maps a peer's buffer into this process WITH THE
 * CALLER'S OWN DEVICE CURRENT and returns a pointer kernels of that device may dereference
 * (peer access over NVLink). rt_peer_close unmaps it, rt_peer_free releases an own buffer
 * (after every peer has closed it). Set-up time calls: they allocate and synchronise.
 * ref: none in racetrack (its collectives are torch.distributed calls); the buffers replace the
 * NCCL staging of the all-reduces at racetrack/realistic_bench.py:315-316,351.
 */
int rt_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle_out);
int rt_peer_open(const unsigned char* handle, void** ptr);
int rt_peer_close(void* ptr);
int rt_peer_free(void* ptr);

/*
 * Device-side barrier of `world` ranks (<= 8). flag_ptrs[q] is rank q's flag array (int32
 * [world + 1], zero at start) as mapped into THIS process (rt_peer_open; flag_ptrs[rank] is the
 * local one). The kernel counts its own barriers in the last slot of the local array, stores
 * that count into slot `rank` of every rank's array and waits until all slots of its own array
 * have reached it; every rank must call the barrier the same number of times. What a rank
 * wrote on `stream` before the barrier is visible to every rank after it. The wait is bounded
 * (about two seconds): a rank that never arrives makes the others record an error, which
 * rt_peer_error_state() reports, instead of hanging them.
 * ref: the rendezvous inside dist.all_reduce of racetrack/realistic_bench.py:315-316,351.
 */
int rt_peer_barrier(int* const* flag_ptrs, int64_t rank, int64_t world, void* stream);
int rt_peer_error_state(void);

/*
 * Reduce-scatter fused with residual add + RMSNorm: for rows [row0, row0 + rows) of the
 * [T, cols] bf16 partial sums that every rank holds (partial_ptrs[q] = rank q's buffer as
 * mapped into this process, row pitch partial_stride elements),
 *   update = bf16(sum over ranks, fp32, rank order)        (what the all-reduce would leave)
 *   hidden = bf16(update + residual)    normed = bf16(weight * (hidden_fp32 * rsqrt(mean^2 + eps)))
 * exactly as rt_residual_norm computes them from `update`. residual / normed / hidden hold
 * only this rank's `rows` rows. Peer memory is read with plain loads over NVLink; call
 * rt_peer_barrier first so that all ranks have finished writing their partial sums.
 * ref: racetrack/realistic_bench.py:315-316,351 (all_reduce SUM) followed by :375-389
 *      (residual add, rms_norm); racetrack/models/deepseek.py:485-495.
 */
int rt_peer_reduce_residual_norm(const void* const* partial_ptrs, int64_t world, int64_t row0,
                                 int64_t partial_stride, const void* residual, const void* weight,
                                 int weight_dtype, void* normed, void* hidden, int64_t rows,
                                 int64_t cols, int64_t residual_stride, float eps, void* stream);

/*
 * All-gather of row-sharded buffers over peer memory: every rank has written its own block
 * (bytes [rank * slice_bytes[b], (rank + 1) * slice_bytes[b]) of buffer b) into its own copy;
 * the call copies the other ranks' blocks out of their copies (peer_ptrs[b * world + q] = buffer
 * b of rank q as mapped into this process) into the local copy, so that afterwards the local
 * buffer holds all blocks. Up to 4 buffers per call, one launch. Call rt_peer_barrier first.
 * Peer memory is read with plain loads over NVLink.
 * ref: the all-gather half of the reference's all-reduce, racetrack/realistic_bench.py:315-316,351,
 *      moved behind the token-wise kernels (RMSNorm, router, quantisation) that follow it.
 */
int rt_peer_gather(const void* const* peer_ptrs, const int64_t* slice_bytes, int64_t n_buffers,
                   int64_t rank, int64_t world, void* stream);

/*
 * The transposing exchange in front of a row-sharded consumer: buffer b of rank q
 * (peer_ptrs[b * world + q], as mapped into this process) holds that rank's column block
 * [T, src_row_bytes[b]] of a [T, world * src_row_bytes[b]] byte matrix for ALL rows; the call
 * assembles this rank's rows of the whole matrix:
 *   dst_b[r, q * src_row_bytes[b] + c] = src_b,q[row0 + r, c]        r < rows
 * dst_ptrs[b] is local memory of rows * world * src_row_bytes[b] bytes. Up to 4 buffers per call,
 * one launch; call rt_peer_barrier first.
 * ref: replaces the all-reduce after the head-sharded output projection,
 *      racetrack/realistic_bench.py:314-316: every rank gathers all heads' attention outputs (FP8
 *      codes + scales, or bf16) for ITS rows and applies the whole w_o to them, so the sum over
 *      heads happens inside one GEMM instead of across ranks.
 */
int rt_peer_gather_cols(const void* const* peer_ptrs, void* const* dst_ptrs, const int64_t* src_row_bytes,
                        int64_t n_buffers, int64_t row0, int64_t rows, int64_t world, void* stream);

/*
 * out[0] = max over ranks of the non-negative fp32 value each rank has stored at slot_ptrs[q]
 * (rank q's slot as mapped into this process). Call rt_peer_barrier first. The tensor-wide amax
 * behind one NVFP4 global scale for all ranks' rows; no counterpart in the reference (it has
 * no NVFP4 arithmetic), it stands where a 4-byte all-reduce MAX would.
 */
int rt_peer_allmax(const void* const* slot_ptrs, int64_t world, float* out, void* stream);

/*
 * Synchronous: reads (and clears) the device-side flag that a tensor-core kernel sets when
 * one of its bounded waits expired. RT_OK when no kernel gave up since the last call,
 * RT_ERR_TIMEOUT otherwise. Call after synchronising the stream; not graph-capturable.
 */
int rt_tc_error_state(void);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
