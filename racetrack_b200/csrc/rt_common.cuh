// Shared device/host helpers for librt_b200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/rt_b200.h"

namespace rt {

// ---------------------------------------------------------------------------
// Host side: error reporting and launch accounting
// ---------------------------------------------------------------------------

// Records a printf-style message in the thread-local error slot and returns `code`.
int fail(int code, const char* fmt, ...);
// Adds `n` to the process-wide launch counter read by rt_launch_count().
void count_launch(int n = 1);
// cudaGetLastError() after a launch; records the kernel name on failure.
int check_launch(const char* kernel_name);
// Opts `kernel` in to `bytes` of dynamic shared memory on the current device; the attribute is
// per device and per kernel, so it is set once for each pair (thread-safe).
int ensure_dynamic_smem(const void* kernel, int bytes, const char* who);

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

#define RT_REQUIRE(cond, code, ...)                 \
    do {                                            \
        if (!(cond)) return ::rt::fail((code), __VA_ARGS__); \
    } while (0)

// ---------------------------------------------------------------------------
// Device side: 128-bit streaming accesses
// ---------------------------------------------------------------------------

#ifdef __CUDACC__

// 16-byte load of data that is read exactly once: bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// 16-byte load of single-use data that the same kernel may overwrite in place
// (no read-only assumption, still no L1 allocation).
__device__ __forceinline__ uint4 ld_once16(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// 16-byte load through the read-only path (reused data: weights, tables).
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// 16-byte store of data that this kernel never reads back: evict-first.
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ void st_stream8(void* p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ---------------------------------------------------------------------------
// bf16 <-> fp32, 8 lanes at a time
// ---------------------------------------------------------------------------

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // bf16 -> fp32 is a 16-bit shift of the bit pattern.
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    // cvt.rn.bf16x2.f32 d, a, b : a -> upper half, b -> lower half
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]);
    v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]);
    v.w = pack_bf16x2(f[6], f[7]);
    return v;
}

// Round an fp32 value to bf16 (nearest even) and widen it back.
__device__ __forceinline__ float round_bf16(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

// ---------------------------------------------------------------------------
// Reductions
// ---------------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Loads 8 consecutive weights as fp32 (weights are tiny and shared by all rows).
template <bool W_BF16>
__device__ __forceinline__ void load_weight8(const void* w, int vec, float (&out)[8]) {
    if constexpr (W_BF16) {
        unpack_bf16x8(ld_cached16(static_cast<const uint4*>(w) + vec), out);
    } else {
        const float4 a = __ldg(static_cast<const float4*>(w) + 2 * vec);
        const float4 b = __ldg(static_cast<const float4*>(w) + 2 * vec + 1);
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
}

// Sum of `a` and of `b` over the whole block; result broadcast to every thread.
// `scratch` is 64 floats of shared memory. blockDim.x must be a multiple of 32.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch) {
    a = warp_sum(a);
    b = warp_sum(b);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) {
        scratch[warp] = a;
        scratch[32 + warp] = b;
    }
    __syncthreads();
    float ra = (lane < nwarp) ? scratch[lane] : 0.f;
    float rb = (lane < nwarp) ? scratch[32 + lane] : 0.f;
    a = warp_sum(ra);
    b = warp_sum(rb);
}

__device__ __forceinline__ float block_sum(float a, float* scratch) {
    a = warp_sum(a);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    float ra = (lane < nwarp) ? scratch[lane] : 0.f;
    return warp_sum(ra);
}

// ---------------------------------------------------------------------------
// Scalar maths that has to agree bit for bit with IEEE fp32 host arithmetic
// ---------------------------------------------------------------------------

// silu(g) * u exactly as `F.silu(g.float()) * u.float()` evaluates it:
// g / (1 + exp(-g)) with an IEEE division, then one multiplication.
__device__ __forceinline__ float swiglu_f32(float g, float u) {
    const float s = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(s, u);
}

// Correctly rounded a / b for a divisor shared by many numerators:
// `rb` must be the correctly rounded reciprocal of b (__frcp_rn(b)). One
// multiplication, an exact remainder and one fused correction give the IEEE
// quotient (Markstein's division theorem); all operands here stay far away
// from the underflow/overflow thresholds where the remainder stops being exact.
// b must be positive: the sign of the quotient is then the sign of a, which is copied
// onto the result because the correction step would turn a/b = -0 into +0.
__device__ __forceinline__ float div_shared(float a, float b, float rb) {
    const float q = __fmul_rn(a, rb);
    const float r = __fmaf_rn(-q, b, a);
    const float c = __fmaf_rn(r, rb, q);
    return __uint_as_float((__float_as_uint(c) & 0x7fffffffu) | (__float_as_uint(a) & 0x80000000u));
}

#endif  // __CUDACC__

}  // namespace rt
