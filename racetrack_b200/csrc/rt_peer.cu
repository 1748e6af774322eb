// Collective steps of the tensor/expert-parallel layer over NVLink peer memory.
//
// One process per GPU; every rank maps the other ranks' exchange buffers into its own address
// space (CUDA IPC, set up by the host side) and the kernels here read or write them with plain
// loads and stores over NVLink / NVSwitch: no multicast, no tensor maps over peer memory.
//
//   peer_barrier_kernel        all ranks have finished writing their partial sums (and have
//                              finished reading the previous ones): every rank stores a step
//                              counter into a flag slot of every peer and waits, with a bounded
//                              spin, until its own slots carry that counter.
//   peer_reduce_norm_kernel    the reduce-scatter of the reference's all-reduce
//                              (racetrack/realistic_bench.py:315-316,351) fused with the token-wise
//                              kernel that follows it: for this rank's rows, the partial sums of
//                              all ranks are read (own memory + peers), added in rank order in
//                              fp32, rounded to bf16 like the all-reduced tensor, then residual
//                              add + RMSNorm exactly as residual_norm_kernel does. The summed
//                              tensor never exists in memory.
//   peer_gather_kernel         the all-gather of row-sharded buffers: every rank has written its
//                              own block of rows into its own copy of the buffer; the kernel pulls
//                              the other ranks' blocks out of their copies into the local one, up
//                              to four buffers per launch (the compact outputs of the token-wise
//                              kernels: latent projection, NVFP4 codes, block scales, routing).
#include <string.h>

#include "rt_common.cuh"

namespace rt {

static __device__ int g_peer_error = 0;

constexpr int kMaxPeers = 8;

struct PeerPtrs {
    const void* p[kMaxPeers];
};
struct PeerFlagPtrs {
    int* p[kMaxPeers];
};

// flags: int32 [world + 1] in every rank's memory; slot r of rank q is written by rank r only,
// slot `world` is the rank's own count of barriers passed (kept on the device, so a barrier
// replayed from a CUDA graph takes the next step like an eagerly launched one).
__global__ void peer_barrier_kernel(PeerFlagPtrs flags, int rank, int world, long long max_cycles) {
    __shared__ int step_s;
    if (threadIdx.x == 0) step_s = ++flags.p[rank][world];
    __syncthreads();
    const int step = step_s;
    const int peer = threadIdx.x;
    if (peer >= world) return;
    // everything this rank wrote before the barrier is visible system-wide before the flag is
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.p[peer] + rank), "r"(step) : "memory");
    const int* mine = flags.p[rank] + peer;
    const long long t0 = clock64();
    while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (v >= step) break;
        if (clock64() - t0 > max_cycles) {    // a peer never arrived: report instead of hanging
            atomicCAS(&g_peer_error, 0, 100 + peer);
            break;
        }
        __nanosleep(64);
    }
}

// One CTA per row of this rank's share. VPT = 16-byte vectors per thread.
template <int VPT, bool W_BF16>
__global__ void __launch_bounds__(512) peer_reduce_norm_kernel(
    PeerPtrs partial, int world, int64_t row0, int64_t pstride,
    const __nv_bfloat16* __restrict__ residual, const void* __restrict__ weight,
    __nv_bfloat16* __restrict__ normed, __nv_bfloat16* __restrict__ hidden, int nvec,
    int64_t rstride, float cols_f, float eps) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const uint4* r = reinterpret_cast<const uint4*>(residual + row * rstride);
    uint4* hrow = reinterpret_cast<uint4*>(hidden) + row * nvec;
    uint4* nrow = reinterpret_cast<uint4*>(normed) + row * nvec;
    float h[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            // all ranks' vectors first (independent loads over NVLink), then the sum in rank order
            uint4 pv[kMaxPeers];
#pragma unroll
            for (int q = 0; q < kMaxPeers; ++q)
                if (q < world)
                    pv[q] = ld_once16(reinterpret_cast<const uint4*>(
                                          static_cast<const __nv_bfloat16*>(partial.p[q]) + (row0 + row) * pstride) + v);
            const uint4 rv = ld_stream16(r + v);
            float acc[8];
            unpack_bf16x8(pv[0], acc);
#pragma unroll
            for (int q = 1; q < kMaxPeers; ++q) {
                if (q < world) {
                    float a[8];
                    unpack_bf16x8(pv[q], a);
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] += a[k];
                }
            }
            float b[8], u[8];
            unpack_bf16x8(pack_bf16x8(acc), u);      // the all-reduced tensor is bf16
            unpack_bf16x8(rv, b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                h[i][k] = u[k] + b[k];
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

constexpr int kMaxGather = 4;
struct GatherArgs {
    const uint4* src[kMaxGather][kMaxPeers];   // buffer b as mapped from rank q
    uint4* dst[kMaxGather];                    // the local copy of buffer b
    int64_t slice_vec[kMaxGather];             // 16-byte vectors per rank's block of buffer b
};

// grid (CTAs, buffers). A CTA walks the (world - 1) foreign blocks of its buffer in 16-byte
// vectors, four loads in flight per thread.
__global__ void __launch_bounds__(256) peer_gather_kernel(GatherArgs a, int rank, int world) {
    const int b = blockIdx.y;
    const int64_t slice = a.slice_vec[b];
    const int64_t total = slice * (world - 1);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    uint4* dst = a.dst[b];
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
        uint4 v[4];
        int64_t off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            off[u] = -1;
            if (i < total) {
                const int k = static_cast<int>(i / slice);
                const int q = k + (k >= rank ? 1 : 0);
                off[u] = static_cast<int64_t>(q) * slice + (i - static_cast<int64_t>(k) * slice);
                v[u] = ld_once16(a.src[b][q] + off[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (off[u] >= 0) dst[off[u]] = v[u];
    }
}

// The transposing exchange in front of a row-sharded consumer ("all-to-all"): buffer b of rank q
// holds that rank's COLUMN block of a [T, world * cols] matrix for ALL rows; this rank wants ITS
// rows [row0, row0 + rows) of the whole matrix: dst[r, q * cols + c] = src_q[row0 + r, c].
// grid (CTAs, buffers); 16-byte vectors, four loads in flight per thread.
struct GatherColsArgs {
    const uint4* src[kMaxGather][kMaxPeers];
    uint4* dst[kMaxGather];
    int64_t row_vec[kMaxGather];               // 16-byte vectors per source row
};

__global__ void __launch_bounds__(256) peer_gather_cols_kernel(GatherColsArgs a, int world, int64_t row0,
                                                               int64_t rows) {
    const int b = blockIdx.y;
    const int64_t rv = a.row_vec[b];
    const int64_t per_peer = rows * rv;
    const int64_t total = per_peer * world;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    uint4* dst = a.dst[b];
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
        uint4 v[4];
        int64_t off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            off[u] = -1;
            if (i < total) {
                const int q = static_cast<int>(i / per_peer);
                const int64_t rem = i - static_cast<int64_t>(q) * per_peer;
                const int64_t r = rem / rv, c = rem - r * rv;
                off[u] = (r * world + q) * rv + c;
                v[u] = ld_once16(a.src[b][q] + (row0 + r) * rv + c);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (off[u] >= 0) dst[off[u]] = v[u];
    }
}

// The maximum of one fp32 value per rank (the tensor-wide amax behind an NVFP4 scale): every rank
// has stored its value in its own slot; after the barrier each rank reads all of them.
__global__ void peer_allmax_kernel(PeerPtrs slots, int world, float* __restrict__ out) {
    float v = 0.f;
    if (static_cast<int>(threadIdx.x) < world) {
        uint32_t bits;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(bits) : "l"(slots.p[threadIdx.x]) : "memory");
        v = __uint_as_float(bits);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x == 0) out[0] = v;
}

}  // namespace rt

using namespace rt;

// Exchange buffers are plain cudaMalloc allocations of the calling process's current device,
// exported with cudaIpcGetMemHandle and opened by the other ranks WITH THEIR OWN DEVICE CURRENT
// (cudaIpcMemLazyEnablePeerAccess then enables the peer mapping for that device), so a kernel on
// a rank's GPU may dereference the returned pointer directly.
extern "C" int rt_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle_out) {
    RT_REQUIRE(bytes > 0 && ptr && handle_out, RT_ERR_BAD_ARG, "rt_peer_alloc: bad arguments");
    void* p = nullptr;
    RT_REQUIRE(cudaMalloc(&p, static_cast<size_t>(bytes)) == cudaSuccess, RT_ERR_CUDA,
               "rt_peer_alloc: cudaMalloc of %lld bytes failed", (long long)bytes);
    if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return fail(RT_ERR_CUDA, "rt_peer_alloc: cannot clear the buffer");
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return fail(RT_ERR_CUDA, "rt_peer_alloc: cudaIpcGetMemHandle failed");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles travel as 64 bytes");
    memcpy(handle_out, &h, 64);
    *ptr = p;
    return RT_OK;
}

extern "C" int rt_peer_open(const unsigned char* handle, void** ptr) {
    RT_REQUIRE(handle && ptr, RT_ERR_BAD_ARG, "rt_peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_peer_open: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    }
    *ptr = p;
    return RT_OK;
}

extern "C" int rt_peer_close(void* ptr) {
    if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_peer_close: cudaIpcCloseMemHandle failed");
    }
    return RT_OK;
}

extern "C" int rt_peer_free(void* ptr) {
    if (ptr && cudaFree(ptr) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_peer_free: cudaFree failed");
    }
    return RT_OK;
}

extern "C" int rt_peer_barrier(int* const* flag_ptrs, int64_t rank, int64_t world, void* stream) {
    RT_REQUIRE(flag_ptrs && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world,
               RT_ERR_BAD_ARG, "rt_peer_barrier: bad arguments (at most %d ranks)", kMaxPeers);
    PeerFlagPtrs f;
    for (int q = 0; q < kMaxPeers; ++q) f.p[q] = q < world ? flag_ptrs[q] : nullptr;
    for (int q = 0; q < world; ++q) RT_REQUIRE(f.p[q], RT_ERR_BAD_ARG, "rt_peer_barrier: null flag pointer");
    // 3e9 SM cycles (about two seconds) of polling, then the error flag
    peer_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(f, (int)rank, (int)world, 3000000000LL);
    count_launch();
    return check_launch("peer_barrier_kernel");
}

extern "C" int rt_peer_error_state(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "rt_peer_error_state: cannot read the device flag");
    }
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_peer_error, &zero, sizeof(int));
        return fail(RT_ERR_TIMEOUT, "a peer barrier gave up waiting for rank %d", v - 100);
    }
    return RT_OK;
}

extern "C" int rt_peer_reduce_residual_norm(const void* const* partial_ptrs, int64_t world, int64_t row0,
                                            int64_t partial_stride, const void* residual,
                                            const void* weight, int weight_dtype, void* normed,
                                            void* hidden, int64_t rows, int64_t cols,
                                            int64_t residual_stride, float eps, void* stream) {
    RT_REQUIRE(partial_ptrs && residual && weight && normed && hidden, RT_ERR_BAD_ARG,
               "rt_peer_reduce_residual_norm: null pointer");
    RT_REQUIRE(world >= 1 && world <= kMaxPeers, RT_ERR_BAD_ARG,
               "rt_peer_reduce_residual_norm: 1 to %d ranks", kMaxPeers);
    RT_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= 32768 && partial_stride % 8 == 0 &&
                   residual_stride % 8 == 0 && row0 >= 0,
               RT_ERR_UNSUPPORTED,
               "rt_peer_reduce_residual_norm: cols must be a multiple of 8 up to 32768, strides multiples of 8");
    RT_REQUIRE(weight_dtype == RT_BF16 || weight_dtype == RT_F32, RT_ERR_BAD_ARG,
               "rt_peer_reduce_residual_norm: weight must be bf16 or fp32");
    if (rows == 0) return RT_OK;
    PeerPtrs p;
    for (int q = 0; q < kMaxPeers; ++q) {
        p.p[q] = q < world ? partial_ptrs[q] : nullptr;
        RT_REQUIRE(q >= world || (p.p[q] && aligned16(p.p[q])), RT_ERR_BAD_ARG,
                   "rt_peer_reduce_residual_norm: partial pointers must be non-null and 16-byte aligned");
    }
    RT_REQUIRE(aligned16(residual) && aligned16(normed) && aligned16(hidden), RT_ERR_BAD_ARG,
               "rt_peer_reduce_residual_norm: pointers must be 16-byte aligned");
    const int nvec = static_cast<int>(cols / 8);
    int vpt = 0, threads = 0;
    for (int cand : {1, 2, 4, 8}) {
        const int th = ((nvec + cand - 1) / cand + 31) / 32 * 32;
        if (th <= 256 || (cand == 8 && th <= 512)) {
            vpt = cand;
            threads = th < 32 ? 32 : th;
            break;
        }
    }
    RT_REQUIRE(vpt, RT_ERR_UNSUPPORTED, "rt_peer_reduce_residual_norm: row too wide");
    const dim3 grid(static_cast<unsigned>(rows));
    cudaStream_t st = as_stream(stream);
    const bool wb = weight_dtype == RT_BF16;
    const auto* res = static_cast<const __nv_bfloat16*>(residual);
    auto* n = static_cast<__nv_bfloat16*>(normed);
    auto* h = static_cast<__nv_bfloat16*>(hidden);
#define RT_LAUNCH_PR(V)                                                                               \
    if (wb)                                                                                           \
        peer_reduce_norm_kernel<V, true><<<grid, threads, 0, st>>>(                                   \
            p, (int)world, row0, partial_stride, res, weight, n, h, nvec, residual_stride, (float)cols, eps); \
    else                                                                                              \
        peer_reduce_norm_kernel<V, false><<<grid, threads, 0, st>>>(                                  \
            p, (int)world, row0, partial_stride, res, weight, n, h, nvec, residual_stride, (float)cols, eps);
    switch (vpt) {
        case 1: RT_LAUNCH_PR(1) break;
        case 2: RT_LAUNCH_PR(2) break;
        case 4: RT_LAUNCH_PR(4) break;
        default: RT_LAUNCH_PR(8) break;
    }
#undef RT_LAUNCH_PR
    count_launch();
    return check_launch("peer_reduce_norm_kernel");
}

extern "C" int rt_peer_gather(const void* const* peer_ptrs, const int64_t* slice_bytes, int64_t n_buffers,
                              int64_t rank, int64_t world, void* stream) {
    RT_REQUIRE(peer_ptrs && slice_bytes, RT_ERR_BAD_ARG, "rt_peer_gather: null pointer");
    RT_REQUIRE(n_buffers >= 1 && n_buffers <= kMaxGather, RT_ERR_BAD_ARG, "rt_peer_gather: 1 to %d buffers",
               kMaxGather);
    RT_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, RT_ERR_BAD_ARG,
               "rt_peer_gather: bad rank / world (at most %d ranks)", kMaxPeers);
    if (world == 1) return RT_OK;
    GatherArgs a;
    int64_t most = 0;
    for (int b = 0; b < kMaxGather; ++b) {
        a.dst[b] = nullptr;
        a.slice_vec[b] = 0;
        for (int q = 0; q < kMaxPeers; ++q) a.src[b][q] = nullptr;
        if (b >= n_buffers) continue;
        RT_REQUIRE(slice_bytes[b] >= 0 && slice_bytes[b] % 16 == 0, RT_ERR_BAD_ARG,
                   "rt_peer_gather: a rank's block must be a multiple of 16 bytes");
        a.slice_vec[b] = slice_bytes[b] / 16;
        for (int q = 0; q < world; ++q) {
            const void* p = peer_ptrs[b * world + q];
            RT_REQUIRE(p && aligned16(p), RT_ERR_BAD_ARG,
                       "rt_peer_gather: buffer pointers must be non-null and 16-byte aligned");
            a.src[b][q] = static_cast<const uint4*>(p);
        }
        a.dst[b] = const_cast<uint4*>(a.src[b][rank]);
        const int64_t total = a.slice_vec[b] * (world - 1);
        if (total > most) most = total;
    }
    if (most == 0) return RT_OK;
    int64_t ctas = (most + 4 * 256 - 1) / (4 * 256);
    if (ctas > 4 * 148) ctas = 4 * 148;
    const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(n_buffers));
    peer_gather_kernel<<<grid, 256, 0, as_stream(stream)>>>(a, (int)rank, (int)world);
    count_launch();
    return check_launch("peer_gather_kernel");
}

extern "C" int rt_peer_gather_cols(const void* const* peer_ptrs, void* const* dst_ptrs,
                                   const int64_t* src_row_bytes, int64_t n_buffers, int64_t row0,
                                   int64_t rows, int64_t world, void* stream) {
    RT_REQUIRE(peer_ptrs && dst_ptrs && src_row_bytes, RT_ERR_BAD_ARG, "rt_peer_gather_cols: null pointer");
    RT_REQUIRE(n_buffers >= 1 && n_buffers <= kMaxGather, RT_ERR_BAD_ARG,
               "rt_peer_gather_cols: 1 to %d buffers", kMaxGather);
    RT_REQUIRE(world >= 1 && world <= kMaxPeers && row0 >= 0 && rows >= 0, RT_ERR_BAD_ARG,
               "rt_peer_gather_cols: bad arguments (at most %d ranks)", kMaxPeers);
    if (rows == 0) return RT_OK;
    GatherColsArgs a;
    int64_t most = 0;
    for (int b = 0; b < kMaxGather; ++b) {
        a.dst[b] = nullptr;
        a.row_vec[b] = 0;
        for (int q = 0; q < kMaxPeers; ++q) a.src[b][q] = nullptr;
        if (b >= n_buffers) continue;
        RT_REQUIRE(src_row_bytes[b] > 0 && src_row_bytes[b] % 16 == 0, RT_ERR_BAD_ARG,
                   "rt_peer_gather_cols: a source row must be a positive multiple of 16 bytes");
        a.row_vec[b] = src_row_bytes[b] / 16;
        for (int q = 0; q < world; ++q) {
            const void* p = peer_ptrs[b * world + q];
            RT_REQUIRE(p && aligned16(p), RT_ERR_BAD_ARG,
                       "rt_peer_gather_cols: buffer pointers must be non-null and 16-byte aligned");
            a.src[b][q] = static_cast<const uint4*>(p);
        }
        RT_REQUIRE(dst_ptrs[b] && aligned16(dst_ptrs[b]), RT_ERR_BAD_ARG,
                   "rt_peer_gather_cols: destination pointers must be non-null and 16-byte aligned");
        a.dst[b] = static_cast<uint4*>(dst_ptrs[b]);
        const int64_t total = a.row_vec[b] * rows * world;
        if (total > most) most = total;
    }
    int64_t ctas = (most + 4 * 256 - 1) / (4 * 256);
    if (ctas > 4 * 148) ctas = 4 * 148;
    const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(n_buffers));
    peer_gather_cols_kernel<<<grid, 256, 0, as_stream(stream)>>>(a, (int)world, row0, rows);
    count_launch();
    return check_launch("peer_gather_cols_kernel");
}

extern "C" int rt_peer_allmax(const void* const* slot_ptrs, int64_t world, float* out, void* stream) {
    RT_REQUIRE(slot_ptrs && out, RT_ERR_BAD_ARG, "rt_peer_allmax: null pointer");
    RT_REQUIRE(world >= 1 && world <= kMaxPeers, RT_ERR_BAD_ARG, "rt_peer_allmax: 1 to %d ranks", kMaxPeers);
    PeerPtrs p;
    for (int q = 0; q < kMaxPeers; ++q) {
        p.p[q] = q < world ? slot_ptrs[q] : nullptr;
        RT_REQUIRE(q >= world || p.p[q], RT_ERR_BAD_ARG, "rt_peer_allmax: null slot pointer");
    }
    peer_allmax_kernel<<<1, 32, 0, as_stream(stream)>>>(p, (int)world, out);
    count_launch();
    return check_launch("peer_allmax_kernel");
}
