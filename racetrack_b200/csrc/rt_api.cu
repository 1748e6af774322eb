// Host-side plumbing shared by every entry point of librt_b200: status
// messages, launch accounting, version.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <utility>

#include "rt_common.cuh"

namespace rt {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char* kernel_name) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return RT_OK;
    return fail(RT_ERR_CUDA, "%s: %s", kernel_name, cudaGetErrorString(e));
}

const char* last_error() { return g_error; }

int ensure_dynamic_smem(const void* kernel, int bytes, const char* who) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> granted;   // (kernel, device) -> bytes
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "%s: no current CUDA device", who);
    }
    std::lock_guard<std::mutex> lock(mu);
    int& have = granted[std::make_pair(kernel, dev)];
    if (have >= bytes) return RT_OK;
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(RT_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
    }
    have = bytes;
    return RT_OK;
}

}  // namespace rt

extern "C" int rt_version(void) { return 1; }

extern "C" const char* rt_last_error(void) { return rt::last_error(); }

extern "C" int64_t rt_launch_count(void) {
    return rt::g_launches.load(std::memory_order_relaxed);
}
