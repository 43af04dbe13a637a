// Status plumbing of the C ABI: version, status strings, thread-local error text, launch counter.
#include "common.cuh"

#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

namespace fm {

static thread_local char t_error[512] = "";
std::atomic<int64_t> g_launches{0};

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int sm_count()
{
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// cudaFuncSetAttribute costs several microseconds of host time per call and the launch paths would repeat it with the
// same value before every launch: the last value set per (kernel, device, attribute) is remembered instead.
cudaError_t func_attr_cached(const void *func, cudaFuncAttribute attr, int value)
{
    static std::mutex mu;
    static std::map<std::tuple<const void *, int, int>, int> last;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_tuple(func, dev, (int)attr);
    auto it = last.find(key);
    if (it != last.end() && it->second == value) return cudaSuccess;
    e = cudaFuncSetAttribute(func, attr, value);
    if (e == cudaSuccess) last[key] = value;
    return e;
}

}  // namespace fm

extern "C" {

int fm_abi_version(void) { return FM_ABI_VERSION; }

const char *fm_status_string(int status)
{
    switch (status) {
    case FM_OK: return "ok";
    case FM_ERR_BAD_ARG: return "bad argument";
    case FM_ERR_UNSUPPORTED: return "unsupported shape or element type";
    case FM_ERR_WORKSPACE: return "workspace too small";
    case FM_ERR_CUDA: return "CUDA error";
    case FM_ERR_DEVICE: return "kernel reported an anomaly";
    default: return "unknown status";
    }
}

const char *fm_last_error(void) { return fm::t_error; }

int64_t fm_launch_count(void) { return fm::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
