// Error text, version and device query of the C ABI.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace fg {

char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

namespace {
std::atomic<long long> g_launches{0};
}
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return (dev >= 0 && dev < kMaxDevices) ? dev : -1;
}

DeviceProps device_props() {
    static std::mutex lock;
    static DeviceProps table[kMaxDevices];
    static bool known[kMaxDevices] = {false};
    const int dev = current_device_slot();
    if (dev < 0) return DeviceProps();
    std::lock_guard<std::mutex> hold(lock);
    if (!known[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            table[dev].sm_count = v;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) == cudaSuccess && v > 0)
            table[dev].l2_bytes = v;
        (void)cudaGetLastError();
        known[dev] = true;
    }
    return table[dev];
}

}  // namespace fg

extern "C" {

int64_t fg_kernel_launch_count(void) { return fg::g_launches.load(std::memory_order_relaxed); }

int fg_version(void) { return 200; }

const char* fg_kernel_signature(void) {
    static char text[512] = {0};
    static std::once_flag once;
    std::call_once(once, [] {
        snprintf(text, sizeof(text), "%s;%s;%s", fg::spmm_signature(), fg::sddmm_signature(),
                 fg::sddmm_plan_signature());
    });
    return text;
}

const char* fg_last_error(void) { return fg::error_buffer(); }

int fg_device_info(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor, int64_t* l2_bytes) {
    int dev = 0;
    FG_CUDA_TRY(cudaGetDevice(&dev));
    int v = 0;
    if (sm_count) {
        FG_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        *sm_count = v;
    }
    if (cc_major) {
        FG_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev));
        *cc_major = v;
    }
    if (cc_minor) {
        FG_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, dev));
        *cc_minor = v;
    }
    if (l2_bytes) {
        FG_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev));
        *l2_bytes = v;
    }
    return FG_OK;
}

}  // extern "C"
