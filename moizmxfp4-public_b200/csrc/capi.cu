// Library-level entry points of the C ABI: version, error text, device query.
#include <atomic>
#include <cstdarg>
#include <cstring>

#include "mxfp4_common.cuh"

namespace mxfp4 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int num_sms() {
    static std::atomic<int> cached[64];      // per device; every writer stores the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace mxfp4

extern "C" int mxfp4_version(void) { return 100; }

extern "C" void mxfp4_last_error(char* buf, size_t n) {
    if (!buf || n == 0) return;
    strncpy(buf, mxfp4::g_err, n - 1);
    buf[n - 1] = '\0';
}

extern "C" int mxfp4_device_info(int* sm_major, int* sm_minor, int* num_sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return mxfp4::cuda_fail(e, "mxfp4_device_info: cudaGetDevice");
    int maj = 0, min = 0, sms = 0;
    if ((e = cudaDeviceGetAttribute(&maj, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&min, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
        return mxfp4::cuda_fail(e, "mxfp4_device_info: cudaDeviceGetAttribute");
    if (sm_major) *sm_major = maj;
    if (sm_minor) *sm_minor = min;
    if (num_sms) *num_sms = sms;
    return MXFP4_OK;
}
