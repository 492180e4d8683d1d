// Error reporting, version and device status word of the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "fq_common.cuh"

namespace fq {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

__device__ int g_fq_status = 0;

// The address is looked up once per device and remembered (relaxed atomics: concurrent host
// threads may race to store the same value).  It goes stale if the host process calls
// cudaDeviceReset(); reload the library in that case.
int* device_status_ptr() {
    constexpr int MAX_DEV = 64;
    static std::atomic<int*> ptrs[MAX_DEV];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
        set_error("device_status_ptr: cannot identify the current device");
        return nullptr;
    }
    int* ptr = ptrs[dev].load(std::memory_order_relaxed);
    if (ptr == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_fq_status);
        if (e != cudaSuccess) {
            set_error("device_status_ptr: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptr = static_cast<int*>(p);
        ptrs[dev].store(ptr, std::memory_order_relaxed);
    }
    return ptr;
}

}  // namespace fq

extern "C" const char* fq_last_error_string(void) { return fq::g_err; }

extern "C" const char* fq_version(void) { return "flashquest_b200 0.1 (sm_100a)"; }

extern "C" int fq_device_status(void) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, fq::g_fq_status, sizeof(int));
    if (e != cudaSuccess) return fq::fail(FQ_ERR_CUDA, "fq_device_status: %s", cudaGetErrorString(e));
    if (v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(fq::g_fq_status, &zero, sizeof(int));
        fq::set_error("a device-side bounded wait timed out (status %d)", v);
    }
    return v;
}
