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

bool pdl_enabled(int kind) {
    static const int mask = [] {
        const char* e = getenv("FQ_PDL");
        return e ? atoi(e) : (PDL_SCORES | PDL_ATTN | PDL_QUANT | PDL_GEMV);
    }();
    return (mask & kind) != 0;
}

DynPos& dyn_pos() {
    static thread_local DynPos d;
    return d;
}

__device__ int g_fq_status = 0;

int* device_status_ptr() {
    constexpr int MAX_DEV = 64;
    static int* ptrs[MAX_DEV] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
        set_error("device_status_ptr: cannot identify the current device");
        return nullptr;
    }
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_fq_status);
        if (e != cudaSuccess) {
            set_error("device_status_ptr: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
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
