// Error reporting and device probes of the C ABI.

#include <stdarg.h>

#include "common.cuh"

namespace pb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail_arg(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return PB_ERR_ARG;
}

int fail_cuda(cudaError_t e, const char* what) {
    snprintf(g_error, sizeof(g_error), "CUDA error: %s (%s) in %s", cudaGetErrorString(e), cudaGetErrorName(e), what);
    return PB_ERR_CUDA;
}

}  // namespace pb

extern "C" const char* pb_last_error(void) { return pb::g_error; }

extern "C" int pb_abi_version(void) { return 1; }

extern "C" int pb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
    }
    return ok;
}

extern "C" int64_t pb_train_state_bytes(void) { return (int64_t)sizeof(pb_train_state); }
