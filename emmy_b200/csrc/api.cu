// Status plumbing of the C ABI.
#include <stdarg.h>

#include "common.cuh"

namespace eq {

static thread_local char g_error[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace eq

extern "C" {

int eq_version(void) { return 100; }

const char* eq_last_error(void) { return eq::g_error; }

const char* eq_status_name(int status) {
    switch (status) {
        case EQ_OK: return "EQ_OK";
        case EQ_ERR_BAD_ARG: return "EQ_ERR_BAD_ARG";
        case EQ_ERR_BAD_ALIGN: return "EQ_ERR_BAD_ALIGN";
        case EQ_ERR_UNSUPPORTED: return "EQ_ERR_UNSUPPORTED";
        case EQ_ERR_CUDA: return "EQ_ERR_CUDA";
        case EQ_ERR_NCCL: return "EQ_ERR_NCCL";
        case EQ_ERR_TIMEOUT: return "EQ_ERR_TIMEOUT";
        case EQ_ERR_WORKSPACE: return "EQ_ERR_WORKSPACE";
        default: return "EQ_ERR_UNKNOWN";
    }
}

}  // extern "C"
