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

// ---- tensor maps (driver entry point fetched at run time: no link-time dependency on libcuda) ------------------
#include <cuda.h>
#include <cudaTypedefs.h>

namespace eq {

int make_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType elem, size_t elem_bytes, uint64_t rows,
                       uint64_t cols, uint64_t pitch, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
            return fail(EQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    EQ_REQUIRE(aligned(base, 16) && pitch % 16 == 0, EQ_ERR_BAD_ALIGN, "tensor map: base and row pitch must be 16-byte aligned");
    EQ_REQUIRE(static_cast<size_t>(box_cols) * elem_bytes % 16 == 0 && box_rows <= 256 && box_cols <= 256, EQ_ERR_BAD_ARG,
               "tensor map: bad box %u x %u", box_rows, box_cols);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, elem, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return EQ_OK;
}

}  // namespace eq
