// Shared helpers of the emmyq kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/emmyq.h"

namespace eq {

// Records the message eq_last_error() returns on this thread and hands the status back.
int fail(int status, const char* fmt, ...);

#define EQ_REQUIRE(cond, status, ...) \
    do {                              \
        if (!(cond)) return ::eq::fail((status), __VA_ARGS__); \
    } while (0)

#define EQ_CUDA_OK(expr)                                                                     \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) return ::eq::fail(EQ_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// Launch check that does not clear a sticky error of somebody else's.
#define EQ_LAUNCH_OK(name)                                                                    \
    do {                                                                                      \
        cudaError_t e__ = cudaPeekAtLastError();                                              \
        if (e__ != cudaSuccess) {                                                             \
            cudaGetLastError();                                                               \
            return ::eq::fail(EQ_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
        }                                                                                     \
    } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device id).
int sm_count();

// ---- device helpers -------------------------------------------------------------------------------------------

// 16-byte streaming load of weights that are read once: bypass L1, read-only path.
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return r;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    // cvt.rn.f16x2.e4m3x2 is exact (e4m3 is a subset of f16); NaN codes map to f16 NaN.
    uint32_t h2;
    uint16_t in = b;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFF)));
}

// The 16 e2m1 values in code order.
__device__ __forceinline__ float e2m1_to_float(uint32_t code) {
    const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    float v = mag[code & 7];
    return (code & 8) ? -v : v;
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(float v) { return v; }

// 16-bit scale stored as raw bits with a run-time dtype tag.
__device__ __forceinline__ float scale16_to_float(uint16_t bits, int dtype) {
    return dtype == EQ_F16 ? __half2float(__ushort_as_half(bits)) : __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

}  // namespace eq
