// Bit-exact decoders of the checkpoint layouts: int4 unpack, AWQ/GPTQ dequantize (with optional g_idx),
// FP8 and NVFP4 weight dequantize.  Load-time / verification kernels: simple, coalesced, not tuned further.
#include "common.cuh"

namespace eq {

// Bit offset of logical nibble i (emmy/compiler/loader/quant.py:86-133).
__device__ __forceinline__ int nibble_shift(int fmt, int i) {
    return fmt == EQ_W4_AWQ ? ((i & 1) * 16 + (i >> 1) * 4) : i * 4;
}

__global__ void unpack_int4_kernel(int fmt, int along_rows, const uint32_t* __restrict__ words, int64_t rows,
                                   int64_t cols, uint8_t* __restrict__ out) {
    int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= rows * cols) return;
    int64_t r = idx / cols, c = idx % cols;
    uint32_t w = words[idx];
    if (along_rows) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[(r * 8 + i) * cols + c] = (w >> nibble_shift(fmt, i)) & 0xF;
    } else {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo |= ((w >> nibble_shift(fmt, i)) & 0xF) << (8 * i);
            hi |= ((w >> nibble_shift(fmt, i + 4)) & 0xF) << (8 * i);
        }
        *reinterpret_cast<uint2*>(out + idx * 8) = make_uint2(lo, hi);
    }
}

// One thread per packed weight word.  AWQ: word (k, j) holds columns 8j..8j+7 of row k.  GPTQ: word (r, n) holds
// rows 8r..8r+7 of column n.  `fast_first` picks which index runs fastest across threads so that the stores of the
// requested orientation coalesce.
template <typename OutT>
__global__ void dequant_w4_kernel(int fmt, const uint32_t* __restrict__ qweight, const uint32_t* __restrict__ qzeros,
                                  const uint16_t* __restrict__ scales, int scale_dtype,
                                  const int32_t* __restrict__ g_idx, int64_t K, int64_t N, int64_t G, int transpose,
                                  OutT* __restrict__ out) {
    const int64_t words_r = fmt == EQ_W4_AWQ ? K : K / 8;      // rows of the word matrix
    const int64_t words_c = fmt == EQ_W4_AWQ ? N / 8 : N;      // columns of the word matrix
    int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= words_r * words_c) return;
    // AWQ stores coalesce along columns for W[K,N] and along rows for W[N,K]; GPTQ words hold a k-run, so the
    // transposed output is the contiguous one.
    const bool rows_fastest = (transpose != 0);
    int64_t r = rows_fastest ? idx % words_r : idx / words_c;
    int64_t c = rows_fastest ? idx / words_r : idx % words_c;
    const uint32_t w = qweight[r * words_c + c];
    const int bias = fmt == EQ_W4_GPTQ ? 1 : 0;
    const int64_t zcols = N / 8;
    if (fmt == EQ_W4_AWQ) {
        const int64_t k = r;
        const int64_t g = g_idx ? g_idx[k] : k / G;
        const uint32_t zw = qzeros[g * zcols + c];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int sh = nibble_shift(EQ_W4_AWQ, i);
            const int64_t n = c * 8 + i;
            const float q = static_cast<float>((w >> sh) & 0xF);
            const float z = static_cast<float>(((zw >> sh) & 0xF) + bias);
            const float v = __fmul_rn(q - z, scale16_to_float(scales[g * N + n], scale_dtype));
            out[transpose ? n * K + k : k * N + n] = from_float<OutT>(v);
        }
    } else {
        const int64_t n = c;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t k = r * 8 + i;
            const int64_t g = g_idx ? g_idx[k] : k / G;
            const uint32_t zw = qzeros[g * zcols + n / 8];
            const float q = static_cast<float>((w >> (4 * i)) & 0xF);
            const float z = static_cast<float>(((zw >> (4 * (n % 8))) & 0xF) + bias);
            const float v = __fmul_rn(q - z, scale16_to_float(scales[g * N + n], scale_dtype));
            out[transpose ? n * K + k : k * N + n] = from_float<OutT>(v);
        }
    }
}

template <typename OutT>
__global__ void dequant_fp8_kernel(const uint8_t* __restrict__ bits, const float* __restrict__ scale, int64_t N,
                                   int64_t K, int64_t srows, int64_t scols, OutT* __restrict__ out) {
    int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= N * K) return;
    const int64_t n = idx / K, k = idx % K;
    const float s = scale[(n / (N / srows)) * scols + k / (K / scols)];
    out[idx] = from_float<OutT>(__fmul_rn(e4m3_to_float(bits[idx]), s));
}

// One thread per 16-element block (8 packed bytes, one scale).
template <typename OutT>
__global__ void dequant_nvfp4_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale_bits,
                                     const float* __restrict__ scale_2, int64_t N, int64_t K,
                                     OutT* __restrict__ out) {
    int64_t blk = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (blk >= N * (K / 16)) return;
    // fused = f32( f16_rne( e4m3(scale) * scale_2 ) ): the one rounding of the two-level scale
    const float fused = __half2float(__float2half_rn(__fmul_rn(e4m3_to_float(scale_bits[blk]), scale_2[0])));
    const uint2 bytes = *reinterpret_cast<const uint2*>(packed + blk * 8);
    const uint32_t w[2] = {bytes.x, bytes.y};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t code = (w[i / 8] >> (4 * (i % 8))) & 0xF;
        out[blk * 16 + i] = from_float<OutT>(__fmul_rn(e2m1_to_float(code), fused));
    }
}

// MXFP4: one thread per 32-value group (16 bytes, one power-of-two scale).  out is [N][K] (the stored orientation).
template <typename OutT>
__global__ void dequant_mxfp4_kernel(const uint8_t* __restrict__ blocks, const uint8_t* __restrict__ scales, int64_t groups_total,
                                     OutT* __restrict__ out) {
    const int64_t grp = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (grp >= groups_total) return;
    const int e = static_cast<int>(scales[grp]) - 127;
    const uint4 bytes = *reinterpret_cast<const uint4*>(blocks + grp * 16);
    const uint32_t w[4] = {bytes.x, bytes.y, bytes.z, bytes.w};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const uint32_t code = (w[i / 8] >> (4 * (i % 8))) & 0xF;
        out[grp * 32 + i] = from_float<OutT>(ldexpf(e2m1_to_float(code), e));  // exact, or infinity at the largest exponents
    }
}

template <typename F>
static int dispatch_out(int out_dtype, F&& f) {
    switch (out_dtype) {
        case EQ_F16: return f(static_cast<__half*>(nullptr));
        case EQ_BF16: return f(static_cast<__nv_bfloat16*>(nullptr));
        case EQ_F32: return f(static_cast<float*>(nullptr));
        default: return fail(EQ_ERR_BAD_ARG, "unknown out_dtype %d", out_dtype);
    }
}

}  // namespace eq

using namespace eq;

extern "C" int eq_unpack_int4(int fmt, int along_rows, const int32_t* words, int64_t rows, int64_t cols, uint8_t* out,
                              void* stream) {
    EQ_REQUIRE(fmt == EQ_W4_AWQ || fmt == EQ_W4_GPTQ || fmt == EQ_W4_CT, EQ_ERR_BAD_ARG, "eq_unpack_int4: unknown format %d", fmt);
    EQ_REQUIRE(words && out, EQ_ERR_BAD_ARG, "eq_unpack_int4: null pointer");
    EQ_REQUIRE(rows >= 0 && cols >= 0, EQ_ERR_BAD_ARG, "eq_unpack_int4: negative extent");
    EQ_REQUIRE(aligned(out, 8), EQ_ERR_BAD_ALIGN, "eq_unpack_int4: out must be 8-byte aligned");
    if (rows * cols == 0) return EQ_OK;
    const int threads = 256;
    unpack_int4_kernel<<<static_cast<unsigned>(ceil_div(rows * cols, threads)), threads, 0,
                         static_cast<cudaStream_t>(stream)>>>(fmt, along_rows, reinterpret_cast<const uint32_t*>(words),
                                                              rows, cols, out);
    EQ_LAUNCH_OK("unpack_int4_kernel");
    return EQ_OK;
}

extern "C" int eq_dequant_w4(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                             int scale_dtype, const int32_t* g_idx, int64_t K, int64_t N, int64_t G, int out_dtype,
                             int transpose, void* out, void* stream) {
    EQ_REQUIRE(fmt == EQ_W4_AWQ || fmt == EQ_W4_GPTQ || fmt == EQ_W4_CT, EQ_ERR_BAD_ARG, "eq_dequant_w4: unknown format %d", fmt);
    EQ_REQUIRE(qweight && qzeros && scales && out, EQ_ERR_BAD_ARG, "eq_dequant_w4: null pointer");
    EQ_REQUIRE(scale_dtype == EQ_F16 || scale_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_dequant_w4: scales must be f16 or bf16");
    EQ_REQUIRE(K > 0 && N > 0, EQ_ERR_BAD_ARG, "eq_dequant_w4: K and N must be positive");
    if (G == -1) G = K;
    // the geometry errors of dequantize_packed_int4 (emmy/compiler/loader/quant.py:546-551)
    EQ_REQUIRE(G > 0 && K % G == 0, EQ_ERR_BAD_ARG, "eq_dequant_w4: group size %lld does not cover K=%lld", (long long)G, (long long)K);
    EQ_REQUIRE(N % 8 == 0 && K % 8 == 0, EQ_ERR_BAD_ARG, "eq_dequant_w4: K and N must be multiples of 8");
    const int64_t words = K * N / 8;
    const int threads = 256;
    return dispatch_out(out_dtype, [&](auto* tag) {
        using OutT = std::remove_pointer_t<decltype(tag)>;
        dequant_w4_kernel<OutT><<<static_cast<unsigned>(ceil_div(words, threads)), threads, 0,
                                  static_cast<cudaStream_t>(stream)>>>(
            fmt, reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const uint32_t*>(qzeros),
            static_cast<const uint16_t*>(scales), scale_dtype, g_idx, K, N, G, transpose, static_cast<OutT*>(out));
        EQ_LAUNCH_OK("dequant_w4_kernel");
        return (int)EQ_OK;
    });
}

extern "C" int eq_dequant_fp8(const uint8_t* bits, const float* scale, int64_t N, int64_t K, int64_t scale_rows,
                              int64_t scale_cols, int out_dtype, void* out, void* stream) {
    EQ_REQUIRE(bits && scale && out, EQ_ERR_BAD_ARG, "eq_dequant_fp8: null pointer");
    EQ_REQUIRE(N > 0 && K > 0 && scale_rows > 0 && scale_cols > 0, EQ_ERR_BAD_ARG, "eq_dequant_fp8: non-positive extent");
    // dequantize's divisibility rule (emmy/compiler/loader/quant.py:160-163)
    EQ_REQUIRE(N % scale_rows == 0 && K % scale_cols == 0, EQ_ERR_BAD_ARG,
               "eq_dequant_fp8: scale shape [%lld,%lld] does not divide weight shape [%lld,%lld]", (long long)scale_rows,
               (long long)scale_cols, (long long)N, (long long)K);
    const int threads = 256;
    return dispatch_out(out_dtype, [&](auto* tag) {
        using OutT = std::remove_pointer_t<decltype(tag)>;
        dequant_fp8_kernel<OutT><<<static_cast<unsigned>(ceil_div(N * K, threads)), threads, 0,
                                   static_cast<cudaStream_t>(stream)>>>(bits, scale, N, K, scale_rows, scale_cols,
                                                                        static_cast<OutT*>(out));
        EQ_LAUNCH_OK("dequant_fp8_kernel");
        return (int)EQ_OK;
    });
}

extern "C" int eq_dequant_nvfp4(const uint8_t* packed, const uint8_t* scale_bits, const float* scale_2, int64_t N,
                                int64_t K, int out_dtype, void* out, void* stream) {
    EQ_REQUIRE(packed && scale_bits && scale_2 && out, EQ_ERR_BAD_ARG, "eq_dequant_nvfp4: null pointer");
    EQ_REQUIRE(N > 0 && K > 0 && K % 16 == 0, EQ_ERR_BAD_ARG, "eq_dequant_nvfp4: K must be a positive multiple of 16");
    EQ_REQUIRE(aligned(packed, 8), EQ_ERR_BAD_ALIGN, "eq_dequant_nvfp4: packed must be 8-byte aligned");
    const int threads = 256;
    return dispatch_out(out_dtype, [&](auto* tag) {
        using OutT = std::remove_pointer_t<decltype(tag)>;
        dequant_nvfp4_kernel<OutT><<<static_cast<unsigned>(ceil_div(N * (K / 16), threads)), threads, 0,
                                     static_cast<cudaStream_t>(stream)>>>(packed, scale_bits, scale_2, N, K,
                                                                          static_cast<OutT*>(out));
        EQ_LAUNCH_OK("dequant_nvfp4_kernel");
        return (int)EQ_OK;
    });
}

extern "C" int eq_dequant_mxfp4(const uint8_t* blocks, const uint8_t* scales, int64_t N, int64_t K, int out_dtype, void* out, void* stream) {
    EQ_REQUIRE(blocks && scales && out, EQ_ERR_BAD_ARG, "eq_dequant_mxfp4: null pointer");
    EQ_REQUIRE(N > 0 && K > 0 && K % 32 == 0, EQ_ERR_BAD_ARG, "eq_dequant_mxfp4: K must be a positive multiple of 32");
    EQ_REQUIRE(aligned(blocks, 16), EQ_ERR_BAD_ALIGN, "eq_dequant_mxfp4: blocks must be 16-byte aligned");
    const int threads = 256;
    const int64_t groups = N * (K / 32);
    return dispatch_out(out_dtype, [&](auto* tag) {
        using OutT = std::remove_pointer_t<decltype(tag)>;
        dequant_mxfp4_kernel<OutT><<<static_cast<unsigned>(ceil_div(groups, threads)), threads, 0, static_cast<cudaStream_t>(stream)>>>(
            blocks, scales, groups, static_cast<OutT*>(out));
        EQ_LAUNCH_OK("dequant_mxfp4_kernel");
        return (int)EQ_OK;
    });
}
