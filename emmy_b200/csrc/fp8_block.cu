// Block-scaled FP8-E4M3 W8A8 linear: 128 x 128 weight blocks, activations quantized per token and per 128 elements of K.
//
// The official DeepSeek / Qwen / GLM FP8 form (weight_block_size [128, 128], `weight_scale_inv` [N/128, K/128] f32, used
// as a multiplier; emmy/compiler/loader/quant.py:136-144, 1581-1593).  The reference spells it as a dynamic activation
// round trip per K group in front of a block-dequantized weight (quant.py:1655-1717); natively
//     y[m, n] = sum_kb ( sum_{k in kb} q_x[m, k] q_w[n, k] ) * s_x[m, kb] * s_w[n / 128, kb]
// with the inner sums exact in f32 over 128 products of e4m3 values.
//
//   quant_fp8_groups_kernel  s_x[m, kb] = max(amax_kb |x|, 1e-12) / 448, q = e4m3_rne_satfinite(x / s_x): the per-token
//                            rule of fp8_linear.cu applied per 128-element group; one warp per group.  Inside the linear
//                            it also clears the status word and lets the kernel behind it start early.
//   fp8_block_tc.cu          tcgen05 with a fresh accumulator per K block and promotion in registers: a swapped-operand
//                            decode tile for M <= 16, 128 x 128 tiles up to 128 rows, 128 x 256 tiles above
//   fp8_block_gemm_kernel    the mma.sync form, kept for an output that is not 16-byte aligned: 128 x 128 output tile per
//                            CTA, K in steps of one scale block, operand tiles by cp.async into XOR-swizzled shared
//                            memory (two stages), fragments by ldmatrix, products by mma.sync m16n8k32 e4m3 into a
//                            per-block accumulator that is folded into the running f32 sum with the block's two scales.
#include "common.cuh"

namespace eq {

int fp8_block_tc_launch(const uint8_t* qx, const float* sx, const uint8_t* w, const float* sw, void* y, int64_t M, int64_t N, int64_t K,
                        int act_dtype, int* status, cudaStream_t stream);  // fp8_block_tc.cu


__device__ __forceinline__ uint16_t e4m3x2_sat(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// One warp per (row, 128-element group); K % 128 == 0.
template <typename InT>
__global__ void __launch_bounds__(256) quant_fp8_groups_kernel(const InT* __restrict__ x, int64_t M, int64_t K, uint8_t* __restrict__ q,
                                                               float* __restrict__ scale, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the linear behind this may start fetching weights
    // inside the linear this kernel is a programmatic dependent itself: the kernel before it (usually the previous
    // linear on this workspace) may still read the codes, scales and status word it rewrites
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (status && blockIdx.x == 0 && threadIdx.x == 0) *status = 0;  // the linear's status word, cleared on the way
    const int64_t groups = K / 128;
    const int64_t gw = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= M * groups) return;
    const InT* src = x + gw * 128 + lane * 4;
    float v[4];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = to_float(src[i]);
        amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
    if (lane == 0) scale[gw] = s;
    const uint32_t lo = e4m3x2_sat(__fdiv_rn(v[0], s), __fdiv_rn(v[1], s)), hi = e4m3x2_sat(__fdiv_rn(v[2], s), __fdiv_rn(v[3], s));
    *reinterpret_cast<uint32_t*>(q + gw * 128 + lane * 4) = lo | (hi << 16);
}

constexpr int kBB = 128;             // tile edge = scale block edge
constexpr int kBlkThreads = 256;     // 8 warps: 2 along M x 4 along N, 64 x 32 outputs per warp
constexpr int kBlkStage = 2 * kBB * kBB;  // A tile + B tile, bytes

__device__ __forceinline__ uint32_t swz(int row, int chunk) { return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ void mma_e4m3_blk(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename OutT>
__global__ void __launch_bounds__(kBlkThreads, 1) fp8_block_gemm_kernel(const uint8_t* __restrict__ qx, const float* __restrict__ sx,
                                                                        const uint8_t* __restrict__ w, const float* __restrict__ sw,
                                                                        OutT* __restrict__ y, int M, int N, int K) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int wm = warp >> 2, wn = warp & 3;  // warp tile origin: rows 64 wm, columns 32 wn
    const int m0 = blockIdx.y * kBB, n0 = blockIdx.x * kBB;
    const int kblocks = K / kBB;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

    // 16-byte chunk `idx` (0..1023) of a tile is (row idx / 8, chunk idx % 8); rows past the matrix are zero-filled
    auto load_stage = [&](int stage, int kb) {
        const uint32_t a_base = smem_base + stage * kBlkStage, b_base = a_base + kBB * kBB;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * kBlkThreads, row = idx >> 3, chunk = idx & 7;
            const int am = m0 + row, bn = n0 + row;
            const uint8_t* asrc = qx + static_cast<size_t>(am < M ? am : 0) * K + static_cast<size_t>(kb) * kBB + chunk * 16;
            const uint8_t* bsrc = w + static_cast<size_t>(bn < N ? bn : 0) * K + static_cast<size_t>(kb) * kBB + chunk * 16;
            const int asz = am < M ? 16 : 0, bsz = bn < N ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_base + swz(row, chunk)), "l"(asrc), "r"(asz) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(b_base + swz(row, chunk)), "l"(bsrc), "r"(bsz) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float total[4][4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) total[a][b][e] = 0.f;

    load_stage(0, 0);
    for (int kb = 0; kb < kblocks; ++kb) {
        const int stage = kb & 1;
        if (kb + 1 < kblocks) {
            load_stage(stage ^ 1, kb + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t a_base = smem_base + stage * kBlkStage, b_base = a_base + kBB * kBB;
        float blk[4][4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int e = 0; e < 4; ++e) blk[a][b][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {  // 32 elements of K per step
            uint32_t bf[4][2];
#pragma unroll
            for (int np = 0; np < 2; ++np) {  // two 8-column tiles per ldmatrix.x4
                const int mat = lane >> 3;
                const int row = wn * 32 + np * 16 + (lane & 7) + (mat >> 1) * 8, chunk = 2 * ks + (mat & 1);
                uint32_t r0, r1, r2, r3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                             : "r"(b_base + swz(row, chunk)));
                bf[2 * np][0] = r0;
                bf[2 * np][1] = r1;
                bf[2 * np + 1][0] = r2;
                bf[2 * np + 1][1] = r3;
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int mat = lane >> 3;
                const int row = wm * 64 + mt * 16 + (lane & 7) + (mat & 1) * 8, chunk = 2 * ks + (mat >> 1);
                uint32_t af[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3])
                             : "r"(a_base + swz(row, chunk)));
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) mma_e4m3_blk(blk[mt][nt], af, bf[nt][0], bf[nt][1]);
            }
        }
        // fold the block in with its scales: s_w is one value for the whole tile, s_x one per row
        const float s_w = sw[static_cast<size_t>(blockIdx.x) * kblocks + kb];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const int r_lo = m0 + wm * 64 + mt * 16 + g, r_hi = r_lo + 8;
            const float s_lo = r_lo < M ? sx[static_cast<size_t>(r_lo) * kblocks + kb] * s_w : 0.f;
            const float s_hi = r_hi < M ? sx[static_cast<size_t>(r_hi) * kblocks + kb] * s_w : 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                total[mt][nt][0] = fmaf(blk[mt][nt][0], s_lo, total[mt][nt][0]);
                total[mt][nt][1] = fmaf(blk[mt][nt][1], s_lo, total[mt][nt][1]);
                total[mt][nt][2] = fmaf(blk[mt][nt][2], s_hi, total[mt][nt][2]);
                total[mt][nt][3] = fmaf(blk[mt][nt][3], s_hi, total[mt][nt][3]);
            }
        }
        __syncthreads();  // every warp is done with this stage before it is refilled
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int col = n0 + wn * 32 + nt * 8 + 2 * j;
            if (col >= N) continue;
            const int r_lo = m0 + wm * 64 + mt * 16 + g, r_hi = r_lo + 8;
            if (r_lo < M) {
                y[static_cast<size_t>(r_lo) * N + col] = from_float<OutT>(total[mt][nt][0]);
                y[static_cast<size_t>(r_lo) * N + col + 1] = from_float<OutT>(total[mt][nt][1]);
            }
            if (r_hi < M) {
                y[static_cast<size_t>(r_hi) * N + col] = from_float<OutT>(total[mt][nt][2]);
                y[static_cast<size_t>(r_hi) * N + col + 1] = from_float<OutT>(total[mt][nt][3]);
            }
        }
    }
}

static size_t blk_align(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace eq

using namespace eq;

static int quant_fp8_groups(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, int* status, cudaStream_t stream) {
    EQ_REQUIRE(M >= 0 && K > 0, EQ_ERR_BAD_ARG, "eq_quant_fp8_per_group: bad extents M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(x && q && scale, EQ_ERR_BAD_ARG, "eq_quant_fp8_per_group: null pointer");
    EQ_REQUIRE(K % 128 == 0, EQ_ERR_UNSUPPORTED, "eq_quant_fp8_per_group: K must be a multiple of 128");
    EQ_REQUIRE(aligned(q, 4), EQ_ERR_BAD_ALIGN, "eq_quant_fp8_per_group: q must be 4-byte aligned");
    const int64_t warps = M * (K / 128);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(warps * 32, 256)));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (status && M <= 128) ? 1 : 0;  // decode-sized calls inside the linear: resident when the kernel before it ends
    switch (in_dtype) {
        case EQ_F16: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_groups_kernel<__half>, static_cast<const __half*>(x), M, K, q, scale, status)); break;
        case EQ_BF16: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_groups_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x), M, K, q, scale, status)); break;
        case EQ_F32: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_groups_kernel<float>, static_cast<const float*>(x), M, K, q, scale, status)); break;
        default: return fail(EQ_ERR_BAD_ARG, "eq_quant_fp8_per_group: unknown dtype %d", in_dtype);
    }
    return EQ_OK;
}

extern "C" int eq_quant_fp8_per_group(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, void* stream_) {
    return quant_fp8_groups(x, M, K, in_dtype, q, scale, nullptr, static_cast<cudaStream_t>(stream_));
}

extern "C" size_t eq_fp8_block_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return blk_align(static_cast<size_t>(M) * K) + blk_align(static_cast<size_t>(M) * (K / 128) * sizeof(float)) + 256;  // codes, scales, status
}

extern "C" int eq_fp8_block_linear(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, int64_t M,
                                   int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(N > 0 && K > 0 && M >= 0, EQ_ERR_BAD_ARG, "eq_fp8_block_linear: bad extents M=%lld K=%lld N=%lld", (long long)M, (long long)K,
               (long long)N);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(weight && weight_scale && x && y, EQ_ERR_BAD_ARG, "eq_fp8_block_linear: null pointer");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_fp8_block_linear: activations must be f16 or bf16");
    EQ_REQUIRE(K % 128 == 0 && N % 128 == 0, EQ_ERR_UNSUPPORTED, "eq_fp8_block_linear: needs whole 128 x 128 blocks (K=%lld N=%lld)", (long long)K,
               (long long)N);
    EQ_REQUIRE(aligned(weight, 16) && aligned(y, 4), EQ_ERR_BAD_ALIGN, "eq_fp8_block_linear: weight must be 16-byte aligned");
    EQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= eq_fp8_block_workspace_bytes(M, K), EQ_ERR_WORKSPACE,
               "eq_fp8_block_linear: workspace of %zu bytes (256-byte aligned) needed, %zu given", eq_fp8_block_workspace_bytes(M, K), workspace_bytes);
    uint8_t* qx = static_cast<uint8_t*>(workspace);
    float* sx = reinterpret_cast<float*>(qx + blk_align(static_cast<size_t>(M) * K));
    int* status = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(sx) + blk_align(static_cast<size_t>(M) * (K / 128) * sizeof(float)));
    int st = quant_fp8_groups(x, M, K, act_dtype, qx, sx, status, stream);
    if (st != EQ_OK) return st;
    // the tensor cores (fp8_block_tc.cu: swapped-operand decode tile up to 16 rows, 128-column tiles up to 128 rows, 256-column
    // tiles above); the mma.sync tile kernel below serves an unaligned y
    if (M <= 16 || aligned(y, 16)) return fp8_block_tc_launch(qx, sx, weight, weight_scale, y, M, N, K, act_dtype, status, stream);
    const dim3 grid(static_cast<unsigned>(N / kBB), static_cast<unsigned>(ceil_div(M, kBB)));
    const size_t smem = 2 * kBlkStage;
    if (act_dtype == EQ_F16) {
        EQ_CUDA_OK(cudaFuncSetAttribute(fp8_block_gemm_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        fp8_block_gemm_kernel<__half><<<grid, kBlkThreads, smem, stream>>>(qx, sx, weight, weight_scale, static_cast<__half*>(y), static_cast<int>(M),
                                                                           static_cast<int>(N), static_cast<int>(K));
    } else {
        EQ_CUDA_OK(cudaFuncSetAttribute(fp8_block_gemm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        fp8_block_gemm_kernel<__nv_bfloat16><<<grid, kBlkThreads, smem, stream>>>(qx, sx, weight, weight_scale, static_cast<__nv_bfloat16*>(y),
                                                                                  static_cast<int>(M), static_cast<int>(N), static_cast<int>(K));
    }
    EQ_LAUNCH_OK("fp8_block_gemm_kernel");
    return EQ_OK;
}

extern "C" int eq_fp8_block_status(const void* workspace, int64_t M, int64_t K, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && K > 0, EQ_ERR_BAD_ARG, "eq_fp8_block_status: bad arguments");
    const unsigned char* base = static_cast<const unsigned char*>(workspace);
    const int* status = reinterpret_cast<const int*>(base + blk_align(static_cast<size_t>(M) * K) + blk_align(static_cast<size_t>(M) * (K / 128) * sizeof(float)));
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_fp8_block_status: a bounded pipeline wait ran out (code %d)", host);
    return EQ_OK;
}
