// Block-scaled FP8 W8A8 linear on the 5th-generation tensor cores.
//
//     y[m, n] = sum_kb ( sum_{k in kb} q_x[m, k] q_w[n, k] ) * s_x[m, kb] * s_w[n / 128, kb]
//
// kind::f8f6f4 accumulates in tensor memory over as many K steps as it is told to, and its block-scaled sibling wants
// power-of-two scales per 32 elements, so f32 scales per 128 elements have to be applied OUTSIDE the MMA.  The kernel
// therefore never accumulates across K blocks in tensor memory: every 128-element K block is four k32 MMAs into a
// FRESH accumulator (two accumulators of 256 columns, or four of 128, rotate and fill TMEM), and the epilogue warps promote each
// finished block into f32 sums they keep in registers -- sum += acc * (s_x[m, kb] * s_w[n / 128, kb]) -- while the tensor
// core works on the next block.  (The reference spells the same arithmetic as a per-group activation round trip in front
// of a block-dequantized weight, emmy/compiler/loader/quant.py:1655-1717.)
//
//   warp 0      TMA producer: A tile 128 rows x 128 bytes, B tile 256 channels x 128 bytes, four 48 KB stages
//   warp 1      MMA issuer: per K block 4 x tcgen05.mma 128 x 256 x 32, commit -> stage free, commit -> accumulator full
//   warps 2..9  promotion and store: quartet q owns columns [128 q, 128 q + 128) = one weight scale block; a thread owns
//               one row and keeps its 128 sums in registers; after reading a block's accumulator it hands it back
// Every wait is bounded and reports through the status word.
#include "tc_common.cuh"

namespace eq {

namespace {

constexpr int kBM = 128, kBK = 128;
constexpr int kTileA = kBM * kBK;

// BN = 256: two weight scale blocks per CTA, eight promotion warps, four 48 KB stages, all of TMEM.  BN = 128 (calls of
// at most 128 rows, where the grid is one row of CTAs): twice as many CTAs stream the weight, six 32 KB stages.
template <int BN>
struct BlkCfg {
    static constexpr int kTileB = BN * kBK;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kQuartets = BN / 128;
    static constexpr int kThreads = 64 + 128 * kQuartets;
    static constexpr size_t kSmem = static_cast<size_t>(kStages) * (kTileA + kTileB) + 1024 + 256;
    static constexpr int kBufs = 512 / BN;  // accumulators that rotate: all of TMEM
    static constexpr uint32_t kTmemCols = 512;
};

template <typename OutT, int BN>
__global__ void __launch_bounds__(BlkCfg<BN>::kThreads, 1)
    fp8_block_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const float* __restrict__ sx, const float* __restrict__ sw, OutT* __restrict__ y, int M, int N, int K,
                        int* __restrict__ status) {
    using Cfg = BlkCfg<BN>;
    constexpr int kBN = BN, kTileB = Cfg::kTileB, kStages = Cfg::kStages, kBufs = Cfg::kBufs;
    constexpr uint32_t kTmemCols = Cfg::kTmemCols;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_a = smem;
    unsigned char* tiles_b = smem + kStages * kTileA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * (kTileA + kTileB));
    uint64_t* full = bars;                    // [kStages] TMA -> MMA
    uint64_t* empty = bars + kStages;         // [kStages] MMA -> TMA
    uint64_t* acc_full = bars + 2 * kStages;  // [kBufs] MMA -> promotion warps
    uint64_t* acc_free = acc_full + kBufs;    // [kBufs] promotion warps -> MMA (one arrival per warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + kBufs);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row tiles run fastest: the CTAs that share a weight tile are co-resident and the weight comes from DRAM once
    const int n0 = blockIdx.y * kBN, m0 = blockIdx.x * kBM;
    const int k_blocks = K / kBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        for (int b = 0; b < kBufs; ++b) {
            tc::mbar_init(tc::smem_u32(acc_full + b), 1);
            tc::mbar_init(tc::smem_u32(acc_free + b), 4 * Cfg::kQuartets);
        }
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_a);
            tc::tma_prefetch_desc(&map_b);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kStages;
                if (kb >= kStages && !tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                tc::mbar_expect_tx(bar, kTileA + kTileB);
                tc::tma_load_2d(tc::smem_u32(tiles_a + s * kTileA), &map_a, kb * kBK, m0, bar);
                tc::tma_load_2d(tc::smem_u32(tiles_b + s * kTileB), &map_b, kb * kBK, n0, bar);
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc(0, 0, kBM, kBN);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kStages, buf = kb % kBufs, use = kb / kBufs;
                // the accumulator's previous block has been read out
                if (use > 0 && !tc::mbar_wait(tc::smem_u32(acc_free + buf), (use - 1) & 1)) {
                    atomicExch(status, 4);
                    break;
                }
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(tiles_a + s * kTileA), b_addr = tc::smem_u32(tiles_b + s * kTileB);
#pragma unroll
                for (int ks = 0; ks < kBK / 32; ++ks)
                    tc::mma_f8f6f4(tmem_base + buf * kBN, tc::smem_desc_k_sw128(a_addr + ks * 32), tc::smem_desc_k_sw128(b_addr + ks * 32), idesc,
                                   ks > 0);  // every K block starts a fresh sum
                tc::mma_commit(tc::smem_u32(empty + s));
                tc::mma_commit(tc::smem_u32(acc_full + buf));
            }
        }
    } else {
        const int quarter = warp & 3;         // TMEM lanes 32 quarter .. + 31
        const int q = (warp - 2) >> 2;        // which 128 columns = which weight scale block
        const int m = m0 + quarter * 32 + lane;
        const int nb = (n0 >> 7) + q;         // row of the weight scales
        const bool cols_live = n0 + q * 128 < N;
        const int kblocks_w = K / 128;
        float sum[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) sum[i] = 0.f;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int buf = kb % kBufs, use = kb / kBufs;
            ok = tc::mbar_wait(tc::smem_u32(acc_full + buf), use & 1);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) {
                if (lane == 0) atomicExch(status, 3);
                break;
            }
            tc::fence_after_sync();
            const float f = (m < M && cols_live) ? __ldg(sx + static_cast<size_t>(m) * kblocks_w + kb) * __ldg(sw + static_cast<size_t>(nb) * kblocks_w + kb) : 0.f;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN + q * 128;
#pragma unroll
            for (int c = 0; c < 128; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(t_row + c, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sum[c + i] = fmaf(__uint_as_float(r[i]), f, sum[c + i]);
            }
            // this warp is done with the accumulator
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(acc_free + buf));
        }
        if (ok && m < M && cols_live) {
            OutT* dst = y + static_cast<size_t>(m) * N + n0 + q * 128;
#pragma unroll
            for (int v = 0; v < 16; ++v) {
                uint32_t pk[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const OutT o0 = from_float<OutT>(sum[8 * v + 2 * i]), o1 = from_float<OutT>(sum[8 * v + 2 * i + 1]);
                    pk[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) | (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                }
                reinterpret_cast<uint4*>(dst)[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- M <= 16: the operands swap roles (a 128-channel weight tile is the MMA's A operand, the rows are B with N = 16), as
// in the per-channel decode kernel of fp8_linear.cu; the promotion is sixteen values per thread and K block.  Two
// accumulators of 16 columns alternate.  A CTA's 128 channels lie in one weight scale block, so a K block's factor is
// s_w[n0 / 128, kb] * s_x[m, kb] for column m.  Six 18 KB stages: two CTAs (of consecutive launches) share an SM.
constexpr int kDbStages = 6;
constexpr int kDbTileW = 128 * 128, kDbTileX = 16 * 128;
constexpr size_t kDbSmem = static_cast<size_t>(kDbStages) * (kDbTileW + kDbTileX) + 1024 + 256;
constexpr int kDbThreads = 6 * 32;
constexpr int kDbBufs = 8;  // accumulators of 16 columns in flight: the hand-over to the promotion warps takes longer than a K block's MMAs

template <typename OutT>
__global__ void __launch_bounds__(kDbThreads, 2)
    fp8_block_decode_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const float* __restrict__ sx,
                               const float* __restrict__ sw, OutT* __restrict__ y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_w = smem;
    unsigned char* tiles_x = smem + kDbStages * kDbTileW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDbStages * (kDbTileW + kDbTileX));
    uint64_t* full = bars;
    uint64_t* empty = bars + kDbStages;
    uint64_t* acc_full = bars + 2 * kDbStages;  // [kDbBufs]
    uint64_t* acc_free = acc_full + kDbBufs;    // [kDbBufs], four arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + kDbBufs);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 128;
    const int k_blocks = K / 128;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDbStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        for (int b = 0; b < kDbBufs; ++b) {
            tc::mbar_init(tc::smem_u32(acc_full + b), 1);
            tc::mbar_init(tc::smem_u32(acc_free + b), 4);
        }
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), 16 * kDbBufs);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_w);
            tc::tma_prefetch_desc(&map_x);
            // the weights never depend on the kernel before (the activation quantize): request them ahead of the wait
            const int ahead = k_blocks < kDbStages ? k_blocks : kDbStages;
            for (int kb = 0; kb < ahead; ++kb) {
                const uint32_t bar = tc::smem_u32(full + kb);
                tc::mbar_expect_tx(bar, kDbTileW + kDbTileX);
                tc::tma_load_2d(tc::smem_u32(tiles_w + kb * kDbTileW), &map_w, kb * 128, n0, bar);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int kb = 0; kb < ahead; ++kb) tc::tma_load_2d(tc::smem_u32(tiles_x + kb * kDbTileX), &map_x, kb * 128, 0, tc::smem_u32(full + kb));
            for (int kb = ahead; kb < k_blocks; ++kb) {
                const int s = kb % kDbStages;
                if (!tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kDbStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                tc::mbar_expect_tx(bar, kDbTileW + kDbTileX);
                tc::tma_load_2d(tc::smem_u32(tiles_w + s * kDbTileW), &map_w, kb * 128, n0, bar);
                tc::tma_load_2d(tc::smem_u32(tiles_x + s * kDbTileX), &map_x, kb * 128, 0, bar);
            }
        }
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // bounded waits count from the moment the codes exist
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc(0, 0, 128, 16);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kDbStages, buf = kb % kDbBufs, use = kb / kDbBufs;
                if (use > 0 && !tc::mbar_wait(tc::smem_u32(acc_free + buf), (use - 1) & 1)) {
                    atomicExch(status, 4);
                    break;
                }
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kDbStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(tiles_w + s * kDbTileW), x_addr = tc::smem_u32(tiles_x + s * kDbTileX);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    tc::mma_f8f6f4(tmem_base + buf * 16, tc::smem_desc_k_sw128(w_addr + ks * 32), tc::smem_desc_k_sw128(x_addr + ks * 32), idesc, ks > 0);
                tc::mma_commit(tc::smem_u32(empty + s));
                tc::mma_commit(tc::smem_u32(acc_full + buf));
            }
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;  // this thread's output channel
        const int kblocks_w = K / 128;
        const float* swr = sw + static_cast<size_t>(n0 >> 7) * kblocks_w;
        float sum[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) sum[m] = 0.f;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int buf = kb % kDbBufs, use = kb / kDbBufs;
            ok = __all_sync(0xFFFFFFFFu, tc::mbar_wait(tc::smem_u32(acc_full + buf), use & 1));
            if (!ok) {
                if (lane == 0) atomicExch(status, 3);
                break;
            }
            tc::fence_after_sync();
            uint32_t r[16];
            tc::tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * 16, r);
            const float wsc = __ldg(swr + kb);
            tc::tmem_ld_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(acc_free + buf));
#pragma unroll
            for (int m = 0; m < 16; ++m)
                if (m < M) sum[m] = fmaf(__uint_as_float(r[m]), wsc * __ldg(sx + static_cast<size_t>(m) * kblocks_w + kb), sum[m]);
        }
        if (ok && n < N) {
#pragma unroll
            for (int m = 0; m < 16; ++m)
                if (m < M) y[static_cast<size_t>(m) * N + n] = from_float<OutT>(sum[m]);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 16 * kDbBufs);
    }
}

template <typename OutT>
int launch_decode(const uint8_t* qx, const float* sx, const uint8_t* w, const float* sw, OutT* y, int64_t M, int64_t N, int64_t K, int* status,
                  cudaStream_t stream) {
    CUtensorMap map_w, map_x;
    int st = make_tensor_map_2d(&map_w, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    st = make_tensor_map_2d(&map_x, qx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, 16, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    auto kernel = fp8_block_decode_tc_kernel<OutT>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kDbSmem)));
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(N, 128)));
    cfg.blockDim = dim3(kDbThreads);
    cfg.dynamicSmemBytes = kDbSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, sx, sw, y, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), status));
    return EQ_OK;
}

template <typename OutT, int BN>
int launch(const uint8_t* qx, const float* sx, const uint8_t* w, const float* sw, OutT* y, int64_t M, int64_t N, int64_t K, int* status,
           cudaStream_t stream) {
    using Cfg = BlkCfg<BN>;
    CUtensorMap map_a, map_b;
    int st = make_tensor_map_2d(&map_a, qx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    st = make_tensor_map_2d(&map_b, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, BN, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    auto kernel = fp8_block_tc_kernel<OutT, BN>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)));
    dim3 grid(static_cast<unsigned>(ceil_div(M, kBM)), static_cast<unsigned>(ceil_div(N, BN)));
    kernel<<<grid, Cfg::kThreads, Cfg::kSmem, stream>>>(map_a, map_b, sx, sw, y, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), status);
    EQ_LAUNCH_OK("fp8_block_tc_kernel");
    return EQ_OK;
}

template <typename OutT>
int launch_any(const uint8_t* qx, const float* sx, const uint8_t* w, const float* sw, OutT* y, int64_t M, int64_t N, int64_t K, int* status,
               cudaStream_t stream) {
    if (M <= 16) return launch_decode<OutT>(qx, sx, w, sw, y, M, N, K, status, stream);
    return M <= 128 ? launch<OutT, 128>(qx, sx, w, sw, y, M, N, K, status, stream) : launch<OutT, 256>(qx, sx, w, sw, y, M, N, K, status, stream);
}

}  // namespace

// qx [M][K] e4m3 codes, sx [M][K / 128]; w [N][K], sw [N / 128][K / 128]; N and K multiples of 128, y 16-byte aligned.
// status: one word, cleared by the caller, set when a bounded pipeline wait ran out.
int fp8_block_tc_launch(const uint8_t* qx, const float* sx, const uint8_t* w, const float* sw, void* y, int64_t M, int64_t N, int64_t K,
                        int act_dtype, int* status, cudaStream_t stream) {
    return act_dtype == EQ_F16 ? launch_any<__half>(qx, sx, w, sw, static_cast<__half*>(y), M, N, K, status, stream)
                               : launch_any<__nv_bfloat16>(qx, sx, w, sw, static_cast<__nv_bfloat16*>(y), M, N, K, status, stream);
}

}  // namespace eq
