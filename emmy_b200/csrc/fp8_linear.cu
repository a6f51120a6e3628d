// FP8-E4M3 W8A8 linear: per-token dynamic activation quantize, then (sum_k q_x q_w) * s_x[m] * s_w[n].
//
//   quant_fp8_rows_kernel   x[M,K] f16/bf16/f32 -> e4m3 bits + one f32 scale per row.  s = max(amax, 1e-12) / 448
//                           and q = e4m3_rne_satfinite(x / s), both with round-to-nearest f32 division: bit-exact
//                           against the numpy rule the reference spells (emmy/compiler/loader/quant.py:1655-1735).
//   quant_fp8_rows_vec_kernel  the same for few rows (decode): one 1024-thread CTA per row, the row held in registers
//                           between the maximum and the encode, 16-byte loads; also clears the status word.
//   fp8_decode_tc_kernel    M <= 16 (decode-shaped): tcgen05 with the operands' roles swapped -- 128-channel weight tiles
//                           are the MMA's A operand, the rows its B operand with N = 16 -- so one TMA thread streams the
//                           weight, 108 KB CTAs of two consecutive launches share an SM, and the weights are requested
//                           before griddepcontrol.wait (the quantize and the linear are both programmatic dependents).
//   fp8_gemm_tc_kernel      M > 16 (prefill-shaped): tcgen05.mma kind::f8f6f4, 256x256 output tile per CTA, K-major
//                           operands brought by TMA with the 128-byte swizzle through a 3-stage mbarrier ring,
//                           f32 accumulators in TMEM, one producer warp, one MMA warp, eight epilogue warps that read
//                           TMEM with tcgen05.ld, apply both scales and store bf16/f16.
// Both scales are hoisted out of the contraction, as in the reference's own native FP8 path
// (tests/compiler/passes/test_fp8_mma.py:111-120).
#include "tc_common.cuh"

namespace eq {

// ------------------------------------------------------------------------------------------------ activation quantize
template <typename InT>
__device__ __forceinline__ float load_as_float(const InT* p) {
    return to_float(*p);
}

__device__ __forceinline__ uint16_t e4m3x2_satfinite(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));  // first source -> upper byte
    return r;
}

template <typename InT>
__global__ void __launch_bounds__(256) quant_fp8_rows_kernel(const InT* __restrict__ x, int64_t K, uint8_t* __restrict__ q,
                                                             float* __restrict__ scale) {
    __shared__ float warp_max[8];
    __shared__ float row_scale;
    const int64_t row = blockIdx.x;
    const InT* xr = x + row * K;
    float amax = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(load_as_float(xr + k)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = warp_max[0];
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        const float s = __fdiv_rn(fmaxf(m, 1e-12f), 448.0f);
        row_scale = s;
        scale[row] = s;
    }
    __syncthreads();
    const float s = row_scale;
    uint8_t* qr = q + row * K;
    // two elements per thread per step; K is even (K % 16 == 0 is required by the callers)
    for (int64_t k = 2 * threadIdx.x; k < K; k += 2 * blockDim.x) {
        const float a = __fdiv_rn(load_as_float(xr + k), s), b = __fdiv_rn(load_as_float(xr + k + 1), s);
        *reinterpret_cast<uint16_t*>(qr + k) = e4m3x2_satfinite(a, b);
    }
}

// RMSNorm in front of the quantize, in one kernel (the fused prologue the reference's compiler realizes around its
// linears, tests/compiler/realization/cases/fused/norm-linear-*.json): h = dtype(dtype(x * rsqrt(mean(x^2) + eps)) * gamma)
// -- the model's RMSNorm, its normalised value rounded to the activation dtype before the weight multiplies it -- then the
// per-token rule on h.  One CTA per row; the row is read three times (sum of squares, maximum, encode) and stays in L1 / L2
// between them; the normalised row is never written.
template <typename InT>
__global__ void __launch_bounds__(256) rmsnorm_quant_fp8_rows_kernel(const InT* __restrict__ x, const InT* __restrict__ gamma, float eps, int64_t K,
                                                                     uint8_t* __restrict__ q, float* __restrict__ scale, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float part[8];
    __shared__ float bcast;
    const int64_t row = blockIdx.x;
    const InT* xr = x + row * K;
    if (status && row == 0 && threadIdx.x == 0) *status = 0;
    auto block_reduce = [&](float v, bool is_max) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v, off);
            v = is_max ? fmaxf(v, o) : v + o;
        }
        __syncthreads();  // the previous use of part[] is over
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = part[0];
            for (int w = 1; w < 8; ++w) m = is_max ? fmaxf(m, part[w]) : m + part[w];
            bcast = m;
        }
        __syncthreads();
        return bcast;
    };
    float ss = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = load_as_float(xr + k);
        ss = fmaf(v, v, ss);
    }
    const float rstd = rsqrtf(__fdiv_rn(block_reduce(ss, false), static_cast<float>(K)) + eps);
    auto normed = [&](int64_t k) {
        const InT n = from_float<InT>(load_as_float(xr + k) * rstd);
        return to_float(from_float<InT>(to_float(n) * load_as_float(gamma + k)));
    };
    float amax = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(normed(k)));
    const float s = __fdiv_rn(fmaxf(block_reduce(amax, true), 1e-12f), 448.0f);
    if (threadIdx.x == 0) scale[row] = s;
    uint8_t* qr = q + row * K;
    for (int64_t k = 2 * threadIdx.x; k < K; k += 2 * blockDim.x)
        *reinterpret_cast<uint16_t*>(qr + k) = e4m3x2_satfinite(__fdiv_rn(normed(k), s), __fdiv_rn(normed(k + 1), s));
}

// ------------------------------------------------------------------------------------------------ decode-shaped
// M <= 16 on tcgen05 with the operands' roles swapped: a 128-channel tile of the WEIGHT is the MMA's A operand (M = 128),
// the activation rows are B (N = 16), so a K step stages 16 KB of weights and 2 KB of rows and the streaming is done by
// one TMA thread instead of 128 lanes' loads.  Six stages are 108 KB: the CTAs of two consecutive launches share an SM,
// the later one requesting its weights before griddepcontrol.wait while the earlier one computes.  The accumulator is
// [channel = TMEM lane][row = column]; the epilogue applies s_x[m] * s_w[n].
constexpr int kDtTileW = 128 * 128;
constexpr int kDtThreads = 6 * 32;
// BX: activation rows per tile (the MMA's N): 16, 32 or 64 (128 rows leave room for three stages only and measured
// slower than the 128 x 128 tile below: 33-35 us against 29-30 us).  As many stages as leave room for a second CTA on the SM.
template <int BX>
struct DtCfg {
    static constexpr int kTileX = BX * 128;
    static constexpr int kStages = BX == 16 ? 6 : BX == 32 ? 5 : 4;
    static constexpr size_t kSmem = static_cast<size_t>(kStages) * (kDtTileW + kTileX) + 1024 + 256;
    static constexpr uint32_t kTmemCols = BX < 32 ? 32 : BX;
};

template <typename OutT, int BX>
__global__ void __launch_bounds__(kDtThreads, 2)
    fp8_decode_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const float* __restrict__ sx,
                         const float* __restrict__ sw, OutT* __restrict__ y, int M, int N, int K, int* __restrict__ status) {
    constexpr int kDtStages = DtCfg<BX>::kStages, kDtTileX = DtCfg<BX>::kTileX;
    constexpr uint32_t kDtTmemCols = DtCfg<BX>::kTmemCols;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_w = smem;
    unsigned char* tiles_x = smem + kDtStages * kDtTileW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDtStages * (kDtTileW + kDtTileX));
    uint64_t* full = bars;
    uint64_t* empty = bars + kDtStages;
    uint64_t* acc_ready = bars + 2 * kDtStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kDtStages + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 128;
    const int k_blocks = K / 128;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDtStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), kDtTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_w);
            tc::tma_prefetch_desc(&map_x);
            // the weights never depend on the kernel before (the activation quantize): request them ahead of the wait
            const int ahead = k_blocks < kDtStages ? k_blocks : kDtStages;
            for (int kb = 0; kb < ahead; ++kb) {
                const uint32_t bar = tc::smem_u32(full + kb);
                tc::mbar_expect_tx(bar, kDtTileW + kDtTileX);
                tc::tma_load_2d(tc::smem_u32(tiles_w + kb * kDtTileW), &map_w, kb * 128, n0, bar);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int kb = 0; kb < ahead; ++kb) tc::tma_load_2d(tc::smem_u32(tiles_x + kb * kDtTileX), &map_x, kb * 128, 0, tc::smem_u32(full + kb));
            for (int kb = ahead; kb < k_blocks; ++kb) {
                const int s = kb % kDtStages;
                if (!tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kDtStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                tc::mbar_expect_tx(bar, kDtTileW + kDtTileX);
                tc::tma_load_2d(tc::smem_u32(tiles_w + s * kDtTileW), &map_w, kb * 128, n0, bar);
                tc::tma_load_2d(tc::smem_u32(tiles_x + s * kDtTileX), &map_x, kb * 128, 0, bar);
            }
        }
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // bounded waits count from the moment the codes exist
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc(0, 0, 128, BX);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kDtStages;
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kDtStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(tiles_w + s * kDtTileW), x_addr = tc::smem_u32(tiles_x + s * kDtTileX);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    tc::mma_f8f6f4(tmem_base, tc::smem_desc_k_sw128(w_addr + ks * 32), tc::smem_desc_k_sw128(x_addr + ks * 32), idesc, kb > 0 || ks > 0);
                tc::mma_commit(tc::smem_u32(empty + s));
            }
            tc::mma_commit(tc::smem_u32(acc_ready));
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;  // this thread's output channel
        const bool ok = tc::mbar_wait(tc::smem_u32(acc_ready), 0);
        if (!ok && lane == 0) atomicExch(status, 3);
        tc::fence_after_sync();
        if (ok) {
            const float wsc = n < N ? sw[n] : 0.f;
#pragma unroll
            for (int c = 0; c < BX; c += 16) {
                uint32_t r[16];
                tc::tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c, r);
                tc::tmem_ld_wait();
                if (n < N) {
#pragma unroll
                    for (int m = 0; m < 16; ++m)
                        if (c + m < M) y[static_cast<size_t>(c + m) * N + n] = from_float<OutT>(__uint_as_float(r[m]) * sx[c + m] * wsc);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, kDtTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------ prefill-shaped
// A CTA computes a 256 x 256 output tile as two 128-row MMAs that share one B tile in shared memory: per byte
// brought in from L2 that is 256 flop, against 170 for a 128 x 256 tile, and L2 -> SM bandwidth is what bounds
// this kernel (a 128 x 256 tile needs ~19 TB/s of it at the tensor peak).  The two f32 accumulators fill TMEM.
// Calls with at most 128 rows (one row tile) run 128 x 128 tiles instead: twice as many CTAs stream the weight, deeper
// stages, and two such CTAs fit an SM.
constexpr int kBK = 128;  // K step in bytes = e4m3 elements
constexpr int kEpilogueWarps = 8;
constexpr int kGemmThreads = (2 + kEpilogueWarps) * 32;

template <int HALVES, int BN>
struct Fp8Cfg {
    static constexpr int kBM = 128 * HALVES;
    static constexpr int kTileA = kBM * kBK, kTileB = BN * kBK;
    static constexpr int kStages = HALVES == 2 ? 3 : 6;
    static constexpr size_t kSmem = static_cast<size_t>(kStages) * (kTileA + kTileB) + 1024 /*alignment*/ + 256 /*barriers*/ + BN * sizeof(float) /*weight scales of the tile*/;
    static constexpr uint32_t kTmemCols = HALVES * BN;
};

template <typename OutT, int HALVES, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    fp8_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const float* __restrict__ sx, const float* __restrict__ sw, OutT* __restrict__ y, int M, int N, int K,
                       int* __restrict__ status) {
    using Cfg = Fp8Cfg<HALVES, BN>;
    constexpr int kBM = Cfg::kBM, kBN = BN, kTileA = Cfg::kTileA, kTileB = Cfg::kTileB, kStages = Cfg::kStages;
    constexpr uint32_t kTmemCols = Cfg::kTmemCols;
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_a = smem;
    unsigned char* tiles_b = smem + kStages * kTileA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * (kTileA + kTileB));
    uint64_t* full = bars;                 // [kStages] TMA -> MMA
    uint64_t* empty = bars + kStages;      // [kStages] MMA -> TMA
    uint64_t* acc_ready = bars + 2 * kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
    float* sw_tile = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 256);  // the tile's BN weight scales

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row tiles run fastest: the CTAs that share a weight tile are co-resident and the weight comes from DRAM once
    const int n0 = blockIdx.y * kBN, m0 = blockIdx.x * kBM;
    const int k_blocks = K / kBK;
    const bool two_halves = HALVES == 2 && M - m0 > 128;  // the second 128 rows hold real rows

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), kTmemCols);
    for (int i = threadIdx.x; i < kBN; i += kGemmThreads) sw_tile[i] = n0 + i < N ? sw[n0 + i] : 0.f;
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer
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
        // ---- MMA issuer
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc(0, 0, 128, kBN);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kStages;
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(tiles_a + s * kTileA), b_addr = tc::smem_u32(tiles_b + s * kTileB);
#pragma unroll
                for (int ks = 0; ks < kBK / 32; ++ks) {
                    // 32 bytes of K per instruction: step the descriptors' start address inside the swizzle atom
                    const uint64_t db = tc::smem_desc_k_sw128(b_addr + ks * 32);
                    tc::mma_f8f6f4(tmem_base, tc::smem_desc_k_sw128(a_addr + ks * 32), db, idesc, kb > 0 || ks > 0);
                    if (two_halves)
                        tc::mma_f8f6f4(tmem_base + kBN, tc::smem_desc_k_sw128(a_addr + 128 * kBK + ks * 32), db, idesc, kb > 0 || ks > 0);
                }
                tc::mma_commit(tc::smem_u32(empty + s));  // stage is free once these MMAs have read it
            }
            tc::mma_commit(tc::smem_u32(acc_ready));  // on a broken pipeline too, so that the epilogue does not sit out its wait
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes 32 (w % 4) .. +31.  Two row halves: warps 2..5 take rows 0..127,
        //      6..9 rows 128..255; one row half: the two quartets take half of the columns each.
        const int quarter = warp & 3;
        const int quartet = (warp - 2) >> 2;
        const int half = HALVES == 2 ? quartet : 0;
        const int c_begin = HALVES == 2 ? 0 : quartet * (kBN / 2);
        const int c_end = HALVES == 2 ? kBN : c_begin + kBN / 2;
        const int m = m0 + half * 128 + quarter * 32 + lane;
        const bool ok = tc::mbar_wait(tc::smem_u32(acc_ready), 0);
        if (!ok && lane == 0) atomicExch(status, 3);
        tc::fence_after_sync();
        if (ok && (half == 0 || two_halves)) {
            const float row_scale = m < M ? sx[m] : 0.f;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * kBN + c, r);
                tc::tmem_ld_wait();
                if (m < M) {
                    OutT* dst = y + static_cast<size_t>(m) * N + n0 + c;
                    if (n0 + c + 32 <= N) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 wsc = *reinterpret_cast<const float2*>(sw_tile + c + 2 * i);  // same address in every lane: a broadcast
                            const float v0 = __uint_as_float(r[2 * i]) * row_scale * wsc.x;
                            const float v1 = __uint_as_float(r[2 * i + 1]) * row_scale * wsc.y;
                            const OutT o0 = from_float<OutT>(v0), o1 = from_float<OutT>(v1);
                            packed[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) |
                                        (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                        }
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c + i < N) dst[i] = from_float<OutT>(__uint_as_float(r[i]) * row_scale * sw_tile[c + i]);
                    }
                }
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

// Few rows (decode): one CTA of 1024 threads per row; the row stays in registers between the two passes.
// kVecs 16-byte vectors per thread cover K <= 1024 * kVecs * (16 / sizeof(InT)) elements.
template <typename InT, int kVecs>
__global__ void __launch_bounds__(1024) quant_fp8_rows_vec_kernel(const InT* __restrict__ x, int64_t K, uint8_t* __restrict__ q,
                                                                  float* __restrict__ scale, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the linear behind this may start fetching weights
    // launched as a programmatic dependent itself: the kernel before it (usually the previous linear on this workspace)
    // may still read the codes, scales and status word this one rewrites
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int kPer = 16 / sizeof(InT);  // elements per 16-byte vector
    __shared__ float warp_max[32];
    __shared__ float row_scale;
    const int64_t row = blockIdx.x;
    if (status && row == 0 && threadIdx.x == 0) *status = 0;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * K);
    const int n_vec = static_cast<int>(K / kPer);
    uint4 v[kVecs];
    float amax = 0.f;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
        const int idx = threadIdx.x + u * 1024;
        v[u] = make_uint4(0, 0, 0, 0);
        if (idx < n_vec) v[u] = __ldg(xr + idx);
        const InT* e = reinterpret_cast<const InT*>(&v[u]);
#pragma unroll
        for (int i = 0; i < kPer; ++i) amax = fmaxf(amax, fabsf(to_float(e[i])));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = warp_max[threadIdx.x];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        if (threadIdx.x == 0) {
            const float s = __fdiv_rn(fmaxf(m, 1e-12f), 448.0f);
            row_scale = s;
            scale[row] = s;
        }
    }
    __syncthreads();
    const float s = row_scale;
    uint8_t* qr = q + row * K;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
        const int idx = threadIdx.x + u * 1024;
        if (idx < n_vec) {
            const InT* e = reinterpret_cast<const InT*>(&v[u]);
            uint16_t out[kPer / 2];
#pragma unroll
            for (int i = 0; i < kPer / 2; ++i) out[i] = e4m3x2_satfinite(__fdiv_rn(to_float(e[2 * i]), s), __fdiv_rn(to_float(e[2 * i + 1]), s));
            if constexpr (kPer == 8)
                *reinterpret_cast<uint2*>(qr + static_cast<size_t>(idx) * kPer) = *reinterpret_cast<const uint2*>(out);
            else
                *reinterpret_cast<uint32_t*>(qr + static_cast<size_t>(idx) * kPer) = *reinterpret_cast<const uint32_t*>(out);
        }
    }
}

// Static activation scale: every row divides by the same calibrated scale.
template <typename InT>
__global__ void __launch_bounds__(256) quant_fp8_static_kernel(const InT* __restrict__ x, int64_t total, const float* __restrict__ input_scale,
                                                               int64_t M, uint8_t* __restrict__ q, float* __restrict__ scale, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float s = input_scale[0];
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx < M) scale[idx] = s;
    if (status && idx == 0) *status = 0;
    const int64_t k = 2 * idx;
    if (k < total) *reinterpret_cast<uint16_t*>(q + k) = e4m3x2_satfinite(__fdiv_rn(to_float(x[k]), s), __fdiv_rn(to_float(x[k + 1]), s));
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace eq

using namespace eq;

template <typename InT>
static int quant_rows_launch(const InT* x, int64_t M, int64_t K, uint8_t* q, float* scale, int* status, cudaStream_t stream) {
    constexpr int kPer = 16 / sizeof(InT);
    const bool vec = M <= 64 && K % kPer == 0 && aligned(x, 16) && aligned(q, 8) && K / kPer <= 4 * 1024;
    if (vec) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(M));
        cfg.blockDim = dim3(1024);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // resident, past its launch latency, when the kernel before it ends
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (K / kPer <= 1024) EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_rows_vec_kernel<InT, 1>, x, K, q, scale, status));
        else if (K / kPer <= 2048) EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_rows_vec_kernel<InT, 2>, x, K, q, scale, status));
        else EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_fp8_rows_vec_kernel<InT, 4>, x, K, q, scale, status));
        return EQ_OK;
    }
    if (status) EQ_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), stream));
    quant_fp8_rows_kernel<InT><<<static_cast<unsigned>(M), 256, 0, stream>>>(x, K, q, scale);
    EQ_LAUNCH_OK("quant_fp8_rows_kernel");
    return EQ_OK;
}

// Quantizes the rows and, when `status` is given, clears that word on the way (the linear's status word).
static int quant_fp8_rows(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, int* status, cudaStream_t stream) {
    switch (in_dtype) {
        case EQ_F16: return quant_rows_launch(static_cast<const __half*>(x), M, K, q, scale, status, stream);
        case EQ_BF16: return quant_rows_launch(static_cast<const __nv_bfloat16*>(x), M, K, q, scale, status, stream);
        case EQ_F32: return quant_rows_launch(static_cast<const float*>(x), M, K, q, scale, status, stream);
        default: return fail(EQ_ERR_BAD_ARG, "eq_quant_fp8_per_token: unknown dtype %d", in_dtype);
    }
}

extern "C" int eq_quant_fp8_per_token(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(M >= 0 && K > 0, EQ_ERR_BAD_ARG, "eq_quant_fp8_per_token: bad extents M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(x && q && scale, EQ_ERR_BAD_ARG, "eq_quant_fp8_per_token: null pointer");
    EQ_REQUIRE(K % 2 == 0 && aligned(q, 2), EQ_ERR_BAD_ALIGN, "eq_quant_fp8_per_token: K must be even and q 2-byte aligned");
    return quant_fp8_rows(x, M, K, in_dtype, q, scale, nullptr, stream);
}

extern "C" size_t eq_fp8_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return align_up(static_cast<size_t>(M) * K, 256) + align_up(static_cast<size_t>(M) * sizeof(float), 256) + 256;
}

template <typename OutT, int HALVES, int BN>
static int fp8_tc_launch(const uint8_t* w, const float* sw, int64_t N, int64_t K, const uint8_t* qx, const float* sx, int64_t M, OutT* y,
                         int* status, cudaStream_t stream) {
    using Cfg = Fp8Cfg<HALVES, BN>;
    CUtensorMap map_a, map_b;
    int st = make_tensor_map_2d(&map_a, qx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, Cfg::kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    st = make_tensor_map_2d(&map_b, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, BN, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    auto kernel = fp8_gemm_tc_kernel<OutT, HALVES, BN>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)));
    dim3 grid(static_cast<unsigned>(ceil_div(M, Cfg::kBM)), static_cast<unsigned>(ceil_div(N, BN)));
    kernel<<<grid, kGemmThreads, Cfg::kSmem, stream>>>(map_a, map_b, sx, sw, y, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                                                       status);
    EQ_LAUNCH_OK("fp8_gemm_tc_kernel");
    return EQ_OK;
}

template <typename OutT>
static int fp8_linear_launch(const uint8_t* w, const float* sw, int64_t N, int64_t K, const uint8_t* qx, const float* sx, int64_t M,
                             OutT* y, int* status, cudaStream_t stream) {
    if (M <= 64) {
        // (measured at K = 5120, N = 17408: 18.4 / 19.0 / 19.8 us at M = 1 / 8 / 16 against 21.0 / 24.4 / 32.7 us for the
        // mma.sync bandwidth kernel this replaced)
        CUtensorMap map_w, map_x;
        const int bx = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        int st = make_tensor_map_2d(&map_w, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EQ_OK) return st;
        st = make_tensor_map_2d(&map_x, qx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, bx, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EQ_OK) return st;
        auto run = [&](auto kernel, size_t smem) -> int {
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(N, 128)));
            cfg.blockDim = dim3(kDtThreads);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, sx, sw, y, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), status));
            return EQ_OK;
        };
        if (bx == 16) return run(fp8_decode_tc_kernel<OutT, 16>, DtCfg<16>::kSmem);
        if (bx == 32) return run(fp8_decode_tc_kernel<OutT, 32>, DtCfg<32>::kSmem);
        return run(fp8_decode_tc_kernel<OutT, 64>, DtCfg<64>::kSmem);
    }
    if (M <= 128) return fp8_tc_launch<OutT, 1, 128>(w, sw, N, K, qx, sx, M, y, status, stream);
    return fp8_tc_launch<OutT, 2, 256>(w, sw, N, K, qx, sx, M, y, status, stream);
}

static int fp8_linear_any(const char* who, const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x,
                          const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                          const void* gamma = nullptr, float eps = 0.f) {
    EQ_REQUIRE(N > 0 && K > 0 && M >= 0, EQ_ERR_BAD_ARG, "%s: bad extents M=%lld K=%lld N=%lld", who, (long long)M, (long long)K, (long long)N);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(weight && weight_scale && x && y, EQ_ERR_BAD_ARG, "%s: null pointer", who);
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "%s: activations must be f16 or bf16", who);
    EQ_REQUIRE(K % 128 == 0 && N % 16 == 0, EQ_ERR_UNSUPPORTED, "%s: needs K %% 128 == 0 and N %% 16 == 0 (K=%lld N=%lld)", who, (long long)K,
               (long long)N);
    EQ_REQUIRE(aligned(weight, 16) && aligned(y, 16), EQ_ERR_BAD_ALIGN, "%s: weight and y must be 16-byte aligned", who);
    EQ_REQUIRE(workspace && workspace_bytes >= eq_fp8_workspace_bytes(M, K), EQ_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who,
               eq_fp8_workspace_bytes(M, K), workspace_bytes);
    EQ_REQUIRE(aligned(workspace, 256), EQ_ERR_BAD_ALIGN, "%s: workspace must be 256-byte aligned", who);
    uint8_t* qx = static_cast<uint8_t*>(workspace);
    float* sx = reinterpret_cast<float*>(qx + align_up(static_cast<size_t>(M) * K, 256));
    int* status = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(sx) + align_up(static_cast<size_t>(M) * sizeof(float), 256));
    int st = EQ_OK;
    if (gamma) {
        // RMSNorm and the per-token quantize in one kernel (a programmatic dependent, like the plain quantize)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(M));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = M <= 128 ? 1 : 0;
        if (act_dtype == EQ_F16)
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, rmsnorm_quant_fp8_rows_kernel<__half>, static_cast<const __half*>(x), static_cast<const __half*>(gamma), eps, K,
                                          qx, sx, status));
        else
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, rmsnorm_quant_fp8_rows_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x),
                                          static_cast<const __nv_bfloat16*>(gamma), eps, K, qx, sx, status));
    } else if (input_scale) {
        const int64_t total = M * K;
        const unsigned grid = static_cast<unsigned>(ceil_div(total / 2 > M ? total / 2 : M, 256));
        if (act_dtype == EQ_F16) quant_fp8_static_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), total, input_scale, M, qx, sx, status);
        else quant_fp8_static_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), total, input_scale, M, qx, sx, status);
        EQ_LAUNCH_OK("quant_fp8_static_kernel");
    } else {
        st = quant_fp8_rows(x, M, K, act_dtype, qx, sx, status, stream);  // also clears the status word
    }
    if (st != EQ_OK) return st;
    if (act_dtype == EQ_F16) return fp8_linear_launch<__half>(weight, weight_scale, N, K, qx, sx, M, static_cast<__half*>(y), status, stream);
    return fp8_linear_launch<__nv_bfloat16>(weight, weight_scale, N, K, qx, sx, M, static_cast<__nv_bfloat16*>(y), status, stream);
}

extern "C" int eq_fp8_linear(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, int64_t M,
                             int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream_) {
    return fp8_linear_any("eq_fp8_linear", weight, weight_scale, N, K, x, nullptr, M, act_dtype, y, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream_));
}

extern "C" int eq_fp8_linear_static(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x,
                                    const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                                    void* stream_) {
    EQ_REQUIRE(input_scale, EQ_ERR_BAD_ARG, "eq_fp8_linear_static: null input_scale");
    return fp8_linear_any("eq_fp8_linear_static", weight, weight_scale, N, K, x, input_scale, M, act_dtype, y, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream_));
}

extern "C" int eq_fp8_linear_rmsnorm(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, const void* gamma,
                                     float eps, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream_) {
    EQ_REQUIRE(gamma, EQ_ERR_BAD_ARG, "eq_fp8_linear_rmsnorm: null norm weight");
    return fp8_linear_any("eq_fp8_linear_rmsnorm", weight, weight_scale, N, K, x, nullptr, M, act_dtype, y, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream_), gamma, eps);
}

extern "C" int eq_fp8_status(const void* workspace, int64_t M, int64_t K, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && K > 0, EQ_ERR_BAD_ARG, "eq_fp8_status: bad arguments");
    const unsigned char* base = static_cast<const unsigned char*>(workspace);
    const int* status = reinterpret_cast<const int*>(base + align_up(static_cast<size_t>(M) * K, 256) +
                                                     align_up(static_cast<size_t>(M) * sizeof(float), 256));
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_fp8_status: a bounded pipeline wait ran out (code %d)", host);
    return EQ_OK;
}
