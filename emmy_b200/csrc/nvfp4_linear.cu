// NVFP4 (e2m1 codes, e4m3 scale per 16 elements of K, f32 global scale) W4A4 linear.
//
//   nvfp4_amax_kernel / nvfp4_scale2_kernel  calibrate-on-the-sample input scale: max(amax, 1e-12) / (6 * 448)
//   quant_nvfp4_act_kernel   static-scale activation quantize, the f32 algebra the reference spells
//                            (emmy/compiler/loader/quant.py:1968-2139, tests/compiler/loader/test_quant.py:1776-1784):
//                            ratio = (amax_blk * f32(1/6)) * f32(1/s2); sbits = e4m3(ratio); fused = dec(sbits) * s2;
//                            codes = e2m1(blk / max(fused, 1e-12)), all round-to-nearest f32.  Bit-exact.
//   nvfp4_tile_scales_kernel re-tiles a plain [rows, K/16] scale matrix into the 512-byte atoms the tensor core's
//                            scale-factor copy reads (load time for weights, inside the quantize for activations)
//   nvfp4_gemm_tc_kernel / nvfp4_gemm_tc_wide_kernel (128 x 128 tiles for M <= 128, 256 x 224 tiles above)
//                            tcgen05.mma kind::mxf4nvf4.block_scale.scale_vec::4X: codes come by TMA (128-byte
//                            swizzle, 256 elements of K per row), scale atoms by bulk copy and then tcgen05.cp into
//                            TMEM, f32 accumulators in TMEM; the epilogue multiplies by the two global scales.
// The hardware applies the raw e4m3 block scale and the global scales are factored out into the epilogue, whereas
// the reference's value path applies f16(block * global) per element: a relative difference of at most 2^-11 per
// operand, far inside the output tolerance; the dequantised-weight export (eq_dequant_nvfp4) stays bit-exact.
#include "tc_common.cuh"

namespace eq {

// ------------------------------------------------------------------------------------------------ calibration
template <typename InT>
__global__ void nvfp4_amax_kernel(const InT* __restrict__ x, int64_t n, unsigned int* __restrict__ amax_bits) {
    float m = 0.f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        m = fmaxf(m, fabsf(to_float(x[i])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));  // non-negative floats order like their bits
}
__global__ void nvfp4_scale2_kernel(const unsigned int* __restrict__ amax_bits, float* __restrict__ scale2) {
    const double amax = fmax(static_cast<double>(__uint_as_float(*amax_bits)), 1e-12);
    *scale2 = static_cast<float>(amax / (6.0 * 448.0));
}

// ------------------------------------------------------------------------------------------------ scale atoms
// Tiled scale layout: [row block of 128][k block of 64 elements][512 B]; inside an atom the scale of (row r, 16-block
// i of the k block) sits at byte (r % 32) * 16 + (r / 32) * 4 + i.  Rows beyond `rows` are zero.
__device__ __forceinline__ size_t sf_tiled_offset(int64_t row, int64_t blk16, int64_t k64_blocks) {
    const int64_t rb = row >> 7, r = row & 127, kb = blk16 >> 2, i = blk16 & 3;
    return static_cast<size_t>((rb * k64_blocks + kb) * 512 + (r & 31) * 16 + (r >> 5) * 4 + i);
}

__global__ void nvfp4_tile_scales_kernel(const uint8_t* __restrict__ plain, int64_t rows, int64_t K, uint8_t* __restrict__ tiled) {
    const int64_t blocks16 = K / 16, k64 = K / 64;
    const int64_t padded_rows = (rows + 127) / 128 * 128;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= padded_rows * blocks16) return;
    const int64_t row = idx / blocks16, b = idx % blocks16;
    tiled[sf_tiled_offset(row, b, k64)] = row < rows ? plain[row * blocks16 + b] : 0;
}

// The same atoms grouped for 224-row column tiles (the prefill kernel's B tile): [tile of 224 rows][two row blocks: rows
// 0..127 and 128..223 of the tile, the rest zero][k block of 64][512 B].
constexpr int kWideBN = 224;
__global__ void nvfp4_tile_scales_wide_kernel(const uint8_t* __restrict__ plain, int64_t rows, int64_t K, uint8_t* __restrict__ tiled) {
    const int64_t blocks16 = K / 16, k64 = K / 64;
    const int64_t tiles = (rows + kWideBN - 1) / kWideBN;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= tiles * 256 * blocks16) return;
    const int64_t t = idx / (256 * blocks16), rem = idx - t * (256 * blocks16);
    const int64_t r256 = rem / blocks16, b = rem - r256 * blocks16;
    const int64_t src = t * kWideBN + r256;
    const int64_t blk = r256 >> 7, r = r256 & 127;
    const size_t off = static_cast<size_t>(((t * 2 + blk) * k64 + (b >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b & 3));
    tiled[off] = (r256 < kWideBN && src < rows) ? plain[src * blocks16 + b] : 0;
}

// ------------------------------------------------------------------------------------------------ activation quantize
__device__ __forceinline__ uint8_t e4m3_satfinite(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
    return static_cast<uint8_t>(r & 0xFF);
}
// two f32 -> one byte: low nibble = code(lo), high nibble = code(hi)
__device__ __forceinline__ uint8_t e2m1x2_satfinite(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return static_cast<uint8_t>(r);
}

// One thread per 16-element block.  Writes the packed codes [M, K/2], the plain scales [M, K/16] (optional) and the
// tiled scales (optional).  `status`, when given, is cleared for the linear that follows in the stream; that linear
// may be launched as a programmatic dependent and fetch its weights while this kernel runs.
template <typename InT>
__global__ void quant_nvfp4_act_kernel(const InT* __restrict__ x, int64_t M, int64_t K, const float* __restrict__ scale2,
                                       uint8_t* __restrict__ codes, uint8_t* __restrict__ sf_plain, uint8_t* __restrict__ sf_tiled,
                                       int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // launched as a programmatic dependent itself when it runs inside the linear: the kernel before it (usually the
    // previous linear on this workspace) still reads the codes and the status word this one rewrites
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t blocks16 = K / 16;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (status && idx == 0) *status = 0;
    if (idx >= M * blocks16) return;
    const int64_t row = idx / blocks16, b = idx % blocks16;
    const InT* src = x + row * K + b * 16;
    float v[16];
    if (sizeof(InT) == 2 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        uint4 raw[2] = {reinterpret_cast<const uint4*>(src)[0], reinterpret_cast<const uint4*>(src)[1]};
        const InT* e = reinterpret_cast<const InT*>(raw);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = to_float(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = to_float(src[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float s2 = scale2[0];
    const float ratio = __fmul_rn(__fmul_rn(amax, __fdiv_rn(1.0f, 6.0f)), __fdiv_rn(1.0f, s2));
    const uint8_t sbits = e4m3_satfinite(ratio);
    const float fused = __fmul_rn(e4m3_to_float(sbits), s2);
    const float div = fmaxf(fused, 1e-12f);
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint8_t byte = e2m1x2_satfinite(__fdiv_rn(v[2 * i], div), __fdiv_rn(v[2 * i + 1], div));
        w[i >> 2] |= static_cast<uint32_t>(byte) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(codes + row * (K / 2) + b * 8) = make_uint2(w[0], w[1]);
    if (sf_plain) sf_plain[idx] = sbits;
    if (sf_tiled) sf_tiled[sf_tiled_offset(row, b, K / 64)] = sbits;
}

// RMSNorm in front of the static quantize, in one kernel: h = dtype(dtype(x * rsqrt(mean(x^2) + eps)) * gamma), the model's
// RMSNorm (its normalised value rounded to the activation dtype before the weight multiplies it), then the block rule on h.
// One CTA per row: the sum of squares first, then one thread per 16-element block; the normalised row is never written.
template <typename InT>
__global__ void __launch_bounds__(256) rmsnorm_quant_nvfp4_rows_kernel(const InT* __restrict__ x, const InT* __restrict__ gamma, float eps, int64_t K,
                                                                       const float* __restrict__ scale2, uint8_t* __restrict__ codes,
                                                                       uint8_t* __restrict__ sf_tiled, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float part[8];
    const int64_t row = blockIdx.x;
    const InT* xr = x + row * K;
    if (status && row == 0 && threadIdx.x == 0) *status = 0;
    float ss = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = to_float(xr[k]);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += part[w];
    const float rstd = rsqrtf(__fdiv_rn(total, static_cast<float>(K)) + eps);
    const float s2 = scale2[0];
    for (int64_t b = threadIdx.x; b < K / 16; b += blockDim.x) {
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const InT n = from_float<InT>(to_float(xr[b * 16 + i]) * rstd);
            v[i] = to_float(from_float<InT>(to_float(n) * to_float(gamma[b * 16 + i])));
            amax = fmaxf(amax, fabsf(v[i]));
        }
        const float ratio = __fmul_rn(__fmul_rn(amax, __fdiv_rn(1.0f, 6.0f)), __fdiv_rn(1.0f, s2));
        const uint8_t sbits = e4m3_satfinite(ratio);
        const float div = fmaxf(__fmul_rn(e4m3_to_float(sbits), s2), 1e-12f);
        uint32_t w[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint8_t byte = e2m1x2_satfinite(__fdiv_rn(v[2 * i], div), __fdiv_rn(v[2 * i + 1], div));
            w[i >> 2] |= static_cast<uint32_t>(byte) << (8 * (i & 3));
        }
        *reinterpret_cast<uint2*>(codes + row * (K / 2) + b * 8) = make_uint2(w[0], w[1]);
        sf_tiled[sf_tiled_offset(row, b, K / 64)] = sbits;
    }
}

// ------------------------------------------------------------------------------------------------ weight quantize
// The two-level weight quantizer (emmy/compiler/loader/quant.py:206-237), one thread per 16-element block:
// block scale = amax_blk / 6 stored as e4m3 relative to scale_2; the divisor is the FUSED scale f16(dec(bits) * scale_2);
// codes = e2m1(blk / fused) with zero where the fused scale is zero.  Every step an f32 round-to-nearest operation, as
// numpy does them: bit-exact with the reference's output.
template <typename InT>
__global__ void quant_nvfp4_weight_kernel(const InT* __restrict__ w, int64_t N, int64_t K, const float* __restrict__ scale2,
                                          uint8_t* __restrict__ codes, uint8_t* __restrict__ sf_plain) {
    const int64_t blocks16 = K / 16;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= N * blocks16) return;
    const InT* src = w + idx * 16;
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        v[i] = to_float(src[i]);
        amax = fmaxf(amax, fabsf(v[i]));
    }
    const float s2 = scale2[0];
    const uint8_t sbits = e4m3_satfinite(__fdiv_rn(__fdiv_rn(amax, 6.0f), s2));
    const float fused = __half2float(__float2half_rn(__fmul_rn(e4m3_to_float(sbits), s2)));
    uint32_t out[2] = {0, 0};
    if (fused != 0.f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint8_t byte = e2m1x2_satfinite(__fdiv_rn(v[2 * i], fused), __fdiv_rn(v[2 * i + 1], fused));
            out[i >> 2] |= static_cast<uint32_t>(byte) << (8 * (i & 3));
        }
    }
    *reinterpret_cast<uint2*>(codes + idx * 8) = make_uint2(out[0], out[1]);
    sf_plain[idx] = sbits;
}

// ------------------------------------------------------------------------------------------------ tensor path
constexpr int kBM = 128;
constexpr int kBKBytes = 128;                 // 256 e2m1 elements of K per stage row
constexpr int kTileA = kBM * kBKBytes;
constexpr int kSfA = 4 * 512;                 // four k64 atoms per stage, one row block
constexpr int kGemmThreads = 192;

// BN = 256 for prefill-shaped calls; BN = 128 when there is a single row tile, so that twice as many CTAs stream the weight.
template <int BN>
struct Fp4Cfg {
    static constexpr int kTileB = BN * kBKBytes;
    static constexpr int kSfB = (BN / 128) * 4 * 512;  // one or two row blocks
    static constexpr int kStageBytes = kTileA + kTileB + kSfA + kSfB;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr size_t kSmem = static_cast<size_t>(kStages) * kStageBytes + 1024 + 256;
    static constexpr uint32_t kTmemCols = BN == 256 ? 512 : 256;  // accumulator columns + 16 (SFA) + 16 or 32 (SFB), as a power of two
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <typename OutT, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    nvfp4_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, const float* __restrict__ gx,
                         const float* __restrict__ gw, OutT* __restrict__ y, int M, int N, int K, int* __restrict__ status) {
    using Cfg = Fp4Cfg<BN>;
    constexpr int kBN = BN, kTileB = Cfg::kTileB, kSfB = Cfg::kSfB, kStages = Cfg::kStages;
    constexpr uint32_t kTmemCols = Cfg::kTmemCols;
    constexpr bool kTwoBlocks = BN == 256;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_a = smem;
    unsigned char* tiles_b = tiles_a + kStages * kTileA;
    unsigned char* sfs_a = tiles_b + kStages * kTileB;
    unsigned char* sfs_b = sfs_a + kStages * kSfA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sfs_b + kStages * kSfB);
    uint64_t* full = bars;
    uint64_t* empty = bars + kStages;
    uint64_t* acc_ready = bars + 2 * kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row tiles run fastest: the CTAs that share a weight tile are co-resident and the weight comes from DRAM once
    const int n0 = blockIdx.y * kBN, m0 = blockIdx.x * kBM;
    const int k_blocks = K / 256;   // stages of 256 elements
    const int k64_blocks = K / 64;  // scale atoms along K
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + kBN;        // 4 columns per k64 step
    const uint32_t tmem_sfb = tmem_base + kBN + 16;   // 8 columns per k64 step

    // The kernel may have been launched as a programmatic dependent of the activation quantize: the weights and their
    // scales never depend on it, so the first ring of weight stages is requested before the dependency is awaited;
    // every other role waits first, so that its bounded waits count from the moment the codes exist.
    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_a);
            tc::tma_prefetch_desc(&map_b);
            const int rb_a = m0 / 128, rb_b = n0 / 128;
            const int n_rb = (N + 127) / 128;
            // the second row block of B may lie beyond N (N not a multiple of 256): it is then not copied
            const bool second = kTwoBlocks && rb_b + 1 < n_rb;
            constexpr int kSfBlock = 4 * 512;
            auto weights = [&](int kb, int s, uint32_t bar) {
                tc::mbar_expect_tx(bar, kTileA + kTileB + kSfA + (second ? 2 * kSfBlock : kSfBlock));
                tc::tma_load_2d(tc::smem_u32(tiles_b + s * kTileB), &map_b, kb * kBKBytes, n0, bar);
                bulk_g2s(tc::smem_u32(sfs_b + s * kSfB), sfb + (static_cast<size_t>(rb_b) * k64_blocks + kb * 4) * 512, kSfBlock, bar);
                if (second)
                    bulk_g2s(tc::smem_u32(sfs_b + s * kSfB + kSfBlock),
                             sfb + (static_cast<size_t>(rb_b + 1) * k64_blocks + kb * 4) * 512, kSfBlock, bar);
            };
            auto codes = [&](int kb, int s, uint32_t bar) {
                tc::tma_load_2d(tc::smem_u32(tiles_a + s * kTileA), &map_a, kb * kBKBytes, m0, bar);
                bulk_g2s(tc::smem_u32(sfs_a + s * kSfA), sfa + (static_cast<size_t>(rb_a) * k64_blocks + kb * 4) * 512, kSfA, bar);
            };
            const int ahead = k_blocks < kStages ? k_blocks : kStages;
            for (int kb = 0; kb < ahead; ++kb) weights(kb, kb, tc::smem_u32(full + kb));
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int kb = 0; kb < ahead; ++kb) codes(kb, kb, tc::smem_u32(full + kb));
            for (int kb = ahead; kb < k_blocks; ++kb) {
                const int s = kb % kStages;
                if (!tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                weights(kb, s, bar);
                codes(kb, s, bar);
            }
        }
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_nvfp4(kBM, kBN, 0, 0);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kStages;
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(tiles_a + s * kTileA), b_addr = tc::smem_u32(tiles_b + s * kTileB);
                const uint32_t sfa_addr = tc::smem_u32(sfs_a + s * kSfA), sfb_addr = tc::smem_u32(sfs_b + s * kSfB);
                // scale atoms of the stage's four k64 steps -> TMEM: A rows 0..127 (4 columns per step), B rows 0..127
                // and 128..255 (8 columns per step); all twelve copies are queued before the first MMA
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    tc::tmem_cp_32x128b_warpx4(tmem_sfa + ks * 4, tc::smem_desc_sf(sfa_addr + ks * 512));
                    tc::tmem_cp_32x128b_warpx4(tmem_sfb + ks * 8, tc::smem_desc_sf(sfb_addr + ks * 512));
                    if constexpr (kTwoBlocks) tc::tmem_cp_32x128b_warpx4(tmem_sfb + ks * 8 + 4, tc::smem_desc_sf(sfb_addr + 4 * 512 + ks * 512));
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t da = tc::smem_desc_k_sw128(a_addr + ks * 32), db = tc::smem_desc_k_sw128(b_addr + ks * 32);
                    tc::mma_mxf4nvf4(tmem_base, da, db, idesc, tmem_sfa + ks * 4, tmem_sfb + ks * 8, kb > 0 || ks > 0);
                }
                tc::mma_commit(tc::smem_u32(empty + s));
            }
            tc::mma_commit(tc::smem_u32(acc_ready));
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int quarter = warp & 3;
        const int m = m0 + quarter * 32 + lane;
        const bool ok = tc::mbar_wait(tc::smem_u32(acc_ready), 0);
        if (!ok && lane == 0) atomicExch(status, 3);
        tc::fence_after_sync();
        if (ok) {
            const float g = gx[0] * gw[0];
#pragma unroll 1
            for (int c = 0; c < kBN; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c, r);
                tc::tmem_ld_wait();
                if (m < M) {
                    OutT* dst = y + static_cast<size_t>(m) * N + n0 + c;
                    if (n0 + c + 32 <= N) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const OutT o0 = from_float<OutT>(__uint_as_float(r[2 * i]) * g), o1 = from_float<OutT>(__uint_as_float(r[2 * i + 1]) * g);
                            packed[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) |
                                        (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                        }
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c + i < N) dst[i] = from_float<OutT>(__uint_as_float(r[i]) * g);
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

// ------------------------------------------------------------------------------------------------ decode tile (M <= 16)
// With a handful of rows the operands swap roles: a 128-channel tile of the WEIGHT is the MMA's A operand (M = 128) and
// the activation rows are B (N = 16), so a K step stages 16 KB of weight codes + 2 KB of activation codes + 2 x 2 KB of
// scale atoms instead of a 16 KB activation tile that is all zeros but its first rows.  Five stages are 110 KB: two
// CTAs fit an SM, and they belong to consecutive launches (programmatic dependent launch: the later one requests its
// weights while the earlier one computes; measured on B200, a launch that streams this matrix alone takes 10.4 us, of
// which 3.5 us are the launch boundary).  The accumulator is [channel (TMEM lane)][row (column)], 16 columns.
constexpr int kDecStages = 5;
constexpr int kDecTileW = 128 * kBKBytes, kDecTileX = 16 * kBKBytes, kDecSf = 4 * 512;
constexpr int kDecStageBytes = kDecTileW + kDecTileX + 2 * kDecSf;
constexpr size_t kDecSmem = static_cast<size_t>(kDecStages) * kDecStageBytes + 1024 + 256;
constexpr uint32_t kDecTmemCols = 64;  // 16 accumulator columns, 16 + 16 scale columns

template <typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 2)
    nvfp4_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        const uint8_t* __restrict__ sfw, const uint8_t* __restrict__ sfx, const float* __restrict__ gx,
                        const float* __restrict__ gw, OutT* __restrict__ y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_w = smem;
    unsigned char* tiles_x = tiles_w + kDecStages * kDecTileW;
    unsigned char* sfs_w = tiles_x + kDecStages * kDecTileX;
    unsigned char* sfs_x = sfs_w + kDecStages * kDecSf;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sfs_x + kDecStages * kDecSf);
    uint64_t* full = bars;
    uint64_t* empty = bars + kDecStages;
    uint64_t* acc_ready = bars + 2 * kDecStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kDecStages + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 128;
    const int k_blocks = K / 256, k64_blocks = K / 64;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDecStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), kDecTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfw = tmem_base + 16, tmem_sfx = tmem_base + 32;  // 4 columns per k64 step each

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_w);
            tc::tma_prefetch_desc(&map_x);
            const int rb_w = n0 / 128;
            auto weights = [&](int kb, int s, uint32_t bar) {
                tc::mbar_expect_tx(bar, kDecStageBytes);
                tc::tma_load_2d(tc::smem_u32(tiles_w + s * kDecTileW), &map_w, kb * kBKBytes, n0, bar);
                bulk_g2s(tc::smem_u32(sfs_w + s * kDecSf), sfw + (static_cast<size_t>(rb_w) * k64_blocks + kb * 4) * 512, kDecSf, bar);
            };
            auto codes = [&](int kb, int s, uint32_t bar) {
                tc::tma_load_2d(tc::smem_u32(tiles_x + s * kDecTileX), &map_x, kb * kBKBytes, 0, bar);
                bulk_g2s(tc::smem_u32(sfs_x + s * kDecSf), sfx + static_cast<size_t>(kb) * 4 * 512, kDecSf, bar);
            };
            // the weights never depend on the kernel before (the activation quantize): request them ahead of the wait
            const int ahead = k_blocks < kDecStages ? k_blocks : kDecStages;
            for (int kb = 0; kb < ahead; ++kb) weights(kb, kb, tc::smem_u32(full + kb));
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int kb = 0; kb < ahead; ++kb) codes(kb, kb, tc::smem_u32(full + kb));
            for (int kb = ahead; kb < k_blocks; ++kb) {
                const int s = kb % kDecStages;
                if (!tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kDecStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                weights(kb, s, bar);
                codes(kb, s, bar);
            }
        }
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // bounded waits count from the moment the codes exist
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_nvfp4(128, 16, 0, 0);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kDecStages;
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kDecStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(tiles_w + s * kDecTileW), x_addr = tc::smem_u32(tiles_x + s * kDecTileX);
                const uint32_t sfw_addr = tc::smem_u32(sfs_w + s * kDecSf), sfx_addr = tc::smem_u32(sfs_x + s * kDecSf);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    tc::tmem_cp_32x128b_warpx4(tmem_sfw + ks * 4, tc::smem_desc_sf(sfw_addr + ks * 512));
                    tc::tmem_cp_32x128b_warpx4(tmem_sfx + ks * 4, tc::smem_desc_sf(sfx_addr + ks * 512));
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t da = tc::smem_desc_k_sw128(w_addr + ks * 32), db = tc::smem_desc_k_sw128(x_addr + ks * 32);
                    tc::mma_mxf4nvf4(tmem_base, da, db, idesc, tmem_sfw + ks * 4, tmem_sfx + ks * 4, kb > 0 || ks > 0);
                }
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
            const float g = gx[0] * gw[0];
            uint32_t r[16];
            tc::tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), r);
            tc::tmem_ld_wait();
            if (n < N) {
#pragma unroll
                for (int m = 0; m < 16; ++m)
                    if (m < M) y[static_cast<size_t>(m) * N + n] = from_float<OutT>(__uint_as_float(r[m]) * g);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, kDecTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------ prefill tile 256 x 224
// Two 128-row accumulators share one 224-column B tile: 448 accumulator columns + 32 (A scales) + 32 (B scales) fill
// TMEM exactly, and a K step moves 68 KB for 256 x 224 x 256 products where the 128 x 256 tile moved 54 KB for 128 x 256
// x 256: 1.4 times fewer bytes per flop through L2, which is what bounded the 128-row form.
constexpr int kWTileA = 256 * kBKBytes, kWTileB = kWideBN * kBKBytes;
constexpr int kWSf = 2 * 4 * 512;  // two row blocks x four k64 atoms, for A and for B
constexpr int kWStages = 3;
constexpr int kWThreads = 320;
constexpr size_t kWSmem = static_cast<size_t>(kWStages) * (kWTileA + kWTileB + 2 * kWSf) + 1024 + 256;

template <typename OutT>
__global__ void __launch_bounds__(kWThreads, 1)
    nvfp4_gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, const float* __restrict__ gx,
                              const float* __restrict__ gw, OutT* __restrict__ y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_a = smem;
    unsigned char* tiles_b = tiles_a + kWStages * kWTileA;
    unsigned char* sfs_a = tiles_b + kWStages * kWTileB;
    unsigned char* sfs_b = sfs_a + kWStages * kWSf;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sfs_b + kWStages * kWSf);
    uint64_t* full = bars;
    uint64_t* empty = bars + kWStages;
    uint64_t* acc_ready = bars + 2 * kWStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kWStages + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * kWideBN, m0 = blockIdx.x * 256;  // row tiles run fastest (see above)
    const int k_blocks = K / 256;
    const int k64_blocks = K / 64;
    const bool two_halves = M - m0 > 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            tc::mbar_init(tc::smem_u32(full + s), 1);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), 512);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + 2 * kWideBN;       // half h, k64 step ks: + 16 h + 4 ks
    const uint32_t tmem_sfb = tmem_base + 2 * kWideBN + 32;  // k64 step ks, row block b: + 8 ks + 4 b

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_a);
            tc::tma_prefetch_desc(&map_b);
            const int rb_a = m0 / 128;
            constexpr int kSfBlock = 4 * 512;
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kWStages;
                if (kb >= kWStages && !tc::mbar_wait(tc::smem_u32(empty + s), ((kb / kWStages) - 1) & 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = tc::smem_u32(full + s);
                tc::mbar_expect_tx(bar, kWTileA + kWTileB + (two_halves ? 2 : 1) * kSfBlock + 2 * kSfBlock);
                tc::tma_load_2d(tc::smem_u32(tiles_a + s * kWTileA), &map_a, kb * kBKBytes, m0, bar);
                tc::tma_load_2d(tc::smem_u32(tiles_b + s * kWTileB), &map_b, kb * kBKBytes, n0, bar);
                bulk_g2s(tc::smem_u32(sfs_a + s * kWSf), sfa + (static_cast<size_t>(rb_a) * k64_blocks + kb * 4) * 512, kSfBlock, bar);
                if (two_halves)
                    bulk_g2s(tc::smem_u32(sfs_a + s * kWSf + kSfBlock), sfa + (static_cast<size_t>(rb_a + 1) * k64_blocks + kb * 4) * 512, kSfBlock, bar);
                const size_t tile_blocks = static_cast<size_t>(blockIdx.y) * 2;
                bulk_g2s(tc::smem_u32(sfs_b + s * kWSf), sfb + (tile_blocks * k64_blocks + kb * 4) * 512, kSfBlock, bar);
                bulk_g2s(tc::smem_u32(sfs_b + s * kWSf + kSfBlock), sfb + ((tile_blocks + 1) * k64_blocks + kb * 4) * 512, kSfBlock, bar);
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_nvfp4(128, kWideBN, 0, 0);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kWStages;
                if (!tc::mbar_wait(tc::smem_u32(full + s), (kb / kWStages) & 1)) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(tiles_a + s * kWTileA), b_addr = tc::smem_u32(tiles_b + s * kWTileB);
                const uint32_t sfa_addr = tc::smem_u32(sfs_a + s * kWSf), sfb_addr = tc::smem_u32(sfs_b + s * kWSf);
                // all scale copies of the stage are queued before its first MMA
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    tc::tmem_cp_32x128b_warpx4(tmem_sfa + ks * 4, tc::smem_desc_sf(sfa_addr + ks * 512));
                    if (two_halves) tc::tmem_cp_32x128b_warpx4(tmem_sfa + 16 + ks * 4, tc::smem_desc_sf(sfa_addr + 4 * 512 + ks * 512));
                    tc::tmem_cp_32x128b_warpx4(tmem_sfb + ks * 8, tc::smem_desc_sf(sfb_addr + ks * 512));
                    tc::tmem_cp_32x128b_warpx4(tmem_sfb + ks * 8 + 4, tc::smem_desc_sf(sfb_addr + 4 * 512 + ks * 512));
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t db = tc::smem_desc_k_sw128(b_addr + ks * 32);
                    tc::mma_mxf4nvf4(tmem_base, tc::smem_desc_k_sw128(a_addr + ks * 32), db, idesc, tmem_sfa + ks * 4, tmem_sfb + ks * 8, kb > 0 || ks > 0);
                    if (two_halves)
                        tc::mma_mxf4nvf4(tmem_base + kWideBN, tc::smem_desc_k_sw128(a_addr + 128 * kBKBytes + ks * 32), db, idesc, tmem_sfa + 16 + ks * 4,
                                         tmem_sfb + ks * 8, kb > 0 || ks > 0);
                }
                tc::mma_commit(tc::smem_u32(empty + s));
            }
            tc::mma_commit(tc::smem_u32(acc_ready));
        }
    } else {
        // epilogue: warps 2..5 rows 0..127, warps 6..9 rows 128..255; warp w touches TMEM lanes 32 (w % 4) .. +31
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int m = m0 + half * 128 + quarter * 32 + lane;
        const bool ok = __all_sync(0xFFFFFFFFu, tc::mbar_wait(tc::smem_u32(acc_ready), 0));
        if (!ok && lane == 0) atomicExch(status, 3);
        tc::fence_after_sync();
        if (ok && (half == 0 || two_halves)) {
            const float g = gx[0] * gw[0];
#pragma unroll 1
            for (int c = 0; c < kWideBN; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * kWideBN + c, r);
                tc::tmem_ld_wait();
                if (m < M && n0 + c < N) {
                    OutT* dst = y + static_cast<size_t>(m) * N + n0 + c;
                    if (n0 + c + 32 <= N) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const OutT o0 = from_float<OutT>(__uint_as_float(r[2 * i]) * g), o1 = from_float<OutT>(__uint_as_float(r[2 * i + 1]) * g);
                            packed[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) |
                                        (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                        }
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c + i < N) dst[i] = from_float<OutT>(__uint_as_float(r[i]) * g);
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t sf_tiled_bytes(int64_t rows, int64_t K) { return static_cast<size_t>((rows + 127) / 128) * (K / 64) * 512; }
static size_t sf_wide_bytes(int64_t rows, int64_t K) { return static_cast<size_t>((rows + kWideBN - 1) / kWideBN) * 2 * (K / 64) * 512; }

}  // namespace eq

using namespace eq;

extern "C" size_t eq_nvfp4_tiled_scale_bytes(int64_t rows, int64_t K) {
    if (rows <= 0 || K <= 0 || K % 64) return 0;
    return sf_tiled_bytes(rows, K);
}

extern "C" int eq_nvfp4_tile_scales(const uint8_t* scale_bits, int64_t rows, int64_t K, uint8_t* tiled, void* stream) {
    EQ_REQUIRE(scale_bits && tiled, EQ_ERR_BAD_ARG, "eq_nvfp4_tile_scales: null pointer");
    EQ_REQUIRE(rows > 0 && K > 0 && K % 64 == 0, EQ_ERR_UNSUPPORTED, "eq_nvfp4_tile_scales: needs K %% 64 == 0 (K=%lld)", (long long)K);
    const int64_t total = (rows + 127) / 128 * 128 * (K / 16);
    nvfp4_tile_scales_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(scale_bits, rows, K, tiled);
    EQ_LAUNCH_OK("nvfp4_tile_scales_kernel");
    return EQ_OK;
}

extern "C" size_t eq_nvfp4_weight_scale_bytes(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0 || K % 64) return 0;
    return align_up(sf_tiled_bytes(N, K), 256) + sf_wide_bytes(N, K);
}

extern "C" int eq_nvfp4_tile_weight_scales(const uint8_t* scale_bits, int64_t N, int64_t K, uint8_t* tiled, void* stream) {
    EQ_REQUIRE(scale_bits && tiled, EQ_ERR_BAD_ARG, "eq_nvfp4_tile_weight_scales: null pointer");
    EQ_REQUIRE(N > 0 && K > 0 && K % 64 == 0, EQ_ERR_UNSUPPORTED, "eq_nvfp4_tile_weight_scales: needs K %% 64 == 0 (K=%lld)", (long long)K);
    EQ_REQUIRE(aligned(tiled, 256), EQ_ERR_BAD_ALIGN, "eq_nvfp4_tile_weight_scales: the output must be 256-byte aligned");
    int st = eq_nvfp4_tile_scales(scale_bits, N, K, tiled, stream);
    if (st != EQ_OK) return st;
    const int64_t total = (N + kWideBN - 1) / kWideBN * 256 * (K / 16);
    nvfp4_tile_scales_wide_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        scale_bits, N, K, tiled + align_up(sf_tiled_bytes(N, K), 256));
    EQ_LAUNCH_OK("nvfp4_tile_scales_wide_kernel");
    return EQ_OK;
}

extern "C" int eq_nvfp4_global_scale(const void* x, int64_t M, int64_t K, int in_dtype, float* scale2, unsigned int* scratch_u32,
                                     void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(x && scale2 && scratch_u32 && M > 0 && K > 0, EQ_ERR_BAD_ARG, "eq_nvfp4_global_scale: bad arguments");
    EQ_CUDA_OK(cudaMemsetAsync(scratch_u32, 0, sizeof(unsigned int), stream));
    const int64_t n = M * K;
    const unsigned grid = static_cast<unsigned>(n / 256 / 8 + 1 < 1184 ? n / 256 / 8 + 1 : 1184);
    switch (in_dtype) {
        case EQ_F16: nvfp4_amax_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), n, scratch_u32); break;
        case EQ_BF16: nvfp4_amax_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n, scratch_u32); break;
        case EQ_F32: nvfp4_amax_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), n, scratch_u32); break;
        default: return fail(EQ_ERR_BAD_ARG, "eq_nvfp4_global_scale: unknown dtype %d", in_dtype);
    }
    EQ_LAUNCH_OK("nvfp4_amax_kernel");
    nvfp4_scale2_kernel<<<1, 1, 0, stream>>>(scratch_u32, scale2);
    EQ_LAUNCH_OK("nvfp4_scale2_kernel");
    return EQ_OK;
}

extern "C" int eq_quant_nvfp4_weight(const void* values, int64_t N, int64_t K, int in_dtype, uint8_t* packed, uint8_t* scale_bits,
                                     float* scale_2, unsigned int* scratch_u32, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(values && packed && scale_bits && scale_2 && scratch_u32, EQ_ERR_BAD_ARG, "eq_quant_nvfp4_weight: null pointer");
    EQ_REQUIRE(N > 0 && K > 0, EQ_ERR_BAD_ARG, "eq_quant_nvfp4_weight: bad extents");
    EQ_REQUIRE(K % 16 == 0, EQ_ERR_UNSUPPORTED, "eq_quant_nvfp4_weight: K must be a multiple of 16");
    EQ_REQUIRE(aligned(packed, 8), EQ_ERR_BAD_ALIGN, "eq_quant_nvfp4_weight: packed must be 8-byte aligned");
    int st = eq_nvfp4_global_scale(values, N, K, in_dtype, scale_2, scratch_u32, stream_);  // the same max(amax, 1e-12) / (6 * 448)
    if (st != EQ_OK) return st;
    const int64_t total = N * (K / 16);
    const unsigned grid = static_cast<unsigned>(ceil_div(total, 128));
    switch (in_dtype) {
        case EQ_F16: quant_nvfp4_weight_kernel<__half><<<grid, 128, 0, stream>>>(static_cast<const __half*>(values), N, K, scale_2, packed, scale_bits); break;
        case EQ_BF16: quant_nvfp4_weight_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(values), N, K, scale_2, packed, scale_bits); break;
        case EQ_F32: quant_nvfp4_weight_kernel<float><<<grid, 128, 0, stream>>>(static_cast<const float*>(values), N, K, scale_2, packed, scale_bits); break;
        default: return fail(EQ_ERR_BAD_ARG, "eq_quant_nvfp4_weight: unknown dtype %d", in_dtype);
    }
    EQ_LAUNCH_OK("quant_nvfp4_weight_kernel");
    return EQ_OK;
}

// `pad_rows`: zero the tiled scales of the rows between M and the end of its 128-row block (what a caller that reads the
// tiled layout expects).  The linear passes false: those rows of A arrive as zeros from the tensor map and the output
// rows they produce are never stored.  `status`: cleared by the kernel for the linear behind it.
static int quant_nvfp4_act(const void* x, int64_t M, int64_t K, int in_dtype, const float* input_scale, uint8_t* codes, uint8_t* scale_bits,
                           uint8_t* scale_tiled, bool pad_rows, int* status, cudaStream_t stream) {
    EQ_REQUIRE(M >= 0 && K > 0, EQ_ERR_BAD_ARG, "eq_quant_nvfp4_act: bad extents");
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(x && input_scale && codes, EQ_ERR_BAD_ARG, "eq_quant_nvfp4_act: null pointer");
    EQ_REQUIRE(K % 16 == 0 && (!scale_tiled || K % 64 == 0), EQ_ERR_UNSUPPORTED, "eq_quant_nvfp4_act: K must be a multiple of 16 (64 with tiled scales)");
    EQ_REQUIRE(aligned(codes, 8), EQ_ERR_BAD_ALIGN, "eq_quant_nvfp4_act: codes must be 8-byte aligned");
    if (scale_tiled && pad_rows) EQ_CUDA_OK(cudaMemsetAsync(scale_tiled, 0, sf_tiled_bytes(M, K), stream));
    const int64_t total = M * (K / 16);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(total, 128)));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = status ? 1 : 0;  // inside the linear: resident, and past its launch latency, when the kernel before it ends
    switch (in_dtype) {
        case EQ_F16: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_nvfp4_act_kernel<__half>, static_cast<const __half*>(x), M, K, input_scale, codes, scale_bits, scale_tiled, status)); break;
        case EQ_BF16: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_nvfp4_act_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x), M, K, input_scale, codes, scale_bits, scale_tiled, status)); break;
        case EQ_F32: EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_nvfp4_act_kernel<float>, static_cast<const float*>(x), M, K, input_scale, codes, scale_bits, scale_tiled, status)); break;
        default: return fail(EQ_ERR_BAD_ARG, "eq_quant_nvfp4_act: unknown dtype %d", in_dtype);
    }
    return EQ_OK;
}

extern "C" int eq_quant_nvfp4_act(const void* x, int64_t M, int64_t K, int in_dtype, const float* input_scale, uint8_t* codes,
                                  uint8_t* scale_bits, uint8_t* scale_tiled, void* stream_) {
    return quant_nvfp4_act(x, M, K, in_dtype, input_scale, codes, scale_bits, scale_tiled, true, nullptr, static_cast<cudaStream_t>(stream_));
}

extern "C" size_t eq_nvfp4_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return align_up(static_cast<size_t>(M) * K / 2, 256) + align_up(sf_tiled_bytes(M, K), 256) + 256;
}

static int nvfp4_linear_any(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N, int64_t K,
                            const void* x, const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                            void* stream_, const void* gamma, float eps);

extern "C" int eq_nvfp4_linear(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N,
                               int64_t K, const void* x, const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace,
                               size_t workspace_bytes, void* stream_) {
    return nvfp4_linear_any(weight, weight_scale_tiled, weight_scale_2, N, K, x, input_scale, M, act_dtype, y, workspace, workspace_bytes, stream_,
                            nullptr, 0.f);
}

extern "C" int eq_nvfp4_linear_rmsnorm(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N, int64_t K,
                                       const void* x, const void* gamma, float eps, const float* input_scale, int64_t M, int act_dtype, void* y,
                                       void* workspace, size_t workspace_bytes, void* stream_) {
    EQ_REQUIRE(gamma, EQ_ERR_BAD_ARG, "eq_nvfp4_linear_rmsnorm: null norm weight");
    return nvfp4_linear_any(weight, weight_scale_tiled, weight_scale_2, N, K, x, input_scale, M, act_dtype, y, workspace, workspace_bytes, stream_, gamma,
                            eps);
}

static int nvfp4_linear_any(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N, int64_t K,
                            const void* x, const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                            void* stream_, const void* gamma, float eps) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(N > 0 && K > 0 && M >= 0, EQ_ERR_BAD_ARG, "eq_nvfp4_linear: bad extents M=%lld K=%lld N=%lld", (long long)M, (long long)K, (long long)N);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(weight && weight_scale_tiled && weight_scale_2 && x && input_scale && y, EQ_ERR_BAD_ARG, "eq_nvfp4_linear: null pointer");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_nvfp4_linear: activations must be f16 or bf16");
    EQ_REQUIRE(K % 256 == 0 && N % 8 == 0, EQ_ERR_UNSUPPORTED, "eq_nvfp4_linear: needs K %% 256 == 0 and N %% 8 == 0 (K=%lld N=%lld)", (long long)K, (long long)N);
    EQ_REQUIRE(aligned(weight, 16) && aligned(weight_scale_tiled, 256) && aligned(y, 16), EQ_ERR_BAD_ALIGN, "eq_nvfp4_linear: weight and scales must be 16-byte aligned");
    EQ_REQUIRE(workspace && workspace_bytes >= eq_nvfp4_workspace_bytes(M, K), EQ_ERR_WORKSPACE, "eq_nvfp4_linear: workspace of %zu bytes needed, %zu given",
               eq_nvfp4_workspace_bytes(M, K), workspace_bytes);
    EQ_REQUIRE(aligned(workspace, 256), EQ_ERR_BAD_ALIGN, "eq_nvfp4_linear: workspace must be 256-byte aligned");
    uint8_t* codes = static_cast<uint8_t*>(workspace);
    uint8_t* sfa = codes + align_up(static_cast<size_t>(M) * K / 2, 256);
    int* status = reinterpret_cast<int*>(sfa + align_up(sf_tiled_bytes(M, K), 256));
    int st = EQ_OK;
    if (gamma) {
        // the model's RMSNorm inside the quantize kernel (a programmatic dependent, like the plain quantize)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(M));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (act_dtype == EQ_F16)
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, rmsnorm_quant_nvfp4_rows_kernel<__half>, static_cast<const __half*>(x), static_cast<const __half*>(gamma), eps,
                                          K, input_scale, codes, sfa, status));
        else
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, rmsnorm_quant_nvfp4_rows_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x),
                                          static_cast<const __nv_bfloat16*>(gamma), eps, K, input_scale, codes, sfa, status));
    } else {
        st = quant_nvfp4_act(x, M, K, act_dtype, input_scale, codes, nullptr, sfa, false, status, stream);
    }
    if (st != EQ_OK) return st;
    CUtensorMap map_a, map_b;
    if (M <= 16) {
        // decode-shaped: weight tiles as the MMA's A operand, the rows as B
        st = make_tensor_map_2d(&map_a, weight, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, 128, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EQ_OK) return st;
        st = make_tensor_map_2d(&map_b, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, K / 2, 16, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EQ_OK) return st;
        auto run = [&](auto kernel, auto* yt) -> int {
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kDecSmem)));
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(N, 128)));
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = kDecSmem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            const uint8_t* sfx = sfa;
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, weight_scale_tiled, sfx, input_scale, weight_scale_2, yt, static_cast<int>(M),
                                          static_cast<int>(N), static_cast<int>(K), status));
            return EQ_OK;
        };
        return act_dtype == EQ_F16 ? run(nvfp4_decode_kernel<__half>, static_cast<__half*>(y))
                                   : run(nvfp4_decode_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16*>(y));
    }
    // codes are bytes holding two e2m1 values: the maps move bytes; 128 bytes = 256 elements of K per tile row
    st = make_tensor_map_2d(&map_a, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, K / 2, kBM, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    // 256 x 224 tiles pay off once there are enough row tiles to fill whole waves; below that the 128-row tiles
    // (128 columns for a single row tile, 256 otherwise) spread the work over more CTAs.
    const bool wide = ceil_div(N, kWideBN) * ceil_div(M, 256) >= 4 * static_cast<int64_t>(sm_count());
    if (!wide) {
        // the 128-row-block scale layout at the front of the blob
        const int bn = M <= 128 ? 128 : 256;
        st = make_tensor_map_2d(&map_b, weight, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, bn, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EQ_OK) return st;
        dim3 grid(static_cast<unsigned>(ceil_div(M, kBM)), static_cast<unsigned>(ceil_div(N, bn)));
        auto run = [&](auto kernel, size_t smem, auto* yt) -> int {
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start (and fetch weights) while the quantize runs
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            const uint8_t* sfa_c = sfa;
            EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, sfa_c, weight_scale_tiled, input_scale, weight_scale_2, yt, static_cast<int>(M),
                                          static_cast<int>(N), static_cast<int>(K), status));
            return EQ_OK;
        };
        if (act_dtype == EQ_F16)
            return bn == 128 ? run(nvfp4_gemm_tc_kernel<__half, 128>, Fp4Cfg<128>::kSmem, static_cast<__half*>(y))
                             : run(nvfp4_gemm_tc_kernel<__half, 256>, Fp4Cfg<256>::kSmem, static_cast<__half*>(y));
        return bn == 128 ? run(nvfp4_gemm_tc_kernel<__nv_bfloat16, 128>, Fp4Cfg<128>::kSmem, static_cast<__nv_bfloat16*>(y))
                         : run(nvfp4_gemm_tc_kernel<__nv_bfloat16, 256>, Fp4Cfg<256>::kSmem, static_cast<__nv_bfloat16*>(y));
    }
    // prefill-shaped: 256 x 224 tiles, the 224-row-tile scale layout behind the first one
    st = make_tensor_map_2d(&map_a, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, K / 2, 256, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    st = make_tensor_map_2d(&map_b, weight, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, kWideBN, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    const uint8_t* sfb_wide = weight_scale_tiled + align_up(sf_tiled_bytes(N, K), 256);
    dim3 grid(static_cast<unsigned>(ceil_div(M, 256)), static_cast<unsigned>(ceil_div(N, kWideBN)));
    auto run = [&](auto kernel, auto* yt) -> int {
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kWSmem)));
        kernel<<<grid, kWThreads, kWSmem, stream>>>(map_a, map_b, sfa, sfb_wide, input_scale, weight_scale_2, yt, static_cast<int>(M),
                                                   static_cast<int>(N), static_cast<int>(K), status);
        EQ_LAUNCH_OK("nvfp4_gemm_tc_wide_kernel");
        return EQ_OK;
    };
    return act_dtype == EQ_F16 ? run(nvfp4_gemm_tc_wide_kernel<__half>, static_cast<__half*>(y))
                               : run(nvfp4_gemm_tc_wide_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16*>(y));
}

extern "C" int eq_nvfp4_status(const void* workspace, int64_t M, int64_t K, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && K > 0, EQ_ERR_BAD_ARG, "eq_nvfp4_status: bad arguments");
    const unsigned char* base = static_cast<const unsigned char*>(workspace);
    const int* status = reinterpret_cast<const int*>(base + align_up(static_cast<size_t>(M) * K / 2, 256) + align_up(sf_tiled_bytes(M, K), 256));
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_nvfp4_status: a bounded pipeline wait ran out (code %d)", host);
    return EQ_OK;
}
