// W4A16 linear for decode-shaped calls (and, in 64-row blocks, for any M): y[M,N] = x[M,K] @ W, W int4 group-wise.
//
// A bandwidth kernel, kept deliberately plain: many small CTAs, no staging phase, nothing between a warp and its
// bytes.  The repacked weight (w4_repack.cu) is a run of 1088-byte ITEM records, [n-tile][item]: 16 output columns x
// 128 input rows of nibbles plus that group's scales and zero points.  A CTA of four warps owns one 16-column tile
// and one K split; its warps take equal runs of items.  Per item a lane
//   - streams its 2 x 16 weight bytes and its 8-byte scale/zero entry (loads are issued kDepth items ahead),
//   - reads the 64 contiguous bytes of x it needs straight from global memory (x is a few KB and lives in L1/L2; the
//     repack deals input rows to lanes so that this is four 16-byte loads),
//   - turns each word into one m16n8k16 A fragment: four lop3 + one shift isolate the nibbles as f16 1024+q (or
//     1024+16q), one f16x2 subtract / fma per pair removes 1024 and the zero point exactly, so the tensor core sees
//     the integers q - z and the f32 accumulator holds sum_k x_k (q_k - z) exactly up to f32 rounding,
//   - folds the item with its scale: y += s * acc.
// Warps of a CTA meet in shared memory.  K splits of one tile meet in an f32 workspace with atomic adds; the CTA
// whose arrival completes the tile converts, stores y and leaves workspace and counter zero.  Nobody waits.
//
// The grid is sized for granularity, not residency: splits are chosen so that there are many more CTAs than CTA
// slots and every CTA streams 8-32 KB, which lets the hardware scheduler even out the SMs.
//
// tcgen05 is not used here: at M <= 16 the contraction fills 1/8 of an MMA tile and the kernel is bound by bytes and
// by integer issue (the nibble isolation), not by tensor throughput; the warp-level MMA keeps operands in registers.
#include "common.cuh"

namespace eq {

constexpr int kTileWarps = 4;
constexpr int kTileThreads = kTileWarps * 32;
constexpr int kDepth = 4;          // items whose weight bytes are in flight per warp
constexpr int kItemBytes = 1088;   // 1024 B of nibbles + 64 B of scales / zero points

struct W4Params {
    const unsigned char* wq;  // [n_tiles][items][1088]
    const int32_t* perm;      // optional [K]: repacked row k' is input feature perm[k']
    const void* x;            // [M][K]
    void* y;                  // [M][N]
    float* wsp;               // [M][N] partial sums (zero between calls)
    int* counters;            // [n_tiles] split arrivals (zero between calls), then one status word
    int K, N, M;
    int items;                // K / 128
    int splits;               // K splits per tile
    int scale_dtype;
};

template <typename ActT>
struct Frag;

template <>
struct Frag<__half> {
    // zero point z (f16 pair, same value twice) -> constants of the exact dequant
    struct Zero {
        uint32_t sub, fma;  // {1024 + z}, {-(64 + z)}
    };
    static __device__ __forceinline__ Zero zero(uint32_t z_pair) {
        Zero r;
        asm("add.f16x2 %0, %1, %2;" : "=r"(r.sub) : "r"(z_pair), "r"(0x64006400u));
        uint32_t t;
        asm("add.f16x2 %0, %1, %2;" : "=r"(t) : "r"(z_pair), "r"(0x54005400u));  // 64 + z
        r.fma = t ^ 0x80008000u;
        return r;
    }
    // one word of a lane -> A fragment registers holding q - z exactly
    static __device__ __forceinline__ void expand(uint32_t w, const Zero& lo, const Zero& hi, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;  // (w & mask) | magic is the f16 pair {1024 + q} or {1024 + 16 q}
        const uint32_t h0 = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        const uint32_t h1 = lop3<0xEA>(w, 0x00F000F0u, kMagic);
        const uint32_t w8 = w >> 8;
        const uint32_t h2 = lop3<0xEA>(w8, 0x000F000Fu, kMagic);
        const uint32_t h3 = lop3<0xEA>(w8, 0x00F000F0u, kMagic);
        constexpr uint32_t kSixteenth = 0x2C002C00u;
        asm("sub.f16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(h0), "r"(lo.sub));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[2]) : "r"(h1), "r"(kSixteenth), "r"(lo.fma));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(a[1]) : "r"(h2), "r"(hi.sub));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[3]) : "r"(h3), "r"(kSixteenth), "r"(hi.fma));
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ void mma0(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
};

template <>
struct Frag<__nv_bfloat16> {
    struct Zero {
        uint32_t sub, fma;  // {128 + z} as bf16 pair; fma unused
    };
    static __device__ __forceinline__ Zero zero(uint32_t z_pair) {
        const float z = __half2float(__ushort_as_half(static_cast<unsigned short>(z_pair & 0xFFFF)));
        const __nv_bfloat162 v = __float2bfloat162_rn(128.f + z);  // exact: at most 144
        Zero r;
        r.sub = *reinterpret_cast<const uint32_t*>(&v);
        r.fma = 0;
        return r;
    }
    static __device__ __forceinline__ void expand(uint32_t w, const Zero& lo, const Zero& hi, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x43004300u;  // 128 + q is exact in bf16
        const uint32_t t0 = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        const uint32_t t1 = lop3<0xEA>(w >> 4, 0x000F000Fu, kMagic);
        const uint32_t t2 = lop3<0xEA>(w >> 8, 0x000F000Fu, kMagic);
        const uint32_t t3 = lop3<0xEA>(w >> 12, 0x000F000Fu, kMagic);
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(t0), "r"(lo.sub));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[2]) : "r"(t1), "r"(lo.sub));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[1]) : "r"(t2), "r"(hi.sub));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[3]) : "r"(t3), "r"(hi.sub));
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ void mma0(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
};

// The 64 bytes of activations lane column j needs for one item of row m: rows 32 j .. 32 j + 31 of the item, the
// first 16 the low k-slots of steps 0..7, the last 16 the high ones.
template <typename ActT>
__device__ __forceinline__ void load_x(const ActT* xrow, const int32_t* perm, int k0, uint4 (&v)[4]) {
    if (!perm) {
        const uint4* src = reinterpret_cast<const uint4*>(xrow + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __ldg(src + i);
    } else {
        uint32_t wds[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const ActT lo = xrow[perm[k0 + 2 * i]], hi = xrow[perm[k0 + 2 * i + 1]];
            wds[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&lo)) |
                     (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = make_uint4(wds[4 * i], wds[4 * i + 1], wds[4 * i + 2], wds[4 * i + 3]);
    }
}

// One output tile (16 columns) x one K split, for a problem (wq, x, y, M).  ONE: a single activation row; every lane
// then reads row 0, the m = 1..7 columns of the product are copies of column 0 and are never looked at.
template <typename ActT, int MT, bool ONE>
__device__ __forceinline__ void w4_tile(const W4Params& p, int tile, int split, float (*red)[MT * 8][16], int* last_flag) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    // this CTA's items, then this warp's
    const int c0 = p.items * split / p.splits, c1 = p.items * (split + 1) / p.splits;
    const int i0 = c0 + (c1 - c0) * warp / kTileWarps, i1 = c0 + (c1 - c0) * (warp + 1) / kTileWarps;
    const unsigned char* rec0 = p.wq + (static_cast<size_t>(tile) * p.items) * kItemBytes + lane * 16;
    const unsigned char* meta0 = p.wq + (static_cast<size_t>(tile) * p.items) * kItemBytes + 1024 + g * 8;
    const ActT* x = static_cast<const ActT*>(p.x);

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.f;

    uint4 w_lo[kDepth], w_hi[kDepth];
    uint2 meta[kDepth];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
        if (i0 + d < i1) {
            const size_t off = static_cast<size_t>(i0 + d) * kItemBytes;
            w_lo[d] = ld_stream_v4(rec0 + off);
            w_hi[d] = ld_stream_v4(rec0 + off + 512);
            meta[d] = __ldg(reinterpret_cast<const uint2*>(meta0 + off));
        }
    }
    // The weights never depend on the kernel before this one; x, y and the workspace may.  Launched with
    // programmatic stream serialization, this grid starts while the previous one drains, has its first weight
    // bytes in flight by now, and only here waits for the previous grid's results to be visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int ib = i0; ib < i1; ib += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            const int it = ib + d;
            if (it < i1) {
                const uint4 wl = w_lo[d], wh = w_hi[d];
                const uint2 mt_ = meta[d];
                if (it + kDepth < i1) {  // refill this register slot
                    const size_t off = static_cast<size_t>(it + kDepth) * kItemBytes;
                    w_lo[d] = ld_stream_v4(rec0 + off);
                    w_hi[d] = ld_stream_v4(rec0 + off + 512);
                    meta[d] = __ldg(reinterpret_cast<const uint2*>(meta0 + off));
                }
                // scale and zero point of the two columns g, g+8
                float s_lo, s_hi;
                if (p.scale_dtype == EQ_F16) {
                    const __half2 s = *reinterpret_cast<const __half2*>(&mt_.x);
                    s_lo = __low2float(s);
                    s_hi = __high2float(s);
                } else {
                    s_lo = __uint_as_float(mt_.x << 16);
                    s_hi = __uint_as_float(mt_.x & 0xFFFF0000u);
                }
                const typename Frag<ActT>::Zero z_lo = Frag<ActT>::zero(__byte_perm(mt_.y, 0, 0x1010));
                const typename Frag<ActT>::Zero z_hi = Frag<ActT>::zero(__byte_perm(mt_.y, 0, 0x3232));
                const uint32_t words[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
                uint4 xv[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int m = ONE ? 0 : mt * 8 + g;
                    if (ONE || m < p.M) {
                        load_x<ActT>(x + static_cast<size_t>(m) * p.K, p.perm, it * 128 + 32 * j, xv[mt]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) xv[mt][i] = make_uint4(0, 0, 0, 0);
                    }
                }
                float acc[MT][4];
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    uint32_t a[4];
                    Frag<ActT>::expand(words[s], z_lo, z_hi, a);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t* lo = reinterpret_cast<const uint32_t*>(&xv[mt][0]);  // 8 words: steps 0..7, low slots
                        const uint32_t* hi = reinterpret_cast<const uint32_t*>(&xv[mt][2]);  // high slots
                        if (s == 0)
                            Frag<ActT>::mma0(acc[mt], a, lo[s], hi[s]);
                        else
                            Frag<ActT>::mma(acc[mt], a, lo[s], hi[s]);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    yacc[mt][0] = fmaf(s_lo, acc[mt][0], yacc[mt][0]);
                    yacc[mt][1] = fmaf(s_lo, acc[mt][1], yacc[mt][1]);
                    yacc[mt][2] = fmaf(s_hi, acc[mt][2], yacc[mt][2]);
                    yacc[mt][3] = fmaf(s_hi, acc[mt][3], yacc[mt][3]);
                }
            }
        }
    }

    // ---- the four warps meet
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][mt * 8 + 2 * j + (e & 1)][g + ((e & 2) ? 8 : 0)] = yacc[mt][e];
    }
    __syncthreads();
    ActT* y = static_cast<ActT*>(p.y);
    const int n_base = tile * 16;
    const int cells = (ONE ? 1 : min(p.M, MT * 8)) * 16;
    if (p.splits == 1) {
        for (int idx = threadIdx.x; idx < cells; idx += kTileThreads) {
            const int m = idx >> 4, n = idx & 15;
            const float v = red[0][m][n] + red[1][m][n] + red[2][m][n] + red[3][m][n];
            y[static_cast<size_t>(m) * p.N + n_base + n] = from_float<ActT>(v);
        }
        return;
    }
    // ---- K splits of the tile meet in the workspace; the last one to arrive finishes
    for (int idx = threadIdx.x; idx < cells; idx += kTileThreads) {
        const int m = idx >> 4, n = idx & 15;
        const float v = red[0][m][n] + red[1][m][n] + red[2][m][n] + red[3][m][n];
        atomicAdd(p.wsp + static_cast<size_t>(m) * p.N + n_base + n, v);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *last_flag = (atomicAdd(p.counters + tile, 1) == p.splits - 1);
    __syncthreads();
    if (!*last_flag) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < cells; idx += kTileThreads) {
        const int m = idx >> 4, n = idx & 15;
        float* w = p.wsp + static_cast<size_t>(m) * p.N + n_base + n;
        y[static_cast<size_t>(m) * p.N + n_base + n] = from_float<ActT>(__ldcg(w));
        __stcg(w, 0.f);
    }
    if (threadIdx.x == 0) p.counters[tile] = 0;
}

template <typename ActT, int MT, bool ONE>
__global__ void __launch_bounds__(kTileThreads) w4a16_tile_kernel(const W4Params p) {
    __shared__ float red[kTileWarps][MT * 8][16];
    __shared__ int last_flag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next grid may start filling free SM slots
    const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
    w4_tile<ActT, MT, ONE>(p, tile, split, red, &last_flag);
}

// K splits per tile: enough CTAs that the hardware scheduler can even out the SMs (about 12 per SM), while a CTA
// still streams at least 8 items (8 KB).
static int plan_splits(int64_t K, int64_t N) {
    const int items = static_cast<int>(K / 128);
    const long long tiles = N / 16;
    const long long want = 12LL * sm_count();
    int s = static_cast<int>(ceil_div(want, tiles));
    if (s < 1) s = 1;
    const int max_s = items >= 8 ? items / 8 : 1;
    if (s > max_s) s = max_s;
    return s;
}

template <typename ActT, int MT, bool ONE>
static int launch_w4_one(const W4Params& p, cudaStream_t stream) {
    const long long ctas = static_cast<long long>(p.N / 16) * p.splits;
    // programmatic dependent launch, as the reference's runtime uses on sm_90+ (crates/emmy-runtime/src/cuda.rs:1299-1327)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kTileThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, w4a16_tile_kernel<ActT, MT, ONE>, p));
    return EQ_OK;
}

template <typename ActT>
static int launch_w4(const W4Params& p, cudaStream_t stream) {
    if (p.M == 1) return launch_w4_one<ActT, 1, true>(p, stream);
    if (p.M <= 8) return launch_w4_one<ActT, 1, false>(p, stream);
    if (p.M <= 16) return launch_w4_one<ActT, 2, false>(p, stream);
    if (p.M <= 32) return launch_w4_one<ActT, 4, false>(p, stream);
    return launch_w4_one<ActT, 8, false>(p, stream);
}

}  // namespace eq

using namespace eq;

extern "C" size_t eq_w4a16_workspace_bytes(int64_t M, int64_t N) {
    if (M <= 0 || N <= 0) return 0;
    const int64_t rows = M < 64 ? M : 64;  // larger M runs in 64-row blocks that reuse the scratch
    return static_cast<size_t>(rows) * N * sizeof(float) + static_cast<size_t>(N / 16 + 1) * sizeof(int);
}

extern "C" int eq_w4a16_linear(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N, int64_t G,
                               const void* x, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                               void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(wq && (M == 0 || (x && y)), EQ_ERR_BAD_ARG, "eq_w4a16_linear: null pointer");
    EQ_REQUIRE(K > 0 && N > 0 && M >= 0, EQ_ERR_BAD_ARG, "eq_w4a16_linear: bad extents M=%lld K=%lld N=%lld", (long long)M,
               (long long)K, (long long)N);
    if (G == -1) G = K;
    EQ_REQUIRE(G > 0 && K % G == 0, EQ_ERR_BAD_ARG, "eq_w4a16_linear: group size %lld does not cover K=%lld", (long long)G,
               (long long)K);
    EQ_REQUIRE(K % 128 == 0 && N % 16 == 0 && G % 128 == 0, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear: needs K %% 128 == 0, N %% 16 == 0, G %% 128 == 0 (K=%lld N=%lld G=%lld)", (long long)K,
               (long long)N, (long long)G);
    EQ_REQUIRE(K < (1 << 24) && N < (1 << 24), EQ_ERR_UNSUPPORTED, "eq_w4a16_linear: extent too large");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_w4a16_linear: activations must be f16 or bf16");
    EQ_REQUIRE(scale_dtype == EQ_F16 || scale_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_w4a16_linear: scales must be f16 or bf16");
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(aligned(wq, 16) && aligned(x, 16) && aligned(y, 2), EQ_ERR_BAD_ALIGN,
               "eq_w4a16_linear: wq and x need 16-byte alignment");
    EQ_REQUIRE(workspace && workspace_bytes >= eq_w4a16_workspace_bytes(M, N), EQ_ERR_WORKSPACE,
               "eq_w4a16_linear: workspace of %zu bytes needed, %zu given", eq_w4a16_workspace_bytes(M, N), workspace_bytes);
    EQ_REQUIRE(aligned(workspace, 16), EQ_ERR_BAD_ALIGN, "eq_w4a16_linear: workspace must be 16-byte aligned");

    const size_t esz = 2;
    for (int64_t m0 = 0; m0 < M; m0 += 64) {
        const int mb = static_cast<int>(M - m0 < 64 ? M - m0 : 64);
        W4Params p;
        p.wq = static_cast<const unsigned char*>(wq);
        p.perm = perm;
        p.x = static_cast<const char*>(x) + static_cast<size_t>(m0) * K * esz;
        p.y = static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz;
        p.wsp = static_cast<float*>(workspace);
        const int64_t ws_rows = M < 64 ? M : 64;
        p.counters = reinterpret_cast<int*>(static_cast<float*>(workspace) + ws_rows * N);
        p.K = static_cast<int>(K);
        p.N = static_cast<int>(N);
        p.M = mb;
        p.items = static_cast<int>(K / 128);
        p.splits = plan_splits(K, N);
        p.scale_dtype = scale_dtype;
        const int st = act_dtype == EQ_F16 ? launch_w4<__half>(p, stream) : launch_w4<__nv_bfloat16>(p, stream);
        if (st != EQ_OK) return st;
    }
    return EQ_OK;
}

// The kernel has no device-side wait; the status word of the workspace is kept for the boundary's sake and is
// always clear.
extern "C" int eq_w4a16_status(const void* workspace, int64_t M, int64_t N, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && N > 0, EQ_ERR_BAD_ARG, "eq_w4a16_status: bad arguments");
    const int64_t ws_rows = M < 64 ? M : 64;
    const int* status = reinterpret_cast<const int*>(static_cast<const float*>(workspace) + ws_rows * N) + N / 16;
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_w4a16_status: the workspace status word is set (%d)", host);
    return EQ_OK;
}

// ---- entry point for callers that cannot allocate ------------------------------------------------------------
// The scratch of eq_w4a16_linear (partial sums, arrival counters, status word) for up to kNoAllocMaxM rows and
// kNoAllocMaxN columns, resident in every device that loads this library until the process exits.
namespace {
constexpr int64_t kNoAllocMaxM = 16;
constexpr int64_t kNoAllocMaxN = 32768;
constexpr size_t kNoAllocBytes = static_cast<size_t>(kNoAllocMaxM) * kNoAllocMaxN * sizeof(float) +
                                 (static_cast<size_t>(kNoAllocMaxN) / 16 + 1) * sizeof(int) + 252;
static __device__ __align__(256) unsigned char g_w4_noalloc_scratch[kNoAllocBytes];

// Device address of the array above on the current device.  The array's name is only a host-side handle; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int noalloc_scratch(void** out) {
    static void* cached[64] = {nullptr};
    int dev = -1;
    EQ_CUDA_OK(cudaGetDevice(&dev));
    EQ_REQUIRE(dev >= 0 && dev < 64, EQ_ERR_UNSUPPORTED, "eq_w4a16_linear_noalloc: device index %d out of range", dev);
    void* ptr = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (!ptr) {
        EQ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_w4_noalloc_scratch));
        EQ_REQUIRE(ptr != nullptr, EQ_ERR_CUDA, "eq_w4a16_linear_noalloc: no device address for the static scratch");
        __atomic_store_n(&cached[dev], ptr, __ATOMIC_RELEASE);
    }
    *out = ptr;
    return EQ_OK;
}
}  // namespace

extern "C" int eq_w4a16_linear_noalloc(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N,
                                       int64_t G, const void* x, int64_t M, int act_dtype, void* y, void* stream_) {
    EQ_REQUIRE(M >= 0 && M <= kNoAllocMaxM, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear_noalloc: M=%lld exceeds the built-in scratch (at most %lld rows); use eq_w4a16_linear with "
               "a caller workspace",
               (long long)M, (long long)kNoAllocMaxM);
    EQ_REQUIRE(N > 0 && N <= kNoAllocMaxN, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear_noalloc: N=%lld exceeds the built-in scratch (at most %lld columns); use eq_w4a16_linear "
               "with a caller workspace",
               (long long)N, (long long)kNoAllocMaxN);
    if (M == 0) return EQ_OK;
    void* scratch = nullptr;
    int st = noalloc_scratch(&scratch);
    if (st != EQ_OK) return st;
    const size_t used = eq_w4a16_workspace_bytes(M, N);
    // all calls share the one array: whatever an earlier (possibly failed) call left there is cleared first
    EQ_CUDA_OK(cudaMemsetAsync(scratch, 0, used, static_cast<cudaStream_t>(stream_)));
    return eq_w4a16_linear(wq, scale_dtype, perm, K, N, G, x, M, act_dtype, y, scratch, used, stream_);
}
