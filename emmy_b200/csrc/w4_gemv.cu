// W4A16 linear for decode-shaped calls (and, in 64-row blocks, for any M): y[M,N] = x[M,K] @ W, W int4 group-wise.
//
// A bandwidth kernel.  The repacked weight (w4_repack.cu) is one flat run of 512-byte tiles, [n-tile][k-chunk], a
// tile being 16 output columns x 64 input rows.  The grid is persistent-sized (a multiple of the SM count) and
// every CTA takes an EQUAL contiguous span of that run, whatever the tile boundaries (stream-K), so all SMs stream
// the same number of bytes.  Inside a CTA each warp takes an equal sub-span.  Per tile-chunk a lane issues one
// 16-byte streaming load (a warp: 512 contiguous bytes), turns its four words into four m16n8k16 A fragments with
// lop3 + one f16x2 subtract/fma per pair of nibbles (exact: (1024+q) - (1024+z)), and feeds mma.sync with the
// activations as the B operand, f32 accumulators.  The per-group scale multiplies the group's partial sum once
// (sum_k x*(q-z) is exact integer-times-activation work; s is applied in f32).
//
// Partial sums of one output tile meet in two levels: warps of a CTA add into shared-memory accumulators and the
// warp that completes the CTA's share of a tile either stores y (tile wholly inside the CTA span, single K slice)
// or adds the CTA's sum into the f32 workspace; the CTA whose contribution completes the tile converts, stores y
// and leaves workspace and counter zero for the next call.  Nobody waits on anybody: "last arriver finishes".
// A CTA handles the tiles it shares with its neighbours FIRST, so that second level is off the tail of the kernel.
//
// K is cut into S slices only when the activations of a whole K run do not fit shared memory (M > 1 and large K).
#include "common.cuh"

namespace eq {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kDepth = 4;  // tile-chunks in flight per warp (registers)

struct W4Params {
    const uint4* wq;       // [n_tiles][chunks][32] lanes
    const uint2* wm;       // [n_tiles][groups][8]: {s[g] | s[g+8] << 16, z[g] | z[g+8] << 8}
    const int32_t* perm;   // optional [K]
    const void* x;         // [M][K]
    void* y;               // [M][N]
    float* wsp;            // [M][N] partial sums (zero between calls)
    int* counters;         // [n_tiles] chunks arrived (zero between calls)
    int K, N, M;
    int chunks;            // K / 64
    int chunks_per_group;  // G / 64
    int groups;            // K / G
    int n_tiles;           // N / 16
    int slices;            // S
    int cs;                // chunks per slice
    int ctas_per_slice;    // P
    int rows;              // activation rows kept per 8-row m-tile in shared memory (M for M < 8, else 8)
    int slots;             // shared accumulator slots (max tiles a CTA span touches)
    int scale_dtype;
};

template <typename ActT>
struct Frag;

template <>
struct Frag<__half> {
    // four words of one lane -> A fragment registers of k16 step `w`, zero point removed
    static __device__ __forceinline__ void dequant(uint32_t w, uint32_t zlo, uint32_t zhi, uint32_t nzlo, uint32_t nzhi,
                                                   uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;  // 1024.0 | 1024.0: (w & mask) | magic == 1024 + q (or 1024 + 16 q)
        const uint32_t h0 = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        const uint32_t h1 = lop3<0xEA>(w, 0x00F000F0u, kMagic);
        const uint32_t w8 = w >> 8;
        const uint32_t h2 = lop3<0xEA>(w8, 0x000F000Fu, kMagic);
        const uint32_t h3 = lop3<0xEA>(w8, 0x00F000F0u, kMagic);
        constexpr uint32_t kSixteenth = 0x2C002C00u;  // 1/16 | 1/16
        asm("sub.f16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(h0), "r"(zlo));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[2]) : "r"(h1), "r"(kSixteenth), "r"(nzlo));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(a[1]) : "r"(h2), "r"(zhi));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[3]) : "r"(h3), "r"(kSixteenth), "r"(nzhi));
    }
    // zero point z (0..16) -> {1024 + z} pair and {-(64 + z)} pair
    static __device__ __forceinline__ void zero_consts(uint32_t z, uint32_t& sub, uint32_t& fma) {
        const __half2 s = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400u)));  // 1024
        const __half2 zz = __half2half2(__uint2half_rn(z));
        const __half2 a = __hadd2(s, zz);
        const __half2 b = __hneg2(__hadd2(__half2half2(__float2half_rn(64.f)), zz));
        sub = *reinterpret_cast<const uint32_t*>(&a);
        fma = *reinterpret_cast<const uint32_t*>(&b);
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <>
struct Frag<__nv_bfloat16> {
    static __device__ __forceinline__ void dequant(uint32_t w, uint32_t zlo, uint32_t zhi, uint32_t, uint32_t,
                                                   uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x43004300u;  // 128.0 | 128.0: 128 + q is exact in bf16
        const uint32_t t0 = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        const uint32_t t1 = lop3<0xEA>(w >> 4, 0x000F000Fu, kMagic);
        const uint32_t t2 = lop3<0xEA>(w >> 8, 0x000F000Fu, kMagic);
        const uint32_t t3 = lop3<0xEA>(w >> 12, 0x000F000Fu, kMagic);
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(t0), "r"(zlo));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[2]) : "r"(t1), "r"(zlo));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[1]) : "r"(t2), "r"(zhi));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(a[3]) : "r"(t3), "r"(zhi));
    }
    static __device__ __forceinline__ void zero_consts(uint32_t z, uint32_t& sub, uint32_t& fma) {
        const __nv_bfloat162 a = __float2bfloat162_rn(128.f + static_cast<float>(z));
        sub = *reinterpret_cast<const uint32_t*>(&a);
        fma = 0;
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

// Position q of a CTA's processing order -> item index.  Order: the partial tile at the head of the span, the
// partial tile at its tail, then the whole tiles between them.
struct SpanOrder {
    int i0, i1, nh, nt;
    __device__ __forceinline__ int item(int q) const {
        if (q < nh) return i0 + q;
        if (q < nh + nt) return i1 - nt + (q - nh);
        return i0 + nh + (q - nh - nt);
    }
};

template <typename ActT, int MT>
__global__ void __launch_bounds__(kThreads, (MT <= 2 ? 3 : 1)) w4a16_streamk_kernel(const W4Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;

    const int slice = blockIdx.x / p.ctas_per_slice;
    const int part = blockIdx.x % p.ctas_per_slice;
    const long long items = static_cast<long long>(p.n_tiles) * p.cs;
    const int i0 = static_cast<int>(items * part / p.ctas_per_slice);
    const int i1 = static_cast<int>(items * (part + 1) / p.ctas_per_slice);

    // shared memory: activations in B-fragment order, accumulator slots, slot counters
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);
    const int xs_vecs = p.cs * MT * 2 * p.rows * 4;
    float* accs = reinterpret_cast<float*>(xs + xs_vecs);           // [slots][MT*8][16]
    int* slot_cnt = reinterpret_cast<int*>(accs + p.slots * MT * 128);  // [slots]

    for (int i = threadIdx.x; i < p.slots * MT * 128; i += kThreads) accs[i] = 0.f;
    for (int i = threadIdx.x; i < p.slots; i += kThreads) slot_cnt[i] = 0;

    // ---- stage this slice of x: word (chunk, mt, half, r, j, wi) = {x[m][k], x[m][k+1]},
    //      k = 64 chunk + 16 (2 half + wi/2) + 8 (wi & 1) + 2 j, m = 8 mt + r
    {
        uint32_t* xw = reinterpret_cast<uint32_t*>(xs);
        const ActT* x = static_cast<const ActT*>(p.x);
        const int total = xs_vecs * 4;
        const int kbase = slice * p.cs * 64;
        for (int idx = threadIdx.x; idx < total; idx += kThreads) {
            const int wi = idx & 3, jj = (idx >> 2) & 3;
            int rest = idx >> 4;
            const int r = rest % p.rows;
            rest /= p.rows;
            const int half = rest & 1;
            rest >>= 1;
            const int mt = rest % MT;
            const int chunk = rest / MT;
            const int k = kbase + 64 * chunk + 16 * (2 * half + (wi >> 1)) + 8 * (wi & 1) + 2 * jj;
            const int m = 8 * mt + r;
            uint32_t v = 0;
            if (m < p.M) {
                if (p.perm) {
                    const ActT lo = x[static_cast<size_t>(m) * p.K + p.perm[k]];
                    const ActT hi = x[static_cast<size_t>(m) * p.K + p.perm[k + 1]];
                    v = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&lo)) |
                        (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
                } else {
                    v = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(m) * p.K + k);
                }
            }
            xw[idx] = v;
        }
    }
    __syncthreads();

    // ---- this warp's share of the CTA span
    const int first_tile = i0 / p.cs;
    SpanOrder order;
    order.i0 = i0;
    order.i1 = i1;
    {
        const int head_end = min(i1, (first_tile + 1) * p.cs);
        order.nh = (i0 % p.cs) ? head_end - i0 : 0;
        const int tail_start = (i1 / p.cs) * p.cs;
        order.nt = (i1 % p.cs && tail_start >= i0 + order.nh) ? i1 - max(tail_start, i0 + order.nh) : 0;
    }
    const int span = i1 - i0;
    const int q0 = static_cast<int>(static_cast<long long>(span) * warp / kWarps);
    const int q1 = static_cast<int>(static_cast<long long>(span) * (warp + 1) / kWarps);

    // register pipeline
    uint4 wbuf[kDepth];
    uint2 mbuf[kDepth];
    int tbuf[kDepth], cbuf[kDepth];

    auto issue = [&](int slot, int q) {
        if (q < q1) {
            const int it = order.item(q);
            const int t = it / p.cs;
            const int c = slice * p.cs + (it - t * p.cs);
            tbuf[slot] = t;
            cbuf[slot] = c;
            wbuf[slot] = ld_stream_v4(p.wq + (static_cast<size_t>(t) * p.chunks + c) * 32 + lane);
            mbuf[slot] = __ldg(p.wm + (static_cast<size_t>(t) * p.groups + c / p.chunks_per_group) * 8 + g);
        }
    };

    float acc[MT][4], yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = yacc[mt][e] = 0.f;

    int cur_t = -1, cur_grp = -1, done_chunks = 0;
    float slo = 0.f, shi = 0.f;
    uint32_t zlo = 0, zhi = 0, nzlo = 0, nzhi = 0;

    auto fold_group = [&]() {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            yacc[mt][0] = fmaf(slo, acc[mt][0], yacc[mt][0]);
            yacc[mt][1] = fmaf(slo, acc[mt][1], yacc[mt][1]);
            yacc[mt][2] = fmaf(shi, acc[mt][2], yacc[mt][2]);
            yacc[mt][3] = fmaf(shi, acc[mt][3], yacc[mt][3]);
            acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
        }
    };

    // Hand this warp's sum for tile `t` to the CTA's slot; the warp that completes the CTA's share finishes it.
    auto flush_tile = [&](int t, int nchunks) {
        const int slot = t - first_tile;
        float* a = accs + slot * MT * 128;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = 8 * mt + 2 * j + (e & 1);
                const int n = g + ((e & 2) ? 8 : 0);
                if (m < p.M) atomicAdd(a + m * 16 + n, yacc[mt][e]);
                yacc[mt][e] = 0.f;
            }
        }
        __syncwarp();
        // this CTA's share of tile t, in chunks
        const int lo = max(i0, t * p.cs), hi = min(i1, (t + 1) * p.cs);
        const int share = hi - lo;
        int last = 0;
        if (lane == 0) {
            __threadfence_block();
            last = (atomicAdd(slot_cnt + slot, nchunks) + nchunks == share);
        }
        last = __shfl_sync(0xFFFFFFFFu, last, 0);
        if (!last) return;
        __threadfence_block();
        ActT* y = static_cast<ActT*>(p.y);
        const int n_base = t * 16;
        const bool whole = (share == p.cs) && (p.slices == 1);
        if (whole) {
            for (int idx = lane; idx < p.M * 16; idx += 32) {
                const int m = idx >> 4, n = idx & 15;
                y[static_cast<size_t>(m) * p.N + n_base + n] = from_float<ActT>(a[m * 16 + n]);
            }
            return;
        }
        // second level: add the CTA's sum into the workspace, then count the CTA's chunks in
        for (int idx = lane; idx < p.M * 16; idx += 32) {
            const int m = idx >> 4, n = idx & 15;
            atomicAdd(p.wsp + static_cast<size_t>(m) * p.N + n_base + n, a[m * 16 + n]);
        }
        __syncwarp();
        int finisher = 0;
        if (lane == 0) {
            __threadfence();
            finisher = (atomicAdd(p.counters + t, share) + share == p.chunks);
        }
        finisher = __shfl_sync(0xFFFFFFFFu, finisher, 0);
        if (!finisher) return;
        __threadfence();
        for (int idx = lane; idx < p.M * 16; idx += 32) {
            const int m = idx >> 4, n = idx & 15;
            float* w = p.wsp + static_cast<size_t>(m) * p.N + n_base + n;
            y[static_cast<size_t>(m) * p.N + n_base + n] = from_float<ActT>(__ldcg(w));
            __stcg(w, 0.f);
        }
        if (lane == 0) p.counters[t] = 0;
    };

    // prologue
#pragma unroll
    for (int d = 0; d < kDepth; ++d) issue(d, q0 + d);

    for (int qb = q0; qb < q1; qb += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            const int q = qb + d;
            if (q < q1) {
                const uint4 w4 = wbuf[d];
                const uint2 meta = mbuf[d];
                const int t = tbuf[d], c = cbuf[d];
                issue(d, q + kDepth);  // refill this register slot
                const int grp = c / p.chunks_per_group;
                if (t != cur_t || grp != cur_grp) {
                    if (cur_t >= 0) fold_group();
                    if (t != cur_t) {
                        if (cur_t >= 0) flush_tile(cur_t, done_chunks);
                        cur_t = t;
                        done_chunks = 0;
                    }
                    cur_grp = grp;
                    slo = scale16_to_float(static_cast<uint16_t>(meta.x & 0xFFFF), p.scale_dtype);
                    shi = scale16_to_float(static_cast<uint16_t>(meta.x >> 16), p.scale_dtype);
                    Frag<ActT>::zero_consts(meta.y & 0xFF, zlo, nzlo);
                    Frag<ActT>::zero_consts((meta.y >> 8) & 0xFF, zhi, nzhi);
                }
                ++done_chunks;
                // B fragments of the four k16 steps of this chunk
                const int c_local = c - slice * p.cs;
                const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
                const uint2* xs2 = reinterpret_cast<const uint2*>(xs);
#pragma unroll
                for (int step = 0; step < 4; ++step) {
                    uint32_t a[4];
                    Frag<ActT>::dequant(words[step], zlo, zhi, nzlo, nzhi, a);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint2 b = make_uint2(0, 0);
                        if (g < p.rows)
                            b = xs2[(((((c_local * MT + mt) * 2 + (step >> 1)) * p.rows + g) * 4 + j) << 1) + (step & 1)];
                        Frag<ActT>::mma(acc[mt], a, b.x, b.y);
                    }
                }
            }
        }
    }
    if (cur_t >= 0) {
        fold_group();
        flush_tile(cur_t, done_chunks);
    }
}

struct W4Plan {
    int mt, rows, slices, cs, ctas_per_slice, slots;
    size_t smem;
};

static int plan_w4(int64_t K, int64_t N, int M, W4Plan& pl) {
    const int chunks = static_cast<int>(K / 64), n_tiles = static_cast<int>(N / 16);
    int mt = (M + 7) / 8;
    pl.mt = mt <= 1 ? 1 : mt <= 2 ? 2 : mt <= 4 ? 4 : 8;
    pl.rows = pl.mt == 1 ? (M < 8 ? M : 8) : 8;
    const int xs_budget = pl.mt <= 2 ? 64 * 1024 : 96 * 1024;
    const int cs_max = xs_budget / (128 * pl.mt * pl.rows);
    EQ_REQUIRE(cs_max >= 1, EQ_ERR_UNSUPPORTED, "plan_w4: activation tile does not fit shared memory");
    int s = static_cast<int>(ceil_div(chunks, cs_max));
    while (chunks % s) ++s;
    pl.slices = s;
    pl.cs = chunks / s;
    const int occupancy = pl.mt <= 2 ? 3 : 1;
    const long long items = static_cast<long long>(n_tiles) * pl.cs;
    int p = sm_count() * occupancy / s;
    if (p < 1) p = 1;
    // keep at least one chunk per warp on average, and bound the accumulator slots of a CTA
    if (static_cast<long long>(p) * kWarps > items) p = static_cast<int>(ceil_div(items, kWarps));
    const int max_slots = pl.mt <= 2 ? 32 : 8;
    long long per_cta = ceil_div(items, p);
    if (ceil_div(per_cta, pl.cs) + 1 > max_slots) {
        per_cta = static_cast<long long>(max_slots - 1) * pl.cs;
        p = static_cast<int>(ceil_div(items, per_cta));
    }
    pl.ctas_per_slice = p;
    per_cta = ceil_div(items, p);
    pl.slots = static_cast<int>(ceil_div(per_cta, pl.cs) + 1);
    pl.smem = static_cast<size_t>(pl.cs) * pl.mt * 2 * pl.rows * 4 * 16 + static_cast<size_t>(pl.slots) * pl.mt * 128 * 4 +
              static_cast<size_t>(pl.slots) * 4;
    return EQ_OK;
}

template <typename ActT, int MT>
static int launch_w4(const W4Params& p, const W4Plan& pl, cudaStream_t stream) {
    auto kernel = w4a16_streamk_kernel<ActT, MT>;
    if (pl.smem > 48 * 1024)
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    kernel<<<static_cast<unsigned>(pl.slices * pl.ctas_per_slice), kThreads, pl.smem, stream>>>(p);
    EQ_LAUNCH_OK("w4a16_streamk_kernel");
    return EQ_OK;
}

}  // namespace eq

using namespace eq;

extern "C" size_t eq_w4a16_workspace_bytes(int64_t M, int64_t N) {
    if (M <= 0 || N <= 0) return 0;
    const int64_t rows = M < 64 ? M : 64;  // larger M runs in 64-row blocks that reuse the scratch
    return static_cast<size_t>(rows) * N * sizeof(float) + static_cast<size_t>(N / 16 + 1) * sizeof(int);
}

extern "C" int eq_w4a16_linear(const void* wq, const void* wm, int scale_dtype, const int32_t* perm, int64_t K,
                               int64_t N, int64_t G, const void* x, int64_t M, int act_dtype, void* y, void* workspace,
                               size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(wq && wm && x && y, EQ_ERR_BAD_ARG, "eq_w4a16_linear: null pointer");
    EQ_REQUIRE(K > 0 && N > 0 && M >= 0, EQ_ERR_BAD_ARG, "eq_w4a16_linear: bad extents M=%lld K=%lld N=%lld", (long long)M,
               (long long)K, (long long)N);
    if (G == -1) G = K;
    EQ_REQUIRE(G > 0 && K % G == 0, EQ_ERR_BAD_ARG, "eq_w4a16_linear: group size %lld does not cover K=%lld", (long long)G,
               (long long)K);
    EQ_REQUIRE(K % 64 == 0 && N % 16 == 0 && G % 64 == 0, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear: needs K %% 64 == 0, N %% 16 == 0, G %% 64 == 0 (K=%lld N=%lld G=%lld)", (long long)K,
               (long long)N, (long long)G);
    EQ_REQUIRE(K < (1 << 24) && N < (1 << 24), EQ_ERR_UNSUPPORTED, "eq_w4a16_linear: extent too large");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_w4a16_linear: activations must be f16 or bf16");
    EQ_REQUIRE(scale_dtype == EQ_F16 || scale_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_w4a16_linear: scales must be f16 or bf16");
    EQ_REQUIRE(aligned(wq, 16) && aligned(wm, 8) && aligned(x, 4) && aligned(y, 2), EQ_ERR_BAD_ALIGN,
               "eq_w4a16_linear: wq needs 16-byte, wm 8-byte, x 4-byte alignment");
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(workspace && workspace_bytes >= eq_w4a16_workspace_bytes(M, N), EQ_ERR_WORKSPACE,
               "eq_w4a16_linear: workspace of %zu bytes needed, %zu given", eq_w4a16_workspace_bytes(M, N), workspace_bytes);
    EQ_REQUIRE(aligned(workspace, 16), EQ_ERR_BAD_ALIGN, "eq_w4a16_linear: workspace must be 16-byte aligned");

    const size_t esz = 2;
    for (int64_t m0 = 0; m0 < M; m0 += 64) {
        const int mb = static_cast<int>(M - m0 < 64 ? M - m0 : 64);
        W4Plan pl;
        int st = plan_w4(K, N, mb, pl);
        if (st != EQ_OK) return st;
        W4Params p;
        p.wq = static_cast<const uint4*>(wq);
        p.wm = static_cast<const uint2*>(wm);
        p.perm = perm;
        p.x = static_cast<const char*>(x) + static_cast<size_t>(m0) * K * esz;
        p.y = static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz;
        p.wsp = static_cast<float*>(workspace);
        const int64_t ws_rows = M < 64 ? M : 64;
        p.counters = reinterpret_cast<int*>(static_cast<float*>(workspace) + ws_rows * N);
        p.K = static_cast<int>(K);
        p.N = static_cast<int>(N);
        p.M = mb;
        p.chunks = static_cast<int>(K / 64);
        p.chunks_per_group = static_cast<int>(G / 64);
        p.groups = static_cast<int>(K / G);
        p.n_tiles = static_cast<int>(N / 16);
        p.slices = pl.slices;
        p.cs = pl.cs;
        p.ctas_per_slice = pl.ctas_per_slice;
        p.rows = pl.rows;
        p.slots = pl.slots;
        p.scale_dtype = scale_dtype;
#define EQ_W4_CASE(MTV)                                                                       \
    case MTV:                                                                                 \
        st = act_dtype == EQ_F16 ? launch_w4<__half, MTV>(p, pl, stream) : launch_w4<__nv_bfloat16, MTV>(p, pl, stream); \
        break;
        switch (pl.mt) {
            EQ_W4_CASE(1)
            EQ_W4_CASE(2)
            EQ_W4_CASE(4)
            EQ_W4_CASE(8)
            default: return fail(EQ_ERR_UNSUPPORTED, "eq_w4a16_linear: no kernel for %d m-tiles", pl.mt);
        }
#undef EQ_W4_CASE
        if (st != EQ_OK) return st;
    }
    return EQ_OK;
}
