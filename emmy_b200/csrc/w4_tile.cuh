// Device code shared by the W4A16 linear (w4_gemv.cu) and the grouped expert kernels (moe.cu): the fragment
// expansion of packed nibbles, the per-lane activation load and the body that computes one 16-column output tile of
// one K split.  See w4_gemv.cu for the description of the kernel built from it.
#pragma once
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
    int span_base, span_rem;  // stream kernel: whole tiles per CTA, plus one for the first span_rem CTAs
    int acc_tiles;            // stream kernel: accumulator slots per CTA (the largest tile count)
    int group_tiles;          // stream kernel, K split: column tiles per CTA group (CTA = group * splits + K slice)
    const int32_t* x_rows;    // optional: activation row m of the problem is row x_rows[m] of x (gather)
    const int32_t* y_rows;    // optional: output row m of the problem is row y_rows[m] of y (scatter)
    const uint64_t* y_ptrs;   // optional (unsplit tiles only): output row m starts at address y_ptrs[m], possibly on a peer GPU
};

// A run of rows of one expert in an expert-ordered row list (grouped expert GEMMs).
struct RowBlock {
    int32_t expert, row0, rows, pad;
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

// The rows of x an item multiplies, as the lane's MMA operands: rows mt * 8 + g, the 32 input positions from
// it * 128 + 32 * j on.  Rows beyond M read as zeros.
template <typename ActT, int MT, bool ONE>
__device__ __forceinline__ void w4_item_x(const W4Params& p, const ActT* x, int it, int g, int j, uint4 (&xv)[MT][4]) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int m = ONE ? 0 : mt * 8 + g;
        if (ONE || m < p.M) {
            const size_t xr = p.x_rows ? static_cast<size_t>(p.x_rows[m]) : static_cast<size_t>(m);
            load_x<ActT>(x + xr * p.K, p.perm, it * 128 + 32 * j, xv[mt]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[mt][i] = make_uint4(0, 0, 0, 0);
        }
    }
}

// One item (128 input rows x 16 columns) of a tile against the rows of x: yacc += s * sum_k x_k (q_k - z).
// wl / wh: the lane's 16 bytes of the item's two nibble tiles; meta: its scale / zero entry (columns g, g+8);
// xv: the lane's operands from w4_item_x.
// PAIRED: the sixteen operand words of a row block come in pair order {low slot, high slot} per k16 step (the staged
// copies are stored that way), so an MMA's two B registers are neighbours of one vector and need no moves; otherwise
// they are the natural order of 32 consecutive activations: words 0..7 the low slots, 8..15 the high ones.
template <typename ActT, int MT, bool PAIRED = false>
__device__ __forceinline__ void w4_item_math(const W4Params& p, const uint4 (&xv)[MT][4], const uint4& wl, const uint4& wh, const uint2& mt_,
                                             float (&yacc)[MT][4]) {
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
    // even and odd k16 steps accumulate into separate registers: two chains of four MMAs instead of one of eight
    float acc[2][MT][4];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        uint32_t a[4];
        Frag<ActT>::expand(words[s], z_lo, z_hi, a);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&xv[mt][0]);
            const uint32_t b0 = PAIRED ? w[2 * s] : w[s], b1 = PAIRED ? w[2 * s + 1] : w[8 + s];
            if (s < 2)
                Frag<ActT>::mma0(acc[s & 1][mt], a, b0, b1);
            else
                Frag<ActT>::mma(acc[s & 1][mt], a, b0, b1);
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        yacc[mt][0] = fmaf(s_lo, acc[0][mt][0] + acc[1][mt][0], yacc[mt][0]);
        yacc[mt][1] = fmaf(s_lo, acc[0][mt][1] + acc[1][mt][1], yacc[mt][1]);
        yacc[mt][2] = fmaf(s_hi, acc[0][mt][2] + acc[1][mt][2], yacc[mt][2]);
        yacc[mt][3] = fmaf(s_hi, acc[0][mt][3] + acc[1][mt][3], yacc[mt][3]);
    }
}

// The same product for three (or more) row blocks whose operands lie in shared memory in the order the lanes read them
// (xs_lane: this lane's first 16 bytes of the item; row block mt, chunk c at (mt * 4 + c) * 512; words in pair order).  The eight weight
// fragments are expanded once and kept; each row block then loads its own operands, so the registers hold one block's
// operands at a time instead of all of them.
template <typename ActT, int MT>
__device__ __forceinline__ void w4_item_math_smem(const W4Params& p, const unsigned char* xs_lane, const uint4& wl, const uint4& wh,
                                                  const uint2& mt_, float (&yacc)[MT][4]) {
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
    uint32_t a[8][4];
#pragma unroll
    for (int s = 0; s < 8; ++s) Frag<ActT>::expand(words[s], z_lo, z_hi, a[s]);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        uint4 xv[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) xv[c] = *reinterpret_cast<const uint4*>(xs_lane + (mt * 4 + c) * 512);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&xv[0]);  // pair order: {low slot, high slot} per step
        float acc[2][4];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s < 2)
                Frag<ActT>::mma0(acc[s & 1], a[s], w[2 * s], w[2 * s + 1]);
            else
                Frag<ActT>::mma(acc[s & 1], a[s], w[2 * s], w[2 * s + 1]);
        }
        yacc[mt][0] = fmaf(s_lo, acc[0][0] + acc[1][0], yacc[mt][0]);
        yacc[mt][1] = fmaf(s_lo, acc[0][1] + acc[1][1], yacc[mt][1]);
        yacc[mt][2] = fmaf(s_hi, acc[0][2] + acc[1][2], yacc[mt][2]);
        yacc[mt][3] = fmaf(s_hi, acc[0][3] + acc[1][3], yacc[mt][3]);
    }
}

template <typename ActT, int MT, bool ONE>
__device__ __forceinline__ void w4_item(const W4Params& p, const ActT* x, int it, const uint4& wl, const uint4& wh, const uint2& mt_,
                                        int g, int j, float (&yacc)[MT][4]) {
    uint4 xv[MT][4];
    w4_item_x<ActT, MT, ONE>(p, x, it, g, j, xv);
    w4_item_math<ActT, MT>(p, xv, wl, wh, mt_, yacc);
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
                w4_item<ActT, MT, ONE>(p, x, it, wl, wh, mt_, g, j, yacc);
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
            if (p.y_ptrs) {
                reinterpret_cast<ActT*>(p.y_ptrs[m])[n_base + n] = from_float<ActT>(v);
            } else {
                const size_t yr = p.y_rows ? static_cast<size_t>(p.y_rows[m]) : static_cast<size_t>(m);
                y[yr * p.N + n_base + n] = from_float<ActT>(v);
            }
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


}  // namespace eq
