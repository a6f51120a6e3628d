// W4A16 linear for decode-shaped calls (and, in 64-row blocks, for any M): y[M,N] = x[M,K] @ W, W int4 group-wise.
//
// A bandwidth kernel.  The repacked weight (w4_repack.cu) is one flat run of 1088-byte ITEM records, [n-tile][item]:
// 16 output columns x 128 input rows of nibbles plus that group's scales and zero points.  The grid is one fat CTA
// per SM and every CTA takes an EQUAL contiguous span of items, whatever the tile boundaries (stream-K), so all SMs
// stream the same number of bytes; the activations are staged once per SM.  Inside a CTA each warp takes an equal
// sub-span and keeps its own ring of kRing slots in shared memory.  A slot holds a BATCH of up to two consecutive
// items and is filled by one bulk asynchronous copy (cp.async.bulk, the 1-D TMA path) that lane 0 issues kRing
// batches ahead and that signals the slot's mbarrier: the weight bytes in flight live in shared memory, not in
// registers.  The (tile, item) walk of a warp is written once into a small descriptor table, so the steady-state
// loop spends its integer instructions on the nibbles.
//
// Per item a lane reads its 2 x 16 bytes and turns each word into one m16n8k16 A fragment with five integer
// instructions (one shift, four lop3): (w & 0x000F000F) | 0x64006400 is the f16 pair {1024 + q, 1024 + q'}.  The
// offset is NOT subtracted per element.  With the activations as the B operand (those of the k-slots that carry
// 1024 + 16 q are stored pre-divided by 16) the tensor core returns
//     acc = sum_k x_k q_k + 1024 * S1,     S1 = sum of the stored B values of the item,
// and the item's contribution is  s * (acc - 1024 S1 - z S2),  S2 = sum_k x_k, with 1024 S1 and S2 computed once
// per CTA while the activations are staged.  (bf16: 128 + q is exact, no pre-division, S1 = S2.)
//
// Partial sums of one output tile meet in two levels: warps of a CTA add into shared-memory accumulators and the
// warp that completes the CTA's share of a tile either stores y (tile wholly inside the CTA span, single K slice)
// or adds the CTA's sum into the f32 workspace; the CTA whose contribution completes the tile converts, stores y
// and leaves workspace and counter zero for the next call.  Nobody waits on anybody: "last arriver finishes".
// A CTA handles the tiles it shares with its neighbours FIRST, so that second level is off the tail of the kernel.
// The only waits are on a warp's own copies; they are bounded, and a wait that runs out sets a status word.
//
// K is cut into S slices only when the activations of a whole K run do not fit shared memory (M > 1 and large K).
#include "common.cuh"

namespace eq {

constexpr int kRing = 3;                 // batch slots per warp
constexpr int kBatch = 2;                // items per batch
constexpr int kItemBytes = 1088;         // 1024 B of nibbles + 64 B of scales / zero points
constexpr int kSlotBytes = kBatch * kItemBytes;
constexpr int kMaxBatches = 32;          // descriptor table entries per warp
constexpr int kXRegs = 4;                // activation vectors a thread has in flight while staging x
constexpr long long kWaitCycles = 2000000000LL;  // about a second: far beyond any real copy latency

struct W4Params {
    const unsigned char* wq;  // [n_tiles][items][1088]
    const int32_t* perm;      // optional [K]
    const void* x;            // [M][K]
    void* y;                  // [M][N]
    float* wsp;               // [M][N] partial sums (zero between calls)
    int* counters;            // [n_tiles] items arrived (zero between calls), then one status word
    int K, N, M;
    int items;                // K / 128
    int n_tiles;              // N / 16
    int slices;               // S
    int cs;                   // items per slice
    int ctas_per_slice;       // P
    int span_base, span_rem;  // items per CTA of a slice: span_base, plus one for the first span_rem CTAs
    int rows;                 // activation rows kept per 8-row m-tile in shared memory (M for M < 8, else 8)
    int slots;                // shared accumulator slots (max tiles a CTA span touches)
    int scale_dtype;
};

template <typename ActT>
struct Frag;

template <>
struct Frag<__half> {
    static constexpr float kOffset = 1024.f;
    static constexpr bool kPrescaleHi = true;
    // one word of a lane -> A fragment registers {1024+q} (a0, a1) and {1024+16q} (a2, a3)
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w, 0x00F000F0u, kMagic);
        const uint32_t w8 = w >> 8;
        a[1] = lop3<0xEA>(w8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w8, 0x00F000F0u, kMagic);
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
    static __device__ __forceinline__ uint32_t sixteenth(uint32_t pair) {
        uint32_t r;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(pair), "r"(0x2C002C00u));
        return r;
    }
    static __device__ __forceinline__ float pair_sum(uint32_t pair) {
        const __half2 h = *reinterpret_cast<const __half2*>(&pair);
        return __low2float(h) + __high2float(h);
    }
};

template <>
struct Frag<__nv_bfloat16> {
    static constexpr float kOffset = 128.f;
    static constexpr bool kPrescaleHi = false;
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x43004300u;  // 128 + q is exact in bf16
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w >> 4, 0x000F000Fu, kMagic);
        a[1] = lop3<0xEA>(w >> 8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w >> 12, 0x000F000Fu, kMagic);
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
    static __device__ __forceinline__ uint32_t sixteenth(uint32_t pair) { return pair; }
    static __device__ __forceinline__ float pair_sum(uint32_t pair) {
        return __uint_as_float(pair << 16) + __uint_as_float(pair & 0xFFFF0000u);
    }
};

// ---- mbarrier / bulk copy ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

#ifdef EQ_W4_TRACE
__device__ unsigned long long g_w4_trace[4096 * 8];
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define EQ_TRACE(slot)                                                                                \
    do {                                                                                              \
        if ((threadIdx.x & 31) == 0 && blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) < 4096)    \
            g_w4_trace[(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 8 + (slot)] = trace_now(); \
    } while (0)
#else
#define EQ_TRACE(slot) \
    do {               \
    } while (0)
#endif

// A CTA's span of items, visited in the order: partial tile at the head of the span, partial tile at its tail,
// then the whole tiles between them.  Position q of that order maps to an item index.
struct SpanOrder {
    int i0, i1, nh, nt;
    __device__ __forceinline__ int item(int q) const {
        if (q < nh) return i0 + q;
        if (q < nh + nt) return i1 - nt + (q - nh);
        return i0 + nh + (q - nh - nt);
    }
    __device__ __forceinline__ int next_jump(int q) const {
        if (q < nh) return nh;
        if (q < nh + nt) return nh + nt;
        return 0x7FFFFFFF;
    }
};

// One batch of a warp's walk: tile and in-slice item index of its first item, whether a second item follows it in
// memory, and that item's coordinates.  Packed as {t0 | n << 24 | tile_step << 28, cl0 | cl1 << 16}.
struct Batch {
    int t0, cl0, t1, cl1, n;
    __device__ __forceinline__ uint2 pack() const {
        return make_uint2(static_cast<uint32_t>(t0) | (static_cast<uint32_t>(n) << 24) |
                              (static_cast<uint32_t>(t1 - t0) << 28),
                          static_cast<uint32_t>(cl0) | (static_cast<uint32_t>(cl1) << 16));
    }
    static __device__ __forceinline__ Batch unpack(uint2 d) {
        Batch b;
        b.t0 = static_cast<int>(d.x & 0xFFFFFFu);
        b.n = static_cast<int>((d.x >> 24) & 0xF);
        b.t1 = b.t0 + static_cast<int>(d.x >> 28);
        b.cl0 = static_cast<int>(d.y & 0xFFFFu);
        b.cl1 = static_cast<int>(d.y >> 16);
        return b;
    }
};

// Walks a warp's positions batch by batch.  Consecutive positions are consecutive items except at the two jumps of
// SpanOrder; the second item joins the first's batch when its record follows the first's in memory.
struct BatchIter {
    int q, q_end, jump, t, cl;
    __device__ __forceinline__ void seek(const SpanOrder& o, int q_, int cs) {
        q = q_;
        const int it = o.item(q);
        t = it / cs;
        cl = it - t * cs;
        jump = o.next_jump(q);
    }
    __device__ __forceinline__ void step(const SpanOrder& o, int cs) {
        ++q;
        if (q < q_end) {
            if (q == jump) {
                seek(o, q, cs);
            } else if (++cl == cs) {
                cl = 0;
                ++t;
            }
        }
    }
    __device__ __forceinline__ Batch next(const SpanOrder& o, int cs, bool single_slice) {
        Batch b;
        b.t0 = t;
        b.cl0 = cl;
        b.n = 1;
        const bool jumps = (q + 1 == jump);
        step(o, cs);
        b.t1 = t;
        b.cl1 = cl;
        const bool contiguous = (q < q_end) && !jumps && (b.t1 == b.t0 || single_slice);
        if (contiguous) {
            b.n = 2;
            step(o, cs);
        } else {
            b.t1 = b.t0;
            b.cl1 = b.cl0;
        }
        return b;
    }
};

struct CtaView {
    float* accs;
    int* slot_cnt;
    int first_tile, i0, i1;
};

// Hand one warp's sum for tile `t` to the CTA's slot; the warp that completes the CTA's share finishes the tile.
template <typename ActT, int MT>
__device__ __noinline__ void flush_tile_impl(const W4Params& p, const CtaView& v, float (&yacc)[MT][4], int t, int nitems) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int slot = t - v.first_tile;
    float* a = v.accs + slot * MT * 128;
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
    const int lo = max(v.i0, t * p.cs), hi = min(v.i1, (t + 1) * p.cs);
    const int share = hi - lo;  // this CTA's items of tile t
    int last = 0;
    if (lane == 0) {
        __threadfence_block();
        last = (atomicAdd(v.slot_cnt + slot, nitems) + nitems == share);
    }
    last = __shfl_sync(0xFFFFFFFFu, last, 0);
    if (!last) return;
    __threadfence_block();
    ActT* y = static_cast<ActT*>(p.y);
    const int n_base = t * 16;
    if (share == p.cs && p.slices == 1) {
        for (int idx = lane; idx < p.M * 16; idx += 32) {
            const int m = idx >> 4, n = idx & 15;
            y[static_cast<size_t>(m) * p.N + n_base + n] = from_float<ActT>(a[m * 16 + n]);
        }
        return;
    }
    // second level: add the CTA's sum into the workspace, then count the CTA's items in
    for (int idx = lane; idx < p.M * 16; idx += 32) {
        const int m = idx >> 4, n = idx & 15;
        atomicAdd(p.wsp + static_cast<size_t>(m) * p.N + n_base + n, a[m * 16 + n]);
    }
    __syncwarp();
    int finisher = 0;
    if (lane == 0) {
        __threadfence();
        finisher = (atomicAdd(p.counters + t, share) + share == p.items);
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
}

// The noinline body takes its sums through memory; the wrapper hands it a copy so that the caller's running sums
// stay in registers across the steady-state loop.
template <typename ActT, int MT>
__device__ __forceinline__ void flush_tile(const W4Params& p, const CtaView& v, float (&yacc)[MT][4], int t, int nitems) {
    float tmp[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            tmp[mt][e] = yacc[mt][e];
            yacc[mt][e] = 0.f;
        }
    flush_tile_impl<ActT, MT>(p, v, tmp, t, nitems);
}

// 128 input rows x 16 columns against MT m-tiles of activations: eight k16 steps chained on one accumulator set.
// The first step multiplies into fresh registers (C = 0), so nothing has to be cleared between items.
// `wl` is the lane's 16 bytes of the first tile of the record, `xb` the lane's B vector of the item's first
// half-chunk; every other operand sits at a compile-time offset from those two.  With a single activation row all
// lanes read row 0: the m = 1..7 columns of the product are then copies of column 0 and are never looked at.
template <typename ActT, int MT, int ROWS>
__device__ __forceinline__ void item_mma(const unsigned char* wl, const uint4* xb, float (&acc)[MT][4]) {
    const uint4 w_lo = *reinterpret_cast<const uint4*>(wl);
    const uint4 w_hi = *reinterpret_cast<const uint4*>(wl + 512);
    const uint32_t words[8] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w, w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
    for (int hs = 0; hs < 4; ++hs) {  // half-chunks: two k16 steps each
        uint32_t a0[4], a1[4];
        Frag<ActT>::expand(words[2 * hs], a0);
        Frag<ActT>::expand(words[2 * hs + 1], a1);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const uint4 b = xb[(((hs >> 1) * MT + mt) * 2 + (hs & 1)) * ROWS * 4];
            if (hs == 0)
                Frag<ActT>::mma0(acc[mt], a0, b.x, b.y);
            else
                Frag<ActT>::mma(acc[mt], a0, b.x, b.y);
            Frag<ActT>::mma(acc[mt], a1, b.z, b.w);
        }
    }
}

// yacc += s * (acc - (offset S1 + z S2)) for one item.  ONE: a single activation row, only column m = 0 is live.
template <typename ActT, int MT, bool ONE>
__device__ __forceinline__ void item_fold(const unsigned char* meta_lane, const float2* xsum_lane, int scale_dtype,
                                          float (&acc)[MT][4], float (&yacc)[MT][4]) {
    const uint2 meta = *reinterpret_cast<const uint2*>(meta_lane);
    float slo, shi;
    if (scale_dtype == EQ_F16) {
        const __half2 s = *reinterpret_cast<const __half2*>(&meta.x);
        slo = __low2float(s);
        shi = __high2float(s);
    } else {
        slo = __uint_as_float(meta.x << 16);
        shi = __uint_as_float(meta.x & 0xFFFF0000u);
    }
    const __half2 z = *reinterpret_cast<const __half2*>(&meta.y);
    const float zlo = __low2float(z), zhi = __high2float(z);
    if constexpr (ONE) {
        const float2 s = xsum_lane[0];  // {offset S1, S2} of row 0
        yacc[0][0] = fmaf(slo, acc[0][0] - fmaf(zlo, s.y, s.x), yacc[0][0]);
        yacc[0][2] = fmaf(shi, acc[0][2] - fmaf(zhi, s.y, s.x), yacc[0][2]);
    } else {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const float4 s = *reinterpret_cast<const float4*>(xsum_lane + mt * 8);  // {offset S1, S2}[m0], [m1]
        yacc[mt][0] = fmaf(slo, acc[mt][0] - fmaf(zlo, s.y, s.x), yacc[mt][0]);
        yacc[mt][1] = fmaf(slo, acc[mt][1] - fmaf(zlo, s.w, s.z), yacc[mt][1]);
        yacc[mt][2] = fmaf(shi, acc[mt][2] - fmaf(zhi, s.y, s.x), yacc[mt][2]);
        yacc[mt][3] = fmaf(shi, acc[mt][3] - fmaf(zhi, s.w, s.z), yacc[mt][3]);
    }
    }
}

template <typename ActT, int MT, int WARPS, bool ONE>
__global__ void __launch_bounds__(WARPS * 32, 1) w4a16_streamk_kernel(const W4Params p) {
    constexpr int kThreads = WARPS * 32;
    constexpr int ROWS = ONE ? 1 : 8;  // activation rows kept per m-tile (rows beyond M are zero)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const int slice = blockIdx.x / p.ctas_per_slice;
    const int part = blockIdx.x - slice * p.ctas_per_slice;
    // equal spans: the first span_rem CTAs of a slice take one item more
    const int i0 = part * p.span_base + min(part, p.span_rem);
    const int i1 = i0 + p.span_base + (part < p.span_rem ? 1 : 0);
    EQ_TRACE(0);

    // ---- shared memory carve-up
    unsigned char* ring = smem_raw + warp * (kRing * kSlotBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + WARPS * kRing * kSlotBytes) + warp * kRing;
    uint2* desc = reinterpret_cast<uint2*>(smem_raw + WARPS * kRing * (kSlotBytes + 8)) + warp * kMaxBatches;
    uint4* xs = reinterpret_cast<uint4*>(smem_raw + WARPS * kRing * (kSlotBytes + 8) + WARPS * kMaxBatches * 8);
    const int xs_vecs = p.cs * 2 * MT * 2 * ROWS * 4;                   // [chunk64][mt][half][row][j]
    float2* xsum = reinterpret_cast<float2*>(xs + xs_vecs);             // [item][MT*8] {offset S1, S2}
    float* accs = reinterpret_cast<float*>(xsum + p.cs * MT * 8);       // [slots][MT*8][16]
    int* slot_cnt = reinterpret_cast<int*>(accs + p.slots * MT * 128);  // [slots]

    // ---- arm this warp's slot barriers, then walk its share of the CTA span: every batch goes into the descriptor
    //      table and the first kRing of them are requested at once, before anything else is touched
    if (lane == 0) {
        for (int s = 0; s < kRing; ++s) mbar_init(smem_addr(bars + s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    CtaView view;
    view.accs = accs;
    view.slot_cnt = slot_cnt;
    view.first_tile = i0 / p.cs;
    view.i0 = i0;
    view.i1 = i1;
    SpanOrder order;
    order.i0 = i0;
    order.i1 = i1;
    {
        const int head_end = min(i1, (view.first_tile + 1) * p.cs);
        order.nh = (i0 % p.cs) ? head_end - i0 : 0;
        const int tail_start = (i1 / p.cs) * p.cs;
        order.nt = (i1 % p.cs && tail_start >= i0 + order.nh) ? i1 - max(tail_start, i0 + order.nh) : 0;
    }
    const int span = i1 - i0;
    const int q0 = span * warp / WARPS;
    const int q1 = span * (warp + 1) / WARPS;
    const size_t slice_item0 = static_cast<size_t>(slice) * p.cs;
    auto request = [&](int slot, const Batch& b) {
        if (lane == 0) {
            const uint32_t bar = smem_addr(bars + slot);
            const uint32_t bytes = b.n * kItemBytes;
            mbar_expect_tx(bar, bytes);
            bulk_g2s(smem_addr(ring + slot * kSlotBytes),
                     p.wq + (static_cast<size_t>(b.t0) * p.items + slice_item0 + b.cl0) * kItemBytes, bytes, bar);
        }
    };
    int nb = 0;
    {
        // every lane walks the span (uniform work), lane 0 writes; nb ends up the same in all lanes
        BatchIter walk;
        walk.q = walk.q_end = q1;
        if (q0 < q1) walk.seek(order, q0, p.cs);
        while (walk.q < walk.q_end && nb < kMaxBatches) {
            const Batch b = walk.next(order, p.cs, p.slices == 1);
            if (nb < kRing) request(nb, b);
            if (lane == 0) desc[nb] = b.pack();
            ++nb;
        }
        if (walk.q < walk.q_end) {  // the host sizes the grid so that this cannot happen; never drop items silently
            if (lane == 0) atomicExch(p.counters + p.n_tiles, 2);
            nb = 0;  // this warp does nothing more, but still meets the CTA barriers below
        }
    }
    EQ_TRACE(1);

    // ---- stage this slice of x in B-fragment order.  Vector v of row m holds x[m][8v .. 8v+7]: one (chunk, step, b)
    //      with k = 64 chunk + 16 step + 8 b + 2 j, j = 0..3.  Word j lands at
    //      ((((chunk MT + mt) 2 + step/2) rows + r) 4 + j) 4 + 2 (step & 1) + b; b = 1 words are pre-divided by 16 (f16).
    {
        const ActT* x = static_cast<const ActT*>(p.x);
        const int kbase = slice * p.cs * 128;
        const int m_rows = min(p.M, MT * 8);
        const int vec_per_row = p.cs * 16;  // uint4 = 8 activations
        const int total_vecs = m_rows * vec_per_row;
        uint32_t* xw = reinterpret_cast<uint32_t*>(xs);
        auto store_vec = [&](int m, int v, uint4 val) {
            const int chunk = v >> 3, step = (v >> 1) & 3, b = v & 1;
            if (Frag<ActT>::kPrescaleHi && b) {
                val.x = Frag<ActT>::sixteenth(val.x);
                val.y = Frag<ActT>::sixteenth(val.y);
                val.z = Frag<ActT>::sixteenth(val.z);
                val.w = Frag<ActT>::sixteenth(val.w);
            }
            const int mt = m >> 3, r = m & 7;
            uint32_t* dst = xw + ((((chunk * MT + mt) * 2 + (step >> 1)) * ROWS + r) * 16) + 2 * (step & 1) + b;
            dst[0] = val.x;
            dst[4] = val.y;
            dst[8] = val.z;
            dst[12] = val.w;
        };
        if (!p.perm) {
            // request kXRegs vectors per thread before storing any, so their latencies overlap
            for (int base = 0; base < total_vecs; base += kXRegs * kThreads) {
                uint4 xr[kXRegs];
                int mm[kXRegs], vv[kXRegs];
#pragma unroll
                for (int u = 0; u < kXRegs; ++u) {
                    const int idx = base + threadIdx.x + u * kThreads;
                    mm[u] = ONE ? 0 : idx / vec_per_row;
                    vv[u] = idx - mm[u] * vec_per_row;
                    if (idx < total_vecs)
                        xr[u] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(mm[u]) * p.K + kbase + vv[u] * 8);
                }
#pragma unroll
                for (int u = 0; u < kXRegs; ++u)
                    if (base + threadIdx.x + u * kThreads < total_vecs) store_vec(mm[u], vv[u], xr[u]);
            }
        } else {
            for (int idx = threadIdx.x; idx < total_vecs; idx += kThreads) {
                const int m = idx / vec_per_row, v = idx - m * vec_per_row;
                uint32_t wds[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int k = kbase + v * 8 + 2 * jj;
                    const ActT lo = x[static_cast<size_t>(m) * p.K + p.perm[k]];
                    const ActT hi = x[static_cast<size_t>(m) * p.K + p.perm[k + 1]];
                    wds[jj] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&lo)) |
                              (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
                }
                store_vec(m, v, make_uint4(wds[0], wds[1], wds[2], wds[3]));
            }
        }
        // rows of the last m-tile beyond M read as zero
        if (!ONE) {
            const int pad_vecs = (MT * 8 - m_rows) * vec_per_row;
            for (int idx = threadIdx.x; idx < pad_vecs; idx += kThreads)
                store_vec(m_rows + idx / vec_per_row, idx % vec_per_row, make_uint4(0, 0, 0, 0));
        }
    }
    for (int i = threadIdx.x; i < p.slots * MT * 128; i += kThreads) accs[i] = 0.f;
    for (int i = threadIdx.x; i < p.slots; i += kThreads) slot_cnt[i] = 0;
    __syncthreads();
    EQ_TRACE(2);
    // ---- per (item, row): offset * S1 (S1 = sum of the stored B values) and S2 = sum of x; eight lanes per pair
    {
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
        constexpr int kRowsAll = ONE ? 1 : MT * 8;
        const int pairs = p.cs * kRowsAll;
        const int sub = threadIdx.x & 7;
        for (int base = 0; base < pairs; base += kThreads / 8) {
            const int idx = base + (threadIdx.x >> 3);
            float s1 = 0.f, s2 = 0.f;
            if (idx < pairs) {
                const int it = idx / kRowsAll, m = idx - it * kRowsAll;
                const int mt = m >> 3, r = m & 7;
                if (r < ROWS) {
                    // this lane: (chunk, half) = sub / 2, words 8 (sub & 1) .. +7 of that 16-word row
                    const int ch = sub >> 2, half = (sub >> 1) & 1;
                    const uint4* src = reinterpret_cast<const uint4*>(
                        xw + (((((it * 2 + ch) * MT + mt) * 2 + half) * ROWS + r) * 16) + 8 * (sub & 1));
                    const uint4 u0 = src[0], u1 = src[1];
                    const uint32_t wd[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                    float even = 0.f, odd = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        even += Frag<ActT>::pair_sum(wd[e]);
                        odd += Frag<ActT>::pair_sum(wd[e + 1]);
                    }
                    s1 = even + odd;
                    s2 = Frag<ActT>::kPrescaleHi ? fmaf(16.f, odd, even) : s1;
                }
            }
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) {
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, off);
                s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, off);
            }
            if (idx < pairs && sub == 0) {
                const int it = idx / kRowsAll, m = idx - it * kRowsAll;
                xsum[it * MT * 8 + m] = make_float2(Frag<ActT>::kOffset * s1, s2);
            }
        }
    }
    __syncthreads();
    EQ_TRACE(3);

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.f;

    int cur_t = -1, done = 0;
    int* status = p.counters + p.n_tiles;
    constexpr int kItemVecs = 2 * MT * 2 * ROWS * 4;  // uint4 per item in xs
    const int g = lane >> 2, j = lane & 3;
    const uint4* xs_lane = xs + (ONE ? j : g * 4 + j);
    const float2* xsum_lane = xsum + (ONE ? 0 : 2 * j);
    const unsigned char* ring_lane = ring + lane * 16;
    const unsigned char* meta_lane = ring + 1024 + g * 8;
    int slot = 0;
    uint32_t parity = 0;

    for (int i = 0; i < nb; ++i) {
        const uint32_t bar = smem_addr(bars + slot);
        if (!mbar_try_wait(bar, parity)) {
            const long long t_start = clock64();
            bool ok = false;
            while (!(ok = mbar_try_wait(bar, parity)) && clock64() - t_start < kWaitCycles) {
            }
            if (!ok) {  // a copy that never landed: report and stop this warp
                if (lane == 0) atomicExch(status, 1);
                return;
            }
        }
        if (i == 0) EQ_TRACE(4);
        const Batch b = Batch::unpack(desc[i]);
        const int rec = slot * kSlotBytes;

        // both items are multiplied unconditionally (a missing second item is stale bytes, its result is dropped)
        float acc0[MT][4], acc1[MT][4];
        item_mma<ActT, MT, ROWS>(ring_lane + rec, xs_lane + b.cl0 * kItemVecs, acc0);
        item_mma<ActT, MT, ROWS>(ring_lane + rec + kItemBytes, xs_lane + b.cl1 * kItemVecs, acc1);

        if (b.t0 != cur_t) {
            if (cur_t >= 0) flush_tile<ActT, MT>(p, view, yacc, cur_t, done);
            cur_t = b.t0;
            done = 0;
        }
        item_fold<ActT, MT, ONE>(meta_lane + rec, xsum_lane + b.cl0 * MT * 8, p.scale_dtype, acc0, yacc);
        ++done;
        if (b.n == 2) {
            if (b.t1 != cur_t) {
                flush_tile<ActT, MT>(p, view, yacc, cur_t, done);
                cur_t = b.t1;
                done = 0;
            }
            item_fold<ActT, MT, ONE>(meta_lane + rec + kItemBytes, xsum_lane + b.cl1 * MT * 8, p.scale_dtype, acc1, yacc);
            ++done;
        }
        // the slot has been read by every lane: refill it
        __syncwarp();
        if (i + kRing < nb) request(slot, Batch::unpack(desc[i + kRing]));
        if (++slot == kRing) {
            slot = 0;
            parity ^= 1;
        }
    }
    EQ_TRACE(5);
    if (cur_t >= 0) flush_tile<ActT, MT>(p, view, yacc, cur_t, done);
    EQ_TRACE(6);
}

struct W4Plan {
    int mt, rows, warps, slices, cs, ctas_per_slice, slots;
    size_t smem;
};

constexpr size_t kSmemLimit = 224 * 1024;

static size_t w4_fixed_smem(int warps) {
    return static_cast<size_t>(warps) * kRing * (kSlotBytes + 8) + static_cast<size_t>(warps) * kMaxBatches * 8;
}
static size_t w4_smem_bytes(int warps, int cs, int mt, int rows, int slots) {
    return w4_fixed_smem(warps) + static_cast<size_t>(cs) * 2 * mt * 2 * rows * 4 * 16 +
           static_cast<size_t>(cs) * mt * 8 * sizeof(float2) + static_cast<size_t>(slots) * mt * 128 * 4 +
           static_cast<size_t>(slots) * 4 + 16;
}

static int plan_w4(int64_t K, int64_t N, int M, W4Plan& pl) {
    const int items = static_cast<int>(K / 128), n_tiles = static_cast<int>(N / 16);
    int mt = (M + 7) / 8;
    pl.mt = mt <= 1 ? 1 : mt <= 2 ? 2 : mt <= 4 ? 4 : 8;
    pl.rows = M == 1 ? 1 : 8;
    pl.warps = pl.mt <= 2 ? 24 : 8;
    const int max_slots = pl.mt <= 2 ? 16 : 4;
    // shared memory left for the activations of one slice after ring, descriptors and accumulator slots
    const size_t reserve = w4_fixed_smem(pl.warps) + static_cast<size_t>(max_slots) * pl.mt * 512 + 1024;
    EQ_REQUIRE(reserve < kSmemLimit, EQ_ERR_UNSUPPORTED, "plan_w4: no shared memory left for activations");
    const size_t per_item = static_cast<size_t>(pl.mt) * pl.rows * 256 + static_cast<size_t>(pl.mt) * 64;
    const int cs_max = static_cast<int>((kSmemLimit - reserve) / per_item);
    EQ_REQUIRE(cs_max >= 1, EQ_ERR_UNSUPPORTED, "plan_w4: activation tile does not fit shared memory");
    int s = static_cast<int>(ceil_div(items, cs_max));
    while (items % s) ++s;
    pl.slices = s;
    pl.cs = items / s;
    const long long all_items = static_cast<long long>(n_tiles) * pl.cs;
    int p = sm_count() / s;
    if (p < 1) p = 1;
    // a warp's descriptor table holds kMaxBatches batches (of one or two items): more CTAs when the span is longer
    const long long per_warp_cap = kMaxBatches - 2;  // worst case one item per batch, uneven split
    if (ceil_div(all_items, static_cast<long long>(p) * pl.warps) > per_warp_cap)
        p = static_cast<int>(ceil_div(all_items, per_warp_cap * pl.warps));
    // bound the accumulator slots of a CTA
    long long per_cta = ceil_div(all_items, p);
    if (ceil_div(per_cta, pl.cs) + 1 > max_slots) {
        per_cta = static_cast<long long>(max_slots - 1) * pl.cs;
        p = static_cast<int>(ceil_div(all_items, per_cta));
    }
    if (p > all_items) p = static_cast<int>(all_items);
    pl.ctas_per_slice = p;
    per_cta = ceil_div(all_items, p);
    pl.slots = static_cast<int>(ceil_div(per_cta, pl.cs) + 1);
    pl.smem = w4_smem_bytes(pl.warps, pl.cs, pl.mt, pl.rows, pl.slots);
    EQ_REQUIRE(pl.smem <= kSmemLimit + 2048, EQ_ERR_UNSUPPORTED, "plan_w4: %zu bytes of shared memory needed", pl.smem);
    return EQ_OK;
}

template <typename ActT, int MT, int WARPS, bool ONE>
static int launch_w4_one(const W4Params& p, const W4Plan& pl, cudaStream_t stream) {
    auto kernel = w4a16_streamk_kernel<ActT, MT, WARPS, ONE>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    kernel<<<static_cast<unsigned>(pl.slices * pl.ctas_per_slice), WARPS * 32, pl.smem, stream>>>(p);
    EQ_LAUNCH_OK("w4a16_streamk_kernel");
    return EQ_OK;
}

template <typename ActT, int MT, int WARPS>
static int launch_w4(const W4Params& p, const W4Plan& pl, cudaStream_t stream) {
    if (MT == 1 && p.M == 1) return launch_w4_one<ActT, 1, WARPS, true>(p, pl, stream);
    return launch_w4_one<ActT, MT, WARPS, false>(p, pl, stream);
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
    EQ_REQUIRE(K / 128 < 65536 && N / 16 < (1 << 24), EQ_ERR_UNSUPPORTED, "eq_w4a16_linear: extent too large");
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
        W4Plan pl;
        int st = plan_w4(K, N, mb, pl);
        if (st != EQ_OK) return st;
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
        p.n_tiles = static_cast<int>(N / 16);
        p.slices = pl.slices;
        p.cs = pl.cs;
        p.ctas_per_slice = pl.ctas_per_slice;
        {
            const long long all_items = static_cast<long long>(p.n_tiles) * pl.cs;
            p.span_base = static_cast<int>(all_items / pl.ctas_per_slice);
            p.span_rem = static_cast<int>(all_items % pl.ctas_per_slice);
        }
        p.rows = pl.rows;
        p.slots = pl.slots;
        p.scale_dtype = scale_dtype;
#define EQ_W4_CASE(MTV, WV)                                                                      \
    case MTV:                                                                                    \
        st = act_dtype == EQ_F16 ? launch_w4<__half, MTV, WV>(p, pl, stream)                     \
                                 : launch_w4<__nv_bfloat16, MTV, WV>(p, pl, stream);             \
        break;
        switch (pl.mt) {
            EQ_W4_CASE(1, 24)
            EQ_W4_CASE(2, 24)
            EQ_W4_CASE(4, 8)
            EQ_W4_CASE(8, 8)
            default: return fail(EQ_ERR_UNSUPPORTED, "eq_w4a16_linear: no kernel for %d m-tiles", pl.mt);
        }
#undef EQ_W4_CASE
        if (st != EQ_OK) return st;
    }
    return EQ_OK;
}

extern "C" int eq_w4a16_status(const void* workspace, int64_t M, int64_t N, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && N > 0, EQ_ERR_BAD_ARG, "eq_w4a16_status: bad arguments");
    const int64_t ws_rows = M < 64 ? M : 64;
    const int* status = reinterpret_cast<const int*>(static_cast<const float*>(workspace) + ws_rows * N) + N / 16;
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_w4a16_status: a device-side wait on a weight copy ran out");
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

#ifdef EQ_W4_TRACE
extern "C" int eq_debug_w4_trace(unsigned long long* host, int n) {
    return cudaMemcpyFromSymbol(host, eq::g_w4_trace, sizeof(unsigned long long) * n) == cudaSuccess ? 0 : -4;
}
#endif
