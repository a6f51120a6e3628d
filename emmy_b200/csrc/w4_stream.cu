// W4A16 linear, M <= 16: the streaming form of the tile kernel (w4_tile.cuh).
//
// The weight is one flat run of item records, [n-tile][item].  The grid is ONE CTA of 32 warps per SM; a CTA owns a
// run of whole column tiles (the tile counts of the CTAs differ by at most one) and its warps take equal contiguous
// spans of the CTA's items, whatever the tile boundaries.  A warp keeps kStreamDepth items in flight in a private
// shared-memory ring filled by cp.async, runs each through w4_item, and when its span leaves a tile it adds its
// sums into the CTA's shared accumulators.  One __syncthreads at the end, then the CTA converts and stores the tiles
// it owns.  No global atomics, no fences, no workspace: measured on B200, the f32 workspace hand-over of an earlier
// form of this kernel (atomic adds, fence, arrival counter) cost 4.6 us of a 10.4 us launch, the stream itself 5.8.
#include "w4_tile.cuh"

namespace eq {

constexpr int kStreamWarps = 32;        // one fat CTA per SM (single-row calls; multi-row calls use half as many warps for twice the registers)
constexpr int kSlot = kItemBytes;       // ring slot: one item record as it lies in global memory

#ifdef EQ_W4_TRACE
__device__ unsigned long long g_w4_trace[4096 * 8];
#define EQ_TRACE(slot)                                                                                            \
    do {                                                                                                          \
        if ((threadIdx.x & 31) == 0 && blockIdx.x * 32 + (threadIdx.x >> 5) < 4096) {                             \
            unsigned long long t_;                                                                                \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                \
            g_w4_trace[(blockIdx.x * 32 + (threadIdx.x >> 5)) * 8 + (slot)] = t_;                                 \
        }                                                                                                         \
    } while (0)
#else
#define EQ_TRACE(slot) \
    do {               \
    } while (0)
#endif

// ---- single activation row: offset-free dequant against activations staged in shared memory --------------------
// (w & 0x000F000F) | 0x64006400 is the f16 pair {1024 + q, 1024 + q'} and (w & 0x00F000F0) | 0x64006400 is
// {1024 + 16 q, ...}; the offsets are NOT subtracted per element.  The staged activations of the high k-slots are
// pre-divided by 16, so the tensor core returns  acc = sum_k x_k q_k + 1024 S1  with S1 the sum of the staged values
// of the item, and the item contributes  s (acc - 1024 S1 - z S2),  S2 = sum_k x_k.  1024 S1 and S2 are computed once
// per CTA.  bf16: 128 + q is exact, nothing is pre-divided and S1 = S2.  Five integer instructions per eight nibbles.
template <typename ActT>
struct Raw;
template <>
struct Raw<__half> {
    static constexpr float kOffset = 1024.f;
    static constexpr bool kPrescaleHi = true;
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w, 0x00F000F0u, kMagic);
        const uint32_t w8 = w >> 8;
        a[1] = lop3<0xEA>(w8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w8, 0x00F000F0u, kMagic);
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
struct Raw<__nv_bfloat16> {
    static constexpr float kOffset = 128.f;
    static constexpr bool kPrescaleHi = false;
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x43004300u;
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w >> 4, 0x000F000Fu, kMagic);
        a[1] = lop3<0xEA>(w >> 8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w >> 12, 0x000F000Fu, kMagic);
    }
    static __device__ __forceinline__ uint32_t sixteenth(uint32_t pair) { return pair; }
    static __device__ __forceinline__ float pair_sum(uint32_t pair) {
        return __uint_as_float(pair << 16) + __uint_as_float(pair & 0xFFFF0000u);
    }
};

// xs_lane: the lane column's 64 staged bytes of the item; sums: {offset S1, S2} of the item.
template <typename ActT>
__device__ __forceinline__ void w4_item_one(int scale_dtype, const uint4* xs_lane, bool feeds_column0, float2 sums, const uint4& wl,
                                            const uint4& wh, const uint2& mt_, float (&yacc)[1][4]) {
    // staged as {low slot, high slot} word pairs per k16 step: a 16-byte read is the B fragment of two steps.  Only
    // column 0 of the product is ever looked at, and its B values sit in lanes 0..3 (g = 0): the other lanes pass
    // zeros and their shared-memory reads are predicated off, a quarter of the wavefronts.
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, x2 = x0, x3 = x0;
    if (feeds_column0) {
        x0 = xs_lane[0];
        x1 = xs_lane[1];
        x2 = xs_lane[2];
        x3 = xs_lane[3];
    }
    const uint32_t lo[8] = {x0.x, x0.z, x1.x, x1.z, x2.x, x2.z, x3.x, x3.z};
    const uint32_t hi[8] = {x0.y, x0.w, x1.y, x1.w, x2.y, x2.w, x3.y, x3.w};
    const uint32_t words[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
    float acc[2][4];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        uint32_t a[4];
        Raw<ActT>::expand(words[s], a);
        if (s < 2)
            Frag<ActT>::mma0(acc[s & 1], a, lo[s], hi[s]);
        else
            Frag<ActT>::mma(acc[s & 1], a, lo[s], hi[s]);
    }
    float s_lo, s_hi;
    if (scale_dtype == EQ_F16) {
        const __half2 sc = *reinterpret_cast<const __half2*>(&mt_.x);
        s_lo = __low2float(sc);
        s_hi = __high2float(sc);
    } else {
        s_lo = __uint_as_float(mt_.x << 16);
        s_hi = __uint_as_float(mt_.x & 0xFFFF0000u);
    }
    const __half2 z = *reinterpret_cast<const __half2*>(&mt_.y);
    // only column m = 0 of the product is live (c0: column g, c2: column g + 8, both in lanes j == 0)
    yacc[0][0] = fmaf(s_lo, (acc[0][0] + acc[1][0]) - fmaf(__low2float(z), sums.y, sums.x), yacc[0][0]);
    yacc[0][2] = fmaf(s_hi, (acc[0][2] + acc[1][2]) - fmaf(__high2float(z), sums.y, sums.x), yacc[0][2]);
}

// Add a warp's sums for one tile into the CTA's shared accumulators [slot][m][16].
template <typename ActT, int MT, bool ONE>
__device__ __forceinline__ void stream_flush(const W4Params& p, float* acc_slot, float (&yacc)[MT][4], int g, int j) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = mt * 8 + 2 * j + (e & 1);
            const int n = g + ((e & 2) ? 8 : 0);
            if (ONE ? (j == 0 && (e & 1) == 0) : (m < p.M)) atomicAdd(acc_slot + m * 16 + n, yacc[mt][e]);
            yacc[mt][e] = 0.f;
        }
    }
}

// DEPTH: items in flight per warp.  A warp of the benchmark's shapes owns six items, so DEPTH = 6 requests its whole
// span before the first item is consumed.
template <typename ActT, int MT, bool ONE, int WARPS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32, 1) w4a16_stream_kernel(const W4Params p) {
    constexpr int kStreamWarps = WARPS;
    constexpr int kStreamDepth = DEPTH;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    EQ_TRACE(0);
    constexpr int kRows = ONE ? 1 : MT * 8;
    extern __shared__ __align__(16) unsigned char smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    // whole tiles per CTA: the first span_rem CTAs take one tile more
    const int cta = blockIdx.x;
    const int tile0 = cta * p.span_base + min(cta, p.span_rem);
    const int ntiles = p.span_base + (cta < p.span_rem ? 1 : 0);
    float* acc_s = reinterpret_cast<float*>(smem_all + kStreamWarps * kStreamDepth * kSlot);  // [ntiles][kRows][16]
    for (int i = threadIdx.x; i < ntiles * kRows * 16; i += kStreamWarps * 32) acc_s[i] = 0.f;
    // equal spans of the CTA's items per warp
    const int cta_items = ntiles * p.items;
    const int q0 = static_cast<int>(static_cast<long long>(cta_items) * warp / kStreamWarps);
    const int q1 = static_cast<int>(static_cast<long long>(cta_items) * (warp + 1) / kStreamWarps);
    const int n = q1 - q0;
    int slot_t = q0 / p.items;          // tile slot inside the CTA
    int it = q0 - slot_t * p.items;     // item inside the tile
    const size_t first = (static_cast<size_t>(tile0) * p.items + q0) * kItemBytes;  // records are contiguous across tiles
    const unsigned char* rec = p.wq + first + lane * 16;
    const unsigned char* met = p.wq + first + 1024 + g * 8;  // lanes of one g share it
    const ActT* x = static_cast<const ActT*>(p.x);
    EQ_TRACE(7);

    // ---- a per-warp ring of kStreamDepth items in shared memory, filled by per-lane asynchronous copies: lane L
    //      copies the 2 x 16 weight bytes it reads later; the eight lanes with j == 0 also copy the 8-byte scale / zero
    //      entry of their column pair, which the other lanes of the pair read too, hence the __syncwarp after the wait.
    //      One commit group per item; iteration i waits until at most kStreamDepth - 1 groups are pending.
    unsigned char* ring = smem_all + warp * (kStreamDepth * kSlot);
    const uint32_t ring_lo = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + lane * 16;
    const uint32_t ring_meta = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + 1024 + g * 8;
    auto issue = [&](int d, int i) {
        if (i < n) {
            const size_t off = static_cast<size_t>(i) * kItemBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kSlot), "l"(rec + off) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kSlot + 512), "l"(rec + off + 512) : "memory");
            if (j == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ring_meta + d * kSlot), "l"(met + off) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int d = 0; d < kStreamDepth; ++d) issue(d, d);
    // weights never depend on the previous grid; x and y may (programmatic dependent launch)
    EQ_TRACE(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- single row: stage x once per SM (high k-slots pre-divided by 16, gathered through perm if any) and the
    //      two sums of every item; the copies above are in flight meanwhile
    uint4* xs = reinterpret_cast<uint4*>(acc_s + ntiles * kRows * 16);  // [K / 8] vectors of 8 activations
    float2* xsum = reinterpret_cast<float2*>(xs + p.K / 8);             // [items]
    if constexpr (ONE) {
        const int n_vec = p.K / 8;
        for (int v = threadIdx.x; v < ((n_vec + 31) & ~31); v += kStreamWarps * 32) {  // whole warps: the sums shuffle
            uint4 val = make_uint4(0, 0, 0, 0);
            if (v >= n_vec) {
            } else if (!p.perm) {
                val = __ldg(reinterpret_cast<const uint4*>(x) + v);
            } else {
                uint32_t wds[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const ActT a = x[p.perm[v * 8 + 2 * i]], b = x[p.perm[v * 8 + 2 * i + 1]];
                    wds[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&a)) |
                             (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&b)) << 16);
                }
                val = make_uint4(wds[0], wds[1], wds[2], wds[3]);
            }
            // rows 16..31 of every 32-row lane block are the high k-slots: vectors 2, 3 of every four
            float s2 = Raw<ActT>::pair_sum(val.x) + Raw<ActT>::pair_sum(val.y) + Raw<ActT>::pair_sum(val.z) + Raw<ActT>::pair_sum(val.w);
            float s1 = s2;
            if (Raw<ActT>::kPrescaleHi && (v & 2)) {
                val.x = Raw<ActT>::sixteenth(val.x);
                val.y = Raw<ActT>::sixteenth(val.y);
                val.z = Raw<ActT>::sixteenth(val.z);
                val.w = Raw<ActT>::sixteenth(val.w);
                s1 = Raw<ActT>::pair_sum(val.x) + Raw<ActT>::pair_sum(val.y) + Raw<ActT>::pair_sum(val.z) + Raw<ActT>::pair_sum(val.w);
            }
            if (v < n_vec) {
                // vector v = 4 (lane block) + q: q & 1 picks steps 0..3 / 4..7, q >> 1 the low / high slots; word i of
                // it is step s = 4 (q & 1) + i and goes to word 2 s + (q >> 1) of the lane block's 16 words
                uint32_t* dst = reinterpret_cast<uint32_t*>(xs) + (v >> 2) * 16 + (v & 1) * 8 + ((v >> 1) & 1);
                dst[0] = val.x;
                dst[2] = val.y;
                dst[4] = val.z;
                dst[6] = val.w;
            }
            // an item is 16 consecutive vectors = 16 consecutive lanes of this warp
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) {
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, off);
                s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, off);
            }
            if (v < n_vec && (v & 15) == 0) xsum[v >> 4] = make_float2(Raw<ActT>::kOffset * s1, s2);
        }
    }
    __syncthreads();  // accumulators are zero, x is staged
    EQ_TRACE(2);

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.f;
    bool dirty = false;

    for (int i = 0; i < n; ++i) {
        const int d = i % kStreamDepth;
        asm volatile("cp.async.wait_group %0;" ::"n"(kStreamDepth - 1) : "memory");
        __syncwarp();  // the scale / zero entry was copied by another lane of the column pair
        const unsigned char* slot = ring + d * kSlot;
        const uint4 wl = *reinterpret_cast<const uint4*>(slot + lane * 16);
        const uint4 wh = *reinterpret_cast<const uint4*>(slot + 512 + lane * 16);
        const uint2 mt_ = *reinterpret_cast<const uint2*>(slot + 1024 + g * 8);
        __syncwarp();  // every lane has read the slot before any lane refills it
        if constexpr (ONE)
            w4_item_one<ActT>(p.scale_dtype, xs + it * 16 + 4 * j, g == 0, xsum[it], wl, wh, mt_, yacc);
        else
            w4_item<ActT, MT, ONE>(p, x, it, wl, wh, mt_, g, j, yacc);
        issue(d, i + kStreamDepth);  // the slot's bytes are in registers: refill it
        if (i == 0) EQ_TRACE(3);
        dirty = true;
        if (++it == p.items) {  // the span leaves this tile
            stream_flush<ActT, MT, ONE>(p, acc_s + slot_t * kRows * 16, yacc, g, j);
            dirty = false;
            it = 0;
            ++slot_t;
        }
    }
    EQ_TRACE(4);
    if (dirty) stream_flush<ActT, MT, ONE>(p, acc_s + slot_t * kRows * 16, yacc, g, j);
    __syncthreads();
    EQ_TRACE(5);
    // ---- the CTA owns its tiles outright: convert and store
    ActT* y = static_cast<ActT*>(p.y);
    const int rows = ONE ? 1 : p.M;
    for (int idx = threadIdx.x; idx < ntiles * rows * 16; idx += kStreamWarps * 32) {
        const int t = idx / (rows * 16), r = idx - t * (rows * 16);
        const int m = r >> 4, nn = r & 15;
        y[static_cast<size_t>(m) * p.N + (tile0 + t) * 16 + nn] = from_float<ActT>(acc_s[(t * kRows + m) * 16 + nn]);
    }
    EQ_TRACE(6);
}

// Shared memory the stream kernel needs for `tiles` column tiles on `ctas` CTAs, or 0 when it does not fit.
static size_t stream_smem(long long tiles, long long ctas, int rows, int K, int warps, int depth) {
    const long long per_cta = ceil_div(tiles, ctas);
    size_t bytes = static_cast<size_t>(warps) * depth * kSlot + static_cast<size_t>(per_cta) * rows * 16 * sizeof(float);
    if (rows == 1) bytes += static_cast<size_t>(K) * 2 + static_cast<size_t>(K / 128) * sizeof(float2);  // staged x and its item sums
    return bytes <= 220 * 1024 ? bytes : 0;
}

template <typename ActT, int MT, bool ONE, int DEPTH>
static int launch_stream_depth(W4Params p, size_t smem, long long ctas, cudaStream_t stream) {
    constexpr int kWarps = ONE ? kStreamWarps : kStreamWarps / 2;
    auto kernel = w4a16_stream_kernel<ActT, MT, ONE, kWarps, DEPTH>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, p));
    return EQ_OK;
}

template <typename ActT, int MT, bool ONE>
static int launch_stream(W4Params p, cudaStream_t stream) {
    constexpr int kWarps = ONE ? kStreamWarps : kStreamWarps / 2;
    const long long tiles = p.N / 16;
    long long ctas = sm_count();
    if (ctas > tiles) ctas = tiles;
    p.span_base = static_cast<int>(tiles / ctas);
    p.span_rem = static_cast<int>(tiles % ctas);
    const int rows = ONE ? 1 : MT * 8;
    // the deepest ring that fits: six items cover a warp's whole span at the Llama MLP shapes
    if (const size_t smem = stream_smem(tiles, ctas, rows, p.K, kWarps, 6)) return launch_stream_depth<ActT, MT, ONE, 6>(p, smem, ctas, stream);
    if (const size_t smem = stream_smem(tiles, ctas, rows, p.K, kWarps, 5)) return launch_stream_depth<ActT, MT, ONE, 5>(p, smem, ctas, stream);
    const size_t smem = stream_smem(tiles, ctas, rows, p.K, kWarps, 4);
    EQ_REQUIRE(smem > 0, EQ_ERR_UNSUPPORTED, "w4a16 stream kernel: accumulators do not fit shared memory");
    return launch_stream_depth<ActT, MT, ONE, 4>(p, smem, ctas, stream);
}

template <typename ActT>
static int stream_dispatch(const W4Params& p, cudaStream_t stream) {
    if (p.M == 1) return launch_stream<ActT, 1, true>(p, stream);
    if (p.M <= 8) return launch_stream<ActT, 1, false>(p, stream);
    return launch_stream<ActT, 2, false>(p, stream);
}

// M <= 16, total items < 2^31.
int w4_stream_launch(const W4Params& p, int act_dtype, cudaStream_t stream) {
    return act_dtype == EQ_F16 ? stream_dispatch<__half>(p, stream) : stream_dispatch<__nv_bfloat16>(p, stream);
}

}  // namespace eq

#ifdef EQ_W4_TRACE
extern "C" int eq_debug_w4_trace(unsigned long long* host, int n) {
    return cudaMemcpyFromSymbol(host, eq::g_w4_trace, sizeof(unsigned long long) * n) == cudaSuccess ? 0 : -4;
}
#endif
