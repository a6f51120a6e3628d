// W4A16 linear, one activation row (M = 1): the weight-streaming kernel of the decode step.
//
// The weight is one flat run of 1088-byte item records, [n-tile][item] (w4_repack.cu).  A launch is ONE wave of
// half-SM CTAs: 16 warps, at most 64 registers per thread and at most 112 KB of shared memory, so that two CTAs fit
// an SM.  One launch fills one of the two places; the other belongs to the launch before or after it in the stream
// (programmatic dependent launch): while launch n computes, the CTAs of launch n + 1 are already resident, have their
// first items in flight (weights never depend on an earlier kernel) and sit in griddepcontrol.wait.  The launches of
// a decode step therefore stream from HBM back to back, instead of each paying its own ramp-up.
//
// Work split.  The item stream is cut into equal spans, one per CTA, at ITEM granularity (the spans differ by at
// most one item, whatever N / 16 is).  A span that starts inside a column tile does that tile's last items first, with
// all warps, and hands the sixteen partial sums to the CTA that owns the tile (the one holding its first item) through
// sixteen words of the workspace; each word carries its own readiness (the bit-inverted f32, zero = not there yet), so
// the owner needs no fence and no flag, and by the time it looks, a whole span later, the words have long arrived.
// The owner's wait is bounded and reports through the status word.  With fewer tiles than CTAs every CTA owns whole
// tiles and nothing is handed over.
//
// Inside a CTA every warp takes an equal contiguous share of the span and keeps DEPTH items in flight in a private
// ring in shared memory, filled by 16-byte cp.async copies that every lane issues for exactly the bytes it reads itself
// later (the eight-byte scale / zero entry is copied once per lane too): no producer warp, no barrier, no __syncwarp.
// A warp adds its sums into the CTA's per-tile accumulators whenever it leaves a tile and counts the items it brought;
// the warp whose count completes a tile converts and stores it there and then, so the kernel has no closing barrier.
//
// Arithmetic (per item = 128 input rows x 16 columns).  (w & 0x000F000F) | 0x64006400 is the f16 pair {1024 + q,
// 1024 + q'} and (w & 0x00F000F0) | 0x64006400 is {1024 + 16 q, ...}; the offsets are NOT removed per element.  The
// activations of the high k-slots are pre-divided by 16 when x is staged, the tensor core (mma.sync m16n8k16, weights
// as A, the activation column as B, f32 accumulate) returns  acc = sum_k x_k q_k + 1024 S1,  and the item contributes
// s (acc - 1024 S1 - z S2)  with S1, S2 the item's sums of the staged / plain activations, computed once per CTA.
// bf16: 128 + q is exact, nothing is pre-divided and S1 = S2.  Five integer instructions per eight nibbles.
// (tcgen05 is not used: at one row the contraction is 1/16 of an MMA tile and the kernel is bound by instruction issue;
// the warp-level MMA keeps the operands in registers.)
#include "w4_gemv1.cuh"

namespace eq {

constexpr int kG1SmemPair = 112 * 1024;    // dynamic shared memory that still lets two CTAs share an SM
constexpr int kG1SmemSolo = 226 * 1024;
constexpr unsigned kG1SpinLimit = 1u << 22;  // polls of the hand-over words before the owner gives up (about a second)

struct G1Params {
    const unsigned char* wq;  // [n_tiles][items][1088]
    const int32_t* perm;      // optional [K]
    const void* x;            // [K]
    void* y;                  // [N]
    uint32_t* xchg;           // [n_tiles][16] hand-over words, zero between calls
    int* status;              // set to 1 when a bounded wait ran out
    int K, N, items;
    uint32_t items_inv;       // floor(2^32 / items) + 1 (0 when items == 1): quotients by one multiply
    int span_base, span_rem;  // items per CTA, plus one for the first span_rem CTAs (tile-aligned mode: tiles)
    int by_items;             // spans are counted in items (1) or in whole tiles (0)
    int acc_tiles;            // accumulator slots per CTA
};

template <typename ActT, bool SCALE_F16, int DEPTH>
__global__ void __launch_bounds__(kG1Threads, 2) w4a16_gemv1_kernel(const G1Params p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int items = p.items;

    // ---- this CTA's span [S, S + L) of the item stream
    const int cta = blockIdx.x;
    int S = cta * p.span_base + min(cta, p.span_rem);
    int L = p.span_base + (cta < p.span_rem ? 1 : 0);
    if (!p.by_items) {
        S *= items;
        L *= items;
    }
    const int t_first = quotient(S, items, p.items_inv);
    const int it_first = S - t_first * items;
    // leading piece: the last items of a tile that the previous CTA owns (handed over); then the tiles owned here,
    // the last of which may be cut short by the end of the span (the next CTA hands its part over)
    const int lenA = it_first ? min(items - it_first, L) : 0;
    const int R = L - lenA;
    const int tile_own = t_first + (it_first ? 1 : 0);  // first owned tile
    const int full = quotient(R, items, p.items_inv);   // owned tiles done whole
    const int lenB = R - full * items;                  // items of the last owned tile done here, 0 = all of them
    const int n_own = full + (lenB ? 1 : 0);            // owned tiles

    // accumulators [1 + n_own][16] (slot 0 is the leading piece), then the items each slot has received so far
    float* acc_s = reinterpret_cast<float*>(smem_all + kG1Warps * DEPTH * kG1Slot);
    int* done_s = reinterpret_cast<int*>(acc_s + p.acc_tiles * 16);
    const int acc_words = p.acc_tiles * 16 + ((p.acc_tiles + 3) & ~3);
    uint4* xs = reinterpret_cast<uint4*>(acc_s + acc_words);  // [K / 8] staged activations
    float2* xsum = reinterpret_cast<float2*>(xs + p.K / 8);   // [items] {offset S1, S2}

    // ---- this warp's two runs: [a0, a1) of the leading piece, [r0, r1) of the rest
    const int a0 = lenA * warp / kG1Warps, a1 = lenA * (warp + 1) / kG1Warps;
    const int r0 = static_cast<int>(static_cast<long long>(R) * warp / kG1Warps);
    const int r1 = static_cast<int>(static_cast<long long>(R) * (warp + 1) / kG1Warps);
    const int nA = a1 - a0, n = nA + (r1 - r0);
    const int r0_tile = quotient(r0, items, p.items_inv);

    // ---- ring of DEPTH items, private to the warp; every lane copies the bytes it reads itself
    const uint32_t ring_w = smem_u32(smem_all) + warp * (DEPTH * kG1Slot) + lane * 16;  // + 512: second nibble tile
    const uint32_t ring_m = ring_w + 1024 - lane * 8;                                   // the lane's own scale / zero entry
    const unsigned char* base_w = p.wq + lane * 16;
    const unsigned char* base_m = p.wq + 1024 + g * 8;
    // the warp's list in order: item v is record phys_a + v of the stream for v < nA, record phys_b + v after that
    const int phys_a = S + a0, phys_b = S + lenA + r0 - nA;
    int v_issue = 0;
    // item v_issue of the list into the slot at byte offset `slot` of the ring (nothing once the list is exhausted); one
    // commit group either way.  (mad.wide keeps the address arithmetic off the integer pipe that the dequant keeps busy.)
    auto issue = [&](uint32_t slot) {
        const uint32_t rec = static_cast<uint32_t>(v_issue + (v_issue < nA ? phys_a : phys_b));
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            ".reg .b64 aw, am;\n"
            "setp.lt.s32 p, %5, %6;\n"
            "mad.wide.u32 aw, %4, 1088, %2;\n"
            "mad.wide.u32 am, %4, 1088, %3;\n"
            "@p cp.async.cg.shared.global [%0], [aw], 16;\n"
            "@p cp.async.cg.shared.global [%0+512], [aw+512], 16;\n"
            "@p cp.async.ca.shared.global [%1], [am], 8;\n"
            "cp.async.commit_group;\n"
            "}\n" ::"r"(ring_w + slot),
            "r"(ring_m + slot), "l"(base_w), "l"(base_m), "r"(rec), "r"(v_issue), "r"(n)
            : "memory");
        ++v_issue;
    };
#pragma unroll 1
    for (int d = 0; d < DEPTH; ++d) issue(d * kG1Slot);

    // weights never depend on the previous grid; x, y and the workspace may
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage x once per CTA (high k-slots pre-divided by 16, gathered through perm if any) with the two sums of
    //      every item; the copies above are in flight meanwhile.  Layout: [item][chunk c][lane column j] of 16 bytes, chunk c
    //      of lane column j holding the {low slot, high slot} word pairs of k16 steps 2c and 2c + 1.
    for (int i = threadIdx.x; i < acc_words; i += kG1Threads) acc_s[i] = 0.f;  // accumulators and counters
    {
        const ActT* x = static_cast<const ActT*>(p.x);
        const int n_vec = p.K / 8;  // a multiple of 16
        constexpr int kBatch = 4;   // loads in flight per thread
        for (int v0 = threadIdx.x; v0 < ((n_vec + 31) & ~31); v0 += kBatch * kG1Threads) {  // whole warps: the sums shuffle
            uint4 vals[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int v = v0 + u * kG1Threads;
                vals[u] = make_uint4(0, 0, 0, 0);
                if (v >= n_vec) {
                } else if (!p.perm) {
                    vals[u] = __ldg(reinterpret_cast<const uint4*>(x) + v);
                } else {
                    uint32_t wds[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const ActT a = x[p.perm[v * 8 + 2 * i]], b = x[p.perm[v * 8 + 2 * i + 1]];
                        wds[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&a)) |
                                 (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&b)) << 16);
                    }
                    vals[u] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int v = v0 + u * kG1Threads;
                if (v >= ((n_vec + 31) & ~31)) break;  // warp-uniform
                stage_vector<ActT>(vals[u], v, v < n_vec, xs, xsum);
            }
        }
    }
    __syncthreads();  // accumulators are zero, x is staged

    // ---- the items.  The list is walked in stretches that end where the warp leaves a tile, finishes the leading
    //      piece, or runs out of items; inside a stretch nothing is tested but the stretch counter.
    float y_lo = 0.f, y_hi = 0.f;                        // columns g and g + 8 of the current tile, live in lanes with j == 0
    int i = 0;                                           // items done
    int it = nA ? it_first + a0 : r0 - r0_tile * items;  // item inside its tile
    int slot_t = nA ? 0 : 1 + r0_tile;                   // accumulator slot: 0 = leading piece, 1.. = owned tiles
    uint32_t slot = 0;
    const uint32_t acc_u32 = smem_u32(acc_s);
    while (i < n) {
        const int stretch = min(items - it, (i < nA ? nA : n) - i);
        uint32_t x_addr = smem_u32(xs) + it * 256 + j * 16;
        uint32_t sum_addr = smem_u32(xsum) + it * 8;
        for (int c = stretch; c > 0; --c) {
            asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
            gemv1_item<ActT, SCALE_F16>(ring_w + slot, ring_m + slot, x_addr, sum_addr, y_lo, y_hi);
            issue(slot);  // the slot's bytes have been consumed: refill it
            slot += kG1Slot;
            if (slot == DEPTH * kG1Slot) slot = 0;
            x_addr += 256;
            sum_addr += 8;
        }
        // ---- end of a stretch: add the sums into the tile's accumulators and count the items brought
        i += stretch;
        it += stretch;
        const bool last_owned = slot_t == n_own;
        int brought = stretch;
        if (last_owned && lenB != 0 && i == n && warp == kG1Warps - 1) {
            // this warp did the last items of the span: it also fetches what the next CTA did of the span's last tile
            // (that CTA did it first thing, so the words are normally there; the wait is bounded)
            if (lane < 16) {
                uint32_t* word = p.xchg + static_cast<size_t>(tile_own + n_own - 1) * 16 + lane;
                uint32_t got = ld_relaxed_gpu(word);
                for (unsigned spins = 0; got == 0 && spins < kG1SpinLimit; ++spins) got = ld_relaxed_gpu(word);
                if (got == 0) {
                    *p.status = 1;
                } else {
                    atomicAdd(acc_s + slot_t * 16 + lane, __uint_as_float(~got));
                    st_relaxed_gpu(word, 0u);  // zero again for the next call
                }
            }
            brought += 1;  // counted like one more item
        }
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.eq.s32 p, %3, 0;\n"
            "@p red.shared.add.f32 [%0], %1;\n"
            "@p red.shared.add.f32 [%0+32], %2;\n"
            "}\n" ::"r"(acc_u32 + (slot_t * 16 + g) * 4),
            "f"(y_lo), "f"(y_hi), "r"(j)
            : "memory");
        y_lo = y_hi = 0.f;
        __syncwarp();
        int complete = 0;
        if (lane == 0) {
            __threadfence_block();
            const int want = slot_t == 0 ? lenA : (last_owned && lenB != 0 ? lenB + 1 : items);
            complete = atomicAdd(done_s + slot_t, brought) + brought == want;
        }
        complete = __shfl_sync(0xFFFFFFFFu, complete, 0);
        if (complete) {
            // every part of this tile is in: convert and store it, or hand the leading piece to its owner (bit-inverted
            // so that zero means "not there yet")
            __threadfence_block();
            if (lane < 16) {
                const float v = *(volatile float*)(acc_s + slot_t * 16 + lane);
                if (slot_t == 0)
                    st_relaxed_gpu(p.xchg + static_cast<size_t>(t_first) * 16 + lane, ~__float_as_uint(v));
                else
                    static_cast<ActT*>(p.y)[static_cast<size_t>(tile_own + slot_t - 1) * 16 + lane] = from_float<ActT>(v);
            }
        }
        if (i == nA) {  // the leading piece is done: continue with the owned tiles
            it = r0 - r0_tile * items;
            slot_t = 1 + r0_tile;
        } else {  // the next tile (or the list is exhausted)
            it = 0;
            ++slot_t;
        }
    }
}

// Shared memory of the kernel, or 0 when it exceeds `limit`.
static size_t g1_smem(int depth, int acc_tiles, int K, size_t limit) {
    const size_t bytes = static_cast<size_t>(kG1Warps) * depth * kG1Slot + static_cast<size_t>(acc_tiles) * 16 * sizeof(float) +
                         static_cast<size_t>((acc_tiles + 3) & ~3) * sizeof(int) + static_cast<size_t>(K) * 2 +
                         static_cast<size_t>(K / 128) * sizeof(float2);
    return bytes <= limit ? bytes : 0;
}

template <typename ActT, bool SCALE_F16, int DEPTH>
static int launch_g1(const G1Params& p, size_t smem, int ctas, cudaStream_t stream) {
    auto kernel = w4a16_gemv1_kernel<ActT, SCALE_F16, DEPTH>;
    static bool configured[64] = {};  // per device: the attributes stick to the function
    int dev = 0;
    EQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kG1SmemSolo));
        // the whole shared-memory / L1 array as shared memory: two CTAs of ~110 KB must fit one SM
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kG1Threads);
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

template <typename ActT, bool SCALE_F16>
static int launch_g1_depth(const G1Params& p, int ctas, cudaStream_t stream, bool* fits) {
    *fits = true;
    // the deepest ring that still lets two launches share an SM; failing that, one CTA per SM
    if (const size_t smem = g1_smem(5, p.acc_tiles, p.K, kG1SmemPair)) return launch_g1<ActT, SCALE_F16, 5>(p, smem, ctas, stream);
    if (const size_t smem = g1_smem(4, p.acc_tiles, p.K, kG1SmemPair)) return launch_g1<ActT, SCALE_F16, 4>(p, smem, ctas, stream);
    if (const size_t smem = g1_smem(3, p.acc_tiles, p.K, kG1SmemPair)) return launch_g1<ActT, SCALE_F16, 3>(p, smem, ctas, stream);
    if (const size_t smem = g1_smem(5, p.acc_tiles, p.K, kG1SmemSolo)) return launch_g1<ActT, SCALE_F16, 5>(p, smem, ctas, stream);
    if (const size_t smem = g1_smem(3, p.acc_tiles, p.K, kG1SmemSolo)) return launch_g1<ActT, SCALE_F16, 3>(p, smem, ctas, stream);
    *fits = false;  // the staged activations alone exceed shared memory
    return EQ_OK;
}

// y[N] = x[K] @ W.  xchg: N zeroed words of workspace (left zero), status: one word.  *fits is cleared, and nothing
// is launched, when K is too large to stage x in shared memory (the caller falls back to the tile kernel).
int w4_gemv1_launch(const unsigned char* wq, int scale_dtype, const int32_t* perm, const void* x, void* y, int64_t N, int64_t K,
                    int act_dtype, uint32_t* xchg, int* status, cudaStream_t stream, bool* fits) {
    const long long tiles = N / 16, items = K / 128;
    const long long total = tiles * items;
    *fits = false;
    if (total >= (1LL << 30)) return EQ_OK;
    G1Params p;
    p.wq = wq;
    p.perm = perm;
    p.x = x;
    p.y = y;
    p.xchg = xchg;
    p.status = status;
    p.K = static_cast<int>(K);
    p.N = static_cast<int>(N);
    p.items = static_cast<int>(items);
    p.items_inv = items == 1 ? 0u : static_cast<uint32_t>((1ULL << 32) / static_cast<unsigned long long>(items)) + 1u;
    long long ctas = sm_count();
    if (tiles >= ctas) {
        // every span is at least one tile long, so a tile is shared by at most two CTAs
        p.by_items = 1;
        p.span_base = static_cast<int>(total / ctas);
        p.span_rem = static_cast<int>(total % ctas);
        p.acc_tiles = static_cast<int>((p.span_base + 1 + items - 1) / items) + 2;
    } else {
        ctas = tiles;
        p.by_items = 0;
        p.span_base = 1;
        p.span_rem = 0;
        p.acc_tiles = 3;
    }
    const int n_ctas = static_cast<int>(ctas);
    if (act_dtype == EQ_F16)
        return scale_dtype == EQ_F16 ? launch_g1_depth<__half, true>(p, n_ctas, stream, fits) : launch_g1_depth<__half, false>(p, n_ctas, stream, fits);
    return scale_dtype == EQ_F16 ? launch_g1_depth<__nv_bfloat16, true>(p, n_ctas, stream, fits)
                                 : launch_g1_depth<__nv_bfloat16, false>(p, n_ctas, stream, fits);
}

}  // namespace eq
