// W4A16 linear, 2 <= M <= 24: the streaming form of the tile kernel (w4_tile.cuh).  (One row has its own kernel,
// w4_gemv1.cu.)
//
// The weight is one flat run of item records, [n-tile][item].  The grid is one CTA of 16 warps per SM; a CTA owns a
// run of whole column tiles (the tile counts of the CTAs differ by at most one) and its warps take equal contiguous
// spans of the CTA's items, whatever the tile boundaries.  A warp keeps kStreamDepth items in flight in a private
// shared-memory ring filled by cp.async, runs each through w4_item, and when its span leaves a tile it adds its
// sums into the CTA's shared accumulators.  One __syncthreads at the end, then the CTA converts and stores the tiles
// it owns.  In this form there are no global atomics, no fences, no workspace: measured on B200, the f32 workspace
// hand-over of an earlier form of this kernel (atomic adds, fence, arrival counter) cost 4.6 us of a 10.4 us launch, the
// stream itself 5.8.  (The K-sliced form below pays for one such hand-over per CTA where x would not fit otherwise.)
//
// Every item multiplies the same M rows of x, 4 KB per item at M = 16: read from global memory that is 117 MB per
// launch through L1 / L2 against 29 MB of weights, and it bounded the launch.  Where M x K fits beside the ring
// (STAGED) the CTA copies x once into shared memory in the order the MMA operands are read (conflict-free 16-byte
// reads, the two B registers of every MMA next to each other).  Where it does not fit, K is cut into slices: a CTA is (group of column tiles, K slice), stages its slice of x,
// and the slices' sums meet in the f32 workspace (SPLIT).  Without a workspace region, or with gathered rows, the rows are
// read from global memory, one item ahead of the weights where registers allow.
#include "w4_tile.cuh"

namespace eq {

constexpr int kStreamWarps = 16;        // one CTA per SM, 128 registers per thread
constexpr int kSlot = kItemBytes;       // ring slot: one item record as it lies in global memory

// Add a warp's sums for one tile into the CTA's shared accumulators [slot][m][16].
template <typename ActT, int MT>
__device__ __forceinline__ void stream_flush(const W4Params& p, float* acc_slot, float (&yacc)[MT][4], int g, int j) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = mt * 8 + 2 * j + (e & 1);
            const int n = g + ((e & 2) ? 8 : 0);
            if (m < p.M) atomicAdd(acc_slot + m * 16 + n, yacc[mt][e]);
            yacc[mt][e] = 0.f;
        }
    }
}

// Shared-memory bytes of the staged x: [item][row block of 8][16-byte chunk 0..3][lane][16 B].
static size_t staged_x_bytes(int64_t K, int rows) { return static_cast<size_t>(K / 128) * (rows / 8) * 2048; }

// DEPTH: items in flight per warp.  STAGED: x lives in shared memory.  SPLIT (implies STAGED): K is cut into p.splits
// slices; CTA = (group of column tiles, K slice) stages only its slice of x, and the slices' partial sums meet in the f32
// workspace (atomic adds; the CTA whose arrival completes a group converts it and leaves workspace and counter zero).
// For shapes whose M x K does not fit shared memory, or whose tiles do not fill the SMs evenly.
template <typename ActT, int MT, int DEPTH, bool STAGED, bool SPLIT = false>
__global__ void __launch_bounds__(kStreamWarps * 32, 1) w4a16_stream_kernel(const W4Params p) {
    constexpr int kStreamDepth = DEPTH;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kRows = MT * 8;
    extern __shared__ __align__(16) unsigned char smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    // whole tiles per CTA: the first span_rem CTAs take one tile more
    const int cta = blockIdx.x;
    int tile0 = cta * p.span_base + min(cta, p.span_rem);
    int ntiles = p.span_base + (cta < p.span_rem ? 1 : 0);
    int i0 = 0, ipp = p.items;  // this CTA's run of items of every tile
    if (SPLIT) {
        const int grp = cta / p.splits, sp = cta - grp * p.splits;
        tile0 = grp * p.group_tiles;
        ntiles = min(p.group_tiles, p.N / 16 - tile0);
        i0 = p.items * sp / p.splits;
        ipp = p.items * (sp + 1) / p.splits - i0;
    }
    float* acc_s = reinterpret_cast<float*>(smem_all + kStreamWarps * kStreamDepth * kSlot);  // [ntiles][kRows][16]
    for (int i = threadIdx.x; i < ntiles * kRows * 16; i += kStreamWarps * 32) acc_s[i] = 0.f;
    // equal spans of the CTA's items per warp
    const int cta_items = ntiles * ipp;
    const int q0 = static_cast<int>(static_cast<long long>(cta_items) * warp / kStreamWarps);
    const int q1 = static_cast<int>(static_cast<long long>(cta_items) * (warp + 1) / kStreamWarps);
    const int n = q1 - q0;
    int slot_t = q0 / ipp;          // tile slot inside the CTA
    int it = q0 - slot_t * ipp;     // item inside the CTA's run of the tile
    // unsplit: records are contiguous across tiles; split: a tile's run starts i0 items into the tile
    const size_t first = SPLIT ? (static_cast<size_t>(tile0 + slot_t) * p.items + i0 + it) * kItemBytes
                               : (static_cast<size_t>(tile0) * p.items + q0) * kItemBytes;
    const unsigned char* rec = p.wq + first + lane * 16;
    const unsigned char* met = p.wq + first + 1024 + g * 8;  // lanes of one g share it
    const ActT* x = static_cast<const ActT*>(p.x);

    // ---- a per-warp ring of kStreamDepth items in shared memory, filled by per-lane asynchronous copies: lane L
    //      copies the 2 x 16 weight bytes it reads later; the eight lanes with j == 0 also copy the 8-byte scale / zero
    //      entry of their column pair, which the other lanes of the pair read too, hence the __syncwarp after the wait.
    //      One commit group per item; iteration i waits until at most kStreamDepth - 1 groups are pending.
    unsigned char* ring = smem_all + warp * (kStreamDepth * kSlot);
    const uint32_t ring_lo = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + lane * 16;
    const uint32_t ring_meta = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + 1024 + g * 8;
    size_t issue_off = 0;        // split: byte offset of the next item to request, and the items left of its tile's run
    int issue_room = ipp - it;
    auto issue = [&](int d, int i) {
        if (i < n) {
            const size_t off = SPLIT ? issue_off : static_cast<size_t>(i) * kItemBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kSlot), "l"(rec + off) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kSlot + 512), "l"(rec + off + 512) : "memory");
            if (j == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ring_meta + d * kSlot), "l"(met + off) : "memory");
            if (SPLIT) {
                issue_off += kItemBytes;
                if (--issue_room == 0) {  // the next item opens the next tile's run
                    issue_off += static_cast<size_t>(p.items - ipp) * kItemBytes;
                    issue_room = ipp;
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int d = 0; d < kStreamDepth; ++d) issue(d, d);
    // weights never depend on the previous grid; x and y may (programmatic dependent launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();  // accumulators are zero

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.f;
    bool dirty = false;
    const unsigned char* xs = smem_all + kStreamWarps * kStreamDepth * kSlot + static_cast<size_t>(p.acc_tiles) * kRows * 16 * sizeof(float);
    if (STAGED) {
        // one warp per (item, row block): lane (g, j) copies the 64 bytes it will read as MMA operands, 16 at a time
        unsigned char* xw = const_cast<unsigned char*>(xs);
        for (int b = warp; b < ipp * MT; b += kStreamWarps) {
            const int bi = b / MT, mt = b - bi * MT;
            const int m = mt * 8 + g;
            uint4 v[4];
            if (m < p.M) {
                load_x<ActT>(x + static_cast<size_t>(m) * p.K, p.perm, (i0 + bi) * 128 + 32 * j, v);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = make_uint4(0, 0, 0, 0);
            }
            // pair order: chunk c holds {low, high} of steps 2c and 2c + 1 (the low slots are words 0..7 of the lane's
            // 32 activations, the high slots words 8..15)
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&v[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(xw + (static_cast<size_t>(b) * 4 + c) * 512 + lane * 16) = make_uint4(w[2 * c], w[8 + 2 * c], w[2 * c + 1], w[9 + 2 * c]);
        }
        __syncthreads();
    }
    // Unstaged with one row block: the rows of x run one item ahead of the weights in registers (they come from L1 /
    // L2, and with four warps per scheduler nothing else would cover that latency); two row blocks would spill.
    constexpr bool kAhead = !STAGED && MT == 1;
    static_assert(STAGED || MT <= 2, "three row blocks read their operands from shared memory, block by block");
    uint4 xv[MT > 2 ? 1 : MT][4];
    if constexpr (kAhead) {
        if (n > 0) w4_item_x<ActT, MT, false>(p, x, it, g, j, xv);
    }

    for (int i = 0; i < n; ++i) {
        const int d = i % kStreamDepth;
        asm volatile("cp.async.wait_group %0;" ::"n"(kStreamDepth - 1) : "memory");
        __syncwarp();  // the scale / zero entry was copied by another lane of the column pair
        const unsigned char* slot = ring + d * kSlot;
        const uint4 wl = *reinterpret_cast<const uint4*>(slot + lane * 16);
        const uint4 wh = *reinterpret_cast<const uint4*>(slot + 512 + lane * 16);
        const uint2 mt_ = *reinterpret_cast<const uint2*>(slot + 1024 + g * 8);
        __syncwarp();  // every lane has read the slot before any lane refills it
        issue(d, i + kStreamDepth);  // the slot's bytes are in registers: refill it
        if constexpr (STAGED && MT > 2) {
            w4_item_math_smem<ActT, MT>(p, xs + static_cast<size_t>(it) * MT * 2048 + lane * 16, wl, wh, mt_, yacc);
        } else if constexpr (STAGED) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    xv[mt][c] = *reinterpret_cast<const uint4*>(xs + (static_cast<size_t>(it * MT + mt) * 4 + c) * 512 + lane * 16);
            w4_item_math<ActT, MT, true>(p, xv, wl, wh, mt_, yacc);
        } else if constexpr (kAhead) {
            uint4 xn[MT][4];
            const int it_next = it + 1 == p.items ? 0 : it + 1;
            if (i + 1 < n) w4_item_x<ActT, MT, false>(p, x, it_next, g, j, xn);
            w4_item_math<ActT, MT>(p, xv, wl, wh, mt_, yacc);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int v = 0; v < 4; ++v) xv[mt][v] = xn[mt][v];
        } else {
            w4_item_x<ActT, MT, false>(p, x, it, g, j, xv);
            w4_item_math<ActT, MT>(p, xv, wl, wh, mt_, yacc);
        }
        dirty = true;
        if (++it == ipp) {  // the span leaves this tile
            stream_flush<ActT, MT>(p, acc_s + slot_t * kRows * 16, yacc, g, j);
            dirty = false;
            it = 0;
            ++slot_t;
        }
    }
    if (dirty) stream_flush<ActT, MT>(p, acc_s + slot_t * kRows * 16, yacc, g, j);
    __syncthreads();
    ActT* y = static_cast<ActT*>(p.y);
    if (SPLIT) {
        // ---- the K slices of a tile group meet in the workspace; the last one to arrive converts and leaves zeros behind
        __shared__ int last_s;
        const int rows_s = p.M, grp = cta / p.splits;
        for (int idx = threadIdx.x; idx < ntiles * rows_s * 16; idx += kStreamWarps * 32) {
            const int t = idx / (rows_s * 16), r = idx - t * (rows_s * 16);
            const int m = r >> 4, nn = r & 15;
            atomicAdd(p.wsp + static_cast<size_t>(m) * p.N + (tile0 + t) * 16 + nn, acc_s[(t * kRows + m) * 16 + nn]);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) last_s = atomicAdd(p.counters + grp, 1) == p.splits - 1;
        __syncthreads();
        if (!last_s) return;
        __threadfence();
        for (int idx = threadIdx.x; idx < ntiles * rows_s * 16; idx += kStreamWarps * 32) {
            const int t = idx / (rows_s * 16), r = idx - t * (rows_s * 16);
            const int m = r >> 4, nn = r & 15;
            float* wv = p.wsp + static_cast<size_t>(m) * p.N + (tile0 + t) * 16 + nn;
            y[static_cast<size_t>(m) * p.N + (tile0 + t) * 16 + nn] = from_float<ActT>(__ldcg(wv));
            __stcg(wv, 0.f);
        }
        if (threadIdx.x == 0) p.counters[grp] = 0;
        return;
    }
    // ---- the CTA owns its tiles outright: convert and store
    const int rows = p.M;
    for (int idx = threadIdx.x; idx < ntiles * rows * 16; idx += kStreamWarps * 32) {
        const int t = idx / (rows * 16), r = idx - t * (rows * 16);
        const int m = r >> 4, nn = r & 15;
        y[static_cast<size_t>(m) * p.N + (tile0 + t) * 16 + nn] = from_float<ActT>(acc_s[(t * kRows + m) * 16 + nn]);
    }
}

// Shared memory the stream kernel needs for `tiles` column tiles on `ctas` CTAs (plus the staged x when asked for), or
// 0 when it does not fit.
static size_t stream_smem(long long tiles, long long ctas, int rows, int depth, size_t staged) {
    const long long per_cta = ceil_div(tiles, ctas);
    const size_t bytes = static_cast<size_t>(kStreamWarps) * depth * kSlot + static_cast<size_t>(per_cta) * rows * 16 * sizeof(float) + staged;
    return bytes <= 220 * 1024 ? bytes : 0;
}

template <typename ActT, int MT, int DEPTH, bool STAGED, bool SPLIT = false>
static int launch_stream_depth(W4Params p, size_t smem, long long ctas, cudaStream_t stream) {
    auto kernel = w4a16_stream_kernel<ActT, MT, DEPTH, STAGED, SPLIT>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kStreamWarps * 32);
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

// K slices for a staged x that does not fit whole: 2, 4 or 8 slices so that a slice does, groups of tiles x slices
// filling the SMs as evenly as whole tiles allow.  Returns the slice count (0: none fits) for a ring of `depth` items.
struct SplitPlan {
    int slices = 0;
    long long ctas = 0, group_tiles = 0;
    size_t smem = 0;
};
static SplitPlan plan_split(const W4Params& p, long long tiles, int rows, int depth) {
    SplitPlan best;
    for (int sp = 2; sp <= 8; sp *= 2) {
        if (p.items < sp) break;
        const size_t slice = staged_x_bytes(static_cast<int64_t>(ceil_div(static_cast<long long>(p.items), sp)) * 128, rows);
        const long long groups_want = sm_count() / sp > 0 ? sm_count() / sp : 1;
        const long long tpg = ceil_div(tiles, groups_want);
        const long long groups = ceil_div(tiles, tpg);
        const size_t smem = stream_smem(tpg, 1, rows, depth, slice);
        if (!smem) continue;
        if (groups * sp > best.ctas) {
            best.ctas = groups * sp;
            best.slices = sp;
            best.group_tiles = tpg;
            best.smem = smem;
        }
    }
    return best;
}

template <typename ActT, int MT>
static int launch_stream(W4Params p, cudaStream_t stream, bool* fits) {
    const long long tiles = p.N / 16;
    long long ctas = sm_count();
    if (ctas > tiles) ctas = tiles;
    p.span_base = static_cast<int>(tiles / ctas);
    p.span_rem = static_cast<int>(tiles % ctas);
    p.acc_tiles = static_cast<int>(ceil_div(tiles, ctas));
    p.splits = 1;
    p.group_tiles = 0;
    const int rows = MT * 8;
    *fits = true;
    // x in shared memory where it fits beside a ring of at least three items (gathered rows are read in place)
    const size_t staged = p.x_rows ? 0 : staged_x_bytes(p.K, rows);
    if (staged) {
        if (const size_t smem = stream_smem(tiles, ctas, rows, 6, staged)) return launch_stream_depth<ActT, MT, 6, true>(p, smem, ctas, stream);
        if (const size_t smem = stream_smem(tiles, ctas, rows, 4, staged)) return launch_stream_depth<ActT, MT, 4, true>(p, smem, ctas, stream);
        if (const size_t smem = stream_smem(tiles, ctas, rows, 3, staged)) return launch_stream_depth<ActT, MT, 3, true>(p, smem, ctas, stream);
        // x does not fit: cut K into slices (needs the f32 workspace)
        if (p.wsp && p.counters) {
            SplitPlan plan = plan_split(p, tiles, rows, 4);
            const bool deep = plan.slices != 0;
            if (!deep) plan = plan_split(p, tiles, rows, 3);
            if (plan.slices) {
                p.splits = plan.slices;
                p.group_tiles = static_cast<int>(plan.group_tiles);
                p.acc_tiles = static_cast<int>(plan.group_tiles);
                return deep ? launch_stream_depth<ActT, MT, 4, true, true>(p, plan.smem, plan.ctas, stream)
                            : launch_stream_depth<ActT, MT, 3, true, true>(p, plan.smem, plan.ctas, stream);
            }
        }
    }
    if constexpr (MT <= 2) {
        // the deepest ring that fits, x read from global memory
        if (const size_t smem = stream_smem(tiles, ctas, rows, 6, 0)) return launch_stream_depth<ActT, MT, 6, false>(p, smem, ctas, stream);
        if (const size_t smem = stream_smem(tiles, ctas, rows, 4, 0)) return launch_stream_depth<ActT, MT, 4, false>(p, smem, ctas, stream);
    }
    *fits = false;  // the accumulators of the CTA's tiles (or, with more than 16 rows, a slice of x) do not fit shared memory
    return EQ_OK;
}

template <typename ActT>
static int stream_dispatch(const W4Params& p, cudaStream_t stream, bool* fits) {
    if (p.M <= 8) return launch_stream<ActT, 1>(p, stream, fits);
    if (p.M <= 16) return launch_stream<ActT, 2>(p, stream, fits);
    return launch_stream<ActT, 3>(p, stream, fits);
}

// 2 <= M <= 24, total items < 2^31.  *fits is cleared, and nothing launched, when the shape does not fit.
int w4_stream_launch(const W4Params& p, int act_dtype, cudaStream_t stream, bool* fits) {
    return act_dtype == EQ_F16 ? stream_dispatch<__half>(p, stream, fits) : stream_dispatch<__nv_bfloat16>(p, stream, fits);
}

}  // namespace eq
