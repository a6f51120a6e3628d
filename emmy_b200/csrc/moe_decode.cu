// The decode tier of the routed MoE layer (a handful of tokens): two launches for the whole layer.
//
// With T <= 16 tokens every pick (token, expert) is one activation row against one expert's weights, and the layer is
// bound by the latency of its launches, not by bytes (eight experts of a Qwen3-30B-A3B layer are 20 MB).  The reference
// runs this case as ONE fixed-shape program over the picks (moe.expert.slots: index_select of the stacked expert
// weights by `sel`, batched products, scores @ partials; emmy/serving/gen_runner.py:3219-3284,
// emmy/compiler/trace/huggingface.py:1455-1471).  Here:
//
//   phase 0  every CTA routes the tokens itself (softmax in f32, top-k with ties to the lowest id, renormalised: the
//            router of moe.cu, one warp per token), then the picks' [gate | up] GEMVs run as ONE stream of weight
//            tiles cut into equal whole-tile spans, one per CTA: virtual tile = pick * (2I / 16) + tile, each tile's
//            records found through the pick's expert id.  Output: gu[pick][2I] in the activation dtype.
//   phase 1  the same over the down projections.  The activation row of a pick is act(silu(gate)) * up, computed
//            while it is staged (the eager form's two roundings, emmy/compiler/trace/huggingface.py:1663-1669), and
//            the routed combine is done by whichever CTA completes a token's tile last: it adds the picks' rows in
//            ascending expert order, products and sum in f32, one rounding (emmy/serving/gen_runner.py:235-287).
//
// Both phases are the single-row kernel of w4_gemv1.cu (ring of items per warp, offset-free dequant, per-tile
// completion) without its cross-CTA hand-over: spans are whole tiles.  No host read, every grid is host-known, the layer
// sits in a CUDA graph.
#include "w4_gemv1.cuh"

namespace eq {

constexpr int kDecMaxTokens = 16;
constexpr int kDecMaxTopK = 16;

struct MoeDecParams {
    const unsigned char* wq;  // this phase's stacked expert weights
    size_t expert_stride;
    const float* logits;      // phase 0: [T][E]
    int32_t* ids;             // [T][topk] (phase 0 writes, phase 1 reads)
    float* scores;            // [T][topk]
    const void* x;            // phase 0: tokens [T][K]; phase 1: gu [T topk][2 K]
    void* out;                // phase 0: gu [T topk][N]; phase 1: expert outputs [T topk][N]
    void* y;                  // phase 1: [T][N]
    int* tile_count;          // [T][N / 16] picks arrived per token tile (phase 0 clears, phase 1 counts and clears)
    int* status;              // phase 0 clears
    int T, E, topk;
    int K, N, items, tiles_per_pick;
    int span_base, span_rem;  // tiles per CTA, plus one for the first span_rem CTAs
    int acc_tiles;
};

// f32 -> a 32-bit key whose unsigned order is the float order (so that one redux.sync finds a warp's maximum).
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k); }

// One warp routes one token: ids ascending, scores renormalised.  (The router of moe.cu, see there.)  The lane's logits
// are read once and kept as order keys in registers (eight per lane cover 256 experts; beyond that they are re-read);
// a round of the top-k is a scan of those registers and two redux.sync (the maximum key, then the lowest expert id that
// holds it), and the exponentials of the winners are taken after the rounds, one lane per pick.
__device__ __forceinline__ void route_token(const float* __restrict__ lg, int E, int topk, int32_t* ids, float* scores) {
    constexpr int kKeep = 8;
    const int lane = threadIdx.x & 31;
    uint32_t key[kKeep];
    uint32_t top = 0;
#pragma unroll
    for (int b = 0; b < kKeep; ++b) {
        const int e = lane + 32 * b;
        key[b] = e < E ? order_key(lg[e]) : 0u;  // 0 is below every real key
        top = max(top, key[b]);
    }
    for (int e = lane + 32 * kKeep; e < E; e += 32) top = max(top, order_key(lg[e]));
    const float mx = key_value(__reduce_max_sync(0xFFFFFFFFu, top));
    float sum = 0.f;
#pragma unroll
    for (int b = 0; b < kKeep; ++b)
        if (lane + 32 * b < E) sum += expf(key_value(key[b]) - mx);
    for (int e = lane + 32 * kKeep; e < E; e += 32) sum += expf(lg[e] - mx);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    unsigned long long taken = 0;  // this lane's experts beyond the kept ones that are already picked (bit = (e - lane) / 32)
    int my_id = 0x7FFFFFFF;        // lane jj keeps pick jj
    uint32_t my_key = 0;
    for (int jj = 0; jj < topk; ++jj) {
        uint32_t best = 0;
        int best_b = 0;
#pragma unroll
        for (int b = 0; b < kKeep; ++b) {
            if (key[b] > best) {  // ascending e: the first of equal values stays
                best = key[b];
                best_b = b;
            }
        }
        int best_e = best ? lane + 32 * best_b : 0x7FFFFFFF;
        for (int e = lane + 32 * kKeep, b = kKeep; e < E; e += 32, ++b) {
            if ((taken >> b) & 1ull) continue;
            const uint32_t k = order_key(lg[e]);
            if (k > best) {
                best = k;
                best_e = e;
            }
        }
        const uint32_t win = __reduce_max_sync(0xFFFFFFFFu, best);
        const int win_e = static_cast<int>(__reduce_min_sync(0xFFFFFFFFu, static_cast<unsigned>(best == win ? best_e : 0x7FFFFFFF)));
        if (win_e < E && (win_e & 31) == lane) {  // this lane's expert: out of the running
            const int b = win_e >> 5;
            if (b < kKeep) {
#pragma unroll
                for (int c = 0; c < kKeep; ++c)
                    if (c == b) key[c] = 0u;
            } else {
                taken |= 1ull << b;
            }
        }
        if (lane == jj) {
            my_id = win_e < E ? win_e : E - 1;
            my_key = win_e < E ? win : 0u;
        }
    }
    float my_p = (lane < topk && my_key) ? expf(key_value(my_key) - mx) / sum : 0.f;
    float psum = my_p;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xFFFFFFFFu, psum, off);
    // ascending expert id (the order the combine adds in): a pick's place is the number of picks with a smaller id
    int place = 0;
    for (int jj = 0; jj < topk; ++jj) {
        const int other = __shfl_sync(0xFFFFFFFFu, my_id, jj);
        place += (other < my_id || (other == my_id && jj < lane)) ? 1 : 0;
    }
    if (lane < topk) {
        ids[place] = my_id;
        scores[place] = my_p / psum;
    }
}

// silu(gate) in f32 rounded to the activation dtype, times up, rounded again.
template <typename ActT>
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t gate, uint32_t up) {
    const ActT* gv = reinterpret_cast<const ActT*>(&gate);
    const ActT* uv = reinterpret_cast<const ActT*>(&up);
    ActT r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float gf = to_float(gv[i]);
        const ActT act = from_float<ActT>(gf / (1.f + expf(-gf)));
        r[i] = from_float<ActT>(to_float(act) * to_float(uv[i]));
    }
    return *reinterpret_cast<const uint32_t*>(r);
}

template <typename ActT, bool SCALE_F16, int DEPTH, int PHASE>
__global__ void __launch_bounds__(kG1Threads, 2) moe_decode_kernel(const MoeDecParams p) {
    // Phase 1 follows phase 0 as a programmatic dependent.  CTA 0 of phase 0 releases it only once the routing is in
    // global memory (every other CTA at once), so phase 1 reads the picks and requests its weights while phase 0 still
    // computes; what phase 0 computes (the gate / up rows) is read behind griddepcontrol.wait.
    if (PHASE == 1 || blockIdx.x != 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char smem_all[];
    __shared__ int32_t ids_s[kDecMaxTokens * kDecMaxTopK];
    __shared__ float scores_s[kDecMaxTokens * kDecMaxTopK];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int items = p.items, tpp = p.tiles_per_pick;
    const int picks = p.T * p.topk;

    // phase 0: everything but the weights comes from the kernel before it (and its weights are chosen by the routing)
    if (PHASE == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- this CTA's whole tiles [tile0, tile0 + ntiles) of the picks' tile stream
    const int cta = blockIdx.x;
    const int tile0 = cta * p.span_base + min(cta, p.span_rem);
    const int ntiles = p.span_base + (cta < p.span_rem ? 1 : 0);
    const int pick0 = tile0 / tpp;                         // the span touches this pick and at most the next one
    const int second_from = (pick0 + 1) * tpp - tile0;     // first tile (relative) of the next pick

    float* acc_s = reinterpret_cast<float*>(smem_all + kG1Warps * DEPTH * kG1Slot);  // [ntiles][16]
    int* done_s = reinterpret_cast<int*>(acc_s + p.acc_tiles * 16);
    const int acc_words = p.acc_tiles * 16 + ((p.acc_tiles + 3) & ~3);
    uint4* xs = reinterpret_cast<uint4*>(acc_s + acc_words);       // [2][K / 8] staged rows of the two picks
    float2* xsum = reinterpret_cast<float2*>(xs + 2 * (p.K / 8));  // [2][items]
    for (int i = threadIdx.x; i < acc_words; i += kG1Threads) acc_s[i] = 0.f;

    // The activation row(s) of the span's picks depend on the pick index only, not on the routing.
    auto stage_rows = [&](int first_warp) {
        const int n_vec = p.K / 8;
        const int rows = second_from < ntiles ? 2 : 1;
        const int stagers = (kG1Warps - first_warp) * 32;
        if (warp < first_warp) return;
        for (int r = 0; r < rows; ++r) {
            const int pick = pick0 + r;
            for (int v = threadIdx.x - first_warp * 32; v < ((n_vec + 31) & ~31); v += stagers) {  // whole warps: the sums shuffle
                uint4 val = make_uint4(0, 0, 0, 0);
                if (v < n_vec) {
                    if (PHASE == 0) {
                        val = __ldg(reinterpret_cast<const uint4*>(static_cast<const ActT*>(p.x) + static_cast<size_t>(pick / p.topk) * p.K) + v);
                    } else {
                        const uint4* gu = reinterpret_cast<const uint4*>(static_cast<const ActT*>(p.x) + static_cast<size_t>(pick) * 2 * p.K);
                        const uint4 gate = __ldcg(gu + v), up = __ldcg(gu + n_vec + v);
                        val = make_uint4(swiglu_pair<ActT>(gate.x, up.x), swiglu_pair<ActT>(gate.y, up.y), swiglu_pair<ActT>(gate.z, up.z),
                                         swiglu_pair<ActT>(gate.w, up.w));
                    }
                }
                stage_vector<ActT>(val, v, v < n_vec, xs + r * n_vec, xsum + r * items);
            }
        }
    };

    if (PHASE == 0) {
        // the routing (the first T warps, one token each); the other warps stage the rows meanwhile
        if (warp < p.T) route_token(p.logits + static_cast<size_t>(warp) * p.E, p.E, p.topk, ids_s + warp * p.topk, scores_s + warp * p.topk);
        // this launch also leaves the arrival counters of phase 1 and the status word zero
        for (int i = blockIdx.x * kG1Threads + threadIdx.x; i < p.T * (p.K / 16); i += gridDim.x * kG1Threads) p.tile_count[i] = 0;
        if (blockIdx.x == 0 && threadIdx.x == 0) *p.status = 0;
        stage_rows(p.T < kG1Warps ? p.T : 0);
        __syncthreads();
        if (blockIdx.x == 0) {
            for (int i = threadIdx.x; i < picks; i += kG1Threads) {
                p.ids[i] = ids_s[i];
                p.scores[i] = scores_s[i];
            }
            __threadfence();  // the routing is in global memory ...
            __syncthreads();
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // ... before phase 1 may start
        }
    } else {
        for (int i = threadIdx.x; i < picks; i += kG1Threads) {
            ids_s[i] = __ldcg(p.ids + i);
            scores_s[i] = __ldcg(p.scores + i);
        }
        __syncthreads();
    }

    // ---- this warp's items: an equal contiguous share of the CTA's ntiles * items
    const int cta_items = ntiles * items;
    const int q0 = cta_items * warp / kG1Warps, q1 = cta_items * (warp + 1) / kG1Warps;
    const int n = q1 - q0;
    int slot_t = q0 / items;       // tile (relative to tile0)
    int it = q0 - slot_t * items;  // item inside the tile
    auto tile_base = [&](int rel) {  // first record of relative tile `rel`
        const int t = tile0 + rel;
        const int pick = t / tpp;
        return p.wq + static_cast<size_t>(ids_s[pick]) * p.expert_stride + static_cast<size_t>(t - pick * tpp) * items * kItemBytes;
    };

    const uint32_t ring_w = smem_u32(smem_all) + warp * (DEPTH * kG1Slot) + lane * 16;
    const uint32_t ring_m = ring_w + 1024 - lane * 8;
    const int meta_delta = 1024 + g * 8 - lane * 16;
    int issue_left = n;            // items not yet requested
    int issue_tile = slot_t;       // tile of the next item to request
    int issue_room = items - it;   // items of that tile not yet requested
    const unsigned char* src = n > 0 ? tile_base(issue_tile) + static_cast<size_t>(it) * kItemBytes + lane * 16 : p.wq;
    auto issue = [&](uint32_t slot) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.gt.s32 p, %4, 0;\n"
            "@p cp.async.cg.shared.global [%0], [%2], 16;\n"
            "@p cp.async.cg.shared.global [%0+512], [%2+512], 16;\n"
            "@p cp.async.ca.shared.global [%1], [%3], 8;\n"
            "cp.async.commit_group;\n"
            "}\n" ::"r"(ring_w + slot),
            "r"(ring_m + slot), "l"(src), "l"(src + meta_delta), "r"(issue_left)
            : "memory");
        --issue_left;
        src += kItemBytes;
        if (--issue_room == 0 && issue_left > 0) {  // the next item opens a new tile, possibly another expert's
            ++issue_tile;
            issue_room = items;
            src = tile_base(issue_tile) + lane * 16;
        }
    };
#pragma unroll 1
    for (int d = 0; d < DEPTH; ++d) issue(d * kG1Slot);

    if (PHASE == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // the picks the weights were requested for are the picks phase 0 ended with: anything else is reported
        for (int i = threadIdx.x; i < picks; i += kG1Threads)
            if (__ldcg(p.ids + i) != ids_s[i]) atomicExch(p.status, 5);
        stage_rows(0);
        __syncthreads();
    }

    float y_lo = 0.f, y_hi = 0.f;
    int i = 0;
    uint32_t slot = 0;
    const uint32_t acc_u32 = smem_u32(acc_s);
    while (i < n) {
        const int stretch = min(items - it, n - i);
        const int which = slot_t >= second_from ? 1 : 0;  // which staged row this tile's pick reads
        uint32_t x_addr = smem_u32(xs + which * (p.K / 8)) + it * 256 + j * 16;
        uint32_t sum_addr = smem_u32(xsum + which * items) + it * 8;
        for (int c = stretch; c > 0; --c) {
            asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
            gemv1_item<ActT, SCALE_F16>(ring_w + slot, ring_m + slot, x_addr, sum_addr, y_lo, y_hi);
            issue(slot);
            slot += kG1Slot;
            if (slot == DEPTH * kG1Slot) slot = 0;
            x_addr += 256;
            sum_addr += 8;
        }
        i += stretch;
        it += stretch;
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
            complete = atomicAdd(done_s + slot_t, stretch) + stretch == items;
        }
        complete = __shfl_sync(0xFFFFFFFFu, complete, 0);
        if (complete) {
            // every warp's part of this tile is in: round it to the activation dtype and store it
            __threadfence_block();
            const int t = tile0 + slot_t;
            const int pick = t / tpp, local = t - pick * tpp;
            ActT* out = static_cast<ActT*>(p.out);
            if (lane < 16) out[static_cast<size_t>(pick) * p.N + local * 16 + lane] = from_float<ActT>(*(volatile float*)(acc_s + slot_t * 16 + lane));
            if (PHASE == 1) {
                // the routed combine: the pick that arrives last at this tile of its token adds all of the token's picks
                const int token = pick / p.topk;
                __threadfence();  // this tile's stores before its arrival is counted
                __syncwarp();
                int last = 0;
                if (lane == 0) last = atomicAdd(p.tile_count + token * tpp + local, 1) == p.topk - 1;
                last = __shfl_sync(0xFFFFFFFFu, last, 0);
                if (last) {
                    __threadfence();  // the other picks' stores after their arrivals were seen
                    if (lane < 16) {
                        float s = 0.f;
                        for (int jj = 0; jj < p.topk; ++jj) {  // ascending expert id, products and sum in f32, one rounding
                            const ActT v = __ldcg(out + static_cast<size_t>(token * p.topk + jj) * p.N + local * 16 + lane);
                            s += to_float(from_float<ActT>(scores_s[token * p.topk + jj])) * to_float(v);
                        }
                        static_cast<ActT*>(p.y)[static_cast<size_t>(token) * p.N + local * 16 + lane] = from_float<ActT>(s);
                    }
                    if (lane == 0) p.tile_count[token * tpp + local] = 0;  // zero again for the next call
                }
            }
        }
        it = 0;
        ++slot_t;
    }
}

static size_t dec_smem(int depth, int acc_tiles, int K) {
    return static_cast<size_t>(kG1Warps) * depth * kG1Slot + static_cast<size_t>(acc_tiles) * 16 * sizeof(float) +
           static_cast<size_t>((acc_tiles + 3) & ~3) * sizeof(int) + 2 * (static_cast<size_t>(K) * 2 + static_cast<size_t>(K / 128) * sizeof(float2));
}

template <typename ActT, bool SCALE_F16, int PHASE, int DEPTH>
static int launch_phase_depth(const MoeDecParams& p, size_t smem, long long ctas, cudaStream_t stream) {
    auto kernel = moe_decode_kernel<ActT, SCALE_F16, DEPTH, PHASE>;
    static bool configured[64] = {};
    int dev = 0;
    EQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
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

template <typename ActT, bool SCALE_F16, int PHASE>
static int launch_phase(MoeDecParams p, cudaStream_t stream) {
    const long long tiles = static_cast<long long>(p.T) * p.topk * p.tiles_per_pick;
    long long ctas = sm_count();
    if (ctas > tiles) ctas = tiles;
    p.span_base = static_cast<int>(tiles / ctas);
    p.span_rem = static_cast<int>(tiles % ctas);
    p.acc_tiles = p.span_base + 1;
    // a warp's share of the CTA's items decides the ring: five slots where that covers more of it and still leaves
    // room for a second CTA on the SM, else four
    const long long per_warp = ceil_div(static_cast<long long>(p.acc_tiles) * p.items, kG1Warps);
    const size_t smem5 = dec_smem(5, p.acc_tiles, p.K);
    if (per_warp > 4 && smem5 <= 112 * 1024) return launch_phase_depth<ActT, SCALE_F16, PHASE, 5>(p, smem5, ctas, stream);
    return launch_phase_depth<ActT, SCALE_F16, PHASE, 4>(p, dec_smem(4, p.acc_tiles, p.K), ctas, stream);
}

// Whether the decode tier serves this layer: few tokens, every CTA's tiles inside two picks, everything in 112 KB.
bool moe_decode_fits(int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I) {
    if (T < 1 || T > kDecMaxTokens || topk > kDecMaxTopK || E > 1024) return false;
    if (H % 128 || I % 128) return false;
    if (topk * I * 2 < (H / 16) * 4) return false;  // the arrival counters live in the (otherwise unused) activation scratch
    const long long ctas = sm_count();
    for (int phase = 0; phase < 2; ++phase) {
        const long long K = phase == 0 ? H : I, tpp = (phase == 0 ? 2 * I : H) / 16;
        const long long tiles = T * topk * tpp;
        const long long per_cta = (tiles + (tiles < ctas ? tiles : ctas) - 1) / (tiles < ctas ? tiles : ctas);
        if (per_cta > tpp) return false;
        if (dec_smem(4, static_cast<int>(per_cta) + 1, static_cast<int>(K)) > 112 * 1024) return false;
    }
    return true;
}

// Whole routed layer for T <= 16 tokens.  gu: [T topk][2 I], rows: [T topk][H] scratch in the activation dtype;
// tile_count: T * H / 16 ints.
int moe_decode_launch(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t topk, int64_t H, int64_t I,
                      const void* x, const float* logits, int64_t T, int act_dtype, void* y, int32_t* ids, float* scores, void* gu, void* rows,
                      int* tile_count, int* status, cudaStream_t stream) {
    MoeDecParams p = {};
    p.logits = logits;
    p.ids = ids;
    p.scores = scores;
    p.tile_count = tile_count;
    p.status = status;
    p.T = static_cast<int>(T);
    p.E = static_cast<int>(E);
    p.topk = static_cast<int>(topk);
    p.y = y;
    int st = EQ_OK;
    for (int phase = 0; phase < 2 && st == EQ_OK; ++phase) {
        p.K = static_cast<int>(phase == 0 ? H : I);
        p.N = static_cast<int>(phase == 0 ? 2 * I : H);
        p.items = p.K / 128;
        p.tiles_per_pick = p.N / 16;
        p.wq = static_cast<const unsigned char*>(phase == 0 ? wq_gate_up : wq_down);
        p.expert_stride = static_cast<size_t>(p.tiles_per_pick) * p.items * kItemBytes;
        p.x = phase == 0 ? x : gu;
        p.out = phase == 0 ? gu : rows;
        const bool f16 = act_dtype == EQ_F16, sf16 = scale_dtype == EQ_F16;
        if (phase == 0) {
            if (f16) st = sf16 ? launch_phase<__half, true, 0>(p, stream) : launch_phase<__half, false, 0>(p, stream);
            else st = sf16 ? launch_phase<__nv_bfloat16, true, 0>(p, stream) : launch_phase<__nv_bfloat16, false, 0>(p, stream);
        } else {
            if (f16) st = sf16 ? launch_phase<__half, true, 1>(p, stream) : launch_phase<__half, false, 1>(p, stream);
            else st = sf16 ? launch_phase<__nv_bfloat16, true, 1>(p, stream) : launch_phase<__nv_bfloat16, false, 1>(p, stream);
        }
    }
    return st;
}

}  // namespace eq
