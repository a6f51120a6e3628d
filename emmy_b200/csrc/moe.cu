// Mixture-of-experts layer on W4A16 (AWQ / GPTQ int4) experts: router, token permute, grouped expert FFN, combine.
// Everything is decided on the device: no host read of the routing, every launch has a host-known grid, so the
// whole layer can sit in a CUDA graph at any token count.
//
//   moe_route_kernel      softmax in f32 over the router logits, top-k with ties to the lowest expert id, picked
//                         probabilities renormalised, picks of a row sorted by ascending expert id (the order the
//                         combine adds them in).  Follows emmy/serving/native/prepare.py:424-463 and the routed
//                         combine's ordering, emmy/serving/gen_runner.py:263-279.
//   moe_count / moe_plan / moe_scatter
//                         histogram of rows per expert, exclusive scan, the list of (expert, first row, rows) row
//                         blocks, and each row's position in expert order: the device-side form of the reference's
//                         stable argsort + counts.tolist() (gen_runner.py:276-283).
//   moe_expert_gemm_kernel  grouped W4A16 GEMM: grid = (column tiles, row blocks); a row block is at most kRowBlock
//                         rows of ONE expert, its weights are that expert's slice of the stacked repacked tensor.
//                         Rows are gathered (first GEMM) / scattered (second GEMM) through index arrays, nothing is
//                         copied.  Body: the W4A16 tile code of w4_tile.cuh.
//                         With many rows per expert the two GEMMs run on the tensor path instead (w4_gemm.cu): rows are
//                         first copied into expert order (moe_gather_rows_kernel) so that TMA can read them, row
//                         blocks are 256 rows, and SwiGLU is fused into the first GEMM's epilogue.
//   streaming tier        up to eight rows per expert on average (and more tokens than the decode tier takes): the plan's
//                         row blocks hold at most eight rows and both grouped linears run through moe_stream.cu, which
//                         streams every touched expert's weights once per block; SwiGLU is a kernel of its own between.
//   moe_swiglu_kernel     h = silu(gate) * up with the roundings of the eager form
//                         (emmy/compiler/trace/huggingface.py:1663-1669).
//   moe_combine_kernel    out[t] = dtype(sum_j f32(score_j) * f32(expert_j(x_t))), picks in ascending expert order,
//                         products and sum in f32, one rounding (gen_runner.py:235-287).
#include <type_traits>

#include "w4_tile.cuh"

namespace eq {

bool moe_decode_fits(int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I);  // moe_decode.cu
int moe_decode_launch(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t topk, int64_t H, int64_t I,
                      const void* x, const float* logits, int64_t T, int act_dtype, void* y, int32_t* ids, float* scores, void* gu, void* rows,
                      int* tile_count, int* status, cudaStream_t stream);
bool moe_stream_fits(int max_blocks, int64_t N);  // moe_stream.cu
int moe_stream_launch(const unsigned char* wq, size_t expert_stride, int scale_dtype, const void* x, void* y, const int32_t* x_rows,
                      const int32_t* y_rows, const uint64_t* y_ptrs, const RowBlock* blocks, const int32_t* n_blocks, int max_blocks, int64_t K,
                      int64_t N, int act_dtype, cudaStream_t stream);
int w4_gemm_tc_grouped_launch(const unsigned char* wq, size_t expert_stride, int scale_dtype, const void* x, void* y, int64_t R, int64_t N,
                              int64_t K, int act_dtype, const RowBlock* blocks, const int32_t* n_blocks, int max_blocks,
                              const int32_t* y_rows, const uint64_t* y_ptrs, bool swiglu, int* status, cudaStream_t stream);  // w4_gemm.cu

constexpr int kMaxTopK = 16;
constexpr int kBadExpertId = 16;  // status code of a row whose expert id is out of range (1..4 are the tensor path's waits)

// ------------------------------------------------------------------------------------------------ router
// One warp per token.  E <= 1024.
__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int topk, int renorm, int32_t* __restrict__ ids,
                                 float* __restrict__ scores) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    const float* lg = logits + static_cast<size_t>(warp) * E;
    // softmax statistics
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(lg[e] - mx);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    // top-k by repeated arg-max on the logits (they order the experts as the probabilities do); ties -> lowest id
    int pick_id[kMaxTopK];
    float pick_p[kMaxTopK];
    unsigned long long taken_lo = 0;  // this lane's experts already picked (bit = (e - lane) / 32)
    float psum = 0.f;
    for (int j = 0; j < topk; ++j) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
        for (int e = lane, b = 0; e < E; e += 32, ++b) {
            if ((taken_lo >> b) & 1ull) continue;
            const float v = lg[e];
            if (v > best || (v == best && e < best_e)) {
                best = v;
                best_e = e;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, off);
            if (ov > best || (ov == best && oe < best_e)) {
                best = ov;
                best_e = oe;
            }
        }
        if (best_e < E && (best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
        const float pr = best_e < E ? expf(best - mx) / sum : 0.f;
        pick_id[j] = best_e < E ? best_e : E - 1;
        pick_p[j] = pr;
        psum += pr;
    }
    if (lane == 0) {
        // ascending expert id (insertion sort of at most 16 picks)
        for (int a = 1; a < topk; ++a) {
            const int id = pick_id[a];
            const float pv = pick_p[a];
            int b = a - 1;
            while (b >= 0 && pick_id[b] > id) {
                pick_id[b + 1] = pick_id[b];
                pick_p[b + 1] = pick_p[b];
                --b;
            }
            pick_id[b + 1] = id;
            pick_p[b + 1] = pv;
        }
        for (int j = 0; j < topk; ++j) {
            ids[static_cast<size_t>(warp) * topk + j] = pick_id[j];
            scores[static_cast<size_t>(warp) * topk + j] = renorm ? pick_p[j] / psum : pick_p[j];
        }
    }
}

// ------------------------------------------------------------------------------------------------ permute
__global__ void moe_count_kernel(const int32_t* __restrict__ eid, int R, int E, int32_t* __restrict__ counts, int32_t* status) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int e = eid[r];
    if (e == -1) return;  // an empty slot of an expert-parallel receive buffer
    if (e < 0 || e >= E) {
        atomicExch(status, kBadExpertId);  // the row is dropped, the caller is told
        return;
    }
    atomicAdd(counts + e, 1);
}

// One CTA: exclusive scan of the counts, row blocks of at most `block_rows` rows, cursors reset.
__global__ void moe_plan_kernel(const int32_t* __restrict__ counts, int E, int block_rows, int32_t* __restrict__ offsets,
                                int32_t* __restrict__ cursor, RowBlock* __restrict__ blocks, int32_t* __restrict__ n_blocks,
                                int max_blocks) {
    extern __shared__ int32_t sh[];  // [E] counts -> offsets, [E] block offsets
    int32_t* off = sh;
    int32_t* boff = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        off[e] = counts[e];
        boff[e] = (counts[e] + block_rows - 1) / block_rows;
        cursor[e] = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t run = 0, brun = 0;
        for (int e = 0; e < E; ++e) {
            const int32_t c = off[e], b = boff[e];
            off[e] = run;
            boff[e] = brun;
            run += c;
            brun += b;
        }
        offsets[E] = run;
        *n_blocks = brun < max_blocks ? brun : max_blocks;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        offsets[e] = off[e];
        const int32_t c = counts[e];
        for (int32_t b = 0, r = 0; r < c; ++b, r += block_rows) {
            if (boff[e] + b < max_blocks) {
                RowBlock rb;
                rb.expert = e;
                rb.row0 = off[e] + r;
                rb.rows = min(block_rows, c - r);
                rb.pad = 0;
                blocks[boff[e] + b] = rb;
            }
        }
    }
}

// pos_of[r]: position of row r in expert order; src_of[pos]: the activation row that feeds position pos; dst_of[pos] = r.
// row_ptr (optional): the address output row r goes to; dst_ptr[pos] carries it into expert order.
__global__ void moe_scatter_kernel(const int32_t* __restrict__ eid, const int32_t* __restrict__ src_row, int R, int E,
                                   const int32_t* __restrict__ offsets, int32_t* __restrict__ cursor, int32_t* __restrict__ src_of,
                                   int32_t* __restrict__ dst_of, const uint64_t* __restrict__ row_ptr, uint64_t* __restrict__ dst_ptr,
                                   int src_div) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int e = eid[r];
    if (e < 0 || e >= E) return;
    const int pos = offsets[e] + atomicAdd(cursor + e, 1);
    src_of[pos] = src_row ? src_row[r] : (src_div > 0 ? r / src_div : r);
    dst_of[pos] = r;
    if (row_ptr) dst_ptr[pos] = row_ptr[r];
}

// The three kernels above in one CTA, for row counts where the launches cost more than the work.
constexpr int kSmallPlanRows = 8192;
__global__ void moe_plan_small_kernel(const int32_t* __restrict__ eid, const int32_t* __restrict__ src_row, int src_div, int R, int E, int block_rows,
                                      int32_t* __restrict__ offsets, RowBlock* __restrict__ blocks, int32_t* __restrict__ n_blocks, int max_blocks,
                                      int32_t* __restrict__ src_of, int32_t* __restrict__ dst_of, const uint64_t* __restrict__ row_ptr,
                                      uint64_t* __restrict__ dst_ptr, int32_t* __restrict__ status) {
    extern __shared__ int32_t sh[];  // counts -> cursors [E], offsets [E], block offsets [E]
    int32_t* cnt = sh;
    int32_t* off = sh + E;
    int32_t* boff = sh + 2 * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        const int e = eid[r];
        if (e == -1) continue;
        if (e < 0 || e >= E)
            atomicExch(status, kBadExpertId);
        else
            atomicAdd(cnt + e, 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t run = 0, brun = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = run;
            boff[e] = brun;
            run += cnt[e];
            brun += (cnt[e] + block_rows - 1) / block_rows;
        }
        offsets[E] = run;
        *n_blocks = brun < max_blocks ? brun : max_blocks;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        offsets[e] = off[e];
        const int32_t c = cnt[e];
        for (int32_t b = 0, r = 0; r < c; ++b, r += block_rows) {
            if (boff[e] + b < max_blocks) {
                RowBlock rb;
                rb.expert = e;
                rb.row0 = off[e] + r;
                rb.rows = min(block_rows, c - r);
                rb.pad = 0;
                blocks[boff[e] + b] = rb;
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;  // now the cursors
    __syncthreads();
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        const int e = eid[r];
        if (e < 0 || e >= E) continue;
        const int pos = off[e] + atomicAdd(cnt + e, 1);
        src_of[pos] = src_row ? src_row[r] : (src_div > 0 ? r / src_div : r);
        dst_of[pos] = r;
        if (row_ptr) dst_ptr[pos] = row_ptr[r];
    }
}

// xp[pos][:] = x[src_of[pos]][:], 16 bytes per thread.
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ src_of, const int32_t* __restrict__ total_rows,
                                       int row_vec, uint4* __restrict__ xp) {
    // a grid-stride loop over the rows that exist: the row list of an expert-parallel receive buffer is mostly empty
    // slots (world x capacity), and a thread per slot would launch hundreds of thousands of CTAs that only return
    const int64_t total = static_cast<int64_t>(*total_rows) * row_vec;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t pos = idx / row_vec, v = idx - pos * row_vec;
        xp[idx] = x[static_cast<int64_t>(src_of[pos]) * row_vec + v];
    }
}

// ------------------------------------------------------------------------------------------------ grouped GEMM
struct GroupedParams {
    const unsigned char* wq;      // [E][n_tiles][items][1088]
    size_t expert_stride;         // bytes between experts
    const void* x;                // activations (rows addressed through x_rows, or contiguous in expert order)
    void* y;                      // outputs (rows addressed through y_rows, or contiguous in expert order)
    const int32_t* x_rows;        // optional [R] gather index in expert order
    const int32_t* y_rows;        // optional [R] scatter index in expert order
    const uint64_t* y_ptrs;       // optional [R] destination address of each row in expert order (overrides y / y_rows)
    const RowBlock* blocks;
    const int32_t* n_blocks;
    int K, N, scale_dtype;
};

template <typename ActT, int MT, bool ONE>
__global__ void __launch_bounds__(kTileThreads) moe_expert_gemm_kernel(const GroupedParams gp) {
    __shared__ float red[kTileWarps][MT * 8][16];
    __shared__ int last_flag;
    if (static_cast<int>(blockIdx.y) >= *gp.n_blocks) return;
    const RowBlock rb = gp.blocks[blockIdx.y];
    W4Params p;
    p.wq = gp.wq + static_cast<size_t>(rb.expert) * gp.expert_stride;
    p.perm = nullptr;
    p.K = gp.K;
    p.N = gp.N;
    p.M = rb.rows;
    p.items = gp.K / 128;
    p.splits = 1;
    p.scale_dtype = gp.scale_dtype;
    p.wsp = nullptr;
    p.counters = nullptr;
    if (gp.x_rows) {
        p.x = gp.x;
        p.x_rows = gp.x_rows + rb.row0;
    } else {
        p.x = static_cast<const ActT*>(gp.x) + static_cast<size_t>(rb.row0) * gp.K;
        p.x_rows = nullptr;
    }
    p.y_ptrs = gp.y_ptrs ? gp.y_ptrs + rb.row0 : nullptr;
    if (gp.y_rows) {
        p.y = gp.y;
        p.y_rows = gp.y_rows + rb.row0;
    } else {
        p.y = static_cast<ActT*>(gp.y) + static_cast<size_t>(rb.row0) * gp.N;
        p.y_rows = nullptr;
    }
    w4_tile<ActT, MT, ONE>(p, blockIdx.x, 0, red, &last_flag);
}

// h[r][i] = act( silu(gate[r][i]) ) * up[r][i], gate = gu[r][i], up = gu[r][I + i]; silu in f32, rounded to the
// activation dtype before the product, product rounded again: the eager form's two roundings.
template <typename ActT>
__global__ void moe_swiglu_kernel(const ActT* __restrict__ gu, const int32_t* __restrict__ total_rows, int I, ActT* __restrict__ h) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t r = idx / I, i = idx % I;
    if (r >= *total_rows) return;
    const float g = to_float(gu[r * 2 * I + i]), u = to_float(gu[r * 2 * I + I + i]);
    const ActT s = from_float<ActT>(g / (1.f + expf(-g)));
    h[idx] = from_float<ActT>(to_float(s) * u);
}

// One thread per output element: f32 products and sum over the row's picks in their stored (ascending id) order.
template <typename ActT>
__global__ void moe_combine_kernel(const ActT* __restrict__ out_rows, const float* __restrict__ scores, int T, int topk, int H,
                                   ActT* __restrict__ y) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= static_cast<int64_t>(T) * H) return;
    const int64_t t = idx / H, hcol = idx % H;
    float acc = 0.f;
    for (int j = 0; j < topk; ++j) {
        // the reference casts the scores to the activation dtype first (gen_runner.py:263)
        const float sc = to_float(from_float<ActT>(scores[t * topk + j]));
        acc = fmaf(sc, to_float(out_rows[(t * topk + j) * H + hcol]), acc);
    }
    y[idx] = from_float<ActT>(acc);
}

// The same, eight columns (16 bytes) per thread: H % 8 == 0 and 16-byte aligned rows.
template <typename ActT>
__global__ void moe_combine_vec_kernel(const uint4* __restrict__ out_rows, const float* __restrict__ scores, int T, int topk, int H8,
                                       uint4* __restrict__ y) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= static_cast<int64_t>(T) * H8) return;
    const int64_t t = idx / H8, c = idx - t * H8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
        const float sc = to_float(from_float<ActT>(scores[t * topk + j]));
        const uint4 v = out_rows[(t * topk + j) * H8 + c];
        const ActT* e = reinterpret_cast<const ActT*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(sc, to_float(e[i]), acc[i]);
    }
    uint4 o;
    ActT* oe = reinterpret_cast<ActT*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) oe[i] = from_float<ActT>(acc[i]);
    y[idx] = o;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct MoeWorkspace {
    int32_t *counts, *offsets, *cursor, *n_blocks, *status, *src_of, *dst_of, *ids, *src_row;
    float* scores;
    uint64_t* dst_ptr;
    RowBlock* blocks;
    unsigned char *h1, *h, *out;
    int max_blocks;
    size_t bytes;
};

// Rows per expert at which the grouped GEMMs move to the tensor path (256-row blocks).
// Up to eight rows per expert on average the layer is a weight stream with a little math attached: row blocks of eight
// rows through the streaming tier (moe_stream.cu; the tile code serves shapes it cannot hold).  Above that the tensor
// path with 256-row blocks.
static bool stream_rows(int64_t R, int64_t E) { return R <= 8 * E; }
static bool tensor_path(int64_t R, int64_t E) { return !stream_rows(R, E); }
static int block_rows_for(int64_t R, int64_t E) { return tensor_path(R, E) ? 256 : 8; }

static MoeWorkspace carve(void* base, int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I) {
    MoeWorkspace w;
    const int64_t R = T * topk;
    unsigned char* p = static_cast<unsigned char*>(base);
    size_t o = 0;
    auto take = [&](size_t bytes) {
        unsigned char* r = p ? p + o : nullptr;
        o += align_up(bytes, 256);
        return r;
    };
    w.counts = reinterpret_cast<int32_t*>(take(E * 4));
    w.offsets = reinterpret_cast<int32_t*>(take((E + 1) * 4));
    w.cursor = reinterpret_cast<int32_t*>(take(E * 4));
    w.n_blocks = reinterpret_cast<int32_t*>(take(4));
    w.status = reinterpret_cast<int32_t*>(take(4));
    w.max_blocks = static_cast<int>(R / block_rows_for(R, E) + E + 1);
    w.blocks = reinterpret_cast<RowBlock*>(take(sizeof(RowBlock) * w.max_blocks));
    w.src_of = reinterpret_cast<int32_t*>(take(R * 4));
    w.dst_of = reinterpret_cast<int32_t*>(take(R * 4));
    w.ids = reinterpret_cast<int32_t*>(take(R * 4));
    w.src_row = reinterpret_cast<int32_t*>(take(R * 4));
    w.scores = reinterpret_cast<float*>(take(R * 4));
    w.dst_ptr = reinterpret_cast<uint64_t*>(take(R * 8));
    w.h1 = take(R * 2 * I * 2);
    w.h = take(R * I * 2);
    w.out = take(R * H * 2);
    w.bytes = o;
    return w;
}

template <typename ActT>
static int launch_grouped(const GroupedParams& gp, int block_rows, int max_blocks, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>(gp.N / 16), static_cast<unsigned>(max_blocks));
    if (block_rows <= 8) moe_expert_gemm_kernel<ActT, 1, false><<<grid, kTileThreads, 0, stream>>>(gp);
    else if (block_rows <= 16) moe_expert_gemm_kernel<ActT, 2, false><<<grid, kTileThreads, 0, stream>>>(gp);
    else moe_expert_gemm_kernel<ActT, 8, false><<<grid, kTileThreads, 0, stream>>>(gp);
    EQ_LAUNCH_OK("moe_expert_gemm_kernel");
    return EQ_OK;
}

// Grouped expert FFN over R rows: row r is activation row src_row[r] (or r) of x and belongs to expert eid[r];
// out[r] = down_e( silu(gate_e(x)) * up_e(x) ).
template <typename ActT>
static int experts_forward(const MoeWorkspace& w, const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t H,
                           int64_t I, const void* x, const int32_t* src_row, int src_div, const int32_t* eid, int64_t R, void* out,
                           const uint64_t* row_ptr, cudaStream_t stream) {
    const int br = block_rows_for(R, E);
    if (R <= kSmallPlanRows) {
        moe_plan_small_kernel<<<1, 1024, 3 * E * sizeof(int32_t), stream>>>(eid, src_row, src_div, static_cast<int>(R), static_cast<int>(E), br, w.offsets,
                                                                            w.blocks, w.n_blocks, w.max_blocks, w.src_of, w.dst_of, row_ptr, w.dst_ptr,
                                                                            w.status);
        EQ_LAUNCH_OK("moe_plan_small_kernel");
    } else {
        EQ_CUDA_OK(cudaMemsetAsync(w.counts, 0, E * 4, stream));
        moe_count_kernel<<<static_cast<unsigned>(ceil_div(R, 256)), 256, 0, stream>>>(eid, static_cast<int>(R), static_cast<int>(E), w.counts, w.status);
        EQ_LAUNCH_OK("moe_count_kernel");
        moe_plan_kernel<<<1, 256, 2 * E * sizeof(int32_t), stream>>>(w.counts, static_cast<int>(E), br, w.offsets, w.cursor, w.blocks, w.n_blocks,
                                                                     w.max_blocks);
        EQ_LAUNCH_OK("moe_plan_kernel");
        moe_scatter_kernel<<<static_cast<unsigned>(ceil_div(R, 256)), 256, 0, stream>>>(eid, src_row, static_cast<int>(R), static_cast<int>(E), w.offsets,
                                                                                      w.cursor, w.src_of, w.dst_of, row_ptr, w.dst_ptr, src_div);
        EQ_LAUNCH_OK("moe_scatter_kernel");
    }
    if (tensor_path(R, E)) {
        // rows into expert order (the region of the second GEMM's output in the workspace is free until then)
        const int act = sizeof(ActT) == 2 && std::is_same<ActT, __half>::value ? EQ_F16 : EQ_BF16;
        const int row_vec = static_cast<int>(H * 2 / 16);
        EQ_REQUIRE(aligned(x, 16) && aligned(out, 16), EQ_ERR_BAD_ALIGN, "grouped expert GEMM: activations and outputs must be 16-byte aligned");
        const int64_t gather_ctas = ceil_div(R * row_vec, 256);
        moe_gather_rows_kernel<<<static_cast<unsigned>(gather_ctas < 32LL * sm_count() ? gather_ctas : 32LL * sm_count()), 256, 0, stream>>>(
            static_cast<const uint4*>(x), w.src_of, w.offsets + E, row_vec, reinterpret_cast<uint4*>(w.out));
        EQ_LAUNCH_OK("moe_gather_rows_kernel");
        int st = w4_gemm_tc_grouped_launch(static_cast<const unsigned char*>(wq_gate_up), static_cast<size_t>(2 * I / 16) * (H / 128) * kItemBytes,
                                           scale_dtype, w.out, w.h, R, 2 * I, H, act, w.blocks, w.n_blocks, w.max_blocks, nullptr, nullptr, true,
                                           w.status, stream);
        if (st != EQ_OK) return st;
        return w4_gemm_tc_grouped_launch(static_cast<const unsigned char*>(wq_down), static_cast<size_t>(H / 16) * (I / 128) * kItemBytes,
                                         scale_dtype, w.h, out, R, H, I, act, w.blocks, w.n_blocks, w.max_blocks, w.dst_of,
                                         row_ptr ? w.dst_ptr : nullptr, false, w.status, stream);
    }
    if (moe_stream_fits(w.max_blocks, 2 * I) && moe_stream_fits(w.max_blocks, H)) {
        const int act = std::is_same<ActT, __half>::value ? EQ_F16 : EQ_BF16;
        int st = moe_stream_launch(static_cast<const unsigned char*>(wq_gate_up), static_cast<size_t>(2 * I / 16) * (H / 128) * kItemBytes, scale_dtype,
                                   x, w.h1, w.src_of, nullptr, nullptr, w.blocks, w.n_blocks, w.max_blocks, H, 2 * I, act, stream);
        if (st != EQ_OK) return st;
        moe_swiglu_kernel<ActT><<<static_cast<unsigned>(ceil_div(R * I, 256)), 256, 0, stream>>>(reinterpret_cast<const ActT*>(w.h1), w.offsets + E,
                                                                                              static_cast<int>(I), reinterpret_cast<ActT*>(w.h));
        EQ_LAUNCH_OK("moe_swiglu_kernel");
        return moe_stream_launch(static_cast<const unsigned char*>(wq_down), static_cast<size_t>(H / 16) * (I / 128) * kItemBytes, scale_dtype, w.h,
                                 out, nullptr, w.dst_of, row_ptr ? w.dst_ptr : nullptr, w.blocks, w.n_blocks, w.max_blocks, I, H, act, stream);
    }
    GroupedParams g1;
    g1.wq = static_cast<const unsigned char*>(wq_gate_up);
    g1.expert_stride = static_cast<size_t>(2 * I / 16) * (H / 128) * kItemBytes;
    g1.x = x;
    g1.y = w.h1;
    g1.x_rows = w.src_of;
    g1.y_rows = nullptr;
    g1.y_ptrs = nullptr;
    g1.blocks = w.blocks;
    g1.n_blocks = w.n_blocks;
    g1.K = static_cast<int>(H);
    g1.N = static_cast<int>(2 * I);
    g1.scale_dtype = scale_dtype;
    int st = launch_grouped<ActT>(g1, br, w.max_blocks, stream);
    if (st != EQ_OK) return st;
    moe_swiglu_kernel<ActT><<<static_cast<unsigned>(ceil_div(R * I, 256)), 256, 0, stream>>>(reinterpret_cast<const ActT*>(w.h1), w.offsets + E,
                                                                                          static_cast<int>(I), reinterpret_cast<ActT*>(w.h));
    EQ_LAUNCH_OK("moe_swiglu_kernel");
    GroupedParams g2 = g1;
    g2.wq = static_cast<const unsigned char*>(wq_down);
    g2.expert_stride = static_cast<size_t>(H / 16) * (I / 128) * kItemBytes;
    g2.x = w.h;
    g2.y = out;
    g2.x_rows = nullptr;
    g2.y_rows = w.dst_of;
    g2.y_ptrs = row_ptr ? w.dst_ptr : nullptr;
    g2.K = static_cast<int>(I);
    g2.N = static_cast<int>(H);
    return launch_grouped<ActT>(g2, br, w.max_blocks, stream);
}


// ------------------------------------------------------------------------------------------------ expert parallel
// Experts sharded E / world per rank; every rank holds T tokens.  The token exchange is done by the kernels themselves
// over peer memory (NVLink): rows are stored straight into the owner's receive buffer IN EXPERT ORDER, so the owner's
// grouped GEMM reads them in place (no row list, no count / scatter / gather pass), the second expert GEMM stores each
// result row straight into the token's rank (per-row destination addresses), and epoch flags written with release /
// read with acquire at system scope order the steps.  No host read, no NCCL call.
//   1. every rank counts its picks per (destination, local expert) and stores that table into EVERY rank's copy of the
//      count tables (a few hundred bytes per peer), then raises flag [0][me] everywhere;
//   2. with all tables in hand every rank knows every destination's layout -- expert e's rows start at the sum of the
//      experts before it, source s's segment inside it at the sum of the sources before it -- so it knows where its
//      own rows go (no second round) and, for its own buffer, the row blocks of the grouped GEMM;
//   3. the dispatch stores each picked row at (its segment's start + the pick's position in the segment) of the
//      owner's buffer, with (source rank, pick index) as the return address; flag [1][me] everywhere;
//   4. grouped FFN over the buffer; the second GEMM's epilogue stores to the sources' `back`; flag [2][me]; combine.
//   rank r's receive buffer: [world * cap rows][H], shared by the sources
//   count tables of rank r: [source][destination][local expert]
//   flags of rank r: [0][s] counts of s arrived, [1][s] rows of s arrived, [2][d] results from d stored into r's `back`
// Waits are bounded (about a second) and report through the status word.
constexpr int kEpOverflow = 32;    // a destination was sent more rows than its receive buffer holds; the excess was dropped
constexpr int kEpWaitReady = 64;   // a peer's rows did not arrive in time
constexpr int kEpWaitDone = 65;    // a peer's results did not arrive in time
constexpr int kEpWaitCounts = 66;  // a peer's count table did not arrive in time
constexpr long long kEpWaitCycles = 2000000000LL;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One thread per pick: its position among this rank's picks for the same (destination, local expert).
__global__ void ep_count_kernel(const int32_t* __restrict__ ids, int picks, int per_rank, int world, int32_t* __restrict__ cnt,
                                int32_t* __restrict__ pos, int32_t* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= picks) return;
    const int id = ids[i];
    if (id < 0 || id >= per_rank * world) {
        atomicExch(status, kBadExpertId);
        pos[i] = -1;
        return;
    }
    pos[i] = atomicAdd(cnt + id, 1);  // id = destination * per_rank + local expert
}

// One CTA: this rank's table [destination][local expert] into every rank's copy, then the flag.
__global__ void ep_publish_counts_kernel(const eq_ep_peers pe, const int32_t* __restrict__ cnt, int per_rank, uint32_t epoch,
                                         const uint32_t* __restrict__ epoch_dev) {
    if (epoch == 0) epoch = *epoch_dev;
    const int entries = pe.world * per_rank;
    for (int d = 0; d < pe.world; ++d) {
        int32_t* dst = pe.recv_count[d] + static_cast<size_t>(pe.rank) * entries;
        for (int i = threadIdx.x; i < entries; i += blockDim.x) dst[i] = cnt[i];
    }
    __threadfence_system();
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < pe.world) st_release_sys(pe.flags[threadIdx.x] + pe.rank, epoch);
}

// which = 0: every source's counts; 1: every source's rows; 2: every destination's results.
__global__ void ep_wait_kernel(const uint32_t* __restrict__ flags, int world, int which, uint32_t epoch, const uint32_t* __restrict__ epoch_dev,
                               int32_t* __restrict__ status) {
    if (static_cast<int>(threadIdx.x) >= world) return;
    if (epoch == 0) epoch = *epoch_dev;
    const uint32_t* f = flags + which * world + threadIdx.x;
    const long long start = clock64();
    while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
        if (clock64() - start > kEpWaitCycles) {
            atomicExch(status, which == 0 ? kEpWaitCounts : which == 1 ? kEpWaitReady : kEpWaitDone);
            return;
        }
    }
}

// One CTA.  From the count tables [source][destination][expert]: where this rank's rows start in every destination's
// buffer (send_base[destination][expert]), and for this rank's own buffer the expert offsets and the grouped GEMM's row
// blocks.  Counts are clamped to what can be true (a table that never arrived is zeros or an older call's), rows beyond a
// buffer's capacity are dropped and reported.  Leaves this rank's own count table zero for the next call.
__global__ void ep_layout_kernel(const eq_ep_peers pe, int per_rank, int block_rows, int max_blocks, int32_t* __restrict__ cnt,
                                 int32_t* __restrict__ send_base, int32_t* __restrict__ offsets, RowBlock* __restrict__ blocks,
                                 int32_t* __restrict__ n_blocks, int32_t* __restrict__ status) {
    extern __shared__ int32_t sh[];  // [world][per_rank] totals per (destination, expert), then starts
    const int world = pe.world, me = pe.rank, entries = world * per_rank;
    const int32_t* tab = pe.recv_count[me];
    const int64_t room = static_cast<int64_t>(world) * pe.cap;
    auto count_of = [&](int s, int de) {
        const int c = tab[static_cast<size_t>(s) * entries + de];
        return c < 0 ? 0 : c > pe.cap ? static_cast<int>(pe.cap) : c;
    };
    for (int de = threadIdx.x; de < entries; de += blockDim.x) {
        int total = 0, before_me = 0;
        for (int s = 0; s < world; ++s) {
            const int c = count_of(s, de);
            if (s < me) before_me += c;
            total += c;
        }
        sh[de] = total;
        send_base[de] = before_me;  // + the expert's start, below
        cnt[de] = 0;
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {  // exclusive scan over the experts of one destination
        const int d = threadIdx.x;
        int64_t run = 0;
        for (int e = 0; e < per_rank; ++e) {
            const int total = sh[d * per_rank + e];
            sh[d * per_rank + e] = static_cast<int>(run < room ? run : room);
            run += total;
        }
        if (run > room) atomicExch(status, kEpOverflow);
        if (d == me) offsets[per_rank] = static_cast<int>(run < room ? run : room);
    }
    __syncthreads();
    for (int de = threadIdx.x; de < entries; de += blockDim.x) send_base[de] += sh[de];
    if (threadIdx.x == 0) {
        int nb = 0;
        const int total_rows = offsets[per_rank];
        for (int e = 0; e < per_rank; ++e) {
            const int start = sh[me * per_rank + e];
            const int end = e + 1 < per_rank ? sh[me * per_rank + e + 1] : total_rows;
            offsets[e] = start;
            for (int r0 = start; r0 < end && nb < max_blocks; r0 += block_rows) {
                blocks[nb].expert = e;
                blocks[nb].row0 = r0;
                blocks[nb].rows = min(block_rows, end - r0);
                blocks[nb].pad = 0;
                ++nb;
            }
        }
        *n_blocks = nb;
    }
}

// One warp per pick: copy the token's row to its place in the owner's buffer and record (source rank, pick index).  The
// last CTA to finish raises this rank's rows-arrived flag at every destination.
__global__ void ep_dispatch_kernel(const eq_ep_peers pe, const uint4* __restrict__ x, const int32_t* __restrict__ ids,
                                   const int32_t* __restrict__ pos, const int32_t* __restrict__ send_base, int picks, int topk, int per_rank,
                                   int row_vec, int32_t* __restrict__ cta_done, uint32_t epoch, const uint32_t* __restrict__ epoch_dev) {
    __shared__ int s_last;
    if (epoch == 0) epoch = *epoch_dev;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp < picks) {
        const int p_in = pos[warp];
        if (p_in >= 0) {
            const int id = ids[warp], dest = id / per_rank;
            const int64_t row = static_cast<int64_t>(send_base[id]) + p_in;
            if (row < static_cast<int64_t>(pe.world) * pe.cap) {  // (the layout kernel reported the overflow)
                uint4* dst = static_cast<uint4*>(pe.recv_x[dest]) + row * row_vec;
                const uint4* src = x + static_cast<size_t>(warp / topk) * row_vec;
                for (int v = lane; v < row_vec; v += 32) dst[v] = src[v];
                if (lane == 0) *reinterpret_cast<int2*>(pe.recv_meta[dest] + 2 * row) = make_int2(pe.rank, warp);
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(cta_done, 1) == static_cast<int>(gridDim.x) - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (static_cast<int>(threadIdx.x) < pe.world) st_release_sys(pe.flags[threadIdx.x] + pe.world + pe.rank, epoch);
    if (threadIdx.x == 0) *cta_done = 0;
}

// Each received row's destination: the pick's row of the source's `back`, as mapped on this rank.
__global__ void ep_row_ptr_kernel(const eq_ep_peers pe, const int32_t* __restrict__ meta, const int32_t* __restrict__ total_rows, size_t row_bytes,
                                  uint64_t* __restrict__ row_ptr) {
    const int total = *total_rows;
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < total; r += gridDim.x * blockDim.x) {
        const int2 m = *reinterpret_cast<const int2*>(meta + 2 * static_cast<size_t>(r));
        row_ptr[r] = (m.x >= 0 && m.x < pe.world && m.y >= 0) ? reinterpret_cast<uint64_t>(static_cast<unsigned char*>(pe.back[m.x]) + static_cast<size_t>(m.y) * row_bytes)
                                                              : 0ull;
    }
}

// The call counter kept on the device (epoch argument 0): every call bumps it once, in lockstep on all ranks, so a
// captured graph of the layer can be replayed.
__global__ void ep_next_epoch_kernel(uint32_t* epoch_dev) { *epoch_dev += 1; }

__global__ void ep_signal_done_kernel(const eq_ep_peers pe, uint32_t epoch, const uint32_t* __restrict__ epoch_dev) {
    if (static_cast<int>(threadIdx.x) >= pe.world) return;
    if (epoch == 0) epoch = *epoch_dev;
    __threadfence_system();
    st_release_sys(pe.flags[threadIdx.x] + 2 * pe.world + pe.rank, epoch);
}

struct EpWorkspace {
    MoeWorkspace moe;
    int32_t *cnt, *send_base, *pos, *cta_done;
    uint32_t* epoch;
    uint64_t* row_ptr;
    RowBlock* blocks;
    int block_rows, max_blocks;  // 8-row blocks through the streaming tier, or 256-row blocks through the tensor tier
    size_t bytes;
};

static EpWorkspace carve_ep(void* base, int64_t world, int64_t cap, int64_t e_local, int64_t H, int64_t I) {
    EpWorkspace w;
    const int64_t R = world * cap;
    w.moe = carve(base, R, e_local, 1, H, I);
    unsigned char* p = static_cast<unsigned char*>(base);
    size_t o = w.moe.bytes;
    auto take = [&](size_t bytes) {
        unsigned char* r = p ? p + o : nullptr;
        o += align_up(bytes, 256);
        return r;
    };
    w.cnt = reinterpret_cast<int32_t*>(take(world * e_local * 4));        // zero between calls
    w.send_base = reinterpret_cast<int32_t*>(take(world * e_local * 4));
    w.pos = reinterpret_cast<int32_t*>(take(R * 4));                      // world * cap >= this rank's picks
    w.cta_done = reinterpret_cast<int32_t*>(take(4));
    w.epoch = reinterpret_cast<uint32_t*>(take(4));
    w.row_ptr = reinterpret_cast<uint64_t*>(take(R * 8));
    // The tier follows the rows a rank expects (about one source's worth: cap), not the buffer's capacity, which is
    // `world` times that; the block list is sized for the capacity.
    const int64_t stream_blocks = R / 8 + e_local + 1;
    const bool stream_tier = stream_rows(cap, e_local) && stream_blocks < (1 << 30) && moe_stream_fits(static_cast<int>(stream_blocks), 2 * I) &&
                             moe_stream_fits(static_cast<int>(stream_blocks), H);
    w.block_rows = stream_tier ? 8 : 256;
    w.max_blocks = static_cast<int>(R / w.block_rows + e_local + 1);
    w.blocks = reinterpret_cast<RowBlock*>(take(sizeof(RowBlock) * w.max_blocks));
    w.bytes = o;
    return w;
}

static int check_moe_shapes(const char* who, int64_t E, int64_t topk, int64_t H, int64_t I, int64_t G) {
    EQ_REQUIRE(E > 0 && E <= 1024 && topk > 0 && topk <= kMaxTopK && topk <= E, EQ_ERR_UNSUPPORTED, "%s: needs 0 < top-k <= 16 and E <= 1024", who);
    if (G == -1) G = 128;
    EQ_REQUIRE(H % 128 == 0 && I % 128 == 0 && G == 128, EQ_ERR_UNSUPPORTED, "%s: needs hidden and intermediate sizes that are multiples of 128 and group 128", who);
    return EQ_OK;
}

}  // namespace eq

using namespace eq;

extern "C" int eq_moe_route(const float* logits, int64_t T, int64_t E, int64_t topk, int renorm, int32_t* ids, float* scores, void* stream) {
    EQ_REQUIRE(T >= 0 && E > 0 && E <= 1024 && topk > 0 && topk <= kMaxTopK && topk <= E, EQ_ERR_UNSUPPORTED,
               "eq_moe_route: needs 0 < top-k <= 16 and E <= 1024");
    if (T == 0) return EQ_OK;
    EQ_REQUIRE(logits && ids && scores, EQ_ERR_BAD_ARG, "eq_moe_route: null pointer");
    moe_route_kernel<<<static_cast<unsigned>(ceil_div(T * 32, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, static_cast<int>(T), static_cast<int>(E), static_cast<int>(topk), renorm, ids, scores);
    EQ_LAUNCH_OK("moe_route_kernel");
    return EQ_OK;
}

extern "C" size_t eq_moe_workspace_bytes(int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I) {
    if (T <= 0 || E <= 0 || topk <= 0 || H <= 0 || I <= 0) return 0;
    return carve(nullptr, T, E, topk, H, I).bytes;
}

extern "C" int eq_moe_experts_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t H, int64_t I, int64_t G,
                                    const void* x, const int32_t* src_row, const int32_t* expert_ids, int64_t R, int act_dtype, void* out,
                                    void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_moe_shapes("eq_moe_experts_w4a16", E, 1, H, I, G);
    if (st != EQ_OK) return st;
    if (R == 0) return EQ_OK;
    EQ_REQUIRE(R > 0 && wq_gate_up && wq_down && x && expert_ids && out, EQ_ERR_BAD_ARG, "eq_moe_experts_w4a16: null pointer or negative row count");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_moe_experts_w4a16: activations must be f16 or bf16");
    EQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= eq_moe_workspace_bytes(R, E, 1, H, I), EQ_ERR_WORKSPACE,
               "eq_moe_experts_w4a16: workspace of %zu bytes (256-byte aligned) needed, %zu given", eq_moe_workspace_bytes(R, E, 1, H, I), workspace_bytes);
    MoeWorkspace w = carve(workspace, R, E, 1, H, I);
    EQ_CUDA_OK(cudaMemsetAsync(w.status, 0, 4, stream));
    if (act_dtype == EQ_F16)
        return experts_forward<__half>(w, wq_gate_up, wq_down, scale_dtype, E, H, I, x, src_row, 0, expert_ids, R, out, nullptr, stream);
    return experts_forward<__nv_bfloat16>(w, wq_gate_up, wq_down, scale_dtype, E, H, I, x, src_row, 0, expert_ids, R, out, nullptr, stream);
}

extern "C" int eq_moe_combine(const void* out_rows, const float* scores, int64_t T, int64_t topk, int64_t H, int act_dtype, void* y, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(T >= 0 && topk > 0 && H > 0, EQ_ERR_BAD_ARG, "eq_moe_combine: bad extents");
    if (T == 0) return EQ_OK;
    EQ_REQUIRE(out_rows && scores && y, EQ_ERR_BAD_ARG, "eq_moe_combine: null pointer");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_moe_combine: activations must be f16 or bf16");
    const int Ti = static_cast<int>(T), ki = static_cast<int>(topk), Hi = static_cast<int>(H);
    if (H % 8 == 0 && aligned(out_rows, 16) && aligned(y, 16)) {
        const unsigned grid = static_cast<unsigned>(ceil_div(T * (H / 8), 256));
        if (act_dtype == EQ_F16)
            moe_combine_vec_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(out_rows), scores, Ti, ki, Hi / 8, static_cast<uint4*>(y));
        else
            moe_combine_vec_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(out_rows), scores, Ti, ki, Hi / 8,
                                                                            static_cast<uint4*>(y));
    } else {
        const unsigned grid = static_cast<unsigned>(ceil_div(T * H, 256));
        if (act_dtype == EQ_F16)
            moe_combine_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(out_rows), scores, Ti, ki, Hi, static_cast<__half*>(y));
        else
            moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out_rows), scores, Ti, ki, Hi,
                                                                        static_cast<__nv_bfloat16*>(y));
    }
    EQ_LAUNCH_OK("moe_combine_kernel");
    return EQ_OK;
}

extern "C" int eq_moe_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t topk, int64_t H, int64_t I, int64_t G,
                            const void* x, const float* router_logits, int64_t T, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                            void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_moe_shapes("eq_moe_w4a16", E, topk, H, I, G);
    if (st != EQ_OK) return st;
    if (T == 0) return EQ_OK;
    EQ_REQUIRE(T > 0 && wq_gate_up && wq_down && x && router_logits && y, EQ_ERR_BAD_ARG, "eq_moe_w4a16: null pointer or negative token count");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_moe_w4a16: activations must be f16 or bf16");
    EQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= eq_moe_workspace_bytes(T, E, topk, H, I), EQ_ERR_WORKSPACE,
               "eq_moe_w4a16: workspace of %zu bytes (256-byte aligned) needed, %zu given", eq_moe_workspace_bytes(T, E, topk, H, I), workspace_bytes);
    MoeWorkspace w = carve(workspace, T, E, topk, H, I);
    const int64_t R = T * topk;
    if (moe_decode_fits(T, E, topk, H, I) && aligned(x, 16))
        // a handful of tokens: router + [gate | up] in one launch, SwiGLU + down + combine in a second one
        return moe_decode_launch(wq_gate_up, wq_down, scale_dtype, E, topk, H, I, x, router_logits, T, act_dtype, y, w.ids, w.scores, w.h1, w.out,
                                 reinterpret_cast<int*>(w.h), w.status, stream);
    EQ_CUDA_OK(cudaMemsetAsync(w.status, 0, 4, stream));
    st = eq_moe_route(router_logits, T, E, topk, 1, w.ids, w.scores, stream_);
    if (st != EQ_OK) return st;
    if (act_dtype == EQ_F16)
        st = experts_forward<__half>(w, wq_gate_up, wq_down, scale_dtype, E, H, I, x, nullptr, static_cast<int>(topk), w.ids, R, w.out, nullptr, stream);
    else
        st = experts_forward<__nv_bfloat16>(w, wq_gate_up, wq_down, scale_dtype, E, H, I, x, nullptr, static_cast<int>(topk), w.ids, R, w.out, nullptr, stream);
    if (st != EQ_OK) return st;
    return eq_moe_combine(w.out, w.scores, T, topk, H, act_dtype, y, stream_);
}

extern "C" int eq_moe_status(const void* workspace, int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && T > 0, EQ_ERR_BAD_ARG, "eq_moe_status: bad arguments");
    MoeWorkspace w = carve(const_cast<void*>(workspace), T, E, topk, H, I);
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, w.status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host != kBadExpertId, EQ_ERR_BAD_ARG, "eq_moe_status: an expert id outside [0, E) was met");
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_moe_status: a bounded pipeline wait of the tensor path ran out (code %d)", host);
    return EQ_OK;
}

extern "C" size_t eq_ep_moe_workspace_bytes(int64_t world, int64_t cap, int64_t E_local, int64_t H, int64_t I) {
    if (world <= 0 || world > EQ_EP_MAX_RANKS || cap <= 0 || E_local <= 0 || H <= 0 || I <= 0) return 0;
    return carve_ep(nullptr, world, cap, E_local, H, I).bytes;
}

extern "C" int eq_ep_moe_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E_local, int64_t topk, int64_t H, int64_t I,
                               int64_t G, const void* x, const int32_t* ids, const float* scores, int64_t T, int act_dtype, void* y,
                               const eq_ep_peers* peers, uint32_t epoch, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(peers && peers->world >= 1 && peers->world <= EQ_EP_MAX_RANKS && peers->rank >= 0 && peers->rank < peers->world && peers->cap > 0,
               EQ_ERR_BAD_ARG, "eq_ep_moe_w4a16: bad peer description");
    const int64_t world = peers->world, cap = peers->cap;
    int st = check_moe_shapes("eq_ep_moe_w4a16", E_local * world, topk, H, I, G);
    if (st != EQ_OK) return st;
    EQ_REQUIRE(T >= 0, EQ_ERR_BAD_ARG, "eq_ep_moe_w4a16: negative token count");
    EQ_REQUIRE(wq_gate_up && wq_down && (T == 0 || (x && ids && scores && y)), EQ_ERR_BAD_ARG, "eq_ep_moe_w4a16: null pointer");
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_ep_moe_w4a16: activations must be f16 or bf16");
    EQ_REQUIRE(T == 0 || aligned(x, 16), EQ_ERR_BAD_ALIGN, "eq_ep_moe_w4a16: x must be 16-byte aligned");
    for (int r = 0; r < world; ++r)
        EQ_REQUIRE(peers->recv_x[r] && peers->recv_meta[r] && peers->recv_count[r] && peers->back[r] && peers->flags[r] &&
                       aligned(peers->recv_x[r], 16) && aligned(peers->back[r], 16) && aligned(peers->recv_meta[r], 8),
                   EQ_ERR_BAD_ARG, "eq_ep_moe_w4a16: peer %d has a null or misaligned buffer", r);
    EQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= eq_ep_moe_workspace_bytes(world, cap, E_local, H, I), EQ_ERR_WORKSPACE,
               "eq_ep_moe_w4a16: workspace of %zu bytes (256-byte aligned, zero on first use) needed, %zu given",
               eq_ep_moe_workspace_bytes(world, cap, E_local, H, I), workspace_bytes);
    EpWorkspace w = carve_ep(workspace, world, cap, E_local, H, I);
    const int me = peers->rank;
    const int64_t picks = T * topk, R = world * cap;
    EQ_REQUIRE(picks <= R, EQ_ERR_UNSUPPORTED, "eq_ep_moe_w4a16: %lld picks exceed the %lld rows the buffers were made for", (long long)picks,
               (long long)R);
    const int row_vec = static_cast<int>(H * 2 / 16);
    const int per_rank = static_cast<int>(E_local);
    EQ_CUDA_OK(cudaMemsetAsync(w.moe.status, 0, 4, stream));
    if (epoch == 0) {
        ep_next_epoch_kernel<<<1, 1, 0, stream>>>(w.epoch);
        EQ_LAUNCH_OK("ep_next_epoch_kernel");
    }
    // 1. this rank's counts per (destination, expert), published to every rank (with or without tokens of its own)
    if (picks > 0) {
        ep_count_kernel<<<static_cast<unsigned>(ceil_div(picks, 256)), 256, 0, stream>>>(ids, static_cast<int>(picks), per_rank, static_cast<int>(world),
                                                                                         w.cnt, w.pos, w.moe.status);
        EQ_LAUNCH_OK("ep_count_kernel");
    }
    ep_publish_counts_kernel<<<1, 256, 0, stream>>>(*peers, w.cnt, per_rank, epoch, w.epoch);
    EQ_LAUNCH_OK("ep_publish_counts_kernel");
    ep_wait_kernel<<<1, 32, 0, stream>>>(peers->flags[me], static_cast<int>(world), 0, epoch, w.epoch, w.moe.status);
    EQ_LAUNCH_OK("ep_wait_kernel");
    // 2. every destination's layout; this rank's row blocks
    const bool stream_tier = w.block_rows == 8;
    const int br = w.block_rows;
    ep_layout_kernel<<<1, 256, world * per_rank * sizeof(int32_t), stream>>>(*peers, per_rank, br, w.max_blocks, w.cnt, w.send_base, w.moe.offsets,
                                                                           w.blocks, w.moe.n_blocks, w.moe.status);
    EQ_LAUNCH_OK("ep_layout_kernel");
    // 3. rows to their owners, in expert order
    const unsigned dgrid = static_cast<unsigned>(picks > 0 ? ceil_div(picks * 32, 256) : 1);
    ep_dispatch_kernel<<<dgrid, 256, 0, stream>>>(*peers, static_cast<const uint4*>(x), ids, w.pos, w.send_base, static_cast<int>(picks),
                                                  static_cast<int>(topk), per_rank, row_vec, w.cta_done, epoch, w.epoch);
    EQ_LAUNCH_OK("ep_dispatch_kernel");
    ep_wait_kernel<<<1, 32, 0, stream>>>(peers->flags[me], static_cast<int>(world), 1, epoch, w.epoch, w.moe.status);
    EQ_LAUNCH_OK("ep_wait_kernel");
    ep_row_ptr_kernel<<<static_cast<unsigned>(4 * sm_count()), 256, 0, stream>>>(*peers, peers->recv_meta[me], w.moe.offsets + E_local,
                                                                                 static_cast<size_t>(H) * 2, w.row_ptr);
    EQ_LAUNCH_OK("ep_row_ptr_kernel");
    // 4. the grouped FFN over the buffer as it lies; results straight to the tokens' ranks
    const size_t stride_gu = static_cast<size_t>(2 * I / 16) * (H / 128) * kItemBytes, stride_dn = static_cast<size_t>(H / 16) * (I / 128) * kItemBytes;
    const unsigned char* gu = static_cast<const unsigned char*>(wq_gate_up);
    const unsigned char* dn = static_cast<const unsigned char*>(wq_down);
    if (stream_tier) {
        st = moe_stream_launch(gu, stride_gu, scale_dtype, peers->recv_x[me], w.moe.h1, nullptr, nullptr, nullptr, w.blocks, w.moe.n_blocks,
                               w.max_blocks, H, 2 * I, act_dtype, stream);
        if (st != EQ_OK) return st;
        const unsigned sgrid = static_cast<unsigned>(ceil_div(R * I, 256));
        if (act_dtype == EQ_F16)
            moe_swiglu_kernel<__half><<<sgrid, 256, 0, stream>>>(reinterpret_cast<const __half*>(w.moe.h1), w.moe.offsets + E_local, static_cast<int>(I),
                                                                 reinterpret_cast<__half*>(w.moe.h));
        else
            moe_swiglu_kernel<__nv_bfloat16><<<sgrid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w.moe.h1), w.moe.offsets + E_local,
                                                                        static_cast<int>(I), reinterpret_cast<__nv_bfloat16*>(w.moe.h));
        EQ_LAUNCH_OK("moe_swiglu_kernel");
        st = moe_stream_launch(dn, stride_dn, scale_dtype, w.moe.h, nullptr, nullptr, nullptr, w.row_ptr, w.blocks, w.moe.n_blocks, w.max_blocks, I, H,
                               act_dtype, stream);
    } else {
        EQ_REQUIRE(aligned(peers->recv_x[me], 16), EQ_ERR_BAD_ALIGN, "eq_ep_moe_w4a16: the receive buffer must be 16-byte aligned");
        st = w4_gemm_tc_grouped_launch(gu, stride_gu, scale_dtype, peers->recv_x[me], w.moe.h, R, 2 * I, H, act_dtype, w.blocks, w.moe.n_blocks,
                                       w.max_blocks, nullptr, nullptr, true, w.moe.status, stream);
        if (st != EQ_OK) return st;
        st = w4_gemm_tc_grouped_launch(dn, stride_dn, scale_dtype, w.moe.h, nullptr, R, H, I, act_dtype, w.blocks, w.moe.n_blocks, w.max_blocks,
                                       nullptr, w.row_ptr, false, w.moe.status, stream);
    }
    if (st != EQ_OK) return st;
    ep_signal_done_kernel<<<1, 32, 0, stream>>>(*peers, epoch, w.epoch);
    EQ_LAUNCH_OK("ep_signal_done_kernel");
    ep_wait_kernel<<<1, 32, 0, stream>>>(peers->flags[me], static_cast<int>(world), 2, epoch, w.epoch, w.moe.status);
    EQ_LAUNCH_OK("ep_wait_kernel");
    if (T == 0) return EQ_OK;
    return eq_moe_combine(peers->back[me], scores, T, topk, H, act_dtype, y, stream_);
}

extern "C" int eq_ep_moe_status(const void* workspace, int64_t world, int64_t cap, int64_t E_local, int64_t H, int64_t I, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && world > 0 && world <= EQ_EP_MAX_RANKS && cap > 0, EQ_ERR_BAD_ARG, "eq_ep_moe_status: bad arguments");
    EpWorkspace w = carve_ep(const_cast<void*>(workspace), world, cap, E_local, H, I);
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, w.moe.status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host != kBadExpertId, EQ_ERR_BAD_ARG, "eq_ep_moe_status: an expert id out of range was met");
    EQ_REQUIRE(host != kEpOverflow, EQ_ERR_UNSUPPORTED, "eq_ep_moe_status: a rank was sent more rows than its receive buffer holds; rows were dropped");
    EQ_REQUIRE(host != kEpWaitReady && host != kEpWaitDone && host != kEpWaitCounts, EQ_ERR_TIMEOUT,
               "eq_ep_moe_status: a peer's %s did not arrive within the wait bound", host == kEpWaitCounts ? "counts" : host == kEpWaitReady ? "rows" : "results");
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_ep_moe_status: a bounded pipeline wait of the tensor path ran out (code %d)", host);
    return EQ_OK;
}
