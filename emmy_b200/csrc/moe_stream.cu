// Grouped expert linear for a few rows per expert (the MoE layer between the decode tier and the tensor tier).
//
// With some tens of tokens every expert is touched by a handful of rows: the layer has to stream ALL expert weights
// (300 MB for a Qwen3-30B-A3B layer) for very little math, which is the multi-row streaming kernel's job (w4_stream.cu),
// not the tensor path's (one 256-row block per expert pays the whole dequantize pipeline for four rows).  The row
// blocks of the plan (at most eight rows of one expert) are laid end to end as one stream of column tiles,
//     virtual tile v = block * (N / 16) + tile,
// cut into equal whole-tile spans, one per CTA (one 16-warp CTA per SM); the number of blocks is known only on the
// device, so every CTA derives its span from it.  Inside a CTA the warps take equal contiguous shares of the span's
// items, keep a ring of items in flight with cp.async, and add into per-tile shared accumulators when they leave a tile,
// exactly as in w4_stream.cu; a tile's weights are found through its block's expert id, its activation rows through the
// plan's gather index (read from global memory one item ahead of the weights), its output rows through the plan's
// scatter index or per-row addresses.
#include "w4_tile.cuh"

namespace eq {

namespace {

constexpr int kMsWarps = 16;
constexpr int kMsSlot = kItemBytes;
constexpr int kMsRows = 8;  // rows per block (one MMA row block)

struct MoeStreamParams {
    const unsigned char* wq;  // [E][N / 16][items][1088]
    size_t expert_stride;
    const void* x;            // rows addressed through x_rows, or contiguous in plan order
    void* y;
    const int32_t* x_rows;    // optional [R] gather index in plan order
    const int32_t* y_rows;    // optional [R] scatter index in plan order
    const uint64_t* y_ptrs;   // optional [R] destination address of each row (overrides y / y_rows)
    const RowBlock* blocks;
    const int32_t* n_blocks;
    int K, N, items, tpe;     // tpe: column tiles per expert
    int scale_dtype;
    int acc_tiles;            // accumulator slots per CTA (the host's bound on tiles per CTA)
};

template <typename ActT, int DEPTH>
__global__ void __launch_bounds__(kMsWarps * 32, 1) moe_stream_kernel(const MoeStreamParams gp) {
    extern __shared__ __align__(16) unsigned char smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int items = gp.items, tpe = gp.tpe;
    // this CTA's whole tiles of the blocks' tile stream
    const long long total = static_cast<long long>(*gp.n_blocks) * tpe;
    const int ctas = gridDim.x, cta = blockIdx.x;
    const int base = static_cast<int>(total / ctas), rem = static_cast<int>(total % ctas);
    const int tile0 = cta * base + min(cta, rem);
    const int ntiles = min(base + (cta < rem ? 1 : 0), gp.acc_tiles);  // (the host sized acc_tiles for the largest plan)
    if (ntiles == 0) return;

    float* acc_s = reinterpret_cast<float*>(smem_all + kMsWarps * DEPTH * kMsSlot);  // [ntiles][8][16]
    for (int i = threadIdx.x; i < ntiles * kMsRows * 16; i += kMsWarps * 32) acc_s[i] = 0.f;

    const int cta_items = ntiles * items;
    const int q0 = static_cast<int>(static_cast<long long>(cta_items) * warp / kMsWarps);
    const int q1 = static_cast<int>(static_cast<long long>(cta_items) * (warp + 1) / kMsWarps);
    const int n = q1 - q0;
    int slot_t = q0 / items;         // tile inside the CTA
    int it = q0 - slot_t * items;    // item inside the tile

    auto tile_base = [&](int rel) {  // first record of the CTA's tile `rel`
        const int v = tile0 + rel;
        const int b = v / tpe;
        return gp.wq + static_cast<size_t>(gp.blocks[b].expert) * gp.expert_stride + static_cast<size_t>(v - b * tpe) * items * kItemBytes;
    };

    // ---- ring of DEPTH items per warp; every lane copies the bytes it reads itself (see w4_stream.cu)
    unsigned char* ring = smem_all + warp * (DEPTH * kMsSlot);
    const uint32_t ring_lo = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + lane * 16;
    const uint32_t ring_meta = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + 1024 + g * 8;
    int issue_left = n, issue_tile = slot_t, issue_room = items - it;
    const unsigned char* src = n > 0 ? tile_base(issue_tile) + static_cast<size_t>(it) * kItemBytes : gp.wq;
    auto issue = [&](int d) {
        if (issue_left > 0) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kMsSlot), "l"(src + lane * 16) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lo + d * kMsSlot + 512), "l"(src + 512 + lane * 16) : "memory");
            if (j == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ring_meta + d * kMsSlot), "l"(src + 1024 + g * 8) : "memory");
            --issue_left;
            src += kItemBytes;
            if (--issue_room == 0 && issue_left > 0) {  // the next item opens a new tile, possibly another expert's
                ++issue_tile;
                issue_room = items;
                src = tile_base(issue_tile);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) issue(d);
    __syncthreads();  // accumulators are zero

    // ---- the row block of the tile the warp is in: its row count, and the lane's own row of x (MMA operand row g, the
    //      32 input positions from 32 j on of every item), found once per block instead of once per item
    W4Params p;
    p.scale_dtype = gp.scale_dtype;
    int rows = 0, cur_block = -1;
    const uint4* xlane = nullptr;  // null: the block has no row g
    auto enter_tile = [&](int rel) {
        const int b = (tile0 + rel) / tpe;
        if (b == cur_block) return;
        cur_block = b;
        const RowBlock rb = gp.blocks[b];
        rows = rb.rows;
        xlane = nullptr;
        if (g < rb.rows) {
            const size_t xr = gp.x_rows ? static_cast<size_t>(gp.x_rows[rb.row0 + g]) : static_cast<size_t>(rb.row0 + g);
            xlane = reinterpret_cast<const uint4*>(static_cast<const ActT*>(gp.x) + xr * gp.K + 32 * j);
        }
    };
    auto item_x = [&](int item, uint4 (&v)[1][4]) {
        if (xlane) {
            const uint4* src = xlane + item * 16;  // 128 activations per item
#pragma unroll
            for (int c = 0; c < 4; ++c) v[0][c] = __ldg(src + c);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) v[0][c] = make_uint4(0, 0, 0, 0);
        }
    };

    float yacc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
    uint4 xv[1][4];
    if (n > 0) {
        enter_tile(slot_t);
        item_x(it, xv);
    }
    int d = 0;  // ring slot of item i
#pragma unroll 2
    for (int i = 0; i < n; ++i) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
        __syncwarp();  // the scale / zero entry was copied by another lane of the column pair
        const unsigned char* slot = ring + d * kMsSlot;
        const uint4 wl = *reinterpret_cast<const uint4*>(slot + lane * 16);
        const uint4 wh = *reinterpret_cast<const uint4*>(slot + 512 + lane * 16);
        const uint2 meta = *reinterpret_cast<const uint2*>(slot + 1024 + g * 8);
        __syncwarp();  // every lane has read the slot before any lane refills it
        issue(d);
        d = d + 1 == DEPTH ? 0 : d + 1;
        const bool leaves = it + 1 == items;
        uint4 xn[1][4];
        if (!leaves && i + 1 < n) item_x(it + 1, xn);  // the rows run one item ahead
        w4_item_math<ActT, 1>(p, xv, wl, wh, meta, yacc);
        if (leaves) {
            // the span leaves this tile: add the sums into the CTA's accumulators, move to the next tile's problem
            float* acc = acc_s + slot_t * kMsRows * 16;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = 2 * j + (e & 1), nn = g + ((e & 2) ? 8 : 0);
                if (m < rows) atomicAdd(acc + m * 16 + nn, yacc[0][e]);
                yacc[0][e] = 0.f;
            }
            it = 0;
            ++slot_t;
            if (i + 1 < n) {
                enter_tile(slot_t);
                item_x(0, xv);
            }
        } else {
            ++it;
#pragma unroll
            for (int v = 0; v < 4; ++v) xv[0][v] = xn[0][v];
        }
    }
    if (it > 0) {  // the span ended inside a tile
        float* acc = acc_s + slot_t * kMsRows * 16;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = 2 * j + (e & 1), nn = g + ((e & 2) ? 8 : 0);
            if (m < rows) atomicAdd(acc + m * 16 + nn, yacc[0][e]);
        }
    }
    __syncthreads();
    // ---- the CTA owns its tiles outright: convert and store, row by row of each tile's block
    for (int idx = threadIdx.x; idx < ntiles * kMsRows * 16; idx += kMsWarps * 32) {
        const int t = idx / (kMsRows * 16), r = idx - t * (kMsRows * 16);
        const int m = r >> 4, nn = r & 15;
        const int v = tile0 + t, b = v / tpe;
        const RowBlock rb = gp.blocks[b];
        if (m >= rb.rows) continue;
        const int col = (v - b * tpe) * 16 + nn;
        const ActT val = from_float<ActT>(acc_s[idx]);
        const int row = rb.row0 + m;
        if (gp.y_ptrs) {
            const uint64_t dst = gp.y_ptrs[row];
            if (dst) reinterpret_cast<ActT*>(dst)[col] = val;
        } else {
            const size_t yr = gp.y_rows ? static_cast<size_t>(gp.y_rows[row]) : static_cast<size_t>(row);
            static_cast<ActT*>(gp.y)[yr * gp.N + col] = val;
        }
    }
}

size_t ms_smem(int depth, int acc_tiles) {
    return static_cast<size_t>(kMsWarps) * depth * kMsSlot + static_cast<size_t>(acc_tiles) * kMsRows * 16 * sizeof(float);
}

template <typename ActT, int DEPTH>
int launch_depth(const MoeStreamParams& gp, size_t smem, int ctas, cudaStream_t stream) {
    auto kernel = moe_stream_kernel<ActT, DEPTH>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    kernel<<<ctas, kMsWarps * 32, smem, stream>>>(gp);
    EQ_LAUNCH_OK("moe_stream_kernel");
    return EQ_OK;
}

}  // namespace

// Whether the streaming tier can serve a plan of at most `max_blocks` row blocks: every CTA's accumulators must fit.
bool moe_stream_fits(int max_blocks, int64_t N) {
    const long long ctas = sm_count();
    const long long per_cta = ceil_div(static_cast<long long>(max_blocks) * (N / 16), ctas);
    return N % 16 == 0 && ms_smem(4, static_cast<int>(per_cta)) <= 220 * 1024;
}

// One grouped linear over the plan's row blocks (at most eight rows each).  Gather / scatter indices and per-row
// destinations as in the tile tier.
int moe_stream_launch(const unsigned char* wq, size_t expert_stride, int scale_dtype, const void* x, void* y, const int32_t* x_rows,
                      const int32_t* y_rows, const uint64_t* y_ptrs, const RowBlock* blocks, const int32_t* n_blocks, int max_blocks, int64_t K,
                      int64_t N, int act_dtype, cudaStream_t stream) {
    MoeStreamParams gp;
    gp.wq = wq;
    gp.expert_stride = expert_stride;
    gp.x = x;
    gp.y = y;
    gp.x_rows = x_rows;
    gp.y_rows = y_rows;
    gp.y_ptrs = y_ptrs;
    gp.blocks = blocks;
    gp.n_blocks = n_blocks;
    gp.K = static_cast<int>(K);
    gp.N = static_cast<int>(N);
    gp.items = static_cast<int>(K / 128);
    gp.tpe = static_cast<int>(N / 16);
    gp.scale_dtype = scale_dtype;
    const int ctas = sm_count();
    gp.acc_tiles = static_cast<int>(ceil_div(static_cast<long long>(max_blocks) * gp.tpe, static_cast<long long>(ctas)));
    const bool f16 = act_dtype == EQ_F16;
    if (const size_t smem = ms_smem(6, gp.acc_tiles); smem <= 220 * 1024)
        return f16 ? launch_depth<__half, 6>(gp, smem, ctas, stream) : launch_depth<__nv_bfloat16, 6>(gp, smem, ctas, stream);
    const size_t smem = ms_smem(4, gp.acc_tiles);
    return f16 ? launch_depth<__half, 4>(gp, smem, ctas, stream) : launch_depth<__nv_bfloat16, 4>(gp, smem, ctas, stream);
}

}  // namespace eq
