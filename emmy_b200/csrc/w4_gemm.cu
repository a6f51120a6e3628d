// W4A16 linear for prefill-shaped calls (M > 16): y[M,N] = x[M,K] @ W on the tcgen05 tensor cores.
//
// The int4 weight never exists as a 16-bit matrix in global memory.  A CTA owns a tile of 128 or 256 activation
// rows by BN output columns and walks K in steps of 64:
//   warp 0        TMA producer: the 64-wide slice of the x rows, 128-byte swizzle, into the stage's A tile
//   warp 1        MMA issuer: tcgen05.mma kind::f16, 128 x BN x 16 per instruction, f32 accumulators in TMEM (one
//                 accumulator per 128 activation rows; both read the same B tile)
//   warps 2..     dequant producers, then the epilogue.  A producer warp reads the packed nibbles of one 16-column
//                 weight tile straight from global memory into registers (one 16-byte load per lane and K step,
//                 issued kAhead steps early), expands them exactly as the decode kernel does (lop3 to 1024 + q, one
//                 subtract / fma removes 1024 and the zero point), multiplies by the group scale in the activation
//                 dtype, which is the value the reference's dequantize-then-matmul path feeds its matmul
//                 (emmy/compiler/loader/quant.py:402-470), and writes the stage's B tile in the same 128-byte-swizzled
//                 K-major layout TMA would have produced.  fence.proxy.async makes the writes visible to the tensor
//                 core; one arrive per warp completes the stage.
// The repack (w4_repack.cu) deals the 128 input rows of an item to lanes so that a lane's four words of one half-tile
// hold, for columns g and g + 8, two runs of eight consecutive rows: exactly two 16-byte chunks of a swizzled row per
// column.  Lanes (g, h, jj) of a warp take the pieces of rows 64 t + 32 jj + 8 h (+16) of K step t of the item, so one
// K step of the MMA is 64 consecutive input rows and x needs no reordering.  Act-order weights (a row permutation)
// gather the columns of x into the workspace first.
#include "tc_common.cuh"
#include "w4_tile.cuh"

namespace eq {

namespace {

constexpr int kGK = 64;             // K per stage: 128 bytes of 16-bit elements
constexpr int kRowBytes = 128;

// HALVES: 128-row activation blocks per CTA; BN: output columns per CTA; DW: dequant (and epilogue) warps;
// AHEAD: items (two K steps each) whose packed bytes are in a warp's registers ahead of use.
template <int HALVES, int BN, int DW, int AHEAD>
struct GemmCfg {
    static constexpr int kDequantWarps = DW;
    static constexpr int kAhead = AHEAD;
    static constexpr int kQuartets = DW / 4;                  // epilogue warp quartets (one warp per TMEM lane quarter)
    static constexpr int kBoxHalves = HALVES == 2 ? 2 : 1;    // 128-row halves per TMA copy of the activation tile
    // With more dequant warps than 16-column tiles the warps also split K: group r of them takes K step r of every item.
    static constexpr int kTiles = BN / 16;
    static constexpr int kKSplit = DW > kTiles ? DW / kTiles : 1;
    static constexpr int kWarpsPerStep = DW / kKSplit;          // warps that fill (and arrive on) one stage
    static constexpr int kTilesPerWarp = kTiles / kWarpsPerStep;
    static constexpr int kThreads = 64 + 32 * kDequantWarps;
    static constexpr int kTileA = HALVES * 128 * kRowBytes;
    static constexpr int kTileB = BN * kRowBytes;
    static constexpr int kStageBytes = kTileA + kTileB;
    static constexpr int kStages = (196608 / kStageBytes) < 4 ? (196608 / kStageBytes) : 4;
    static constexpr size_t kSmem = static_cast<size_t>(kStages) * kStageBytes + 1024 + 256;
    static constexpr uint32_t kAccCols = HALVES * BN;
    static constexpr uint32_t kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
    static_assert(kTilesPerWarp >= 1 && kTilesPerWarp * kWarpsPerStep == kTiles && (kKSplit == 1 || kKSplit == 2),
                  "every dequant warp needs whole weight tiles, and an item has two K steps to split");
    static_assert(DW % 4 == 0 && BN % 64 == 0, "the epilogue works in warp quartets on 32-column chunks");
    static_assert(kAccCols <= 512, "the accumulators must fit TMEM");
};


// 8-byte read-only load that stays where it is written (issued kAhead steps before its use).
__device__ __forceinline__ uint2 ld_pinned_v2(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename ActT>
struct ScaleMul;
template <>
struct ScaleMul<__half> {
    static constexpr uint32_t kFmt = 0;
    // raw scale bits -> the same value twice in the activation dtype; CVT: the scales are stored in the other 16-bit type
    template <bool CVT>
    static __device__ __forceinline__ uint32_t pair(uint32_t raw) {
        if constexpr (CVT) raw = __half_as_ushort(__float2half_rn(__uint_as_float(raw << 16)));
        return __byte_perm(raw, 0, 0x1010);
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t v, uint32_t s) {
        uint32_t r;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(s));
        return r;
    }
};
template <>
struct ScaleMul<__nv_bfloat16> {
    static constexpr uint32_t kFmt = 1;
    template <bool CVT>
    static __device__ __forceinline__ uint32_t pair(uint32_t raw) {
        if constexpr (CVT) raw = __bfloat16_as_ushort(__float2bfloat16_rn(__half2float(__ushort_as_half(static_cast<unsigned short>(raw)))));
        return __byte_perm(raw, 0, 0x1010);
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t v, uint32_t s) {
        uint32_t r;
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(s));
        return r;
    }
};

// xg[m][k'] = x[m][perm[k']]
template <typename ActT>
__global__ void gather_cols_kernel(const ActT* __restrict__ x, const int32_t* __restrict__ perm, int64_t M, int64_t K,
                                   ActT* __restrict__ xg) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= M * K) return;
    const int64_t m = idx / K, k = idx - m * K;
    xg[idx] = x[m * K + perm[k]];
}

// Rows of the TMA box of the activation tile for single-half plain tiles: the row count rounded up to a swizzle atom.
__host__ __device__ inline int a_box_rows(int M) { return M >= 121 ? 128 : (M + 7) / 8 * 8; }

// MODE: kPlain: one weight, CTA row tile = blockIdx.y.  kGrouped: blockIdx.y walks a device-side list of row blocks, each
// a run of rows of ONE expert in an expert-ordered activation matrix; the weight is that expert's slice of a stacked
// tensor and output rows may be scattered through y_rows.  kGroupedSwiGLU: the same, with the first 128 columns of the
// CTA's B tile taken from the gate half and the last 128 from the up half of a [gate | up] weight, and the epilogue
// writing act(silu(gate)) * up (emmy/compiler/trace/huggingface.py:1663-1669) into a matrix of N / 2 columns.
enum GemmMode { kPlain = 0, kGrouped = 1, kGroupedSwiGLU = 2 };

struct GroupArgs {
    const RowBlock* blocks;
    const int32_t* n_blocks;
    const int32_t* y_rows;   // optional: output row m goes to row y_rows[m]
    const uint64_t* y_ptrs;  // optional: output row m starts at address y_ptrs[m] (0 = drop the row); may be a peer GPU's memory
    size_t expert_stride;    // bytes between the experts' repacked weights
};

// SPLIT (plain mode only): gridDim.z CTAs share one output tile, each contracting a run of whole items of K.  Partial
// sums meet in an f32 scratch [M][N] by vector reductions; the CTA whose arrival completes the tile converts it, stores y
// and leaves scratch and counter zero.  Nobody waits.
struct SplitArgs {
    float* partial;     // [M][N], zero between calls
    int* counters;      // one per column tile of this kernel, zero between calls
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename ActT, int HALVES, int BN, int DW, int AHEAD, bool CVT, int MODE, bool SPLIT = false>
__global__ void __launch_bounds__(GemmCfg<HALVES, BN, DW, AHEAD>::kThreads)
    w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const unsigned char* __restrict__ wq, ActT* __restrict__ y,
                         int M, int N, int K, int* __restrict__ status, const GroupArgs grp, const SplitArgs split) {
    using Cfg = GemmCfg<HALVES, BN, DW, AHEAD>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kAhead = Cfg::kAhead;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* tiles_a = smem;
    unsigned char* tiles_b = smem + kStages * Cfg::kTileA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
    uint64_t* full_a = bars;                  // [kStages] TMA -> MMA
    uint64_t* full_b = bars + kStages;        // [kStages] dequant warps -> MMA
    uint64_t* empty = bars + 2 * kStages;     // [kStages] MMA -> producers
    uint64_t* acc_ready = bars + 3 * kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 1);

    // Plain launches are programmatic dependents (launch_cfg): the next grid may start its prologue and its first weight
    // loads while this one runs, and this one does the same behind its predecessor.  Weights never depend on the
    // previous grid; x, y and the split-K scratch may, so the warps that touch them wait below.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    int m0 = blockIdx.y * (128 * HALVES), m_end = M;
    if constexpr (MODE != kPlain) {
        if (static_cast<int>(blockIdx.y) >= *grp.n_blocks) return;  // the whole CTA, before any barrier exists
        const RowBlock rb = grp.blocks[blockIdx.y];
        m0 = rb.row0;
        m_end = rb.row0 + rb.rows;
        wq += static_cast<size_t>(rb.expert) * grp.expert_stride;
    }
    const int items = K / 128;
    // this CTA's run of items (all of K unless SPLIT), in K steps of 64
    int item_lo = 0, item_hi = items;
    if constexpr (SPLIT) {
        item_lo = static_cast<int>(static_cast<long long>(items) * blockIdx.z / gridDim.z);
        item_hi = static_cast<int>(static_cast<long long>(items) * (blockIdx.z + 1) / gridDim.z);
    }
    const int kb_lo = 2 * item_lo;
    const int k_blocks = 2 * (item_hi - item_lo);
    const int live_halves = min(HALVES, (m_end - m0 + 127) / 128);  // 128-row blocks of this tile that hold rows

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(tc::smem_u32(full_a + s), 1);
            tc::mbar_init(tc::smem_u32(full_b + s), Cfg::kWarpsPerStep);
            tc::mbar_init(tc::smem_u32(empty + s), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_ready), 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(tmem_slot), Cfg::kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // shared-window addresses, computed once: barrier s of a ring sits 8 s bytes on
    const uint32_t full_a_addr = tc::smem_u32(full_a), full_b_addr = tc::smem_u32(full_b), empty_addr = tc::smem_u32(empty);
    const uint32_t a_base = tc::smem_u32(tiles_a), b_base = tc::smem_u32(tiles_b);

    if (warp == 0) {
        // ---- TMA producer of the activation tiles
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&map_x);
            asm volatile("griddepcontrol.wait;" ::: "memory");  // x may be the previous grid's output
            int stage = 0;
            uint32_t phase = 0;
            bool first = true;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!first && !tc::mbar_wait(empty_addr + 8 * stage, phase ^ 1)) {
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t bar = full_a_addr + 8 * stage;
                // one copy per TMA box (Cfg::kBoxHalves 128-row halves); halves without rows are not fetched
                constexpr int kBoxBytes = Cfg::kBoxHalves * 128 * kRowBytes;
                const int boxes = (live_halves + Cfg::kBoxHalves - 1) / Cfg::kBoxHalves;
                // single-half plain tiles of fewer than 128 rows use a shorter box (see a_box_rows): rows past it keep
                // whatever the stage held, and the accumulator rows they feed are never stored
                const int box_bytes = (HALVES == 1 && MODE == kPlain) ? a_box_rows(M) * kRowBytes : kBoxBytes;
                tc::mbar_expect_tx(bar, boxes * box_bytes);
                for (int bx = 0; bx < boxes; ++bx)
                    tc::tma_load_2d(a_base + stage * Cfg::kTileA + bx * kBoxBytes, &map_x, (kb_lo + kb) * kGK, m0 + 128 * Cfg::kBoxHalves * bx, bar);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                    first = false;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc(ScaleMul<ActT>::kFmt, ScaleMul<ActT>::kFmt, 128, BN);
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < k_blocks; ++kb) {
                const bool got_a = tc::mbar_wait(full_a_addr + 8 * stage, phase);
                const bool got_b = got_a && tc::mbar_wait(full_b_addr + 8 * stage, phase);
                if (!got_b) {
                    atomicExch(status, 2);
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a_addr = a_base + stage * Cfg::kTileA, b_addr = b_base + stage * Cfg::kTileB;
#pragma unroll
                for (int ks = 0; ks < kGK / 16; ++ks) {
                    const uint64_t db = tc::smem_desc_k_sw128(b_addr + ks * 32);
#pragma unroll
                    for (int hh = 0; hh < HALVES; ++hh)
                        if (hh < live_halves)
                            tc::mma_f16(tmem_base + hh * BN, tc::smem_desc_k_sw128(a_addr + hh * 128 * kRowBytes + ks * 32), db, idesc, kb > 0 || ks > 0);
                }
                tc::mma_commit(empty_addr + 8 * stage);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            tc::mma_commit(tc::smem_u32(acc_ready));  // on a broken pipeline too: the epilogue must not sit out its wait
        }
    } else {
        // ---- dequant producers
        const int dw = warp - 2;
        const int kgrp = dw / Cfg::kWarpsPerStep;  // which K step of an item this warp fills when the warps split K
        const int g = lane & 7, h = (lane >> 3) & 1, jj = lane >> 4;
        // Shared-memory byte offsets of the lane's four 16-byte chunks inside a B tile: row r = 16 tile + g (+8) is an
        // output column, chunk q = 4 jj + 2 high + h of its 128 bytes is swizzled with r & 7 = g.
        const unsigned char* wp[Cfg::kTilesPerWarp];   // the lane's 16 bytes of K step 0 of item 0; K step 1 is 32 bytes on
        const unsigned char* mp[Cfg::kTilesPerWarp];   // its scale / zero record of item 0
        uint32_t off_lo[Cfg::kTilesPerWarp];
        bool live[Cfg::kTilesPerWarp];
#pragma unroll
        for (int nt = 0; nt < Cfg::kTilesPerWarp; ++nt) {
            const int tile_in_cta = (dw % Cfg::kWarpsPerStep) * Cfg::kTilesPerWarp + nt;
            int tile = n0 / 16 + tile_in_cta;
            if constexpr (MODE == kGroupedSwiGLU) {
                constexpr int kHalfTiles = BN / 32;  // gate tiles of this CTA, then as many up tiles
                const int col_tile = n0 / 32 + (tile_in_cta % kHalfTiles);
                tile = col_tile < N / 32 ? col_tile + (tile_in_cta / kHalfTiles) * (N / 32) : N / 16;
            }
            live[nt] = tile < N / 16;
            const unsigned char* rec = wq + static_cast<size_t>(live[nt] ? tile : 0) * items * kItemBytes;
            wp[nt] = rec + static_cast<size_t>(item_lo) * kItemBytes + h * 512 + (4 * g + jj) * 16;
            mp[nt] = rec + static_cast<size_t>(item_lo) * kItemBytes + 1024 + g * 8;
            off_lo[nt] = static_cast<uint32_t>((tile_in_cta * 16 + g) * kRowBytes + (((4 * jj + h) ^ g) << 4));
        }
        // register ring of whole items (two K steps each)
        uint4 w0[kAhead][Cfg::kTilesPerWarp], w1[kAhead][Cfg::kTilesPerWarp];
        uint2 meta[kAhead][Cfg::kTilesPerWarp];
        const int my_items = item_hi - item_lo;
#pragma unroll
        for (int d = 0; d < kAhead; ++d) {
            if (d < my_items) {
#pragma unroll
                for (int nt = 0; nt < Cfg::kTilesPerWarp; ++nt) {
                    if (Cfg::kKSplit == 1 || kgrp == 0) w0[d][nt] = ld_stream_v4(wp[nt] + static_cast<size_t>(d) * kItemBytes);
                    if (Cfg::kKSplit == 1 || kgrp == 1) w1[d][nt] = ld_stream_v4(wp[nt] + static_cast<size_t>(d) * kItemBytes + 32);
                    meta[d][nt] = ld_pinned_v2(mp[nt] + static_cast<size_t>(d) * kItemBytes);
                }
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");  // these warps store y / add into the split-K scratch later
        bool broken = false, first = true;
        int stage = 0;
        uint32_t phase = 0;
        for (int it0 = 0; it0 < my_items && !broken; it0 += kAhead) {
#pragma unroll
            for (int d = 0; d < kAhead; ++d) {
                const int it = it0 + d;
                if (it >= my_items || broken) continue;
                // the item's constants: exact-dequant zero terms and the scale pair of columns g and g + 8
                typename Frag<ActT>::Zero z_lo[Cfg::kTilesPerWarp], z_hi[Cfg::kTilesPerWarp];
                uint32_t s_lo[Cfg::kTilesPerWarp], s_hi[Cfg::kTilesPerWarp];
#pragma unroll
                for (int nt = 0; nt < Cfg::kTilesPerWarp; ++nt) {
                    const uint2 mt = meta[d][nt];
                    z_lo[nt] = Frag<ActT>::zero(__byte_perm(mt.y, 0, 0x1010));
                    z_hi[nt] = Frag<ActT>::zero(__byte_perm(mt.y, 0, 0x3232));
                    s_lo[nt] = ScaleMul<ActT>::template pair<CVT>(mt.x & 0xFFFFu);
                    s_hi[nt] = ScaleMul<ActT>::template pair<CVT>(mt.x >> 16);
                }
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (broken) continue;
                    if (Cfg::kKSplit == 2 && t != kgrp) {  // the other warp group's K step
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1;
                            first = false;
                        }
                        continue;
                    }
                    if (!first && !tc::mbar_wait(empty_addr + 8 * stage, phase ^ 1)) {
                        if (lane == 0) atomicExch(status, 4);
                        broken = true;
                        continue;
                    }
                    const uint32_t tile_addr = b_base + stage * Cfg::kTileB;
#pragma unroll
                    for (int nt = 0; nt < Cfg::kTilesPerWarp; ++nt) {
                        const uint4 w = t == 0 ? w0[d][nt] : w1[d][nt];
                        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
                        uint32_t a[4][4];
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi) Frag<ActT>::expand(wv[wi], z_lo[nt], z_hi[nt], a[wi]);
                        // a[wi][0]: column g, low run; [2]: column g, high run; [1] / [3]: the same for column g + 8
                        if (live[nt]) {
                            const uint32_t addr = tile_addr + off_lo[nt];
                            st_shared_v4(addr, ScaleMul<ActT>::mul(a[0][0], s_lo[nt]), ScaleMul<ActT>::mul(a[1][0], s_lo[nt]),
                                         ScaleMul<ActT>::mul(a[2][0], s_lo[nt]), ScaleMul<ActT>::mul(a[3][0], s_lo[nt]));
                            st_shared_v4(addr ^ 32u, ScaleMul<ActT>::mul(a[0][2], s_lo[nt]), ScaleMul<ActT>::mul(a[1][2], s_lo[nt]),
                                         ScaleMul<ActT>::mul(a[2][2], s_lo[nt]), ScaleMul<ActT>::mul(a[3][2], s_lo[nt]));
                            st_shared_v4(addr + 8 * kRowBytes, ScaleMul<ActT>::mul(a[0][1], s_hi[nt]), ScaleMul<ActT>::mul(a[1][1], s_hi[nt]),
                                         ScaleMul<ActT>::mul(a[2][1], s_hi[nt]), ScaleMul<ActT>::mul(a[3][1], s_hi[nt]));
                            st_shared_v4((addr ^ 32u) + 8 * kRowBytes, ScaleMul<ActT>::mul(a[0][3], s_hi[nt]), ScaleMul<ActT>::mul(a[1][3], s_hi[nt]),
                                         ScaleMul<ActT>::mul(a[2][3], s_hi[nt]), ScaleMul<ActT>::mul(a[3][3], s_hi[nt]));
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(full_b_addr + 8 * stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                        first = false;
                    }
                }
                if (it + kAhead < my_items) {  // refill this ring slot
#pragma unroll
                    for (int nt = 0; nt < Cfg::kTilesPerWarp; ++nt) {
                        const size_t off = static_cast<size_t>(it + kAhead) * kItemBytes;
                        if (Cfg::kKSplit == 1 || kgrp == 0) w0[d][nt] = ld_stream_v4(wp[nt] + off);
                        if (Cfg::kKSplit == 1 || kgrp == 1) w1[d][nt] = ld_stream_v4(wp[nt] + off + 32);
                        meta[d][nt] = ld_pinned_v2(mp[nt] + off);
                    }
                }
            }
        }

        // ---- epilogue: warp w may touch TMEM lanes 32 (w % 4) .. +31
        const int quarter = warp & 3;
        const int quartet = dw >> 2;
        const bool ok = __all_sync(0xFFFFFFFFu, tc::mbar_wait(tc::smem_u32(acc_ready), 0));
        if (!ok && lane == 0) atomicExch(status, 3);
        tc::fence_after_sync();
        // Work units: (128-row half, 32-column chunk of the output), dealt round-robin to the warp quartets.  Everything
        // that decides whether a unit runs is warp-uniform: the TMEM loads are warp-wide instructions.
        constexpr int kChunks = (MODE == kGroupedSwiGLU ? BN / 2 : BN) / 32;
        // Rows that leave for their own addresses (possibly on a peer GPU): a thread's 64 bytes of its own row would make
        // every warp-wide store 32 separate 16-byte pieces, which NVLink carries at a fraction of its rate (measured: the
        // expert-parallel down projection took 480 us against 195 us with local stores).  The warp turns its 32 rows x 64
        // columns in shared memory (the stages are idle once the accumulator is complete) and stores 128 contiguous bytes
        // of one row with every eight lanes.
        bool turned = false;
        if constexpr (MODE == kGrouped) turned = N % 64 == 0;  // scattered local rows (y_rows) gain from whole lines too
        if (turned) {
            constexpr int kChunks64 = BN / 64;
            unsigned char* stg = smem + dw * 4096;  // [32 rows][8 x 16 B], chunk v of row r at v ^ (r & 7)
            const uint32_t stg_w = tc::smem_u32(stg) + lane * 128;
#pragma unroll 1
            for (int unit = quartet; ok && unit < HALVES * kChunks64; unit += Cfg::kQuartets) {
                const int half = unit / kChunks64, c = (unit - half * kChunks64) * 64;
                if (half >= live_halves) break;
                const int row0 = m0 + half * 128 + quarter * 32;
                const int m = row0 + lane;
                uint64_t mine = 0ull;  // lane r holds row r's destination
                if (m < m_end)
                    mine = grp.y_ptrs ? grp.y_ptrs[m]
                                      : reinterpret_cast<uint64_t>(y + (grp.y_rows ? static_cast<size_t>(grp.y_rows[m]) : static_cast<size_t>(m)) * N);
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * BN;
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(t_row + c + 32 * part, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint32_t pk[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const ActT o0 = from_float<ActT>(__uint_as_float(r[8 * v + 2 * i])), o1 = from_float<ActT>(__uint_as_float(r[8 * v + 2 * i + 1]));
                            pk[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) |
                                    (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                        }
                        const uint32_t at = stg_w + (((4 * part + v) ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
                    }
                }
                __syncwarp();
                const int v = lane & 7;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const uint64_t dst = __shfl_sync(0xFFFFFFFFu, mine, rr);
                    const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((v ^ (rr & 7)) << 4));
                    if (dst != 0ull && n0 + c + 8 * v < N)
                        *reinterpret_cast<uint4*>(dst + static_cast<size_t>(n0 + c + 8 * v) * sizeof(ActT)) = val;
                }
                __syncwarp();
            }
        }
#pragma unroll 1
        for (int unit = quartet; ok && !turned && unit < HALVES * kChunks; unit += Cfg::kQuartets) {
            const int half = unit / kChunks, c = (unit - half * kChunks) * 32;
            if (half >= live_halves) break;
            const int m = m0 + half * 128 + quarter * 32 + lane;
            bool row_ok = m < m_end;
            size_t out_row = static_cast<size_t>(m);
            ActT* out_base = y;
            if constexpr (MODE != kPlain) {
                if (row_ok && grp.y_ptrs) {
                    // the row's own destination: results go straight to the rank that owns the token
                    out_base = reinterpret_cast<ActT*>(grp.y_ptrs[m]);
                    out_row = 0;
                    row_ok = out_base != nullptr;
                } else if (row_ok && grp.y_rows) {
                    out_row = static_cast<size_t>(grp.y_rows[m]);
                }
            }
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * BN;
            if constexpr (MODE == kGroupedSwiGLU) {
                // gate columns [0, BN/2) and up columns [BN/2, BN) of the accumulator -> BN/2 columns of the output
                const int out_n = N / 2, out0 = n0 / 2;
                {
                    uint32_t rg[32], ru[32];
                    tc::tmem_ld_32x32(t_row + c, rg);
                    tc::tmem_ld_32x32(t_row + BN / 2 + c, ru);
                    tc::tmem_ld_wait();
                    if (row_ok && out0 + c < out_n) {
                        ActT* dst = out_base + out_row * out_n + out0 + c;
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = to_float(from_float<ActT>(__uint_as_float(rg[i])));
                            const float u = to_float(from_float<ActT>(__uint_as_float(ru[i])));
                            const ActT sg = from_float<ActT>(g / (1.f + expf(-g)));
                            const ActT o = from_float<ActT>(to_float(sg) * u);
                            const uint32_t bits = *reinterpret_cast<const uint16_t*>(&o);
                            if (i & 1)
                                packed[i >> 1] |= bits << 16;
                            else
                                packed[i >> 1] = bits;
                        }
                        if (out0 + c + 32 <= out_n) {
#pragma unroll
                            for (int v = 0; v < 4; ++v)
                                reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (out0 + c + i < out_n) reinterpret_cast<uint16_t*>(dst)[i] = static_cast<uint16_t>(packed[i >> 1] >> (16 * (i & 1)));
                        }
                    }
                }
            } else if constexpr (SPLIT) {
                {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(t_row + c, r);
                    tc::tmem_ld_wait();
                    if (row_ok && n0 + c < N) {
                        float* dst = split.partial + static_cast<size_t>(m) * N + n0 + c;
                        if (n0 + c + 32 <= N) {
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                red_add_v4(dst + 4 * v, __uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                           __uint_as_float(r[4 * v + 3]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (n0 + c + i < N) atomicAdd(dst + i, __uint_as_float(r[i]));
                        }
                    }
                }
            } else {
                {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(t_row + c, r);
                    tc::tmem_ld_wait();
                    if (row_ok && n0 + c < N) {
                        ActT* dst = out_base + out_row * N + n0 + c;
                        if (n0 + c + 32 <= N) {
                            uint32_t packed[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const ActT o0 = from_float<ActT>(__uint_as_float(r[2 * i])), o1 = from_float<ActT>(__uint_as_float(r[2 * i + 1]));
                                packed[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) |
                                            (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                            }
#pragma unroll
                            for (int v = 0; v < 4; ++v)
                                reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (n0 + c + i < N) dst[i] = from_float<ActT>(__uint_as_float(r[i]));
                        }
                    }
                }
            }
        }
        if constexpr (SPLIT) {
            // the epilogue warps of this CTA meet, one of them counts the CTA in; the last CTA of the tile finishes it
            __shared__ int s_last;
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(Cfg::kDequantWarps * 32) : "memory");
            if (dw == 0 && lane == 0) s_last = atomicAdd(split.counters + blockIdx.x, 1) == static_cast<int>(gridDim.z) - 1;
            asm volatile("bar.sync 1, %0;" ::"n"(Cfg::kDequantWarps * 32) : "memory");
            if (s_last) {
                __threadfence();
                const int rows = min(m_end - m0, 128 * HALVES);
                const int cols = min(BN, N - n0);  // multiples of 16
                for (int idx = (dw * 32 + lane) * 4; idx < rows * cols; idx += Cfg::kDequantWarps * 32 * 4) {
                    const int rr = idx / cols, cc = idx - rr * cols;
                    float4* src = reinterpret_cast<float4*>(split.partial + static_cast<size_t>(m0 + rr) * N + n0 + cc);
                    const float4 v = __ldcg(src);
                    __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
                    const ActT o0 = from_float<ActT>(v.x), o1 = from_float<ActT>(v.y), o2 = from_float<ActT>(v.z), o3 = from_float<ActT>(v.w);
                    uint2 pk;
                    pk.x = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o0)) | (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o1)) << 16);
                    pk.y = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o2)) | (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&o3)) << 16);
                    *reinterpret_cast<uint2*>(y + static_cast<size_t>(m0 + rr) * N + n0 + cc) = pk;
                }
                if (dw == 0 && lane == 0) split.counters[blockIdx.x] = 0;
            }
        }
        if (lane == 0 && dw == 0) {
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// Launch, as a programmatic dependent of the stream's previous kernel when asked (plain linears; the grouped modes read a
// block list the previous kernel wrote before anything else and stay ordinary launches).
template <typename Kernel, typename... Args>
int launch_pdl(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t stream, bool dependent, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, args...));
    return EQ_OK;
}

template <typename ActT, int HALVES, int BN, int DW, int AHEAD, int MODE>
int launch_cfg(const unsigned char* wq, int scale_dtype, const ActT* x, ActT* y, int64_t M, int64_t N, int64_t K, int* status,
               const GroupArgs& grp, unsigned grid_y, cudaStream_t stream) {
    using Cfg = GemmCfg<HALVES, BN, DW, AHEAD>;
    CUtensorMap map_x;
    const CUtensorMapDataType elem = ScaleMul<ActT>::kFmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int box_rows = (HALVES == 1 && MODE == kPlain) ? a_box_rows(static_cast<int>(M)) : 128 * Cfg::kBoxHalves;
    int st = make_tensor_map_2d(&map_x, x, elem, 2, M, K, K * 2, box_rows, kGK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    const bool cvt = scale_dtype != (ScaleMul<ActT>::kFmt == 0 ? EQ_F16 : EQ_BF16);
    auto kernel = cvt ? w4a16_gemm_tc_kernel<ActT, HALVES, BN, DW, AHEAD, true, MODE> : w4a16_gemm_tc_kernel<ActT, HALVES, BN, DW, AHEAD, false, MODE>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)));
    dim3 grid(static_cast<unsigned>(ceil_div(N, BN)), grid_y);
    return launch_pdl(kernel, grid, Cfg::kThreads, Cfg::kSmem, stream, MODE == kPlain, map_x, wq, y, static_cast<int>(M), static_cast<int>(N),
                      static_cast<int>(K), status, grp, SplitArgs{nullptr, nullptr});
}

// Up to 128 * HALVES rows: one row tile of 128 * HALVES x 256 with K split over gridDim.z so that about one CTA per SM runs.
template <typename ActT, int HALVES>
int launch_split(const unsigned char* wq, int scale_dtype, const ActT* x, ActT* y, int64_t M, int64_t N, int64_t K, int* status,
                 float* partial, int* counters, cudaStream_t stream) {
    using Cfg = GemmCfg<HALVES, 256, 16, 2>;
    CUtensorMap map_x;
    const CUtensorMapDataType elem = ScaleMul<ActT>::kFmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int box_rows = HALVES == 1 ? a_box_rows(static_cast<int>(M)) : 128 * Cfg::kBoxHalves;
    int st = make_tensor_map_2d(&map_x, x, elem, 2, M, K, K * 2, box_rows, kGK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EQ_OK) return st;
    const int64_t tiles = ceil_div(N, 256), items = K / 128;
    int64_t splits = sm_count() / tiles;
    if (splits > items) splits = items;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
    const bool cvt = scale_dtype != (ScaleMul<ActT>::kFmt == 0 ? EQ_F16 : EQ_BF16);
    const GroupArgs none = {nullptr, nullptr, nullptr, nullptr, 0};
    const SplitArgs sp = {partial, counters};
    dim3 grid(static_cast<unsigned>(tiles), 1, static_cast<unsigned>(splits));
    if (splits == 1) {
        auto kernel = cvt ? w4a16_gemm_tc_kernel<ActT, HALVES, 256, 16, 2, true, kPlain, false> : w4a16_gemm_tc_kernel<ActT, HALVES, 256, 16, 2, false, kPlain, false>;
        EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)));
        return launch_pdl(kernel, grid, Cfg::kThreads, Cfg::kSmem, stream, true, map_x, wq, y, static_cast<int>(M), static_cast<int>(N),
                          static_cast<int>(K), status, none, sp);
    }
    auto kernel = cvt ? w4a16_gemm_tc_kernel<ActT, HALVES, 256, 16, 2, true, kPlain, true> : w4a16_gemm_tc_kernel<ActT, HALVES, 256, 16, 2, false, kPlain, true>;
    EQ_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)));
    return launch_pdl(kernel, grid, Cfg::kThreads, Cfg::kSmem, stream, true, map_x, wq, y, static_cast<int>(M), static_cast<int>(N),
                      static_cast<int>(K), status, none, sp);
}

template <typename ActT>
int launch_typed(const unsigned char* wq, int scale_dtype, const int32_t* perm, const ActT* x, ActT* y, int64_t M, int64_t N,
                 int64_t K, ActT* gathered, int* status, float* partial, int* counters, cudaStream_t stream) {
    if (perm) {
        const int64_t total = M * K;
        gather_cols_kernel<ActT><<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, stream>>>(x, perm, M, K, gathered);
        EQ_LAUNCH_OK("gather_cols_kernel");
        x = gathered;
    }
    const GroupArgs none = {nullptr, nullptr, nullptr, nullptr, 0};
    if (M <= 128) {
        // wide matrices fill the SMs with 64-column tiles; narrow ones split K over 256-column tiles instead
        if (ceil_div(N, 64) >= sm_count())
            return launch_cfg<ActT, 1, 64, 8, 4, kPlain>(wq, scale_dtype, x, y, M, N, K, status, none, 1, stream);
        return launch_split<ActT, 1>(wq, scale_dtype, x, y, M, N, K, status, partial, counters, stream);
    }
    if (M <= 512 && ceil_div(N, 128) * ceil_div(M, 256) * 2 <= sm_count()) {
        // a few hundred rows of a narrow matrix would leave most SMs idle on whole-K tiles: run 256-row blocks through the
        // split-K form instead (each block streams the weight once more, which is still far cheaper; the dequantisation,
        // not the MMA, bounds these calls, so a 256-row block costs what a 128-row block costs)
        for (int64_t m0 = 0; m0 < M; m0 += 256) {
            const int64_t mb = M - m0 < 256 ? M - m0 : 256;
            const int st = mb > 128 ? launch_split<ActT, 2>(wq, scale_dtype, x + m0 * K, y + m0 * N, mb, N, K, status, partial, counters, stream)
                                    : launch_split<ActT, 1>(wq, scale_dtype, x + m0 * K, y + m0 * N, mb, N, K, status, partial, counters, stream);
            if (st != EQ_OK) return st;
        }
        return EQ_OK;
    }
    if (ceil_div(N, 256) * ceil_div(M, 256) >= sm_count())
        return launch_cfg<ActT, 2, 256, 16, 2, kPlain>(wq, scale_dtype, x, y, M, N, K, status, none, static_cast<unsigned>(ceil_div(M, 256)), stream);
    return launch_cfg<ActT, 2, 128, 16, 3, kPlain>(wq, scale_dtype, x, y, M, N, K, status, none, static_cast<unsigned>(ceil_div(M, 256)), stream);
}

}  // namespace

// gathered: M * K elements of scratch when perm is given.  status: one word, set by a bounded wait that ran out.
// partial / counters: f32 [min(M, 256)][N] and one int per 256 columns, zero between calls (used by the split-K forms).
int w4_gemm_tc_launch(const unsigned char* wq, int scale_dtype, const int32_t* perm, const void* x, void* y, int64_t M, int64_t N,
                      int64_t K, int act_dtype, void* gathered, int* status, float* partial, int* counters, cudaStream_t stream) {
    if (act_dtype == EQ_F16)
        return launch_typed<__half>(wq, scale_dtype, perm, static_cast<const __half*>(x), static_cast<__half*>(y), M, N, K,
                                    static_cast<__half*>(gathered), status, partial, counters, stream);
    return launch_typed<__nv_bfloat16>(wq, scale_dtype, perm, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), M,
                                       N, K, static_cast<__nv_bfloat16*>(gathered), status, partial, counters, stream);
}

// Grouped expert GEMM on the tensor path.  x: [R][K] activations in expert order; blocks / n_blocks: device-side list of
// row blocks of at most 256 rows; wq: E stacked repacked weights expert_stride bytes apart, each [N][K] logical.
// swiglu: N is the width of the [gate | up] weight and y has N / 2 columns.  max_blocks bounds the grid.
int w4_gemm_tc_grouped_launch(const unsigned char* wq, size_t expert_stride, int scale_dtype, const void* x, void* y, int64_t R, int64_t N,
                              int64_t K, int act_dtype, const RowBlock* blocks, const int32_t* n_blocks, int max_blocks,
                              const int32_t* y_rows, const uint64_t* y_ptrs, bool swiglu, int* status, cudaStream_t stream) {
    const GroupArgs grp = {blocks, n_blocks, y_rows, y_ptrs, expert_stride};
    const unsigned gy = static_cast<unsigned>(max_blocks);
    if (act_dtype == EQ_F16) {
        const __half* xa = static_cast<const __half*>(x);
        __half* ya = static_cast<__half*>(y);
        return swiglu ? launch_cfg<__half, 2, 256, 16, 2, kGroupedSwiGLU>(wq, scale_dtype, xa, ya, R, N, K, status, grp, gy, stream)
                      : launch_cfg<__half, 2, 256, 16, 2, kGrouped>(wq, scale_dtype, xa, ya, R, N, K, status, grp, gy, stream);
    }
    const __nv_bfloat16* xa = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* ya = static_cast<__nv_bfloat16*>(y);
    return swiglu ? launch_cfg<__nv_bfloat16, 2, 256, 16, 2, kGroupedSwiGLU>(wq, scale_dtype, xa, ya, R, N, K, status, grp, gy, stream)
                  : launch_cfg<__nv_bfloat16, 2, 256, 16, 2, kGrouped>(wq, scale_dtype, xa, ya, R, N, K, status, grp, gy, stream);
}

}  // namespace eq
