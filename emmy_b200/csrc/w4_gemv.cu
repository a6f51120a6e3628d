// W4A16 linear: the entry points and their dispatch.
//
//   M == 1         w4a16_gemv1_kernel (w4_gemv1.cu): half-SM CTAs, equal item spans, launches overlap in pairs.
//   2 <= M <= 24   w4a16_stream_kernel (w4_stream.cu): one fat CTA per SM streams whole column tiles, x staged in shared
//                  memory (whole, or a K slice per CTA with the slices meeting in the workspace).  From 17 rows on only
//                  where a slice of x fits; otherwise the next line.
//   M > 16         w4a16_gemm_tc_kernel (w4_gemm.cu): tcgen05, weights dequantised into shared memory.
//   w4a16_tile_kernel below: M > 16 with an output that is not 16-byte aligned (in 64-row blocks), and decode
//   shapes whose activations do not fit shared memory (K beyond about 100 k at M == 1).
//
// w4a16_tile_kernel is the plain form the other two grew out of, and the body the small-row MoE GEMMs still use
// (w4_tile.cuh): many small CTAs of four warps, one 16-column tile and one K split each, nothing between a warp and
// its bytes.  Per item (128 input rows x 16 columns, 1088 bytes) a lane
//   - streams its 2 x 16 weight bytes and its 8-byte scale/zero entry (loads are issued kDepth items ahead),
//   - reads the 64 contiguous bytes of x it needs straight from global memory (the repack deals input rows to lanes so
//     that this is four 16-byte loads),
//   - turns each word into one m16n8k16 A fragment: four lop3 + one shift isolate the nibbles as f16 1024+q (or
//     1024+16q), one f16x2 subtract / fma per pair removes 1024 and the zero point exactly, so the tensor core sees
//     the integers q - z and the f32 accumulator holds sum_k x_k (q_k - z) exactly up to f32 rounding,
//   - folds the item with its scale: y += s * acc.
// Warps of a CTA meet in shared memory.  K splits of one tile meet in an f32 workspace with atomic adds; the CTA
// whose arrival completes the tile converts, stores y and leaves workspace and counter zero.  Nobody waits.
#include "w4_tile.cuh"

namespace eq {

int w4_stream_launch(const W4Params& p, int act_dtype, cudaStream_t stream, bool* fits);  // w4_stream.cu
int w4_gemv1_launch(const unsigned char* wq, int scale_dtype, const int32_t* perm, const void* x, void* y, int64_t N, int64_t K,
                    int act_dtype, uint32_t* xchg, int* status, cudaStream_t stream, bool* fits);  // w4_gemv1.cu
int w4_gemm_tc_launch(const unsigned char* wq, int scale_dtype, const int32_t* perm, const void* x, void* y, int64_t M, int64_t N,
                      int64_t K, int act_dtype, void* gathered, int* status, float* partial, int* counters, cudaStream_t stream);  // w4_gemm.cu

template <typename ActT, int MT, bool ONE>
__global__ void __launch_bounds__(kTileThreads) w4a16_tile_kernel(const W4Params p) {
    __shared__ float red[kTileWarps][MT * 8][16];
    __shared__ int last_flag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next grid may start filling free SM slots
    const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
    w4_tile<ActT, MT, ONE>(p, tile, split, red, &last_flag);
}

// K splits per tile: enough CTAs that the hardware scheduler can even out the SMs (about 12 per SM), while a CTA
// still streams at least 8 items (8 KB).
static int plan_splits(int64_t K, int64_t N) {
    const int items = static_cast<int>(K / 128);
    const long long tiles = N / 16;
    const long long want = 12LL * sm_count();
    int s = static_cast<int>(ceil_div(want, tiles));
    if (s < 1) s = 1;
    const int max_s = items >= 8 ? items / 8 : 1;
    if (s > max_s) s = max_s;
    return s;
}

template <typename ActT, int MT, bool ONE>
static int launch_w4_one(const W4Params& p, cudaStream_t stream) {
    const long long ctas = static_cast<long long>(p.N / 16) * p.splits;
    // programmatic dependent launch, as the reference's runtime uses on sm_90+ (crates/emmy-runtime/src/cuda.rs:1299-1327)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kTileThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, w4a16_tile_kernel<ActT, MT, ONE>, p));
    return EQ_OK;
}

template <typename ActT>
static int launch_w4(const W4Params& p, cudaStream_t stream) {
    if (p.M == 1) return launch_w4_one<ActT, 1, true>(p, stream);
    if (p.M <= 8) return launch_w4_one<ActT, 1, false>(p, stream);
    if (p.M <= 16) return launch_w4_one<ActT, 2, false>(p, stream);
    if (p.M <= 32) return launch_w4_one<ActT, 4, false>(p, stream);
    return launch_w4_one<ActT, 8, false>(p, stream);
}

}  // namespace eq

using namespace eq;

// Workspace layout: a 256-byte header whose first word is the status word (fixed place, whatever M and N are), then
// f32 partial sums of up to 256 rows and one arrival counter per 16-column tile.  Calls with M > 16 add room for the
// column-gathered copy of x that act-order weights need on the tensor path.
static constexpr size_t kW4Header = 256;
static int64_t w4_front_rows(int64_t M) { return M < 256 ? M : 256; }
static size_t w4_front_bytes(int64_t M, int64_t N) {
    const int64_t rows = w4_front_rows(M);
    return kW4Header + static_cast<size_t>(rows) * N * sizeof(float) + static_cast<size_t>(N / 16) * sizeof(int);
}
static size_t w4_gather_offset(int64_t M, int64_t N) { return (w4_front_bytes(M, N) + 255) / 256 * 256; }

extern "C" size_t eq_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M <= 16) return w4_front_bytes(M, N);
    return w4_gather_offset(M, N) + static_cast<size_t>(M) * K * 2;
}

static int w4a16_check(const char* who, const void* wq, int scale_dtype, int64_t K, int64_t N, int64_t* G, const void* x, int64_t M,
                       int act_dtype, const void* y) {
    EQ_REQUIRE(wq && (M == 0 || (x && y)), EQ_ERR_BAD_ARG, "%s: null pointer", who);
    EQ_REQUIRE(K > 0 && N > 0 && M >= 0, EQ_ERR_BAD_ARG, "%s: bad extents M=%lld K=%lld N=%lld", who, (long long)M, (long long)K,
               (long long)N);
    if (*G == -1) *G = K;
    EQ_REQUIRE(*G > 0 && K % *G == 0, EQ_ERR_BAD_ARG, "%s: group size %lld does not cover K=%lld", who, (long long)*G, (long long)K);
    EQ_REQUIRE(K % 128 == 0 && N % 16 == 0 && *G % 128 == 0, EQ_ERR_UNSUPPORTED,
               "%s: needs K %% 128 == 0, N %% 16 == 0, G %% 128 == 0 (K=%lld N=%lld G=%lld)", who, (long long)K, (long long)N,
               (long long)*G);
    EQ_REQUIRE(K < (1 << 24) && N < (1 << 24), EQ_ERR_UNSUPPORTED, "%s: extent too large", who);
    EQ_REQUIRE(act_dtype == EQ_F16 || act_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "%s: activations must be f16 or bf16", who);
    EQ_REQUIRE(scale_dtype == EQ_F16 || scale_dtype == EQ_BF16, EQ_ERR_BAD_ARG, "%s: scales must be f16 or bf16", who);
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(aligned(wq, 16) && aligned(x, 16) && aligned(y, 2), EQ_ERR_BAD_ALIGN, "%s: wq and x need 16-byte alignment", who);
    return EQ_OK;
}

static W4Params w4_params(const void* wq, const int32_t* perm, const void* x, void* y, float* partial, int* counters, int64_t K, int64_t N, int M,
                          int scale_dtype) {
    W4Params p;
    p.wq = static_cast<const unsigned char*>(wq);
    p.perm = perm;
    p.x = x;
    p.y = y;
    p.wsp = partial;
    p.counters = counters;
    p.K = static_cast<int>(K);
    p.N = static_cast<int>(N);
    p.M = M;
    p.items = static_cast<int>(K / 128);
    p.splits = plan_splits(K, N);
    p.scale_dtype = scale_dtype;
    p.x_rows = nullptr;
    p.y_rows = nullptr;
    p.y_ptrs = nullptr;
    return p;
}

extern "C" int eq_w4a16_linear(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N, int64_t G,
                               const void* x, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                               void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int checked = w4a16_check("eq_w4a16_linear", wq, scale_dtype, K, N, &G, x, M, act_dtype, y);
    if (checked != EQ_OK || M == 0) return checked;
    EQ_REQUIRE(workspace && workspace_bytes >= eq_w4a16_workspace_bytes(M, N, K), EQ_ERR_WORKSPACE,
               "eq_w4a16_linear: workspace of %zu bytes needed, %zu given", eq_w4a16_workspace_bytes(M, N, K), workspace_bytes);
    EQ_REQUIRE(aligned(workspace, 16), EQ_ERR_BAD_ALIGN, "eq_w4a16_linear: workspace must be 16-byte aligned");

    int* status = static_cast<int*>(workspace);
    float* partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kW4Header);
    int* counters = reinterpret_cast<int*>(partial + w4_front_rows(M) * N);

    const bool streamable = static_cast<long long>(N / 16) * (K / 128) < (1LL << 30);
    if (M > 16 && M <= 24 && streamable) {
        // up to 24 rows still stream the weight once through the mma.sync tile (x staged in shared memory, K sliced where
        // it does not fit); a shape that does not fit falls through to the tensor path
        W4Params p = w4_params(wq, perm, x, y, partial, counters, K, N, static_cast<int>(M), scale_dtype);
        bool fits = false;
        const int st = w4_stream_launch(p, act_dtype, stream, &fits);
        if (st != EQ_OK || fits) return st;
    }
    if (M > 16 && aligned(y, 16)) {
        // prefill-shaped: the tcgen05 kernel; its bounded waits report through the status word.  No call clears the
        // word (a clear would be one more node between this kernel and the one before it, which it overlaps as a
        // programmatic dependent): it stays set until eq_w4a16_status has reported it.
        void* gathered = static_cast<unsigned char*>(workspace) + w4_gather_offset(M, N);
        const int st = w4_gemm_tc_launch(static_cast<const unsigned char*>(wq), scale_dtype, perm, x, y, M, N, K, act_dtype, gathered, status,
                                         partial, counters, stream);
        // Everything behind the header is zero between calls, whatever their shapes: a later call of another shape keeps its
        // partial sums or hand-over words where this one kept the gathered copy of x, so that copy is wiped again.
        if (st == EQ_OK && perm) EQ_CUDA_OK(cudaMemsetAsync(gathered, 0, static_cast<size_t>(M) * K * 2, stream));
        return st;
    }
    if (M == 1) {
        // the decode step's GEMV; the workspace carries its sixteen-word hand-overs between neighbouring CTAs
        bool fits = false;
        const int st = w4_gemv1_launch(static_cast<const unsigned char*>(wq), scale_dtype, perm, x, y, N, K, act_dtype,
                                       reinterpret_cast<uint32_t*>(partial), status, stream, &fits);
        if (st != EQ_OK || fits) return st;
    }

    const size_t esz = 2;
    for (int64_t m0 = 0; m0 < M; m0 += 64) {
        const int mb = static_cast<int>(M - m0 < 64 ? M - m0 : 64);
        W4Params p = w4_params(wq, perm, static_cast<const char*>(x) + static_cast<size_t>(m0) * K * esz,
                               static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz, partial, counters, K, N, mb, scale_dtype);
        int st = EQ_OK;
        bool fits = false;
        if (mb > 1 && mb <= 16 && streamable)
            st = w4_stream_launch(p, act_dtype, stream, &fits);  // decode-shaped: one wave of equal spans
        if (st != EQ_OK) return st;
        if (!fits)  // shapes whose staging does not fit shared memory, and row blocks of an unaligned output: K splits
                    // of small CTAs that meet in the workspace
            st = act_dtype == EQ_F16 ? launch_w4<__half>(p, stream) : launch_w4<__nv_bfloat16>(p, stream);
        if (st != EQ_OK) return st;
    }
    return EQ_OK;
}

// ---- gate / up + SwiGLU in one call ---------------------------------------------------------------------------
// h[M, I] = act(silu(x W_gate)) * (x W_up) for a [gate | up] weight (the two projections concatenated along N, as the
// reference stores them: emmy/compiler/trace/huggingface.py:1663-1669, 2110-2141), with the eager form's two roundings.
// M > 16: the tensor path's SwiGLU tile (128 gate + 128 up columns per CTA, the activation in the epilogue) over row
// blocks of the dense matrix; fewer rows: the [gate | up] linear into scratch, then an elementwise pass.
namespace eq {
namespace {

__global__ void dense_row_blocks_kernel(RowBlock* __restrict__ blocks, int32_t* __restrict__ n_blocks, int M) {
    const int nb = (M + 255) / 256;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        blocks[b].expert = 0;
        blocks[b].row0 = b * 256;
        blocks[b].rows = min(256, M - b * 256);
        blocks[b].pad = 0;
    }
    if (threadIdx.x == 0) *n_blocks = nb;
}

// h[r][i] = act(silu(gu[r][i])) * gu[r][I + i], eight columns per thread (I is a multiple of 16).  A programmatic
// dependent of the linear that wrote gu, and a primary of the kernel after it: that one is resident, with its weights on
// the way, while this one runs.
template <typename ActT>
__global__ void swiglu_rows_kernel(const ActT* __restrict__ gu, int64_t M, int64_t I, ActT* __restrict__ h) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t idx = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 8;
    if (idx >= M * I) return;
    const int64_t r = idx / I, i = idx - r * I;
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + r * 2 * I + i), uv = *reinterpret_cast<const uint4*>(gu + r * 2 * I + I + i);
    const ActT* ge = reinterpret_cast<const ActT*>(&gv);
    const ActT* ue = reinterpret_cast<const ActT*>(&uv);
    uint4 out;
    ActT* oe = reinterpret_cast<ActT*>(&out);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float g = to_float(ge[e]);
        const ActT s = from_float<ActT>(g / (1.f + expf(-g)));
        oe[e] = from_float<ActT>(to_float(s) * to_float(ue[e]));
    }
    if ((reinterpret_cast<uintptr_t>(h) & 15) == 0) {
        *reinterpret_cast<uint4*>(h + idx) = out;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) h[idx + e] = oe[e];
    }
}

template <typename ActT>
int launch_swiglu_rows(const void* gu, int64_t M, int64_t I, void* h, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(M * I / 8, 256)));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, swiglu_rows_kernel<ActT>, static_cast<const ActT*>(gu), M, I, static_cast<ActT*>(h)));
    return EQ_OK;
}

size_t gu_align(size_t v) { return (v + 255) / 256 * 256; }
size_t gu_blocks_bytes(int64_t M) { return gu_align((static_cast<size_t>((M + 255) / 256) + 1) * sizeof(RowBlock)); }

}  // namespace

int w4_gemm_tc_grouped_launch(const unsigned char* wq, size_t expert_stride, int scale_dtype, const void* x, void* y, int64_t R, int64_t N,
                              int64_t K, int act_dtype, const RowBlock* blocks, const int32_t* n_blocks, int max_blocks,
                              const int32_t* y_rows, const uint64_t* y_ptrs, bool swiglu, int* status, cudaStream_t stream);  // w4_gemm.cu

}  // namespace eq

extern "C" size_t eq_w4a16_gate_up_workspace_bytes(int64_t M, int64_t I, int64_t K) {
    if (M <= 0 || I <= 0 || K <= 0) return 0;
    // the linear's own workspace, then the row-block list (M > 16) or the [M, 2 I] scratch (M <= 16)
    return gu_align(eq_w4a16_workspace_bytes(M, 2 * I, K)) + (M > 16 ? gu_blocks_bytes(M) : gu_align(static_cast<size_t>(M) * 2 * I * 2));
}

extern "C" int eq_w4a16_gate_up_swiglu(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t I, int64_t G, const void* x,
                                       int64_t M, int act_dtype, void* h, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = w4a16_check("eq_w4a16_gate_up_swiglu", wq, scale_dtype, K, 2 * I, &G, x, M, act_dtype, h);
    if (st != EQ_OK) return st;
    if (M == 0) return EQ_OK;
    EQ_REQUIRE(I % 16 == 0, EQ_ERR_UNSUPPORTED, "eq_w4a16_gate_up_swiglu: the intermediate size must be a multiple of 16 (I=%lld)", (long long)I);
    EQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= eq_w4a16_gate_up_workspace_bytes(M, I, K), EQ_ERR_WORKSPACE,
               "eq_w4a16_gate_up_swiglu: workspace of %zu bytes (256-byte aligned) needed, %zu given", eq_w4a16_gate_up_workspace_bytes(M, I, K),
               workspace_bytes);
    const size_t inner = gu_align(eq_w4a16_workspace_bytes(M, 2 * I, K));
    unsigned char* extra = static_cast<unsigned char*>(workspace) + inner;
    if (M > 16 && !perm && aligned(h, 16)) {
        int* status = static_cast<int*>(workspace);  // sticky until eq_w4a16_status reports it, as in eq_w4a16_linear
        RowBlock* blocks = reinterpret_cast<RowBlock*>(extra);
        const int nb = static_cast<int>((M + 255) / 256);
        int32_t* n_blocks = reinterpret_cast<int32_t*>(blocks + nb);
        dense_row_blocks_kernel<<<1, 256, 0, stream>>>(blocks, n_blocks, static_cast<int>(M));
        EQ_LAUNCH_OK("dense_row_blocks_kernel");
        return w4_gemm_tc_grouped_launch(static_cast<const unsigned char*>(wq), 0, scale_dtype, x, h, M, 2 * I, K, act_dtype, blocks, n_blocks, nb, nullptr,
                                         nullptr, true, status, stream);
    }
    // few rows, scattered act-order groups or an unaligned output: the [gate | up] linear, then the activation
    EQ_REQUIRE(M <= 16, EQ_ERR_UNSUPPORTED, "eq_w4a16_gate_up_swiglu: M > 16 needs a 16-byte aligned output and a weight without a row permutation");
    void* gu = extra;  // [M][2 I] scratch
    st = eq_w4a16_linear(wq, scale_dtype, perm, K, 2 * I, G, x, M, act_dtype, gu, workspace, inner, stream_);
    if (st != EQ_OK) return st;
    return act_dtype == EQ_F16 ? launch_swiglu_rows<__half>(gu, M, I, h, stream) : launch_swiglu_rows<__nv_bfloat16>(gu, M, I, h, stream);
}

// The tensor-path kernel and the GEMV's hand-over wait are bounded; one that runs out sets the status word.
extern "C" int eq_w4a16_status(const void* workspace, int64_t M, int64_t N, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(workspace && M > 0 && N > 0, EQ_ERR_BAD_ARG, "eq_w4a16_status: bad arguments");
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    if (host != 0) {  // reported once: the next calls start from a clean word
        EQ_CUDA_OK(cudaMemsetAsync(const_cast<void*>(workspace), 0, sizeof(int), stream));
        EQ_CUDA_OK(cudaStreamSynchronize(stream));
    }
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_w4a16_status: the workspace status word is set (%d)", host);
    return EQ_OK;
}

// ---- entry point for callers that cannot allocate ------------------------------------------------------------
// The scratch of eq_w4a16_linear (status word, hand-over words / partial sums, arrival counters) for up to kNoAllocMaxM
// rows and kNoAllocMaxN columns, resident in every device that loads this library until the process exits.
namespace {
constexpr int64_t kNoAllocMaxM = 16;
constexpr int64_t kNoAllocMaxN = 32768;
constexpr size_t kNoAllocBytes = kW4Header + static_cast<size_t>(kNoAllocMaxM) * kNoAllocMaxN * sizeof(float) +
                                 (static_cast<size_t>(kNoAllocMaxN) / 16) * sizeof(int) + 256;
static __device__ __align__(256) unsigned char g_w4_noalloc_scratch[kNoAllocBytes];  // zero when the module loads

struct NoAllocState {
    void* ptr;   // device address of the array on this device
    int dirty;   // a call failed after it may have launched: clear the array before the next use
};

// Device address of the array above on the current device.  The array's name is only a host-side handle; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int noalloc_state(NoAllocState** out) {
    static NoAllocState state[64] = {};
    int dev = -1;
    EQ_CUDA_OK(cudaGetDevice(&dev));
    EQ_REQUIRE(dev >= 0 && dev < 64, EQ_ERR_UNSUPPORTED, "eq_w4a16_linear_noalloc: device index %d out of range", dev);
    void* ptr = __atomic_load_n(&state[dev].ptr, __ATOMIC_ACQUIRE);
    if (!ptr) {
        EQ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_w4_noalloc_scratch));
        EQ_REQUIRE(ptr != nullptr, EQ_ERR_CUDA, "eq_w4a16_linear_noalloc: no device address for the static scratch");
        __atomic_store_n(&state[dev].ptr, ptr, __ATOMIC_RELEASE);
    }
    *out = &state[dev];
    return EQ_OK;
}
}  // namespace

extern "C" int eq_w4a16_linear_noalloc(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N,
                                       int64_t G, const void* x, int64_t M, int act_dtype, void* y, void* stream_) {
    const int checked = w4a16_check("eq_w4a16_linear_noalloc", wq, scale_dtype, K, N, &G, x, M, act_dtype, y);
    if (checked != EQ_OK) return checked;
    EQ_REQUIRE(M <= kNoAllocMaxM, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear_noalloc: M=%lld exceeds the built-in scratch (at most %lld rows); use eq_w4a16_linear with "
               "a caller workspace",
               (long long)M, (long long)kNoAllocMaxM);
    EQ_REQUIRE(N <= kNoAllocMaxN, EQ_ERR_UNSUPPORTED,
               "eq_w4a16_linear_noalloc: N=%lld exceeds the built-in scratch (at most %lld columns); use eq_w4a16_linear "
               "with a caller workspace",
               (long long)N, (long long)kNoAllocMaxN);
    if (M == 0) return EQ_OK;
    NoAllocState* state = nullptr;
    int st = noalloc_state(&state);
    if (st != EQ_OK) return st;
    const size_t used = eq_w4a16_workspace_bytes(M, N, K);
    // The array starts out zero and every kernel leaves the words it used zero again, so nothing is cleared on the
    // way in; only after a call that failed part-way is the whole array cleared before the next one.
    if (__atomic_load_n(&state->dirty, __ATOMIC_ACQUIRE)) {
        EQ_CUDA_OK(cudaMemsetAsync(state->ptr, 0, kNoAllocBytes, static_cast<cudaStream_t>(stream_)));
        __atomic_store_n(&state->dirty, 0, __ATOMIC_RELEASE);
    }
    st = eq_w4a16_linear(wq, scale_dtype, perm, K, N, G, x, M, act_dtype, y, state->ptr, used, stream_);
    if (st != EQ_OK) __atomic_store_n(&state->dirty, 1, __ATOMIC_RELEASE);
    return st;
}

// Reads the built-in array's status word (synchronizes the stream): EQ_ERR_TIMEOUT if a bounded wait of an earlier
// eq_w4a16_linear_noalloc call on this device ran out; the array is then cleared before its next use.
extern "C" int eq_w4a16_noalloc_status(void* stream_) {
    NoAllocState* state = nullptr;
    int st = noalloc_state(&state);
    if (st != EQ_OK) return st;
    st = eq_w4a16_status(state->ptr, 1, 16, stream_);
    if (st != EQ_OK) __atomic_store_n(&state->dirty, 1, __ATOMIC_RELEASE);
    return st;
}
