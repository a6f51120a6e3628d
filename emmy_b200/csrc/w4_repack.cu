// Load-time re-tiling of AWQ / GPTQ int4 weights into the stream the W4A16 kernels read.
//
// The repacked weight is a flat run of 1088-byte ITEM records, [n-tile][item]: 16 output columns x 128 input rows.
//   bytes    0..1023  two 16(n) x 64(k) tiles of nibbles, 512 B each
//   bytes 1024..1087  the scales and zero points of the item's group: eight 8-byte records, one per column pair
//                     (g, g+8): {scale[g] | scale[g+8] << 16 (raw 16-bit patterns), f16(zero[g]) | f16(zero[g+8]) << 16}
//                     with the family's zero bias already added (0..16)
// so one bulk copy brings everything a warp needs for 128 input rows of 16 columns, and a tile's whole K run is
// contiguous.  (A group wider than 128 rows repeats its record in each of its items.)
// Inside a 512-byte tile lane L = 4g + j of a warp owns 16 bytes, word c of the lane is k16 step s = 4 tile + c of
// the item, and the eight nibbles p of a word are
//     p:        0          4          1           5           2          6          3           5+2
//     row:  32j+2s     32j+2s+1   32j+16+2s   32j+17+2s    32j+2s     32j+2s+1   32j+16+2s   32j+17+2s   (in the item)
//     n:        g          g          g           g          g+8        g+8        g+8         g+8       (in the tile)
// so that (w & 0x000F000F), (w & 0x00F000F0), ((w >> 8) & 0x000F000F), ((w >> 8) & 0x00F000F0) are the four
// registers of an m16n8k16 A fragment.
#include "common.cuh"

namespace eq {

__device__ __forceinline__ uint32_t read_nibble(int fmt, const uint32_t* __restrict__ qweight, int64_t K, int64_t N,
                                                int64_t k, int64_t n) {
    if (fmt == EQ_W4_AWQ) {
        const int i = static_cast<int>(n & 7);
        return (qweight[k * (N / 8) + n / 8] >> ((i & 1) * 16 + (i >> 1) * 4)) & 0xF;
    }
    return (qweight[(k / 8) * N + n] >> (4 * (k & 7))) & 0xF;
}

// Input row of nibble p of word wi (k16 step s = 4 (c & 1) + wi of the item) in lane j.  The rows of an item are
// dealt to the four lane columns j in blocks of 32; inside a block the first 16 rows are the "low" fragment slots
// (k-slots 2j, 2j+1 of the steps), the last 16 the "high" ones (k-slots 2j+8, 2j+9), two rows per step:
//     row = 128 item + 32 j + 16 high + 2 s + odd
// so the activations one lane needs for a whole item are 64 contiguous bytes of x.
__device__ __forceinline__ int64_t item_row(int64_t c, int wi, int j, int p) {
    const int s = 4 * static_cast<int>(c & 1) + wi;
    return (c >> 1) * 128 + 32 * j + ((p & 1) ? 16 : 0) + 2 * s + ((p >> 2) & 1);
}

constexpr int64_t kItemRecord = 1088;  // 1024 B of nibbles + 64 B of scales / zero points

// byte offset of word (tile t, 64-row chunk c, lane, word wi) in the repacked stream
__device__ __forceinline__ int64_t word_offset(int64_t K, int64_t t, int64_t c, int lane, int wi) {
    return (t * (K / 128) + (c >> 1)) * kItemRecord + (c & 1) * 512 + lane * 16 + wi * 4;
}

// One thread per output word.
__global__ void w4_repack_kernel(int fmt, const uint32_t* __restrict__ qweight, const int32_t* __restrict__ perm,
                                 int64_t K, int64_t N, unsigned char* __restrict__ wq) {
    // blockIdx.y: the expert of a stacked call (inputs and outputs of the experts lie back to back)
    qweight += blockIdx.y * (K * N / 8);
    wq += blockIdx.y * ((N / 16) * (K / 128) * kItemRecord);
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= K * N / 8) return;
    const int wi = static_cast<int>(idx & 3);
    const int lane = static_cast<int>((idx >> 2) & 31);
    const int64_t tile_chunk = idx >> 7;
    const int64_t chunks = K / 64;
    const int64_t t = tile_chunk / chunks, c = tile_chunk % chunks;
    const int g = lane >> 2, j = lane & 3;
    uint32_t w = 0;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int64_t kk = item_row(c, wi, j, p);
        const int64_t n = t * 16 + g + ((p & 2) ? 8 : 0);
        const int64_t ksrc = perm ? perm[kk] : kk;
        w |= read_nibble(fmt, qweight, K, N, ksrc, n) << (4 * p);
    }
    *reinterpret_cast<uint32_t*>(wq + word_offset(K, t, c, lane, wi)) = w;
}

// Scales and zero points: one thread per (n-tile, item, g) writes the 8-byte record of columns g and g+8.
// The source group of repacked group `grp` is g_idx[perm[grp * G]] when act-order information is present.
__global__ void w4_repack_meta_kernel(int fmt, const uint32_t* __restrict__ qzeros, const uint16_t* __restrict__ scales,
                                      const int32_t* __restrict__ g_idx, const int32_t* __restrict__ perm, int64_t K,
                                      int64_t N, int64_t G, unsigned char* __restrict__ wq) {
    qzeros += blockIdx.y * ((K / G) * (N / 8));
    scales += blockIdx.y * ((K / G) * N);
    wq += blockIdx.y * ((N / 16) * (K / 128) * kItemRecord);
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t items = K / 128;
    if (idx >= items * (N / 2)) return;
    const int g = static_cast<int>(idx & 7);
    const int64_t ti = idx >> 3;
    const int64_t t = ti / items, item = ti % items;
    const int64_t grp = item * 128 / G;
    int64_t src = grp;
    if (g_idx) src = g_idx[perm ? perm[grp * G] : grp * G];
    uint32_t sc = 0, zz = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int64_t n = t * 16 + g + 8 * h;
        const int ni = static_cast<int>(n & 7);
        const int sh = fmt == EQ_W4_AWQ ? ((ni & 1) * 16 + (ni >> 1) * 4) : 4 * ni;
        const uint32_t z = ((qzeros[src * (N / 8) + n / 8] >> sh) & 0xF) + (fmt == EQ_W4_GPTQ ? 1u : 0u);
        sc |= static_cast<uint32_t>(scales[src * N + n]) << (16 * h);
        zz |= static_cast<uint32_t>(__half_as_ushort(__uint2half_rn(z))) << (16 * h);
    }
    *reinterpret_cast<uint2*>(wq + ti * kItemRecord + 1024 + g * 8) = make_uint2(sc, zz);
}

// flags[0] |= 1 when some aligned G-block of g_idx is not constant; flags[1] |= 1 on an out-of-range entry.
__global__ void g_idx_check_kernel(const int32_t* __restrict__ g_idx, int64_t K, int64_t G, int32_t* flags) {
    const int64_t k = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (k >= K) return;
    const int32_t g = g_idx[k];
    if (g < 0 || g >= K / G) atomicOr(&flags[1], 1);
    if (g != g_idx[(k / G) * G]) atomicOr(&flags[0], 1);
}

// One block per group: the rows of that group, in ascending k, become repacked rows [g*G, (g+1)*G).
// flags[1] |= 2 when a group does not hold exactly G rows.
__global__ void g_idx_sort_kernel(const int32_t* __restrict__ g_idx, int64_t K, int64_t G, int32_t* __restrict__ perm,
                                  int32_t* flags) {
    __shared__ int warp_counts[32];
    __shared__ int base;
    const int g = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int64_t k0 = 0; k0 < K; k0 += blockDim.x) {
        const int64_t k = k0 + threadIdx.x;
        const bool mine = k < K && g_idx[k] == g;
        const unsigned ballot = __ballot_sync(0xFFFFFFFFu, mine);
        if (lane == 0) warp_counts[warp] = __popc(ballot);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_counts[w];
        const int pos = before + __popc(ballot & ((1u << lane) - 1));
        if (mine && pos < G) perm[static_cast<int64_t>(g) * G + pos] = static_cast<int32_t>(k);
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < nwarps; ++w) total += warp_counts[w];
            base += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && base != G) atomicOr(&flags[1], 2);
}

__global__ void w4_unpack_repacked_kernel(const unsigned char* __restrict__ wq, int64_t K, int64_t N,
                                          uint8_t* __restrict__ out) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= K * N / 8) return;
    const int wi = static_cast<int>(idx & 3);
    const int lane = static_cast<int>((idx >> 2) & 31);
    const int64_t tile_chunk = idx >> 7;
    const int64_t chunks = K / 64;
    const int64_t t = tile_chunk / chunks, c = tile_chunk % chunks;
    const int g = lane >> 2, j = lane & 3;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(wq + word_offset(K, t, c, lane, wi));
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int64_t kk = item_row(c, wi, j, p);
        const int64_t n = t * 16 + g + ((p & 2) ? 8 : 0);
        out[kk * N + n] = (w >> (4 * p)) & 0xF;
    }
}

static int check_geometry(const char* who, int64_t K, int64_t N, int64_t& G) {
    EQ_REQUIRE(K > 0 && N > 0, EQ_ERR_BAD_ARG, "%s: K and N must be positive", who);
    if (G == -1) G = K;
    EQ_REQUIRE(G > 0 && K % G == 0, EQ_ERR_BAD_ARG, "%s: group size %lld does not cover K=%lld", who, (long long)G, (long long)K);
    EQ_REQUIRE(K % 128 == 0 && N % 16 == 0, EQ_ERR_UNSUPPORTED, "%s: needs K %% 128 == 0 and N %% 16 == 0 (K=%lld N=%lld)", who,
               (long long)K, (long long)N);
    EQ_REQUIRE(G % 128 == 0, EQ_ERR_UNSUPPORTED, "%s: group size %lld is not a multiple of 128", who, (long long)G);
    return EQ_OK;
}

}  // namespace eq

using namespace eq;

extern "C" int eq_w4_repack_sizes(int64_t K, int64_t N, int64_t G, size_t* wq_bytes, size_t* perm_bytes) {
    int st = check_geometry("eq_w4_repack_sizes", K, N, G);
    if (st != EQ_OK) return st;
    if (wq_bytes) *wq_bytes = static_cast<size_t>(N / 16) * (K / 128) * kItemRecord;
    // K row indices followed by four status words the repack itself uses
    if (perm_bytes) *perm_bytes = static_cast<size_t>(K + 4) * sizeof(int32_t);
    return EQ_OK;
}

extern "C" int eq_w4_repack(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                            const int32_t* g_idx, int64_t K, int64_t N, int64_t G, void* wq, int32_t* perm, int* uses_perm,
                            void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(fmt == EQ_W4_AWQ || fmt == EQ_W4_GPTQ || fmt == EQ_W4_CT, EQ_ERR_BAD_ARG, "eq_w4_repack: unknown format %d", fmt);
    EQ_REQUIRE(qweight && qzeros && scales && wq, EQ_ERR_BAD_ARG, "eq_w4_repack: null pointer");
    int st = check_geometry("eq_w4_repack", K, N, G);
    if (st != EQ_OK) return st;
    EQ_REQUIRE(aligned(wq, 16), EQ_ERR_BAD_ALIGN, "eq_w4_repack: wq must be 16-byte aligned");
    if (uses_perm) *uses_perm = 0;
    const int32_t* row_perm = nullptr;
    if (g_idx) {
        EQ_REQUIRE(perm, EQ_ERR_BAD_ARG, "eq_w4_repack: g_idx given without a perm buffer");
        int32_t* flags = perm + K;
        EQ_CUDA_OK(cudaMemsetAsync(flags, 0, 4 * sizeof(int32_t), stream));
        g_idx_check_kernel<<<static_cast<unsigned>(ceil_div(K, 256)), 256, 0, stream>>>(g_idx, K, G, flags);
        EQ_LAUNCH_OK("g_idx_check_kernel");
        int32_t host_flags[4] = {0, 0, 0, 0};
        EQ_CUDA_OK(cudaMemcpyAsync(host_flags, flags, sizeof(host_flags), cudaMemcpyDeviceToHost, stream));
        EQ_CUDA_OK(cudaStreamSynchronize(stream));
        EQ_REQUIRE(host_flags[1] == 0, EQ_ERR_BAD_ARG, "eq_w4_repack: g_idx has entries outside [0, K/G)");
        if (host_flags[0]) {
            // rows of one group are scattered: sort rows by group and gather x through perm at run time
            g_idx_sort_kernel<<<static_cast<unsigned>(K / G), 256, 0, stream>>>(g_idx, K, G, perm, flags);
            EQ_LAUNCH_OK("g_idx_sort_kernel");
            EQ_CUDA_OK(cudaMemcpyAsync(host_flags, flags, sizeof(host_flags), cudaMemcpyDeviceToHost, stream));
            EQ_CUDA_OK(cudaStreamSynchronize(stream));
            EQ_REQUIRE(host_flags[1] == 0, EQ_ERR_UNSUPPORTED, "eq_w4_repack: a g_idx group does not hold exactly G rows");
            row_perm = perm;
            if (uses_perm) *uses_perm = 1;
        }
    }
    const int threads = 256;
    w4_repack_kernel<<<static_cast<unsigned>(ceil_div(K * N / 8, threads)), threads, 0, stream>>>(
        fmt, reinterpret_cast<const uint32_t*>(qweight), row_perm, K, N, static_cast<unsigned char*>(wq));
    EQ_LAUNCH_OK("w4_repack_kernel");
    w4_repack_meta_kernel<<<static_cast<unsigned>(ceil_div((K / 128) * (N / 2), threads)), threads, 0, stream>>>(
        fmt, reinterpret_cast<const uint32_t*>(qzeros), static_cast<const uint16_t*>(scales), g_idx, row_perm, K, N, G,
        static_cast<unsigned char*>(wq));
    EQ_LAUNCH_OK("w4_repack_meta_kernel");
    return EQ_OK;
}

// E stacked weights (the experts of an MoE layer: qweight [E, ...], qzeros [E, ...], scales [E, K/G, N], each expert in
// its checkpoint layout) -> E repacked blobs back to back, in two launches for the whole stack.  No g_idx (expert
// checkpoints with act-order go through eq_w4_repack one by one).
extern "C" int eq_w4_repack_stack(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales, int64_t E, int64_t K, int64_t N,
                                  int64_t G, void* wq, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(fmt == EQ_W4_AWQ || fmt == EQ_W4_GPTQ || fmt == EQ_W4_CT, EQ_ERR_BAD_ARG, "eq_w4_repack_stack: unknown format %d", fmt);
    EQ_REQUIRE(E > 0 && E <= 65535 && qweight && qzeros && scales && wq, EQ_ERR_BAD_ARG, "eq_w4_repack_stack: null pointer or bad expert count");
    int st = check_geometry("eq_w4_repack_stack", K, N, G);
    if (st != EQ_OK) return st;
    EQ_REQUIRE(aligned(wq, 16), EQ_ERR_BAD_ALIGN, "eq_w4_repack_stack: wq must be 16-byte aligned");
    const int threads = 256;
    const dim3 g1(static_cast<unsigned>(ceil_div(K * N / 8, threads)), static_cast<unsigned>(E));
    w4_repack_kernel<<<g1, threads, 0, stream>>>(fmt, reinterpret_cast<const uint32_t*>(qweight), nullptr, K, N, static_cast<unsigned char*>(wq));
    EQ_LAUNCH_OK("w4_repack_kernel");
    const dim3 g2(static_cast<unsigned>(ceil_div((K / 128) * (N / 2), threads)), static_cast<unsigned>(E));
    w4_repack_meta_kernel<<<g2, threads, 0, stream>>>(fmt, reinterpret_cast<const uint32_t*>(qzeros), static_cast<const uint16_t*>(scales), nullptr,
                                                       nullptr, K, N, G, static_cast<unsigned char*>(wq));
    EQ_LAUNCH_OK("w4_repack_meta_kernel");
    return EQ_OK;
}

extern "C" int eq_w4_unpack_repacked(const void* wq, int64_t K, int64_t N, uint8_t* out, void* stream) {
    EQ_REQUIRE(wq && out, EQ_ERR_BAD_ARG, "eq_w4_unpack_repacked: null pointer");
    EQ_REQUIRE(K > 0 && N > 0 && K % 128 == 0 && N % 16 == 0, EQ_ERR_UNSUPPORTED,
               "eq_w4_unpack_repacked: needs K %% 128 == 0 and N %% 16 == 0");
    const int threads = 256;
    w4_unpack_repacked_kernel<<<static_cast<unsigned>(ceil_div(K * N / 8, threads)), threads, 0,
                                static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned char*>(wq), K, N, out);
    EQ_LAUNCH_OK("w4_unpack_repacked_kernel");
    return EQ_OK;
}
