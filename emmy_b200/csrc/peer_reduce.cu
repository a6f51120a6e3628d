// Sum of the ranks' partial results of a row-parallel linear, over NVLink peer mappings (small results: decode steps).
//
// A row-parallel linear leaves every rank with a full [M, N] partial in the activation dtype, and the layer's output is
// their sum in f32, rounded once (the reference reduces a rank's partial sums over the tensor-parallel group the same
// way: emmy/serving/vllm_model_gen.py:986-991).  For a decode step that is a few hundred KB, and a library all-reduce
// costs tens of microseconds of launch and protocol latency.  Here one kernel does it in one NVLink round:
//
//   push    block b of every rank stores its 2048-element piece of the rank's partial into the same place of every
//           peer's receive buffer, slot (epoch & 1), region [source rank], by plain 16-byte peer stores;
//   signal  a system-scope fence, then one release store per peer into that peer's flag (slot, source, b) = epoch;
//   wait    the block waits (bounded, about a second) until its own flags (slot, every source, b) carry the epoch;
//   sum     it adds the W pieces in rank order in f32 -- every rank adds the same values in the same order, so all
//           ranks hold bit-identical results -- rounds once and stores its piece of y.
//
// Blocks only ever wait for the block of the same index on the other GPUs, never for a block of their own grid, so no
// co-residency is needed.  The epoch lives on the device (the last block to finish advances it), which makes the call
// replayable from a captured CUDA graph.  A slot is reused every second call: a peer can push epoch e + 2 into it only
// after it has seen this rank's flag of epoch e + 1, which this rank stores in a kernel that starts after the kernel of
// epoch e has finished reading.  The traffic is (W - 1) x the result per rank, so this is for small results; large ones
// belong to a bandwidth-optimal all-reduce (NCCL), and emmy_b200/shard.py switches on the size.
#include "common.cuh"

namespace eq {

namespace {

constexpr int kArThreads = 256;
constexpr int kArPiece = kArThreads * 8;            // elements per block: 16 bytes per thread
constexpr long long kArWaitCycles = 2000000000LL;   // about a second
constexpr int kArTimeout = 70;                      // status: a peer's piece did not arrive in time

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += to_float(e[i]);
}

// state: [0] status, [1] epoch of the last finished call, [2] blocks finished in the running call
template <typename T>
__global__ void __launch_bounds__(kArThreads) peer_allreduce_kernel(const eq_ar_peers pe, const T* __restrict__ partial, T* __restrict__ y,
                                                                    long long count, uint32_t* state) {
    // launched as a programmatic dependent: the grid is resident while the linear before it drains; nothing of that
    // linear (nor of this kernel's previous call) is touched before the wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(state + 1) + 1;  // stable until the last block finishes
    const int slot = static_cast<int>(epoch & 1u);
    const int world = pe.world, rank = pe.rank;
    const long long i0 = static_cast<long long>(blockIdx.x) * kArPiece + threadIdx.x * 8;
    const bool live = i0 < count;  // count is a multiple of 8
    const size_t region = static_cast<size_t>(pe.cap);  // elements per (slot, source)

    uint4 mine = make_uint4(0, 0, 0, 0);
    if (live) {
        mine = *reinterpret_cast<const uint4*>(partial + i0);
        for (int p = 0; p < world; ++p) {
            if (p == rank) continue;
            T* dst = static_cast<T*>(pe.recv[p]) + (static_cast<size_t>(slot) * world + rank) * region + i0;
            *reinterpret_cast<uint4*>(dst) = mine;
        }
    }
    __threadfence_system();
    __syncthreads();
    const size_t flag_at = (static_cast<size_t>(slot) * world) * pe.max_blocks + blockIdx.x;  // + source * max_blocks
    const int t = static_cast<int>(threadIdx.x);
    if (t < world && t != rank) st_release_sys_u32(pe.flags[t] + flag_at + static_cast<size_t>(rank) * pe.max_blocks, epoch);

    int ok = 1;
    if (t < world && t != rank) {
        const uint32_t* f = pe.flags[rank] + flag_at + static_cast<size_t>(t) * pe.max_blocks;
        const long long start = clock64();
        while (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) < 0) {
            if (clock64() - start > kArWaitCycles) {
                atomicExch(reinterpret_cast<int*>(state), kArTimeout);
                ok = 0;
                break;
            }
        }
    }
    ok = __syncthreads_and(ok);

    if (live && ok) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const T* own = static_cast<const T*>(pe.recv[rank]);
        for (int p = 0; p < world; ++p) {
            if (p == rank) {
                add8<T>(acc, mine);
            } else {  // pushed by a peer since the last call: read past L1
                const uint4 v = __ldcg(reinterpret_cast<const uint4*>(own + (static_cast<size_t>(slot) * world + p) * region + i0));
                add8<T>(acc, v);
            }
        }
        uint4 out;
        T* o = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = from_float<T>(acc[i]);
        *reinterpret_cast<uint4*>(y + i0) = out;
    }
    __syncthreads();
    if (t == 0) {
        __threadfence();
        if (atomicAdd(state + 2, 1u) == gridDim.x - 1) {  // every block has read the epoch by now
            state[2] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(state + 1) = epoch;
        }
    }
}

}  // namespace

}  // namespace eq

extern "C" size_t eq_peer_allreduce_recv_bytes(int64_t world, int64_t cap) {
    if (world <= 0 || cap <= 0) return 0;
    return static_cast<size_t>(2) * world * cap * 2;
}

extern "C" size_t eq_peer_allreduce_flag_bytes(int64_t world, int64_t cap) {
    if (world <= 0 || cap <= 0) return 0;
    return static_cast<size_t>(2) * world * eq::ceil_div(cap, eq::kArPiece) * sizeof(uint32_t);
}

extern "C" size_t eq_peer_allreduce_state_bytes(void) { return 256; }

extern "C" int eq_peer_allreduce(const eq_ar_peers* peers, const void* partial, int64_t count, int dtype, void* y, void* state, void* stream_) {
    using namespace eq;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(peers && state && (count == 0 || (partial && y)), EQ_ERR_BAD_ARG, "eq_peer_allreduce: null pointer");
    EQ_REQUIRE(peers->world >= 1 && peers->world <= EQ_EP_MAX_RANKS && peers->rank >= 0 && peers->rank < peers->world, EQ_ERR_BAD_ARG,
               "eq_peer_allreduce: bad world / rank %d / %d", peers->world, peers->rank);
    EQ_REQUIRE(dtype == EQ_F16 || dtype == EQ_BF16, EQ_ERR_BAD_ARG, "eq_peer_allreduce: values must be f16 or bf16");
    EQ_REQUIRE(count >= 0 && count % 8 == 0 && count <= peers->cap, EQ_ERR_UNSUPPORTED,
               "eq_peer_allreduce: %lld values: needs a multiple of 8, at most the buffers' capacity %lld", (long long)count, (long long)peers->cap);
    EQ_REQUIRE(peers->cap % 8 == 0 && peers->max_blocks == ceil_div(peers->cap, kArPiece), EQ_ERR_BAD_ARG,
               "eq_peer_allreduce: max_blocks must be ceil(cap / %d) and cap a multiple of 8", kArPiece);
    for (int r = 0; r < peers->world; ++r)
        EQ_REQUIRE(peers->recv[r] && peers->flags[r] && aligned(peers->recv[r], 16), EQ_ERR_BAD_ARG, "eq_peer_allreduce: rank %d has no buffers", r);
    EQ_REQUIRE(aligned(partial, 16) && aligned(y, 16) && aligned(state, 16), EQ_ERR_BAD_ALIGN, "eq_peer_allreduce: partial, y and state need 16-byte alignment");
    if (count == 0) return EQ_OK;  // (every rank passes the same count: nobody waits for this call)
    const unsigned blocks = static_cast<unsigned>(ceil_div(count, kArPiece));
    uint32_t* st = static_cast<uint32_t*>(state);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long n = count;
    if (dtype == EQ_F16)
        EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<__half>, *peers, static_cast<const __half*>(partial), static_cast<__half*>(y), n, st));
    else
        EQ_CUDA_OK(cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<__nv_bfloat16>, *peers, static_cast<const __nv_bfloat16*>(partial),
                                      static_cast<__nv_bfloat16*>(y), n, st));
    return EQ_OK;
}

extern "C" int eq_peer_allreduce_status(const void* state, void* stream_) {
    using namespace eq;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    EQ_REQUIRE(state, EQ_ERR_BAD_ARG, "eq_peer_allreduce_status: null state");
    int host = 0;
    EQ_CUDA_OK(cudaMemcpyAsync(&host, state, sizeof(int), cudaMemcpyDeviceToHost, stream));
    EQ_CUDA_OK(cudaStreamSynchronize(stream));
    EQ_REQUIRE(host == 0, EQ_ERR_TIMEOUT, "eq_peer_allreduce_status: a peer's piece did not arrive in time (%d)", host);
    return EQ_OK;
}
