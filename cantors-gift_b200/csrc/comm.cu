// comm.cu - the one collective of the path: an in-place all-gather of M- or batch-sharded
// outputs over NCCL (NVLink 5 / NVSwitch inside one box).
//
// The reference has no collective and no multi-device runtime; its only parallel execution
// is the std::thread fan-out of include/cg/backend/parallel_executor.hpp:49-92. One process
// drives one GPU; rank 0 makes the id, the caller ships it to the other ranks.
//
// NCCL is bound at run time with dlopen so that a process which already holds an NCCL (for
// instance through torch.distributed) shares that copy instead of loading a second one.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace cgb {

struct NcclId {
    char internal[CG_B200_COMM_ID_BYTES];
};
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);

struct NcclApi {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllGatherFn all_gather = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    bool ok = false;
};

static NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
        api.get_unique_id = (GetUniqueIdFn)dlsym(api.handle, "ncclGetUniqueId");
        api.comm_init_rank = (CommInitRankFn)dlsym(api.handle, "ncclCommInitRank");
        api.all_gather = (AllGatherFn)dlsym(api.handle, "ncclAllGather");
        api.comm_destroy = (CommDestroyFn)dlsym(api.handle, "ncclCommDestroy");
        api.ok = api.get_unique_id && api.comm_init_rank && api.all_gather && api.comm_destroy;
    });
    return api;
}

struct Comm {
    void* nccl_comm;
    int world;
    int rank;
    void* token = nullptr;   // world * 8 bytes for cg_b200_comm_barrier
};

// ---- flag barrier over peer memory (PeerBarrier, peer_flag_exchange: common.cuh) ---------------------
// A barrier of its own is one tiny kernel: lane r handles peer r, after a system fence that orders the
// preceding kernel's peer stores before the flags.
__global__ void peer_barrier_kernel(unsigned long long* const* flags, int world, int rank, unsigned long long epoch,
                                    unsigned long long wait_limit_ns, uint32_t* err_word) {
    const int r = threadIdx.x;
    if (r >= world || r == rank) return;
    __threadfence_system();
    peer_flag_exchange(flags, rank, r, epoch, wait_limit_ns, err_word);
}

// Pushes `bytes` (a multiple of 16) from `src` into the same offset of up to 7 peer buffers: each 16-byte
// packet is loaded once and stored to every peer. With a flag table it ends in the barrier: the last
// CTA to finish publishes the epoch and waits for the peers'.
struct PeerPointers {
    int4* p[7];
};

__global__ void __launch_bounds__(512)
peer_push_kernel(const int4* __restrict__ src, const PeerPointers peers, int n_peer, size_t packets,
                 unsigned long long* const* flags, int world, int rank, unsigned long long epoch,
                 unsigned long long wait_limit_ns, unsigned int* done_counter, uint32_t* err_word) {
    __shared__ int4* dst[7];
    __shared__ bool last;
    if (threadIdx.x < 7) dst[threadIdx.x] = threadIdx.x < n_peer ? peers.p[threadIdx.x] : nullptr;
    __syncthreads();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    constexpr int kUnroll = 4;   // independent loads in flight per thread
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < packets; i += kUnroll * stride) {
        int4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = __ldcs(src + i + u * stride);
        for (int d = 0; d < n_peer; ++d) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) dst[d][i + u * stride] = v[u];
        }
    }
    for (; i < packets; i += stride) {
        const int4 v = __ldcs(src + i);
        for (int d = 0; d < n_peer; ++d) dst[d][i] = v;
    }
    if (!flags) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(done_counter, 1u);
        last = prev == gridDim.x - 1;
        if (last) *done_counter = 0;   // every CTA has counted itself: ready for the next launch
    }
    __syncthreads();
    if (!last) return;
    __threadfence_system();
    const int r = threadIdx.x;
    if (r < world && r != rank) peer_flag_exchange(flags, rank, r, epoch, wait_limit_ns, err_word);
}

}  // namespace cgb

using namespace cgb;

extern "C" int cg_b200_peer_barrier_create(void** barrier, void* const* flag_buffers, int world, int rank) {
    if (!barrier || !flag_buffers) return CG_B200_ERR_NULL_POINTER;
    *barrier = nullptr;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CG_B200_ERR_INVALID_ARG;
    for (int r = 0; r < world; ++r)
        if (!flag_buffers[r] || !aligned_to(flag_buffers[r], 8)) return flag_buffers[r] ? CG_B200_ERR_MISALIGNED : CG_B200_ERR_NULL_POINTER;
    int st = require_sm100();
    if (st) return st;
    PeerBarrier* b = new PeerBarrier;
    b->world = world;
    b->rank = rank;
    // the flag table, then the done counter of the fused kernels, in one small allocation
    if (cudaMalloc(&b->table_dev, 16 * sizeof(void*)) != cudaSuccess || cudaMemset(b->table_dev, 0, 16 * sizeof(void*)) != cudaSuccess ||
        cudaMemcpy(b->table_dev, flag_buffers, (size_t)world * sizeof(void*), cudaMemcpyHostToDevice) != cudaSuccess) {
        delete b;
        return CG_B200_ERR_CUDA;
    }
    b->done_counter = reinterpret_cast<unsigned int*>(b->table_dev + 8);
    *barrier = b;
    return CG_B200_OK;
}

extern "C" int cg_b200_peer_barrier(void* barrier, void* stream) {
    if (!barrier) return CG_B200_ERR_NULL_POINTER;
    PeerBarrier* b = static_cast<PeerBarrier*>(barrier);
    ++b->epoch;
    if (b->world == 1) return CG_B200_OK;
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(reinterpret_cast<unsigned long long* const*>(b->table_dev), b->world,
                                                             b->rank, b->epoch, b->wait_limit_ns, device_error_word());
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}

extern "C" int cg_b200_peer_push(const void* src, void* const* peer_dst, int world, int rank, size_t bytes, void* barrier,
                                 void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CG_B200_ERR_INVALID_ARG;
    if (bytes % 16) return CG_B200_ERR_INVALID_ARG;
    PeerBarrier* b = static_cast<PeerBarrier*>(barrier);
    if (b && (b->world != world || b->rank != rank)) return CG_B200_ERR_INVALID_ARG;
    if (b) ++b->epoch;   // every rank calls with a barrier the same number of times, whatever its byte count
    if (world == 1 || (bytes == 0 && !b)) return CG_B200_OK;
    if (!peer_dst || (bytes && !src)) return CG_B200_ERR_NULL_POINTER;
    if (!aligned_to(src, 16)) return CG_B200_ERR_MISALIGNED;
    int st = require_sm100();
    if (st) return st;
    PeerPointers peers{};
    int n = 0;
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        if (!peer_dst[r]) return CG_B200_ERR_NULL_POINTER;
        if (!aligned_to(peer_dst[r], 16)) return CG_B200_ERR_MISALIGNED;
        peers.p[n++] = static_cast<int4*>(peer_dst[r]);
    }
    // a grid that fits beside a persistent compute kernel: at most one CTA of 512 threads per SM, fewer for
    // small transfers (four packets per thread per pass)
    const size_t packets = bytes / 16;
    const size_t want = (packets + 512 * 4 - 1) / (512 * 4);
    const size_t cap = (size_t)sm_count();
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
    peer_push_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(
        static_cast<const int4*>(src), peers, n, packets, b ? reinterpret_cast<unsigned long long* const*>(b->table_dev) : nullptr,
        world, rank, b ? b->epoch : 0ull, b ? b->wait_limit_ns : 0ull, b ? b->done_counter : nullptr, device_error_word());
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}

extern "C" int cg_b200_peer_barrier_set_timeout(void* barrier, uint64_t nanoseconds) {
    if (!barrier) return CG_B200_ERR_NULL_POINTER;
    if (nanoseconds == 0 || nanoseconds > 60000000000ull) return CG_B200_ERR_INVALID_ARG;
    static_cast<PeerBarrier*>(barrier)->wait_limit_ns = nanoseconds;
    return CG_B200_OK;
}

extern "C" int cg_b200_peer_barrier_destroy(void* barrier) {
    if (!barrier) return CG_B200_OK;
    PeerBarrier* b = static_cast<PeerBarrier*>(barrier);
    if (b->table_dev) cudaFree(b->table_dev);
    delete b;
    return CG_B200_OK;
}

extern "C" int cg_b200_comm_unique_id(void* host_unique_id) {
    if (!host_unique_id) return CG_B200_ERR_NULL_POINTER;
    NcclApi& api = nccl();
    if (!api.ok) return CG_B200_ERR_COMM;
    NcclId id;
    if (api.get_unique_id(&id) != 0) return CG_B200_ERR_COMM;
    memcpy(host_unique_id, &id, sizeof(id));
    return CG_B200_OK;
}

extern "C" int cg_b200_comm_init_rank(void** comm, int world, int rank, const void* host_unique_id) {
    if (!comm || !host_unique_id) return CG_B200_ERR_NULL_POINTER;
    *comm = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return CG_B200_ERR_INVALID_ARG;
    int st = require_sm100();
    if (st) return st;
    NcclApi& api = nccl();
    if (!api.ok) return CG_B200_ERR_COMM;
    NcclId id;
    memcpy(&id, host_unique_id, sizeof(id));
    void* c = nullptr;
    if (api.comm_init_rank(&c, world, id, rank) != 0) return CG_B200_ERR_COMM;
    Comm* out = new Comm{c, world, rank};
    if (cudaMalloc(&out->token, (size_t)world * 8) != cudaSuccess || cudaMemset(out->token, 0, (size_t)world * 8) != cudaSuccess) {
        api.comm_destroy(c);
        delete out;
        return CG_B200_ERR_CUDA;
    }
    *comm = out;
    return CG_B200_OK;
}

extern "C" int cg_b200_allgather_inplace(void* comm, void* buf, size_t shard_bytes, void* stream) {
    if (!comm) return CG_B200_ERR_NULL_POINTER;
    if (shard_bytes == 0) return CG_B200_OK;
    if (!buf) return CG_B200_ERR_NULL_POINTER;
    Comm* c = static_cast<Comm*>(comm);
    const char* send = static_cast<const char*>(buf) + (size_t)c->rank * shard_bytes;
    // datatype 0 = ncclInt8: the shards are opaque bytes
    if (nccl().all_gather(send, buf, shard_bytes, 0, c->nccl_comm, (cudaStream_t)stream) != 0) return CG_B200_ERR_COMM;
    return CG_B200_OK;
}

extern "C" int cg_b200_comm_barrier(void* comm, void* stream) {
    if (!comm) return CG_B200_ERR_NULL_POINTER;
    Comm* c = static_cast<Comm*>(comm);
    // an 8-byte all-gather: it completes on a rank only after every rank has reached it in its stream
    const char* send = static_cast<const char*>(c->token) + (size_t)c->rank * 8;
    if (nccl().all_gather(send, c->token, 8, 0, c->nccl_comm, (cudaStream_t)stream) != 0) return CG_B200_ERR_COMM;
    return CG_B200_OK;
}

extern "C" int cg_b200_comm_destroy(void* comm) {
    if (!comm) return CG_B200_OK;
    Comm* c = static_cast<Comm*>(comm);
    if (c->token) cudaFree(c->token);
    int r = nccl().comm_destroy(c->nccl_comm);
    delete c;
    return r == 0 ? CG_B200_OK : CG_B200_ERR_COMM;
}
