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

// ---- flag barrier over peer memory ------------------------------------------------------------------
// One 64-bit slot per rank in every rank's flag buffer. A barrier is one tiny kernel: lane r
// publishes this rank's epoch into rank r's buffer (release at system scope, after a system fence
// that orders the preceding kernel's peer stores before it) and then waits, bounded, until rank r's
// epoch has arrived in the local buffer. The kernels that wait on each other run on different GPUs.
struct PeerBarrier {
    unsigned long long* table_dev = nullptr;   // device copy of the `world` flag-buffer pointers
    int world = 1, rank = 0;
    unsigned long long epoch = 0;
    unsigned long long wait_limit_ns = 2000000000ull;
};

__global__ void peer_barrier_kernel(unsigned long long* const* flags, int world, int rank, unsigned long long epoch,
                                    unsigned long long wait_limit_ns, uint32_t* err_word) {
    const int r = threadIdx.x;
    if (r >= world || r == rank) return;
    __threadfence_system();
    unsigned long long* remote = flags[r] + rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(remote), "l"(epoch) : "memory");
    const unsigned long long* mine = flags[rank] + r;
    unsigned long long t0 = 0, seen = 0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t it = 0;; ++it) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
        if (seen >= epoch) break;
        if ((it & 0x3f) == 0x3f) {
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > wait_limit_ns) {   // a peer never arrived: report and return
                if (err_word) atomicCAS(err_word, 0u, 0x500u + (uint32_t)r);
                break;
            }
            __nanosleep(100);
        }
    }
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
    if (cudaMalloc(&b->table_dev, 8 * sizeof(void*)) != cudaSuccess ||
        cudaMemcpy(b->table_dev, flag_buffers, (size_t)world * sizeof(void*), cudaMemcpyHostToDevice) != cudaSuccess) {
        delete b;
        return CG_B200_ERR_CUDA;
    }
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
