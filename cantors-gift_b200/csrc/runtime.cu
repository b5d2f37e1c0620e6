// runtime.cu - device, memory, stream and event entry points of the cg_b200 C ABI.
//
// These stand behind the reference's host-only runtime interfaces (Allocator, Stream,
// Event, Device in include/cg/runtime/runtime.hpp:44-79), whose only implementation is a
// malloc-backed CPU device (src/runtime/runtime.cpp:15-60).
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace cgb {

static thread_local char g_cuda_err[256] = "";

void note_cuda_error(cudaError_t e, const char* where) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e), where);
    cudaGetLastError();  // clear the sticky-free error state
}

static constexpr int kMaxDevices = 64;
static int g_cc_major[kMaxDevices];
static int g_sm_count[kMaxDevices];
static bool g_dev_known[kMaxDevices];
static uint32_t* g_err_word[kMaxDevices];
static std::mutex g_mu;

static int current_device_info(int* dev_out) {
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return CG_B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev_known[dev]) {
        int major = 0, sms = 0;
        CGB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        CGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_cc_major[dev] = major;
        g_sm_count[dev] = sms;
        g_dev_known[dev] = true;
    }
    *dev_out = dev;
    return CG_B200_OK;
}

int require_sm100() {
    int dev;
    int st = current_device_info(&dev);
    if (st) return st;
    return g_cc_major[dev] == 10 ? CG_B200_OK : CG_B200_ERR_NOT_SM100;
}

int sm_count() {
    int dev;
    if (current_device_info(&dev)) return 148;
    return g_sm_count[dev] > 0 ? g_sm_count[dev] : 148;
}

uint32_t* device_error_word() {
    int dev;
    if (current_device_info(&dev)) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_err_word[dev]) {
        uint32_t* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 256) != cudaSuccess) return nullptr;
        g_err_word[dev] = p;
    }
    return g_err_word[dev];
}

}  // namespace cgb

using namespace cgb;

extern "C" {

int cg_b200_version(void) { return (CG_B200_VERSION_MAJOR << 16) | CG_B200_VERSION_MINOR; }

const char* cg_b200_status_string(int status) {
    switch (status) {
        case CG_B200_OK: return "ok";
        case CG_B200_ERR_INVALID_ARG: return "invalid argument";
        case CG_B200_ERR_NULL_POINTER: return "null pointer";
        case CG_B200_ERR_MISALIGNED: return "misaligned pointer or stride";
        case CG_B200_ERR_UNSUPPORTED: return "unsupported configuration";
        case CG_B200_ERR_CUDA: return "CUDA call failed";
        case CG_B200_ERR_NO_DEVICE: return "no CUDA device (this library has no CPU fallback)";
        case CG_B200_ERR_WORKSPACE: return "workspace missing or too small";
        case CG_B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case CG_B200_ERR_COMM: return "NCCL failure";
        case CG_B200_ERR_FUSED_IR: return "IR carries lossy fusion markers (fused_chain / fused_with)";
        case CG_B200_ERR_NOT_SM100: return "device is not compute capability 10.x";
        default: return "unknown status";
    }
}

const char* cg_b200_last_cuda_error(void) { return g_cuda_err; }

int cg_b200_device_count(int* count) {
    if (!count) return CG_B200_ERR_NULL_POINTER;
    *count = 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        if (e != cudaSuccess) note_cuda_error(e, "cudaGetDeviceCount");
        return CG_B200_ERR_NO_DEVICE;
    }
    *count = n;
    return CG_B200_OK;
}

int cg_b200_device_props(int device, cg_b200_props* out) {
    if (!out) return CG_B200_ERR_NULL_POINTER;
    memset(out, 0, sizeof(*out));
    cudaDeviceProp p;
    CGB_CUDA(cudaGetDeviceProperties(&p, device));
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->sm_count = p.multiProcessorCount;
    out->max_smem_per_block = (int32_t)p.sharedMemPerBlockOptin;
    out->l2_bytes = p.l2CacheSize;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) out->sm_clock_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) out->mem_clock_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, device) == cudaSuccess) out->mem_bus_bits = v;
    out->hbm_bytes = p.totalGlobalMem;
    out->tmem_bytes_per_sm = p.major == 10 ? 256u * 1024u : 0u;
    return CG_B200_OK;
}

int cg_b200_set_device(int device) {
    CGB_CUDA(cudaSetDevice(device));
    return CG_B200_OK;
}

int cg_b200_malloc(void** dev_ptr, size_t bytes) {
    if (!dev_ptr) return CG_B200_ERR_NULL_POINTER;
    *dev_ptr = nullptr;
    if (bytes == 0) return CG_B200_OK;
    CGB_CUDA(cudaMalloc(dev_ptr, bytes));  // cudaMalloc returns >= 256-byte aligned pointers
    return CG_B200_OK;
}

int cg_b200_free(void* dev_ptr) {
    if (!dev_ptr) return CG_B200_OK;
    CGB_CUDA(cudaFree(dev_ptr));
    return CG_B200_OK;
}

int cg_b200_malloc_host(void** host_ptr, size_t bytes) {
    if (!host_ptr) return CG_B200_ERR_NULL_POINTER;
    *host_ptr = nullptr;
    if (bytes == 0) return CG_B200_OK;
    CGB_CUDA(cudaMallocHost(host_ptr, bytes));
    return CG_B200_OK;
}

int cg_b200_free_host(void* host_ptr) {
    if (!host_ptr) return CG_B200_OK;
    CGB_CUDA(cudaFreeHost(host_ptr));
    return CG_B200_OK;
}

int cg_b200_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes, void* stream) {
    if (bytes == 0) return CG_B200_OK;
    if (!dev_dst || !host_src) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes, void* stream) {
    if (bytes == 0) return CG_B200_OK;
    if (!host_dst || !dev_src) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_memset(void* dev_dst, int byte, size_t bytes, void* stream) {
    if (bytes == 0) return CG_B200_OK;
    if (!dev_dst) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaMemsetAsync(dev_dst, byte, bytes, (cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_stream_create(void** stream) {
    if (!stream) return CG_B200_ERR_NULL_POINTER;
    cudaStream_t s;
    CGB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return CG_B200_OK;
}

int cg_b200_stream_destroy(void* stream) {
    if (!stream) return CG_B200_OK;
    CGB_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_stream_sync(void* stream) {
    CGB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_event_create(void** event) {
    if (!event) return CG_B200_ERR_NULL_POINTER;
    cudaEvent_t e;
    CGB_CUDA(cudaEventCreate(&e));
    *event = e;
    return CG_B200_OK;
}

int cg_b200_event_destroy(void* event) {
    if (!event) return CG_B200_OK;
    CGB_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return CG_B200_OK;
}

int cg_b200_event_record(void* event, void* stream) {
    if (!event) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return CG_B200_OK;
}

int cg_b200_event_sync(void* event) {
    if (!event) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaEventSynchronize((cudaEvent_t)event));
    return CG_B200_OK;
}

int cg_b200_stream_wait_event(void* stream, void* event) {
    if (!event) return CG_B200_ERR_NULL_POINTER;
    CGB_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return CG_B200_OK;
}

int cg_b200_event_elapsed_sec(void* earlier, void* later, double* seconds) {
    if (!earlier || !later || !seconds) return CG_B200_ERR_NULL_POINTER;
    float ms = 0.f;
    CGB_CUDA(cudaEventElapsedTime(&ms, (cudaEvent_t)earlier, (cudaEvent_t)later));
    *seconds = (double)ms * 1e-3;
    return CG_B200_OK;
}

int cg_b200_ipc_export(const void* dev_ptr, void* host_handle) {
    if (!dev_ptr || !host_handle) return CG_B200_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == CG_B200_IPC_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    CGB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr)));
    memcpy(host_handle, &h, sizeof(h));
    return CG_B200_OK;
}

int cg_b200_ipc_open(const void* host_handle, void** peer_ptr) {
    if (!host_handle || !peer_ptr) return CG_B200_ERR_NULL_POINTER;
    *peer_ptr = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, host_handle, sizeof(h));
    CGB_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return CG_B200_OK;
}

int cg_b200_ipc_close(void* peer_ptr) {
    if (!peer_ptr) return CG_B200_OK;
    CGB_CUDA(cudaIpcCloseMemHandle(peer_ptr));
    return CG_B200_OK;
}

int cg_b200_last_device_error(void* stream, uint32_t* word) {
    if (!word) return CG_B200_ERR_NULL_POINTER;
    *word = 0;
    uint32_t* d = device_error_word();
    if (!d) return CG_B200_ERR_CUDA;
    CGB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    CGB_CUDA(cudaMemcpy(word, d, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (*word != 0) CGB_CUDA(cudaMemset(d, 0, sizeof(uint32_t)));
    return CG_B200_OK;
}

}  // extern "C"
