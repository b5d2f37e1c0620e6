// common.cuh - shared host/device helpers of the cg_b200 library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cg_b200.h"

namespace cgb {

// ---- host-side status plumbing -------------------------------------------------------------
// Last CUDA error text seen by this thread, appended to cg_b200_status_string(ERR_CUDA)
// callers that want detail can read it through cg_b200_last_cuda_error().
void note_cuda_error(cudaError_t e, const char* where);

#define CGB_CUDA(call)                                        \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) {                             \
            ::cgb::note_cuda_error(e__, #call);               \
            return e__ == cudaErrorNoDevice || e__ == cudaErrorInsufficientDriver \
                       ? CG_B200_ERR_NO_DEVICE                \
                       : CG_B200_ERR_CUDA;                    \
        }                                                     \
    } while (0)

// CG_B200_OK when a device of compute capability 10.x is current; cached per device.
int require_sm100();
int sm_count();

inline bool dtype_ok(int dt) { return dt == CG_B200_F16 || dt == CG_B200_BF16 || dt == CG_B200_F32; }
inline size_t dtype_bytes(int dt) { return dt == CG_B200_F32 ? 4 : 2; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Device error word shared by kernels with bounded waits (0 = no error).
uint32_t* device_error_word();   // device pointer, lazily allocated per device; nullptr on failure

// ---- flag barrier over peer memory ----------------------------------------------------------------
// One 64-bit slot per rank in every rank's flag buffer. Rank `rank` publishes its epoch into slot `rank`
// of rank r's buffer and waits, bounded, until rank r's epoch has arrived in slot r of its own buffer.
// The kernels that wait on each other run on different GPUs.
struct PeerBarrier {
    unsigned long long* table_dev = nullptr;   // device copy of the `world` flag-buffer pointers
    unsigned int* done_counter = nullptr;      // device word: CTAs of a fused kernel that have finished; returns to 0
    int world = 1, rank = 0;
    unsigned long long epoch = 0;
    unsigned long long wait_limit_ns = 2000000000ull;
};

// What one thread does for one peer. Everything this GPU wrote to peer memory before the caller's
// system fence is visible to the peer once it sees the epoch. A peer that never arrives is reported
// (0x500 + its rank) and the wait ends.
__device__ __forceinline__ void peer_flag_exchange(unsigned long long* const* flags, int rank, int r,
                                                   unsigned long long epoch, unsigned long long wait_limit_ns,
                                                   uint32_t* err_word) {
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
            if (t1 - t0 > wait_limit_ns) {
                if (err_word) atomicCAS(err_word, 0u, 0x500u + (uint32_t)r);
                break;
            }
            __nanosleep(100);
        }
    }
}

// ---- device-side element conversion -----------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int dtype = CG_B200_F32;
    __device__ static float to_f32(float v) { return v; }
    __device__ static float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int dtype = CG_B200_BF16;
    __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
    static constexpr int dtype = CG_B200_F16;
    __device__ static float to_f32(__half v) { return __half2float(v); }
    __device__ static __half from_f32(float v) { return __float2half_rn(v); }
};

// A 16-byte packet of T.
template <typename T> struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld_stream(const T* p) {
    // read-once data: bypass L1 allocation
    const int4 r = __ldcs(reinterpret_cast<const int4*>(p));
    Vec16<T> o;
    *reinterpret_cast<int4*>(&o) = r;
    return o;
}
template <typename T>
__device__ __forceinline__ Vec16<T> ld_keep(const T* p) {
    const int4 r = __ldg(reinterpret_cast<const int4*>(p));
    Vec16<T> o;
    *reinterpret_cast<int4*>(&o) = r;
    return o;
}
template <typename T>
__device__ __forceinline__ void st_stream(T* p, const Vec16<T>& v) {
    __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}

// 16-byte packet <-> fp32 lanes with the cheapest conversions the type allows: bf16 is the top
// half of an fp32 (a shift or a mask per element), and two fp32 pack into one cvt.rn.*x2.
template <typename T>
__device__ __forceinline__ void unpack16(const Vec16<T>& v, float (&f)[Vec16<T>::N]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int l = 0; l < 4; ++l) f[l] = v.v[l];
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            f[2 * l] = __uint_as_float(w[l] << 16);
            f[2 * l + 1] = __uint_as_float(w[l] & 0xffff0000u);
        }
    } else {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const float2 t = __half22float2(h[l]);
            f[2 * l] = t.x;
            f[2 * l + 1] = t.y;
        }
    }
}

template <typename T>
__device__ __forceinline__ Vec16<T> pack16(const float (&f)[Vec16<T>::N]) {
    Vec16<T> v;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int l = 0; l < 4; ++l) v.v[l] = f[l];
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) h[l] = __floats2bfloat162_rn(f[2 * l], f[2 * l + 1]);
    } else {
        __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) h[l] = __floats2half2_rn(f[2 * l], f[2 * l + 1]);
    }
    return v;
}

// Rounds fp32 lanes to T and back (what storing and reloading a tensor of type T does).
template <typename T>
__device__ __forceinline__ void round_through16(float (&f)[Vec16<T>::N]) {
    if constexpr (sizeof(T) != 4) {
        const Vec16<T> v = pack16<T>(f);
        unpack16<T>(v, f);
    }
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// gelu, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), every product rounded
// separately so the value does not depend on contraction choices.
__device__ __forceinline__ float gelu_tanh_f32(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float x3 = __fmul_rn(__fmul_rn(x, x), x);
    float t = __fadd_rn(x, __fmul_rn(k1, x3));
    float u = __fmul_rn(k0, t);
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(u)));
}

}  // namespace cgb
