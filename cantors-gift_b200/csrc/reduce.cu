// reduce.cu - reduce_sum / reduce_max / reduce_mean over a run of adjacent axes.
//
// The reference defines the three ops with an `axes` list and `keep_dims` (src/ir/ops.cpp:74-102,
// 417-436; include/cg/ir/builder.hpp:62-63) and lowers them to VectorLoad, Reduce, VectorStore
// (src/lowering/tensor_to_codegen.cpp:332); the PTX emitter prints a comment for CGOpcode::Reduce
// (src/backend/ptx/ptx_emitter.cpp:136-142), so nothing is ever reduced. Here: a row-major tensor whose
// reduced axes are adjacent is a [outer, reduce, inner] box (keep_dims changes the result's shape,
// not its bytes), out[o, i] = op over r of in[o, r, i], accumulated in fp32 and rounded once to the
// storage type; mean = sum / reduce.
//
// HBM-bound: algorithmic bytes = (outer * reduce * inner + outer * inner) * sizeof(T).
// inner == 1 (last axes reduced): rows are contiguous; one warp per row for short rows, one CTA per row
// for long ones, 16-byte loads where the row allows them. inner > 1: threads run along `inner`
// (coalesced), the CTA's y dimension splits `reduce` and combines through shared memory.
#include <math.h>

#include "common.cuh"

namespace cgb {

struct ReduceParams {
    const void* in;
    void* out;
    long long outer, reduce, inner;
    int op;
};

__device__ __forceinline__ float red_identity(int op) { return op == CG_B200_REDUCE_MAX ? -INFINITY : 0.0f; }
__device__ __forceinline__ float red_apply(int op, float a, float b) { return op == CG_B200_REDUCE_MAX ? fmaxf(a, b) : a + b; }
__device__ __forceinline__ float red_finish(int op, float a, long long n) {
    return op == CG_B200_REDUCE_MEAN ? a / (float)n : a;
}
__device__ __forceinline__ float warp_reduce(int op, float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = red_apply(op, v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

// this lane's share of one contiguous row: 16-byte packets where the row's start allows, elements at the edges
template <typename T>
__device__ __forceinline__ float row_partial(const T* row, long long n, int op, int lane, int lanes) {
    constexpr int L = Vec16<T>::N;
    float acc = red_identity(op);
    const uintptr_t addr = reinterpret_cast<uintptr_t>(row);
    long long head = ((16 - (addr & 15)) & 15) / sizeof(T);   // elements before the first 16-byte boundary
    if (head > n) head = n;
    const long long packets = (n - head) / L;
    for (long long i = lane; i < head; i += lanes) acc = red_apply(op, acc, Elem<T>::to_f32(row[i]));
    const T* body = row + head;
    for (long long k = lane; k < packets; k += lanes) {
        float f[L];
        unpack16<T>(ld_stream<T>(body + k * L), f);
#pragma unroll
        for (int j = 0; j < L; ++j) acc = red_apply(op, acc, f[j]);
    }
    for (long long i = head + packets * L + lane; i < n; i += lanes) acc = red_apply(op, acc, Elem<T>::to_f32(row[i]));
    return acc;
}

// inner == 1, short rows: one warp per row
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_warp_kernel(ReduceParams p) {
    const T* in = static_cast<const T*>(p.in);
    T* out = static_cast<T*>(p.out);
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long step = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long row = warp0; row < p.outer; row += step) {
        const float v = warp_reduce(p.op, row_partial<T>(in + row * p.reduce, p.reduce, p.op, lane, 32));
        if (lane == 0) out[row] = Elem<T>::from_f32(red_finish(p.op, v, p.reduce));
    }
}

// inner == 1, long rows: one CTA per row
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_cta_kernel(ReduceParams p) {
    __shared__ float part[8];
    const T* in = static_cast<const T*>(p.in);
    T* out = static_cast<T*>(p.out);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long row = blockIdx.x; row < p.outer; row += gridDim.x) {
        float v = warp_reduce(p.op, row_partial<T>(in + row * p.reduce, p.reduce, p.op, (int)threadIdx.x, 256));
        if (lane == 0) part[warp] = v;
        __syncthreads();
        if (warp == 0) {
            v = warp_reduce(p.op, lane < 8 ? part[lane] : red_identity(p.op));
            if (lane == 0) out[row] = Elem<T>::from_f32(red_finish(p.op, v, p.reduce));
        }
        __syncthreads();
    }
}

// inner > 1: x runs along inner, y splits reduce
template <typename T>
__global__ void __launch_bounds__(256) reduce_strided_kernel(ReduceParams p, long long tiles_x) {
    __shared__ float part[8][32];
    const T* in = static_cast<const T*>(p.in);
    T* out = static_cast<T*>(p.out);
    const long long units = p.outer * tiles_x;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const long long o = u / tiles_x, i = (u % tiles_x) * 32 + threadIdx.x;
        float acc = red_identity(p.op);
        if (i < p.inner) {
            const T* base = in + o * p.reduce * p.inner + i;
            for (long long r = threadIdx.y; r < p.reduce; r += 8) acc = red_apply(p.op, acc, Elem<T>::to_f32(base[r * p.inner]));
        }
        part[threadIdx.y][threadIdx.x] = acc;
        __syncthreads();
        if (threadIdx.y == 0 && i < p.inner) {
#pragma unroll
            for (int y = 1; y < 8; ++y) acc = red_apply(p.op, acc, part[y][threadIdx.x]);
            out[o * p.inner + i] = Elem<T>::from_f32(red_finish(p.op, acc, p.reduce));
        }
        __syncthreads();
    }
}

template <typename T>
static int launch_reduce(const ReduceParams& p, cudaStream_t s) {
    const long long cap = (long long)sm_count() * 16;
    if (p.inner == 1) {
        if (p.reduce * (long long)sizeof(T) <= 8192) {   // up to sixteen 512-byte trips of a warp
            const long long blocks = (p.outer + 7) / 8;
            reduce_rows_warp_kernel<T><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(p);
        } else {
            reduce_rows_cta_kernel<T><<<(unsigned)(p.outer < cap ? p.outer : cap), 256, 0, s>>>(p);
        }
    } else {
        const long long tiles_x = (p.inner + 31) / 32;
        const long long units = p.outer * tiles_x;
        reduce_strided_kernel<T><<<(unsigned)(units < cap ? units : cap), dim3(32, 8), 0, s>>>(p, tiles_x);
    }
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}

}  // namespace cgb

extern "C" int cg_b200_reduce(int dtype, int op, const void* in, void* out, int64_t outer, int64_t reduce, int64_t inner,
                              void* stream) {
    using namespace cgb;
    if (!dtype_ok(dtype) || outer < 0 || reduce < 0 || inner < 0) return CG_B200_ERR_INVALID_ARG;
    if (op != CG_B200_REDUCE_SUM && op != CG_B200_REDUCE_MAX && op != CG_B200_REDUCE_MEAN) return CG_B200_ERR_INVALID_ARG;
    if (outer == 0 || inner == 0) return CG_B200_OK;           // nothing to write
    if (reduce == 0) return CG_B200_ERR_INVALID_ARG;           // no identity to write for max / mean of nothing
    if (!in || !out) return CG_B200_ERR_NULL_POINTER;
    const size_t esz = dtype_bytes(dtype);
    if (!aligned_to(in, esz) || !aligned_to(out, esz)) return CG_B200_ERR_MISALIGNED;
    int st = require_sm100();
    if (st) return st;
    const ReduceParams p{in, out, outer, reduce, inner, op};
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
        case CG_B200_F32: return launch_reduce<float>(p, s);
        case CG_B200_BF16: return launch_reduce<__nv_bfloat16>(p, s);
        default: return launch_reduce<__half>(p, s);
    }
}
