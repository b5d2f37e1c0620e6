// rowreduce.cu - last-axis softmax, layernorm and layernorm(softmax) in one HBM pass.
//
// The reference defines softmax and layernorm as attribute-less Tensor-IR ops over the last
// axis (src/ir/ops.cpp:536-556) but never executes them: lowering falls through to an
// "unknown opcode" Const (src/lowering/tensor_to_codegen.cpp:350-356) and the PTX emitter
// prints a comment for CGOpcode::Reduce (src/backend/ptx/ptx_emitter.cpp:136-142); its
// shuffle emission (ptx_emitter.cpp:165-189) is the only hint at a warp reduction.
// Definitions used: max-subtracted softmax (include/cg/egraph/rewrite_rules.hpp:96-101);
// layernorm = mean, biased variance, normalise, scale + shift
// (src/analysis/arithmetic_intensity.cpp:138-146).
//
// HBM-bound: algorithmic bytes per row = 2 * cols * sizeof(T) (read once, write once).
// Layout: [rows, cols] row-major. Register path: one CTA per row, the row lives in
// registers as fp32 (CHUNKS 16-byte packets per thread, packet j of thread t is packet
// j*THREADS + t of the row, so a warp reads 512 contiguous bytes); reductions are
// shfl.bfly inside a warp plus one shared-memory hop across warps. Rows that are too long
// or not 16-byte tiled take the streaming path, which re-reads the row (from L2) per pass.
#include <math.h>

#include "common.cuh"

namespace cgb {

enum RowMode { kSoftmax = 0, kLayerNorm = 1, kSoftmaxLayerNorm = 2 };

struct RowParams {
    const void* in;
    void* out;
    const void* gamma;
    const void* beta;
    long long rows;
    long long cols;
    float eps;
};

struct MaxOp {
    __device__ static float identity() { return -INFINITY; }
    __device__ static float apply(float a, float b) { return fmaxf(a, b); }
};
struct SumOp {
    __device__ static float identity() { return 0.0f; }
    __device__ static float apply(float a, float b) { return a + b; }
};

// All threads of the CTA get the reduction of v. `scratch` holds one float per warp; `phase`
// alternates between two scratch halves so back-to-back reductions need one barrier each.
template <typename Op, int THREADS>
__device__ __forceinline__ float block_reduce(float v, float* scratch, int& phase) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
    if constexpr (THREADS == 32) {
        return v;
    } else {
        constexpr int W = THREADS / 32;
        float* s = scratch + (phase & 1) * 32;
        phase ^= 1;
        if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
        __syncthreads();
        float r = (threadIdx.x & 31) < W ? s[threadIdx.x & 31] : Op::identity();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r = Op::apply(r, __shfl_xor_sync(0xffffffffu, r, o));
        return r;
    }
}

// exp(x - m) as ex2(x * log2(e) - m * log2(e)): one FMA and one MUFU per element. The relative
// error (about 2^-22 plus the rounding of the scaled argument) is far inside the path's 1e-4 bound.
constexpr float kLog2e = 1.4426950408889634f;

template <typename T, int THREADS, int CHUNKS, int MODE>
__global__ void __launch_bounds__(THREADS) row_reg_kernel(const __grid_constant__ RowParams p) {
    constexpr int L = 16 / sizeof(T);
    __shared__ float scratch[64];
    int phase = 0;
    const long long n_pkt = p.cols / L;  // cols % L == 0 on this path
    const float inv_cols = 1.0f / (float)p.cols;

    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T* in = static_cast<const T*>(p.in) + row * p.cols;
        T* out = static_cast<T*>(p.out) + row * p.cols;
        float x[CHUNKS][L];
        bool live[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j) {
            const long long pk = (long long)j * THREADS + threadIdx.x;
            live[j] = pk < n_pkt;
            if (live[j]) unpack16<T>(ld_stream(in + pk * L), x[j]);
        }

        if constexpr (MODE == kSoftmax || MODE == kSoftmaxLayerNorm) {
            float m = -INFINITY;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
#pragma unroll
                    for (int l = 0; l < L; ++l) m = fmaxf(m, x[j][l]);
                }
            m = block_reduce<MaxOp, THREADS>(m, scratch, phase);
            const float neg_m = -m * kLog2e;
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
#pragma unroll
                    for (int l = 0; l < L; ++l) {
                        x[j][l] = ex2_approx(fmaf(x[j][l], kLog2e, neg_m));
                        s += x[j][l];
                    }
                }
            s = block_reduce<SumOp, THREADS>(s, scratch, phase);
            const float inv = 1.0f / s;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
#pragma unroll
                    for (int l = 0; l < L; ++l) x[j][l] = x[j][l] * inv;
                    // the tensor between the two ops has storage type T
                    if constexpr (MODE == kSoftmaxLayerNorm) round_through16<T>(x[j]);
                }
        }

        if constexpr (MODE == kLayerNorm || MODE == kSoftmaxLayerNorm) {
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
#pragma unroll
                    for (int l = 0; l < L; ++l) s += x[j][l];
                }
            const float mean = block_reduce<SumOp, THREADS>(s, scratch, phase) * inv_cols;
            float q = 0.0f;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
#pragma unroll
                    for (int l = 0; l < L; ++l) {
                        x[j][l] -= mean;
                        q = fmaf(x[j][l], x[j][l], q);
                    }
                }
            const float var = block_reduce<SumOp, THREADS>(q, scratch, phase) * inv_cols;
            const float rstd = rsqrtf(var + p.eps);
            const T* gamma = static_cast<const T*>(p.gamma);
            const T* beta = static_cast<const T*>(p.beta);
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) {
                    const long long pk = (long long)j * THREADS + threadIdx.x;
#pragma unroll
                    for (int l = 0; l < L; ++l) x[j][l] *= rstd;
                    if (gamma) {
                        float g[L];
                        unpack16<T>(ld_keep(gamma + pk * L), g);
#pragma unroll
                        for (int l = 0; l < L; ++l) x[j][l] *= g[l];
                    }
                    if (beta) {
                        float b[L];
                        unpack16<T>(ld_keep(beta + pk * L), b);
#pragma unroll
                        for (int l = 0; l < L; ++l) x[j][l] += b[l];
                    }
                }
        }

#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) {
                const long long pk = (long long)j * THREADS + threadIdx.x;
                st_stream(out + pk * L, pack16<T>(x[j]));
            }
    }
}

// ---- fused layernorm(softmax(x)), register path, packed arithmetic ---------------------------------
// This kernel is issue-bound before it is HBM-bound (the first version spent 23 instructions per
// element), so its inner loops work on pairs: fp32x2 add / mul / fma (one issue slot for two
// elements on sm_100), bf16x2 / f16x2 max on the raw input words, two-element pack/unpack.
// The layernorm statistics are taken about c = 1/cols, the mean a softmax row has before rounding:
// sum(p - c) and sum((p - c)^2) come out of ONE block reduction, and with the shift the one-pass
// variance has no cancellation (the correction term (mean - c)^2 is rounding noise).
struct Sum2Op {
    __device__ static float2 apply(float2 a, float2 b) { return __fadd2_rn(a, b); }
};

template <int THREADS>
__device__ __forceinline__ float2 block_reduce_sum2(float2 v, float2* scratch, int& phase) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float2 t;
        t.x = __shfl_xor_sync(0xffffffffu, v.x, o);
        t.y = __shfl_xor_sync(0xffffffffu, v.y, o);
        v = __fadd2_rn(v, t);
    }
    if constexpr (THREADS == 32) {
        return v;
    } else {
        constexpr int W = THREADS / 32;
        float2* sc = scratch + (phase & 1) * 32;
        phase ^= 1;
        if ((threadIdx.x & 31) == 0) sc[threadIdx.x >> 5] = v;
        __syncthreads();
        float2 r = sc[threadIdx.x & (W - 1)];      // every lane reads one of the W partials
#pragma unroll
        for (int o = W / 2; o > 0; o >>= 1) {       // butterfly over W lanes: all lanes end with the total
            float2 t;
            t.x = __shfl_xor_sync(0xffffffffu, r.x, o);
            t.y = __shfl_xor_sync(0xffffffffu, r.y, o);
            r = __fadd2_rn(r, t);
        }
        return r;
    }
}

template <typename Op, int THREADS>
__device__ __forceinline__ float block_reduce_fast(float v, float* scratch, int& phase) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
    if constexpr (THREADS == 32) {
        return v;
    } else {
        constexpr int W = THREADS / 32;
        float* sc = scratch + (phase & 1) * 32;
        phase ^= 1;
        if ((threadIdx.x & 31) == 0) sc[threadIdx.x >> 5] = v;
        __syncthreads();
        float r = sc[threadIdx.x & (W - 1)];
#pragma unroll
        for (int o = W / 2; o > 0; o >>= 1) r = Op::apply(r, __shfl_xor_sync(0xffffffffu, r, o));
        return r;
    }
}

// packet -> L/2 fp32 pairs
template <typename T>
__device__ __forceinline__ void unpack_pairs(const Vec16<T>& v, float2 (&f)[Vec16<T>::N / 2]) {
    if constexpr (sizeof(T) == 4) {
        f[0] = make_float2(v.v[0], v.v[1]);
        f[1] = make_float2(v.v[2], v.v[3]);
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) f[l] = make_float2(__uint_as_float(w[l] << 16), __uint_as_float(w[l] & 0xffff0000u));
    } else {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) f[l] = __half22float2(h[l]);
    }
}

// fp32 pair -> rounded to T and back
template <typename T>
__device__ __forceinline__ float2 round_pair(float2 a) {
    if constexpr (sizeof(T) == 4) {
        return a;
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a.x, a.y);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    } else {
        return __half22float2(__floats2half2_rn(a.x, a.y));
    }
}

template <typename T>
__device__ __forceinline__ Vec16<T> pack_pairs(const float2 (&f)[Vec16<T>::N / 2]) {
    Vec16<T> v;
    if constexpr (sizeof(T) == 4) {
        v.v[0] = f[0].x; v.v[1] = f[0].y; v.v[2] = f[1].x; v.v[3] = f[1].y;
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) h[l] = __floats2bfloat162_rn(f[l].x, f[l].y);
    } else {
        __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
        for (int l = 0; l < 4; ++l) h[l] = __floats2half2_rn(f[l].x, f[l].y);
    }
    return v;
}

// max over the 16 bytes of a packet, on the packed words where the type allows it
template <typename T>
__device__ __forceinline__ float packet_max(const Vec16<T>& v) {
    if constexpr (sizeof(T) == 4) {
        return fmaxf(fmaxf(v.v[0], v.v[1]), fmaxf(v.v[2], v.v[3]));
    } else if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const __nv_bfloat162 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        return fmaxf(__bfloat162float(m.x), __bfloat162float(m.y));
    } else {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        return fmaxf(__half2float(m.x), __half2float(m.y));
    }
}

// FULL: the row is exactly THREADS * CHUNKS packets, so no packet needs a bounds predicate (the
// predicates and the re-convergence points around them were a seventh of the instructions issued,
// and this kernel is bound by instruction issue, not by DRAM).
// AFFINE: gamma or beta is given. Without them their code must not exist at all: the compiler turns the
// "if (gamma)" blocks into predicated instructions, which are issued (and counted) even when the
// predicate is false - a quarter of this kernel's issue slots.
template <typename T, int THREADS, int CHUNKS, int MIN_CTAS, bool FULL, bool AFFINE>
__global__ void __launch_bounds__(THREADS, MIN_CTAS) softmax_layernorm_reg_kernel(const __grid_constant__ RowParams p) {
    constexpr int L = 16 / sizeof(T);
    constexpr int P = L / 2;   // pairs per packet
    __shared__ float scratch[64];
    __shared__ float2 scratch2[64];
    int phase = 0, phase2 = 0;
    const long long n_pkt = p.cols / L;
    const float inv_cols = 1.0f / (float)p.cols;
    const float2 log2e2 = make_float2(kLog2e, kLog2e);
    const float2 neg_c2 = make_float2(-inv_cols, -inv_cols);
    const T* gamma = static_cast<const T*>(p.gamma);
    const T* beta = static_cast<const T*>(p.beta);

    // Persistent over rows with a one-row software prefetch: the next row's packets are requested
    // into their own registers before the current row's three dependent reductions, so the CTA
    // always has HBM requests in flight (without it the memory pipe idles while the CTA computes;
    // issuing the prefetch later, into the registers the unpack frees, measured far slower).
    bool live[CHUNKS];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) live[j] = FULL || (long long)j * THREADS + threadIdx.x < n_pkt;
    Vec16<T> raw[CHUNKS], nxt[CHUNKS];
    long long row = blockIdx.x;
    if (row < p.rows) {
        const T* in0 = static_cast<const T*>(p.in) + row * p.cols;
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) raw[j] = ld_stream(in0 + ((long long)j * THREADS + threadIdx.x) * L);
    }
    // one row: `cur` holds it, `nx` receives the row after it (the two buffers swap roles from row to
    // row, so no packet is copied between registers)
    auto one_row = [&](Vec16<T> (&raw)[CHUNKS], Vec16<T> (&nxt)[CHUNKS], long long row) {
        T* out = static_cast<T*>(p.out) + row * p.cols;
        const long long row_next = row + gridDim.x;
        if (row_next < p.rows) {
            const T* in_next = static_cast<const T*>(p.in) + row_next * p.cols;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j)
                if (live[j]) nxt[j] = ld_stream(in_next + ((long long)j * THREADS + threadIdx.x) * L);
        }
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) m = fmaxf(m, packet_max<T>(raw[j]));
        m = block_reduce_fast<MaxOp, THREADS>(m, scratch, phase);

        const float nm = -m * kLog2e;
        const float2 neg_m2 = make_float2(nm, nm);
        float2 x[CHUNKS][P];
        float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) {
                unpack_pairs<T>(raw[j], x[j]);
#pragma unroll
                for (int l = 0; l < P; ++l) {
                    const float2 t = __ffma2_rn(x[j][l], log2e2, neg_m2);
                    x[j][l] = make_float2(ex2_approx(t.x), ex2_approx(t.y));
                    s2 = __fadd2_rn(s2, x[j][l]);
                }
            }
        const float ssum = block_reduce_fast<SumOp, THREADS>(s2.x + s2.y, scratch, phase);
        const float inv = 1.0f / ssum;
        const float2 inv2 = make_float2(inv, inv);

        // p = e / sum rounded to the storage type; d = p - c; one reduction for sum(d), sum(d^2)
        float2 sd = make_float2(0.0f, 0.0f), sq = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) {
#pragma unroll
                for (int l = 0; l < P; ++l) {
                    const float2 pr = round_pair<T>(__fmul2_rn(x[j][l], inv2));
                    const float2 d = __fadd2_rn(pr, neg_c2);
                    x[j][l] = d;
                    sd = __fadd2_rn(sd, d);
                    sq = __ffma2_rn(d, d, sq);
                }
            }
        const float2 tot = block_reduce_sum2<THREADS>(make_float2(sd.x + sd.y, sq.x + sq.y), scratch2, phase2);
        const float dm = tot.x * inv_cols;                       // mean - c
        const float var = fmaxf(tot.y * inv_cols - dm * dm, 0.0f);
        const float rstd = rsqrtf(var + p.eps);
        const float2 rstd2 = make_float2(rstd, rstd);
        const float sh = -dm * rstd;
        const float2 shift2 = make_float2(sh, sh);
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j)
            if (live[j]) {
                const long long pk = (long long)j * THREADS + threadIdx.x;
#pragma unroll
                for (int l = 0; l < P; ++l) x[j][l] = __ffma2_rn(x[j][l], rstd2, shift2);
                if constexpr (AFFINE) {
                    if (gamma) {
                        float2 g[P];
                        unpack_pairs<T>(ld_keep(gamma + pk * L), g);
#pragma unroll
                        for (int l = 0; l < P; ++l) x[j][l] = __fmul2_rn(x[j][l], g[l]);
                    }
                    if (beta) {
                        float2 b[P];
                        unpack_pairs<T>(ld_keep(beta + pk * L), b);
#pragma unroll
                        for (int l = 0; l < P; ++l) x[j][l] = __fadd2_rn(x[j][l], b[l]);
                    }
                }
                st_stream(out + pk * L, pack_pairs<T>(x[j]));
            }
    };
    for (; row < p.rows; row += 2LL * gridDim.x) {
        one_row(raw, nxt, row);
        if (row + gridDim.x < p.rows) one_row(nxt, raw, row + gridDim.x);
    }
}

// Streaming path: any cols, element-aligned. One CTA per row, several passes over the row.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) row_stream_kernel(const __grid_constant__ RowParams p) {
    constexpr int THREADS = 256;
    __shared__ float scratch[64];
    int phase = 0;
    const float inv_cols = 1.0f / (float)p.cols;
    const T* gamma = static_cast<const T*>(p.gamma);
    const T* beta = static_cast<const T*>(p.beta);
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T* in = static_cast<const T*>(p.in) + row * p.cols;
        T* out = static_cast<T*>(p.out) + row * p.cols;
        float m = 0.0f, inv = 1.0f;
        if constexpr (MODE != kLayerNorm) {
            m = -INFINITY;
            for (long long c = threadIdx.x; c < p.cols; c += THREADS) m = fmaxf(m, Elem<T>::to_f32(in[c]));
            m = block_reduce<MaxOp, THREADS>(m, scratch, phase);
            float s = 0.0f;
            for (long long c = threadIdx.x; c < p.cols; c += THREADS)
                s += ex2_approx(fmaf(Elem<T>::to_f32(in[c]), kLog2e, -m * kLog2e));
            s = block_reduce<SumOp, THREADS>(s, scratch, phase);
            inv = 1.0f / s;
        }
        // value of the tensor that enters the layernorm stage (or the softmax result)
        auto staged = [&](long long c) -> float {
            float v = Elem<T>::to_f32(in[c]);
            if constexpr (MODE != kLayerNorm) v = ex2_approx(fmaf(v, kLog2e, -m * kLog2e)) * inv;
            if constexpr (MODE == kSoftmaxLayerNorm) v = Elem<T>::to_f32(Elem<T>::from_f32(v));
            return v;
        };
        if constexpr (MODE == kSoftmax) {
            // `in == out` is allowed: every element is read and written by the same thread
            for (long long c = threadIdx.x; c < p.cols; c += THREADS) out[c] = Elem<T>::from_f32(staged(c));
        } else {
            float s = 0.0f;
            for (long long c = threadIdx.x; c < p.cols; c += THREADS) s += staged(c);
            const float mean = block_reduce<SumOp, THREADS>(s, scratch, phase) * inv_cols;
            float q = 0.0f;
            for (long long c = threadIdx.x; c < p.cols; c += THREADS) {
                const float d = staged(c) - mean;
                q += d * d;
            }
            const float var = block_reduce<SumOp, THREADS>(q, scratch, phase) * inv_cols;
            const float rstd = rsqrtf(var + p.eps);
            __syncthreads();  // all reads of `in` for the statistics are done before any in-place write
            for (long long c = threadIdx.x; c < p.cols; c += THREADS) {
                float t = (staged(c) - mean) * rstd;
                if (gamma) t = t * Elem<T>::to_f32(gamma[c]);
                if (beta) t = t + Elem<T>::to_f32(beta[c]);
                out[c] = Elem<T>::from_f32(t);
            }
        }
    }
}

template <typename T, int THREADS, int CHUNKS, int MODE>
static void launch_reg(const RowParams& p, int blocks, cudaStream_t s) {
    if constexpr (MODE == kSoftmaxLayerNorm)
        {
        // persistent: the prefetching loop wants several rows per CTA
        constexpr int kMinCtas = 512 / THREADS > 0 ? 512 / THREADS : 1;   // 4 CTAs of 128 threads: no spills
        const long long cap = (long long)sm_count() * 8;
        const int g = (int)(p.rows < cap ? p.rows : cap);
        (void)blocks;
        constexpr int L = 16 / sizeof(T);
        const bool full = p.cols / L == (long long)THREADS * CHUNKS, affine = p.gamma || p.beta;
        if (full && !affine) softmax_layernorm_reg_kernel<T, THREADS, CHUNKS, kMinCtas, true, false><<<g, THREADS, 0, s>>>(p);
        else if (full) softmax_layernorm_reg_kernel<T, THREADS, CHUNKS, kMinCtas, true, true><<<g, THREADS, 0, s>>>(p);
        else if (!affine) softmax_layernorm_reg_kernel<T, THREADS, CHUNKS, kMinCtas, false, false><<<g, THREADS, 0, s>>>(p);
        else softmax_layernorm_reg_kernel<T, THREADS, CHUNKS, kMinCtas, false, true><<<g, THREADS, 0, s>>>(p);
    }
    else
        row_reg_kernel<T, THREADS, CHUNKS, MODE><<<blocks, THREADS, 0, s>>>(p);
}

template <typename T, int MODE>
static int launch_mode(const RowParams& p, cudaStream_t s) {
    constexpr int L = 16 / sizeof(T);
    const long long n_pkt = p.cols / L;
    bool vec = (p.cols % L) == 0 && aligned_to(p.in, 16) && aligned_to(p.out, 16) &&
               (!p.gamma || aligned_to(p.gamma, 16)) && (!p.beta || aligned_to(p.beta, 16));
    const long long max_blocks = (long long)sm_count() * 32;
    const int blocks = (int)(p.rows < max_blocks ? p.rows : max_blocks);
    if (vec && n_pkt <= 32) launch_reg<T, 32, 1, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 64) launch_reg<T, 64, 1, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 128) launch_reg<T, 128, 1, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 256) launch_reg<T, 128, 2, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 512) launch_reg<T, 128, 4, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 1024) launch_reg<T, 256, 4, MODE>(p, blocks, s);
    else if (vec && n_pkt <= 2048) launch_reg<T, 512, 4, MODE>(p, blocks, s);
    else row_stream_kernel<T, MODE><<<blocks, 256, 0, s>>>(p);
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}

static int row_entry(int mode, int dtype, const void* in, const void* gamma, const void* beta, float eps, void* out,
                     int64_t rows, int64_t cols, void* stream) {
    if (!dtype_ok(dtype) || rows < 0 || cols < 0) return CG_B200_ERR_INVALID_ARG;
    if (mode != kSoftmax && !(eps >= 0.0f)) return CG_B200_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return CG_B200_OK;
    if (!in || !out) return CG_B200_ERR_NULL_POINTER;
    const size_t esz = dtype_bytes(dtype);
    if (!aligned_to(in, esz) || !aligned_to(out, esz) || !aligned_to(gamma, esz) || !aligned_to(beta, esz))
        return CG_B200_ERR_MISALIGNED;
    int st = require_sm100();
    if (st) return st;
    RowParams p{in, out, gamma, beta, rows, cols, eps};
    cudaStream_t s = (cudaStream_t)stream;
#define CGB_ROW_DISPATCH(T)                                                     \
    switch (mode) {                                                             \
        case kSoftmax: return launch_mode<T, kSoftmax>(p, s);                   \
        case kLayerNorm: return launch_mode<T, kLayerNorm>(p, s);               \
        default: return launch_mode<T, kSoftmaxLayerNorm>(p, s);                \
    }
    switch (dtype) {
        case CG_B200_F32: CGB_ROW_DISPATCH(float)
        case CG_B200_BF16: CGB_ROW_DISPATCH(__nv_bfloat16)
        default: CGB_ROW_DISPATCH(__half)
    }
#undef CGB_ROW_DISPATCH
}

}  // namespace cgb

extern "C" int cg_b200_softmax(int dtype, const void* in, void* out, int64_t rows, int64_t cols, void* stream) {
    return cgb::row_entry(cgb::kSoftmax, dtype, in, nullptr, nullptr, 0.0f, out, rows, cols, stream);
}

extern "C" int cg_b200_layernorm(int dtype, const void* in, const void* gamma, const void* beta, float eps, void* out,
                                 int64_t rows, int64_t cols, void* stream) {
    return cgb::row_entry(cgb::kLayerNorm, dtype, in, gamma, beta, eps, out, rows, cols, stream);
}

extern "C" int cg_b200_softmax_layernorm(int dtype, const void* in, const void* gamma, const void* beta, float eps,
                                         void* out, int64_t rows, int64_t cols, void* stream) {
    return cgb::row_entry(cgb::kSoftmaxLayerNorm, dtype, in, gamma, beta, eps, out, rows, cols, stream);
}
