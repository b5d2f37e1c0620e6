// eltwise.cu - fused elementwise chains: one HBM pass per chain, 128-bit accesses.
//
// Stands where the reference lowers each Tensor-IR elementwise op to one un-looped
// VectorLoad / Add|Mul / VectorStore group (src/lowering/tensor_to_codegen.cpp:60-135) and
// prints straight-line ld/st PTX for it (src/backend/ptx/ptx_emitter.cpp:60-232). The
// executable anchor for the arithmetic is the reference's hand-built x86 loop kernels
// (benchmarks/benchmark_multithread.py:54-124): separately rounded mul / add / max.
//
// HBM-bound: algorithmic bytes per element = (number of full-size inputs + 1) * sizeof(T).
// Layout: every operand is a flat row-major array; a thread owns one 16-byte packet per operand.
//
// The chain is a postfix program. Two evaluators share one code path:
//   - compile-time programs (a table of common chains): the evaluation loop unrolls and the
//     value stack turns into plain registers;
//   - the run-time interpreter for everything else: the stack is four register slots that
//     shift on push/pop, so there is no indexed local memory.
#include <string.h>

#include "common.cuh"

namespace cgb {

struct EltParams {
    const void* in[CG_B200_EW_MAX_INPUTS];
    void* out;
    unsigned long long n;        // elements
    long long inner;             // broadcast period
    int n_instr;
    int round_each_op;
    unsigned char op[CG_B200_EW_MAX_INSTR];
    unsigned char arg[CG_B200_EW_MAX_INSTR];
    float imm[CG_B200_EW_MAX_INSTR];
    unsigned char bcast[CG_B200_EW_MAX_INPUTS];
};

// ---- program views ----------------------------------------------------------------------------
struct DynProg {
    static constexpr bool kStatic = false;
    const EltParams& p;
    __device__ explicit DynProg(const EltParams& q) : p(q) {}
    __device__ int n() const { return p.n_instr; }
    __device__ int op(int i) const { return p.op[i]; }
    __device__ int arg(int i) const { return p.arg[i]; }
};

// Compile-time chains. Immediates and dtypes stay run-time values; only the op/arg sequence
// is fixed. All inputs of a static chain are full-size (no broadcast).
template <int... Code>
struct StaticProg {
    static constexpr bool kStatic = true;
    static constexpr int kN = sizeof...(Code) / 2;
    __host__ __device__ static constexpr int code(int i) {
        constexpr int c[sizeof...(Code)] = {Code...};
        return c[i];
    }
    __host__ __device__ explicit StaticProg(const EltParams&) {}
    __host__ __device__ constexpr int n() const { return kN; }
    __host__ __device__ constexpr int op(int i) const { return code(2 * i); }
    __host__ __device__ constexpr int arg(int i) const { return code(2 * i + 1); }
};

#define EW_IN(i) CG_B200_EW_INPUT, i
#define EW_OP(o) o, 0
// relu(a*b + c) * s
using ProgMulAddReluScale = StaticProg<EW_IN(0), EW_IN(1), EW_OP(CG_B200_EW_MUL), EW_IN(2), EW_OP(CG_B200_EW_ADD),
                                       EW_OP(CG_B200_EW_RELU), EW_OP(CG_B200_EW_IMM), EW_OP(CG_B200_EW_MUL)>;
using ProgAdd = StaticProg<EW_IN(0), EW_IN(1), EW_OP(CG_B200_EW_ADD)>;
using ProgMul = StaticProg<EW_IN(0), EW_IN(1), EW_OP(CG_B200_EW_MUL)>;
using ProgMulRelu = StaticProg<EW_IN(0), EW_IN(1), EW_OP(CG_B200_EW_MUL), EW_OP(CG_B200_EW_RELU)>;
using ProgMulAdd = StaticProg<EW_IN(0), EW_IN(1), EW_OP(CG_B200_EW_MUL), EW_IN(2), EW_OP(CG_B200_EW_ADD)>;
using ProgRelu = StaticProg<EW_IN(0), EW_OP(CG_B200_EW_RELU)>;
using ProgGelu = StaticProg<EW_IN(0), EW_OP(CG_B200_EW_GELU_TANH)>;

// ---- one op on L lanes ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float rnd_store(float v, bool rnd) {
    if constexpr (sizeof(T) == 4) {
        return v;
    } else {
        return rnd ? Elem<T>::to_f32(Elem<T>::from_f32(v)) : v;
    }
}

__device__ __forceinline__ float apply_binary(int op, float a, float b) {
    switch (op) {
        case CG_B200_EW_ADD: return __fadd_rn(a, b);
        case CG_B200_EW_SUB: return __fsub_rn(a, b);
        case CG_B200_EW_MUL: return __fmul_rn(a, b);
        case CG_B200_EW_DIV: return __fdiv_rn(a, b);
        case CG_B200_EW_MAX: return a > b ? a : b;
        default: return a < b ? a : b;
    }
}

__device__ __forceinline__ float apply_unary(int op, float a) {
    switch (op) {
        case CG_B200_EW_NEG: return -a;
        case CG_B200_EW_ABS: return fabsf(a);
        case CG_B200_EW_RELU: return a > 0.0f ? a : 0.0f;
        case CG_B200_EW_GELU_TANH: return gelu_tanh_f32(a);
        case CG_B200_EW_TANH: return tanhf(a);
        case CG_B200_EW_SIGMOID: return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-a)));
        case CG_B200_EW_EXP: return expf(a);
        case CG_B200_EW_LOG: return logf(a);
        case CG_B200_EW_SQRT: return __fsqrt_rn(a);
        default: return __fdiv_rn(1.0f, __fsqrt_rn(a));
    }
}

// Load L consecutive elements of input `which` for output elements [e0, e0 + L).
// kVector: e0 is a multiple of L, L*sizeof(T) == 16 and full-size inputs are 16-byte aligned.
template <typename T, int L, bool kVector>
__device__ __forceinline__ void load_lanes(const EltParams& p, int which, unsigned long long e0, float (&dst)[L]) {
    const T* base = static_cast<const T*>(p.in[which]);
    const int kind = p.bcast[which];
    if (kind == CG_B200_BC_FULL) {
        if constexpr (kVector) {
            Vec16<T> v = ld_stream(base + e0);
#pragma unroll
            for (int l = 0; l < L; ++l) dst[l] = Elem<T>::to_f32(v.v[l]);
        } else {
#pragma unroll
            for (int l = 0; l < L; ++l) dst[l] = Elem<T>::to_f32(base[e0 + l]);
        }
    } else if (kind == CG_B200_BC_SCALAR) {
        float s = Elem<T>::to_f32(__ldg(base));
#pragma unroll
        for (int l = 0; l < L; ++l) dst[l] = s;
    } else if (kind == CG_B200_BC_ROW) {
        unsigned long long inner = (unsigned long long)p.inner;
        unsigned long long c0 = e0 % inner;
        if (kVector && (inner % L) == 0 && ((reinterpret_cast<uintptr_t>(base) & 15) == 0)) {
            Vec16<T> v = ld_keep(base + c0);
#pragma unroll
            for (int l = 0; l < L; ++l) dst[l] = Elem<T>::to_f32(v.v[l]);
        } else {
#pragma unroll
            for (int l = 0; l < L; ++l) {
                unsigned long long c = c0 + l;
                if (c >= inner) c %= inner;
                dst[l] = Elem<T>::to_f32(__ldg(base + c));
            }
        }
    } else {  // BC_COL
        unsigned long long inner = (unsigned long long)p.inner;
        unsigned long long r0 = e0 / inner;
        unsigned long long left = inner - (e0 - r0 * inner);  // elements left in this row
#pragma unroll
        for (int l = 0; l < L; ++l) {
            unsigned long long r = r0;
            if ((unsigned long long)l >= left) r = (e0 + l) / inner;
            dst[l] = Elem<T>::to_f32(__ldg(base + r));
        }
    }
}

// Evaluate the program for L lanes starting at element e0. Result in res[].
template <typename T, int L, bool kVector, typename Prog>
__device__ __forceinline__ void eval_lanes(const EltParams& p, const Prog& prog, unsigned long long e0,
                                           float (&res)[L]) {
    float s0[L], s1[L], s2[L], s3[L];
#pragma unroll
    for (int l = 0; l < L; ++l) s0[l] = s1[l] = s2[l] = s3[l] = 0.0f;
    const bool rnd = sizeof(T) == 2 && p.round_each_op != 0;
    auto push = [&](const float (&v)[L]) {
#pragma unroll
        for (int l = 0; l < L; ++l) {
            s3[l] = s2[l];
            s2[l] = s1[l];
            s1[l] = s0[l];
            s0[l] = v[l];
        }
    };
    auto step = [&](int i) {
        const int op = prog.op(i);
        if (op == CG_B200_EW_INPUT) {
            float v[L];
            load_lanes<T, L, kVector>(p, prog.arg(i), e0, v);
            push(v);
        } else if (op == CG_B200_EW_IMM) {
            float v[L];
            float c = rnd_store<T>(p.imm[i], rnd);
#pragma unroll
            for (int l = 0; l < L; ++l) v[l] = c;
            push(v);
        } else if (op <= CG_B200_EW_MIN) {
#pragma unroll
            for (int l = 0; l < L; ++l) {
                s0[l] = rnd_store<T>(apply_binary(op, s1[l], s0[l]), rnd);
                s1[l] = s2[l];
                s2[l] = s3[l];
            }
        } else {
#pragma unroll
            for (int l = 0; l < L; ++l) s0[l] = rnd_store<T>(apply_unary(op, s0[l]), rnd);
        }
    };
    if constexpr (Prog::kStatic) {
#pragma unroll
        for (int i = 0; i < Prog::kN; ++i) step(i);
    } else {
        const int n = prog.n();
#pragma unroll 1
        for (int i = 0; i < n; ++i) step(i);
    }
#pragma unroll
    for (int l = 0; l < L; ++l) res[l] = s0[l];
}

// One 16-byte packet per thread per trip; the ragged tail (n % L elements) is done scalar by
// block 0. The grid normally covers the whole array (see launch_typed), so most threads make one
// trip: with the registers of a single packet the kernel runs at full occupancy, which measured
// faster on B200 than two packets per thread at half occupancy.
// A 16-bit packet is eight fp32 lanes per stack slot. The run-time interpreter for those types keeps four slots
// alive and spilled heavily under the 32 registers of eight resident CTAs (0.85 TB/s on gelu(a*b)+c in bf16); built
// for four CTAs (64 registers) it runs at 1.9 TB/s. The compile-time chains spill a few words at 32 registers and
// measured the same or faster that way (4.6 vs 4.2 TB/s on relu(a*b+c)*s in bf16), so they keep eight.
template <typename T, typename Prog>
constexpr int vec_min_ctas() { return (sizeof(T) == 2 && !Prog::kStatic) ? 4 : 8; }

template <typename T, typename Prog>
__global__ void __launch_bounds__(256, (vec_min_ctas<T, Prog>())) eltwise_vec_kernel(const __grid_constant__ EltParams p) {
    constexpr int L = 16 / sizeof(T);
    const Prog prog(p);
    T* out = static_cast<T*>(p.out);
    const unsigned long long n_pkt = p.n / L;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long v = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_pkt; v += stride) {
        float r0[L];
        eval_lanes<T, L, true>(p, prog, v * L, r0);
        Vec16<T> o0;
#pragma unroll
        for (int l = 0; l < L; ++l) o0.v[l] = Elem<T>::from_f32(r0[l]);
        st_stream(out + v * L, o0);
    }
    if (blockIdx.x == 0) {
        unsigned long long e = n_pkt * L + threadIdx.x;
        if (e < p.n) {
            float r[1];
            eval_lanes<T, 1, false>(p, prog, e, r);
            out[e] = Elem<T>::from_f32(r[0]);
        }
    }
}

// Element-aligned fallback when a pointer is not 16-byte aligned.
template <typename T, typename Prog>
__global__ void __launch_bounds__(256) eltwise_scalar_kernel(const __grid_constant__ EltParams p) {
    const Prog prog(p);
    T* out = static_cast<T*>(p.out);
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < p.n; e += stride) {
        float r[1];
        eval_lanes<T, 1, false>(p, prog, e, r);
        out[e] = Elem<T>::from_f32(r[0]);
    }
}

// ---- host side ----------------------------------------------------------------------------------
static int validate(const cg_b200_eltwise_desc* d, int n_inputs) {
    if (!d) return CG_B200_ERR_NULL_POINTER;
    if (!dtype_ok(d->dtype)) return CG_B200_ERR_INVALID_ARG;
    if (d->n_instr < 1 || d->n_instr > CG_B200_EW_MAX_INSTR) return CG_B200_ERR_INVALID_ARG;
    if (n_inputs < 0 || n_inputs > CG_B200_EW_MAX_INPUTS) return CG_B200_ERR_INVALID_ARG;
    if (d->inner < 1) return CG_B200_ERR_INVALID_ARG;
    int depth = 0;
    for (int i = 0; i < d->n_instr; ++i) {
        const int op = d->prog[i].op;
        if (op < 0 || op >= CG_B200_EW_OP_COUNT) return CG_B200_ERR_INVALID_ARG;
        if (op == CG_B200_EW_INPUT) {
            const int a = d->prog[i].arg;
            if (a < 0 || a >= n_inputs) return CG_B200_ERR_INVALID_ARG;
            if (d->bcast[a] < CG_B200_BC_FULL || d->bcast[a] > CG_B200_BC_COL) return CG_B200_ERR_INVALID_ARG;
            ++depth;
        } else if (op == CG_B200_EW_IMM) {
            ++depth;
        } else if (op <= CG_B200_EW_MIN) {
            if (depth < 2) return CG_B200_ERR_INVALID_ARG;
            --depth;
        } else if (depth < 1) {
            return CG_B200_ERR_INVALID_ARG;
        }
        if (depth > CG_B200_EW_MAX_STACK) return CG_B200_ERR_INVALID_ARG;
    }
    return depth == 1 ? CG_B200_OK : CG_B200_ERR_INVALID_ARG;
}

template <typename Prog>
static bool matches(const EltParams& p) {
    if (p.n_instr != Prog::kN) return false;
    for (int i = 0; i < Prog::kN; ++i) {
        if (p.op[i] != Prog::code(2 * i)) return false;
        if (p.op[i] == CG_B200_EW_INPUT) {
            if (p.arg[i] != Prog::code(2 * i + 1)) return false;
            if (p.bcast[p.arg[i]] != CG_B200_BC_FULL) return false;
        }
    }
    return true;
}

template <typename T, typename Prog>
static void launch_vec(const EltParams& p, int blocks, cudaStream_t s) {
    eltwise_vec_kernel<T, Prog><<<blocks, 256, 0, s>>>(p);
}

template <typename T>
static int launch_typed(const EltParams& p, bool vector_ok, cudaStream_t s) {
    const int sms = sm_count();
    if (!vector_ok) {
        unsigned long long want = (p.n + 255) / 256;
        int blocks = (int)(want < (unsigned long long)sms * 8 ? want : (unsigned long long)sms * 8);
        eltwise_scalar_kernel<T, DynProg><<<blocks, 256, 0, s>>>(p);
        CGB_CUDA(cudaGetLastError());
        return CG_B200_OK;
    }
    constexpr int L = 16 / sizeof(T);
    // One thread per packet. Measured on B200: for this streaming pattern a grid that covers the
    // whole array (tens of thousands of short-lived CTAs) sustains about 10 % more HBM bandwidth
    // than a persistent grid of 8 CTAs per SM; the grid-stride loop only matters when the array
    // exceeds the grid limit.
    (void)sms;
    unsigned long long want = (p.n / L + 255) / 256;
    const unsigned long long cap = 0x7fffffffull;
    int blocks = (int)(want < cap ? (want == 0 ? 1 : want) : cap);
    if (matches<ProgMulAddReluScale>(p)) launch_vec<T, ProgMulAddReluScale>(p, blocks, s);
    else if (matches<ProgAdd>(p)) launch_vec<T, ProgAdd>(p, blocks, s);
    else if (matches<ProgMul>(p)) launch_vec<T, ProgMul>(p, blocks, s);
    else if (matches<ProgMulRelu>(p)) launch_vec<T, ProgMulRelu>(p, blocks, s);
    else if (matches<ProgMulAdd>(p)) launch_vec<T, ProgMulAdd>(p, blocks, s);
    else if (matches<ProgRelu>(p)) launch_vec<T, ProgRelu>(p, blocks, s);
    else if (matches<ProgGelu>(p)) launch_vec<T, ProgGelu>(p, blocks, s);
    else launch_vec<T, DynProg>(p, blocks, s);
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}

}  // namespace cgb

using namespace cgb;

extern "C" int cg_b200_eltwise_validate(const cg_b200_eltwise_desc* desc, int n_inputs) {
    return validate(desc, n_inputs);
}

extern "C" int cg_b200_eltwise(const cg_b200_eltwise_desc* desc, const void* const* inputs, int n_inputs,
                               void* out, size_t n, void* stream) {
    int st = validate(desc, n_inputs);
    if (st) return st;
    if (n == 0) return CG_B200_OK;
    if (!inputs || !out) return CG_B200_ERR_NULL_POINTER;
    const size_t esz = dtype_bytes(desc->dtype);
    EltParams p;
    memset(&p, 0, sizeof(p));
    bool vector_ok = aligned_to(out, 16);
    if (!aligned_to(out, esz)) return CG_B200_ERR_MISALIGNED;
    for (int i = 0; i < n_inputs; ++i) {
        if (!inputs[i]) return CG_B200_ERR_NULL_POINTER;
        if (!aligned_to(inputs[i], esz)) return CG_B200_ERR_MISALIGNED;
        if (desc->bcast[i] == CG_B200_BC_FULL && !aligned_to(inputs[i], 16)) vector_ok = false;
        p.in[i] = inputs[i];
        p.bcast[i] = (unsigned char)desc->bcast[i];
    }
    p.out = out;
    p.n = n;
    p.inner = desc->inner;
    p.n_instr = desc->n_instr;
    p.round_each_op = desc->round_each_op;
    for (int i = 0; i < desc->n_instr; ++i) {
        p.op[i] = (unsigned char)desc->prog[i].op;
        p.arg[i] = (unsigned char)desc->prog[i].arg;
        p.imm[i] = desc->prog[i].imm;
    }
    st = require_sm100();
    if (st) return st;
    cudaStream_t s = (cudaStream_t)stream;
    switch (desc->dtype) {
        case CG_B200_F32: return launch_typed<float>(p, vector_ok, s);
        case CG_B200_BF16: return launch_typed<__nv_bfloat16>(p, vector_ok, s);
        default: return launch_typed<__half>(p, vector_ok, s);
    }
}
