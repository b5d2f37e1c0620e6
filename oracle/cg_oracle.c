/*
 * cg_oracle.c - CPU restatement of the op semantics the B200 path must reproduce.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA kernels and the timed
 * CPU baseline; nothing in the product path may call it.
 *
 * Parity status per function:
 *   - cgo_eltwise (add/sub/mul/max/relu chains) and cgo_gemm in f32 sequential-FMA mode
 *     are PINNED: tests compare them bit for bit with the reference's own hand-built x86
 *     kernels (built from the reference's X86Emitter sources into oracle/_ref) and with
 *     golden outputs of those kernels committed under tests/golden/.
 *   - gelu, softmax, layernorm, bf16/f16 rounding, batched GEMM: PARITY UNPINNED. The
 *     reference defines these ops (files cited per function) but holds no executable
 *     implementation and no test value for them, so these are restatements of the
 *     definitions only.
 *
 * Reference citations are paths inside the cantors-gift tree.
 */
#include "../include/cg_b200.h"

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ---- element types ----------------------------------------------------------------
 * Sizes follow dtype_size (include/cg/core/dtype.hpp:44-63). bf16 is the upper half of an
 * fp32 with round-to-nearest-even; f16 is IEEE binary16. */
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

static inline uint16_t f32_to_f16(float f) {
    _Float16 v = (_Float16)f;
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

static inline int dtype_ok(int dt) { return dt == CG_B200_F16 || dt == CG_B200_BF16 || dt == CG_B200_F32; }
static inline size_t dtype_bytes(int dt) { return dt == CG_B200_F32 ? 4 : 2; }

static inline float load_as_f32(const void* p, int dt, size_t i) {
    switch (dt) {
        case CG_B200_F32: return ((const float*)p)[i];
        case CG_B200_BF16: return bf16_to_f32(((const uint16_t*)p)[i]);
        default: return f16_to_f32(((const uint16_t*)p)[i]);
    }
}

static inline void store_from_f32(void* p, int dt, size_t i, float v) {
    switch (dt) {
        case CG_B200_F32: ((float*)p)[i] = v; break;
        case CG_B200_BF16: ((uint16_t*)p)[i] = f32_to_bf16(v); break;
        default: ((uint16_t*)p)[i] = f32_to_f16(v); break;
    }
}

static inline float round_to(int dt, float v) {
    switch (dt) {
        case CG_B200_F32: return v;
        case CG_B200_BF16: return bf16_to_f32(f32_to_bf16(v));
        default: return f16_to_f32(f32_to_f16(v));
    }
}

void cgo_f32_to_bf16(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
void cgo_bf16_to_f32(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
void cgo_f32_to_f16(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f32_to_f16(in[i]);
}
void cgo_f16_to_f32(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f16_to_f32(in[i]);
}

/* ---- host threading: static contiguous chunks over pthreads (no OpenMP runtime is
 * assumed on the host). */
static int g_threads = 0;

int cgo_num_threads(void) {
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

void cgo_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*range_fn)(int64_t lo, int64_t hi, void* ctx);
typedef struct { range_fn fn; void* ctx; int64_t lo, hi; } range_task;

static void* range_thread(void* p) {
    range_task* t = (range_task*)p;
    t->fn(t->lo, t->hi, t->ctx);
    return NULL;
}

static void parallel_for(int64_t n, int64_t min_chunk, range_fn fn, void* ctx) {
    int nt = cgo_num_threads();
    if (min_chunk < 1) min_chunk = 1;
    if ((int64_t)nt > (n + min_chunk - 1) / min_chunk) nt = (int)((n + min_chunk - 1) / min_chunk);
    if (nt <= 1) {
        if (n > 0) fn(0, n, ctx);
        return;
    }
    pthread_t* th = (pthread_t*)malloc((size_t)nt * sizeof(pthread_t));
    range_task* tk = (range_task*)malloc((size_t)nt * sizeof(range_task));
    int64_t per = n / nt, extra = n % nt, off = 0;
    for (int t = 0; t < nt; ++t) {
        int64_t len = per + (t < extra ? 1 : 0);
        tk[t].fn = fn; tk[t].ctx = ctx; tk[t].lo = off; tk[t].hi = off + len;
        off += len;
        pthread_create(&th[t], NULL, range_thread, &tk[t]);
    }
    for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
    free(th);
    free(tk);
}

/* ---- scalar op definitions ----------------------------------------------------------
 * gelu is the tanh form with constants 0.5, sqrt(2/pi), 0.044715
 * (include/cg/egraph/rewrite_rules.hpp:96-101). relu/max follow the x86 maxps operand
 * order the reference's kernels use (benchmarks/benchmark_multithread.py:112:
 * vmaxps(x, zero) returns the second operand unless x > 0). */
static inline float op_gelu_tanh(float x) {
    const float k0 = 0.7978845608028654f; /* sqrt(2/pi) */
    const float k1 = 0.044715f;
    float x3 = (x * x) * x;
    float t = x + k1 * x3;
    float u = k0 * t;
    return (0.5f * x) * (1.0f + tanhf(u));
}

static inline float op_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

/* ---- fused elementwise chain ---------------------------------------------------------
 * Elementwise op set and broadcast rule: src/ir/ops.cpp:277-420,
 * src/shape/inference.cpp:11-31. The executable anchor is the reference's hand-built x86
 * kernels: separately rounded vmulps / vaddps / vmaxps per 4-float group
 * (benchmarks/benchmark_multithread.py:54-124, benchmarks/benchmark.py:260-323). This
 * file is compiled with -ffp-contract=off so a*b+c stays two roundings. */
int cgo_eltwise_validate(const cg_b200_eltwise_desc* d, int n_inputs) {
    if (!d) return CG_B200_ERR_NULL_POINTER;
    if (!dtype_ok(d->dtype)) return CG_B200_ERR_INVALID_ARG;
    if (d->n_instr < 1 || d->n_instr > CG_B200_EW_MAX_INSTR) return CG_B200_ERR_INVALID_ARG;
    if (n_inputs < 0 || n_inputs > CG_B200_EW_MAX_INPUTS) return CG_B200_ERR_INVALID_ARG;
    if (d->inner < 1) return CG_B200_ERR_INVALID_ARG;
    int depth = 0;
    for (int i = 0; i < d->n_instr; ++i) {
        int op = d->prog[i].op;
        if (op < 0 || op >= CG_B200_EW_OP_COUNT) return CG_B200_ERR_INVALID_ARG;
        if (op == CG_B200_EW_INPUT) {
            int a = d->prog[i].arg;
            if (a < 0 || a >= n_inputs) return CG_B200_ERR_INVALID_ARG;
            if (d->bcast[a] < CG_B200_BC_FULL || d->bcast[a] > CG_B200_BC_COL) return CG_B200_ERR_INVALID_ARG;
            ++depth;
        } else if (op == CG_B200_EW_IMM) {
            ++depth;
        } else if (op >= CG_B200_EW_ADD && op <= CG_B200_EW_MIN) {
            if (depth < 2) return CG_B200_ERR_INVALID_ARG;
            --depth;
        } else {
            if (depth < 1) return CG_B200_ERR_INVALID_ARG;
        }
        if (depth > CG_B200_EW_MAX_STACK) return CG_B200_ERR_INVALID_ARG;
    }
    return depth == 1 ? CG_B200_OK : CG_B200_ERR_INVALID_ARG;
}

typedef struct {
    const cg_b200_eltwise_desc* d;
    const void* const* inputs;
    void* out;
} eltwise_ctx;

static void eltwise_range(int64_t lo, int64_t hi, void* p) {
    const eltwise_ctx* c = (const eltwise_ctx*)p;
    const cg_b200_eltwise_desc* d = c->d;
    const int dt = d->dtype;
    const int rnd = (dt != CG_B200_F32) && d->round_each_op;
    const int64_t inner = d->inner;
    for (int64_t e = lo; e < hi; ++e) {
        float s[CG_B200_EW_MAX_STACK] = {0.0f, 0.0f, 0.0f, 0.0f};
        int sp = 0;
        for (int i = 0; i < d->n_instr; ++i) {
            const cg_b200_eltwise_instr* in = &d->prog[i];
            if (in->op == CG_B200_EW_INPUT) {
                size_t idx;
                switch (d->bcast[in->arg]) {
                    case CG_B200_BC_SCALAR: idx = 0; break;
                    case CG_B200_BC_ROW: idx = (size_t)(e % inner); break;
                    case CG_B200_BC_COL: idx = (size_t)(e / inner); break;
                    default: idx = (size_t)e; break;
                }
                s[sp++] = load_as_f32(c->inputs[in->arg], dt, idx);
                continue;
            }
            if (in->op == CG_B200_EW_IMM) {
                s[sp++] = rnd ? round_to(dt, in->imm) : in->imm;
                continue;
            }
            float r;
            if (in->op <= CG_B200_EW_MIN) {
                float b = s[--sp];
                float a = s[--sp];
                switch (in->op) {
                    case CG_B200_EW_ADD: r = a + b; break;
                    case CG_B200_EW_SUB: r = a - b; break;
                    case CG_B200_EW_MUL: r = a * b; break;
                    case CG_B200_EW_DIV: r = a / b; break;
                    case CG_B200_EW_MAX: r = a > b ? a : b; break;
                    default: r = a < b ? a : b; break;
                }
            } else {
                float a = s[--sp];
                switch (in->op) {
                    case CG_B200_EW_NEG: r = -a; break;
                    case CG_B200_EW_ABS: r = fabsf(a); break;
                    case CG_B200_EW_RELU: r = a > 0.0f ? a : 0.0f; break;
                    case CG_B200_EW_GELU_TANH: r = op_gelu_tanh(a); break;
                    case CG_B200_EW_TANH: r = tanhf(a); break;
                    case CG_B200_EW_SIGMOID: r = op_sigmoid(a); break;
                    case CG_B200_EW_EXP: r = expf(a); break;
                    case CG_B200_EW_LOG: r = logf(a); break;
                    case CG_B200_EW_SQRT: r = sqrtf(a); break;
                    default: r = 1.0f / sqrtf(a); break;
                }
            }
            s[sp++] = rnd ? round_to(dt, r) : r;
        }
        store_from_f32(c->out, dt, (size_t)e, s[0]);
    }
}

int cgo_eltwise(const cg_b200_eltwise_desc* d, const void* const* inputs, int n_inputs,
                void* out, size_t n) {
    int st = cgo_eltwise_validate(d, n_inputs);
    if (st) return st;
    if (n == 0) return CG_B200_OK;
    if (!out || !inputs) return CG_B200_ERR_NULL_POINTER;
    eltwise_ctx c = {d, inputs, out};
    parallel_for((int64_t)n, 1 << 14, eltwise_range, &c);
    return CG_B200_OK;
}

/* ---- GEMM + epilogue -----------------------------------------------------------------
 * OP_MATMUL semantics: [.., M, K] x [.., K, N] with broadcast batch dims
 * (src/ir/ops.cpp matmul verifier, src/shape/inference.cpp:168-198). The accumulation is
 * the reference's only executable matmul: acc = 0; for k ascending: acc = fma(A[m,k],
 * B[k,n], acc) in fp32 (benchmarks/benchmark.py:326-438, vfmadd231ss on xmm0). acc64 != 0
 * accumulates in double instead (used to report error against exact arithmetic).
 * `rows` optionally limits the work to flat row indices b*M + m (C is written only there). */
/* Element offset of operand X of GEMM `b`: one batch level, or outer/inner levels when
 * batch_inner > 1 (include/cg_b200.h, cg_b200_gemm_desc). */
static inline int64_t batch_offset(const cg_b200_gemm_desc* d, int64_t b, int64_t stride, int64_t inner_stride) {
    if (d->batch_inner > 1) return (b / d->batch_inner) * stride + (b % d->batch_inner) * inner_stride;
    return b * stride;
}

typedef struct {
    const void* src; int dt; int64_t cols, ld; int transposed; float* dst;
} convert_ctx;

static void convert_range(int64_t lo, int64_t hi, void* p) {
    const convert_ctx* c = (const convert_ctx*)p;
    for (int64_t r = lo; r < hi; ++r)
        for (int64_t k = 0; k < c->cols; ++k) {
            size_t idx = c->transposed ? (size_t)(k * c->ld + r) : (size_t)(r * c->ld + k);
            c->dst[r * c->cols + k] = load_as_f32(c->src, c->dt, idx);
        }
}

typedef struct {
    const cg_b200_gemm_desc* d;
    const char* Ap; const float* Bf; const void* bias; const void* residual; void* C;
    const int64_t* rows; int64_t start, b; int acc64;
} gemm_ctx;

static void gemm_range(int64_t lo, int64_t hi, void* p) {
    const gemm_ctx* c = (const gemm_ctx*)p;
    const cg_b200_gemm_desc* d = c->d;
    const int64_t M = d->M, N = d->N, K = d->K;
    const int epi = d->epilogue;
    const int need_bias = epi == CG_B200_EPI_BIAS || epi == CG_B200_EPI_BIAS_RELU ||
                          epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_BIAS_RESIDUAL;
    const int need_res = epi == CG_B200_EPI_BIAS_RESIDUAL || epi == CG_B200_EPI_RESIDUAL;
    float* accf = (float*)malloc((size_t)N * sizeof(float));
    double* accd = c->acc64 ? (double*)malloc((size_t)N * sizeof(double)) : NULL;
    for (int64_t ri = c->start + lo; ri < c->start + hi; ++ri) {
        int64_t flat = c->rows ? c->rows[ri] : ri;
        int64_t m = flat - c->b * M;
        if (c->acc64) {
            for (int64_t n = 0; n < N; ++n) accd[n] = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                double a = (double)load_as_f32(c->Ap, d->in_dtype, (size_t)(m * d->lda + k));
                const float* br = c->Bf + k * N;
                for (int64_t n = 0; n < N; ++n) accd[n] += a * (double)br[n];
            }
            for (int64_t n = 0; n < N; ++n) accf[n] = (float)accd[n];
        } else {
            for (int64_t n = 0; n < N; ++n) accf[n] = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                float a = load_as_f32(c->Ap, d->in_dtype, (size_t)(m * d->lda + k));
                const float* br = c->Bf + k * N;
                for (int64_t n = 0; n < N; ++n) accf[n] = fmaf(a, br[n], accf[n]);
            }
        }
        size_t crow = (size_t)(batch_offset(d, c->b, d->batch_stride_c, d->inner_stride_c) + m * d->ldc);
        for (int64_t n = 0; n < N; ++n) {
            float v = accf[n];
            if (epi == CG_B200_EPI_SCALE) v = v * d->alpha;
            if (need_bias) v = v + load_as_f32(c->bias, d->out_dtype, (size_t)n);
            if (epi == CG_B200_EPI_BIAS_RELU || epi == CG_B200_EPI_RELU) v = v > 0.0f ? v : 0.0f;
            if (epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_GELU_TANH) v = op_gelu_tanh(v);
            if (need_res) v = v + load_as_f32(c->residual, d->out_dtype, crow + (size_t)n);
            store_from_f32(c->C, d->out_dtype, crow + (size_t)n, v);
        }
    }
    free(accf);
    free(accd);
}

int cgo_gemm(const cg_b200_gemm_desc* d, const void* A, const void* B, const void* bias,
             const void* residual, void* C, const int64_t* rows, int64_t n_rows, int acc64) {
    if (!d) return CG_B200_ERR_NULL_POINTER;
    if (!dtype_ok(d->in_dtype) || !dtype_ok(d->out_dtype)) return CG_B200_ERR_INVALID_ARG;
    if (d->M < 0 || d->N < 0 || d->K < 0 || d->batch < 1) return CG_B200_ERR_INVALID_ARG;
    if (d->batch_inner > 1 && d->batch % d->batch_inner != 0) return CG_B200_ERR_INVALID_ARG;
    if (d->M == 0 || d->N == 0) return CG_B200_OK;
    if (!A || !B || !C) return CG_B200_ERR_NULL_POINTER;
    const int epi = d->epilogue;
    const int need_bias = epi == CG_B200_EPI_BIAS || epi == CG_B200_EPI_BIAS_RELU ||
                          epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_BIAS_RESIDUAL;
    const int need_res = epi == CG_B200_EPI_BIAS_RESIDUAL || epi == CG_B200_EPI_RESIDUAL;
    if (need_bias && !bias) return CG_B200_ERR_NULL_POINTER;
    if (need_res && !residual) return CG_B200_ERR_NULL_POINTER;
    const int64_t M = d->M, N = d->N, K = d->K;
    const size_t in_sz = dtype_bytes(d->in_dtype);
    const int64_t total_rows = rows ? n_rows : d->batch * M;

    float* Bf = (float*)malloc((size_t)(K > 0 ? K : 1) * (size_t)N * sizeof(float));
    if (!Bf) return CG_B200_ERR_INVALID_ARG;
    int64_t cached_b = -1;
    /* consecutive rows of the same batch share one converted copy of B */
    for (int64_t start = 0; start < total_rows;) {
        int64_t flat0 = rows ? rows[start] : start;
        int64_t b = flat0 / M;
        int64_t end = start;
        while (end < total_rows && (rows ? rows[end] : end) / M == b) ++end;
        int64_t bb = batch_offset(d, b, d->batch_stride_b, d->inner_stride_b);
        if (bb != cached_b) {
            convert_ctx cc = {(const char*)B + (size_t)bb * in_sz, d->in_dtype, N, d->ldb, d->b_transposed, Bf};
            parallel_for(K, 16, convert_range, &cc);
            cached_b = bb;
        }
        gemm_ctx gc = {d, (const char*)A + (size_t)batch_offset(d, b, d->batch_stride_a, d->inner_stride_a) * in_sz, Bf, bias,
                       residual, C, rows, start, b, acc64};
        parallel_for(end - start, 1, gemm_range, &gc);
        start = end;
    }
    free(Bf);
    return CG_B200_OK;
}

/* ---- row reductions ------------------------------------------------------------------
 * softmax / layernorm act on the last axis and carry no attributes
 * (src/ir/ops.cpp:536-556). softmax is the max-subtracted form
 * (include/cg/egraph/rewrite_rules.hpp:96-101); layernorm is mean, variance, normalise,
 * scale + shift (src/analysis/arithmetic_intensity.cpp:138-146) with eps = 1e-5 in the
 * reference's transformer benchmark (benchmarks/benchmark_transformer.py:115). Sums are
 * accumulated in double so the restatement does not depend on summation order. */
static void softmax_row(const float* x, float* y, int64_t cols) {
    float m = -INFINITY;
    for (int64_t c = 0; c < cols; ++c) m = x[c] > m ? x[c] : m;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
        y[c] = expf(x[c] - m);
        s += (double)y[c];
    }
    float inv = (float)(1.0 / s);
    for (int64_t c = 0; c < cols; ++c) y[c] = y[c] * inv;
}

static void layernorm_row(const float* x, const float* g, const float* b, float eps, float* y,
                          int64_t cols) {
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += (double)x[c];
    double mean = s / (double)cols;
    double v = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
        double dlt = (double)x[c] - mean;
        v += dlt * dlt;
    }
    double var = v / (double)cols;
    float rstd = (float)(1.0 / sqrt(var + (double)eps));
    float meanf = (float)mean;
    for (int64_t c = 0; c < cols; ++c) {
        float t = (x[c] - meanf) * rstd;
        if (g) t = t * g[c];
        if (b) t = t + b[c];
        y[c] = t;
    }
}

static float* vec_to_f32(const void* p, int dt, int64_t n) {
    if (!p) return NULL;
    float* f = (float*)malloc((size_t)n * sizeof(float));
    for (int64_t i = 0; i < n; ++i) f[i] = load_as_f32(p, dt, (size_t)i);
    return f;
}

/* mode: 0 = softmax, 1 = layernorm, 2 = layernorm(softmax) with the intermediate rounded
 * to `dt` (what two kernels exchanging a `dt` tensor would produce). */
typedef struct {
    int mode, dt; const void* in; const float* g; const float* b; float eps; void* out; int64_t cols;
} row_ctx;

static void row_range(int64_t lo, int64_t hi, void* p) {
    const row_ctx* c = (const row_ctx*)p;
    const int64_t cols = c->cols;
    float* x = (float*)malloc((size_t)cols * sizeof(float));
    float* y = (float*)malloc((size_t)cols * sizeof(float));
    for (int64_t r = lo; r < hi; ++r) {
        size_t base = (size_t)(r * cols);
        for (int64_t k = 0; k < cols; ++k) x[k] = load_as_f32(c->in, c->dt, base + (size_t)k);
        if (c->mode == 0) {
            softmax_row(x, y, cols);
        } else if (c->mode == 1) {
            layernorm_row(x, c->g, c->b, c->eps, y, cols);
        } else {
            softmax_row(x, y, cols);
            for (int64_t k = 0; k < cols; ++k) x[k] = round_to(c->dt, y[k]);
            layernorm_row(x, c->g, c->b, c->eps, y, cols);
        }
        for (int64_t k = 0; k < cols; ++k) store_from_f32(c->out, c->dt, base + (size_t)k, y[k]);
    }
    free(x);
    free(y);
}

static int row_op(int mode, int dt, const void* in, const void* gamma, const void* beta, float eps,
                  void* out, int64_t rows, int64_t cols) {
    if (!dtype_ok(dt) || rows < 0 || cols < 0) return CG_B200_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return CG_B200_OK;
    if (!in || !out) return CG_B200_ERR_NULL_POINTER;
    float* g = vec_to_f32(gamma, dt, cols);
    float* b = vec_to_f32(beta, dt, cols);
    row_ctx c = {mode, dt, in, g, b, eps, out, cols};
    parallel_for(rows, 1, row_range, &c);
    free(g);
    free(b);
    return CG_B200_OK;
}

int cgo_softmax(int dt, const void* in, void* out, int64_t rows, int64_t cols) {
    return row_op(0, dt, in, NULL, NULL, 0.0f, out, rows, cols);
}

int cgo_layernorm(int dt, const void* in, const void* gamma, const void* beta, float eps, void* out,
                  int64_t rows, int64_t cols) {
    return row_op(1, dt, in, gamma, beta, eps, out, rows, cols);
}

int cgo_softmax_layernorm(int dt, const void* in, const void* gamma, const void* beta, float eps,
                          void* out, int64_t rows, int64_t cols) {
    return row_op(2, dt, in, gamma, beta, eps, out, rows, cols);
}
