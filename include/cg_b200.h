/*
 * cg_b200.h - C ABI of the B200 (sm_100a) execution path for cantors-gift Executables.
 *
 * Every entry point returns an int status (0 = CG_B200_OK); no exception crosses this
 * boundary. Unless a parameter is named host_*, every data pointer is a device pointer
 * on the CUDA device that is current on the calling thread. `stream` is a cudaStream_t
 * passed as void* (NULL = the default stream). Launches are asynchronous on `stream`;
 * cg_b200_stream_sync is the only blocking call besides the host copies.
 *
 * There is no CPU fallback: without a usable CUDA device the compute entry points
 * return CG_B200_ERR_NO_DEVICE.
 *
 * Each declaration cites the interface of the reference project (cantors-gift, paths
 * relative to its root) that it stands behind.
 */
#ifndef CG_B200_H
#define CG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define CG_B200_VERSION_MAJOR 0
#define CG_B200_VERSION_MINOR 1

/* ---- status codes --------------------------------------------------------------- */
enum cg_b200_status {
    CG_B200_OK = 0,
    CG_B200_ERR_INVALID_ARG = 1,    /* bad size, count, enum value or program            */
    CG_B200_ERR_NULL_POINTER = 2,   /* a required pointer is NULL                        */
    CG_B200_ERR_MISALIGNED = 3,     /* a pointer or stride breaks the stated alignment   */
    CG_B200_ERR_UNSUPPORTED = 4,    /* valid request that no kernel here implements      */
    CG_B200_ERR_CUDA = 5,           /* a CUDA runtime/driver call failed                 */
    CG_B200_ERR_NO_DEVICE = 6,      /* no CUDA device (there is no CPU fallback)         */
    CG_B200_ERR_WORKSPACE = 7,      /* workspace missing or too small                    */
    CG_B200_ERR_DEVICE_TIMEOUT = 8, /* a bounded device-side wait ran out                */
    CG_B200_ERR_COMM = 9,           /* NCCL failure                                      */
    CG_B200_ERR_FUSED_IR = 10,      /* IR carries the reference's lossy fusion markers   */
    CG_B200_ERR_NOT_SM100 = 11      /* device is not compute capability 10.x             */
};

/* Element types. Numbering equals the reference's cg::DType (include/cg/core/dtype.hpp:14-40). */
enum cg_b200_dtype {
    CG_B200_F16 = 0,
    CG_B200_BF16 = 1,
    CG_B200_F32 = 2
};

/* ---- library / device ----------------------------------------------------------- */

/* Packed version: (major << 16) | minor. */
int cg_b200_version(void);
/* Static, never-NULL description of a status code. */
const char* cg_b200_status_string(int status);
/* Text of the last CUDA error this thread saw inside the library ("" if none). */
const char* cg_b200_last_cuda_error(void);
/* Number of CUDA devices; *count = 0 and CG_B200_ERR_NO_DEVICE when there is none. */
int cg_b200_device_count(int* count);

/* Static capabilities of one device. Stands behind TargetInfo / HardwareModel
 * (include/cg/backend/backend.hpp:48-65, src/cost/hardware_model.cpp:71-106), whose
 * generic NVIDIA model holds A100-class constants. */
typedef struct cg_b200_props {
    char     name[64];
    int32_t  cc_major, cc_minor;
    int32_t  sm_count;
    int32_t  max_smem_per_block;   /* opt-in bytes */
    int32_t  l2_bytes;
    int32_t  sm_clock_khz;
    int32_t  mem_clock_khz;
    int32_t  mem_bus_bits;
    uint64_t hbm_bytes;
    uint64_t tmem_bytes_per_sm;    /* 256 KiB on sm_100 */
} cg_b200_props;
int cg_b200_device_props(int device, cg_b200_props* out);
int cg_b200_set_device(int device);

/* ---- memory: stands behind cg::Allocator (include/cg/runtime/runtime.hpp:44-49) --- */
/* Returned pointers are 256-byte aligned, as Allocator::allocate's default alignment. */
int cg_b200_malloc(void** dev_ptr, size_t bytes);
int cg_b200_free(void* dev_ptr);
int cg_b200_malloc_host(void** host_ptr, size_t bytes);   /* pinned */
int cg_b200_free_host(void* host_ptr);
int cg_b200_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes, void* stream);
int cg_b200_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes, void* stream);
int cg_b200_memset(void* dev_dst, int byte, size_t bytes, void* stream);

/* ---- streams / events: cg::Stream, cg::Event (include/cg/runtime/runtime.hpp:51-63) */
int cg_b200_stream_create(void** stream);
int cg_b200_stream_destroy(void* stream);
int cg_b200_stream_sync(void* stream);
int cg_b200_event_create(void** event);
int cg_b200_event_destroy(void* event);
int cg_b200_event_record(void* event, void* stream);
int cg_b200_event_sync(void* event);
/* Work submitted to `stream` after this call starts only when `event` has completed; the host does
 * not block. With it a caller overlaps the copy of one slab with the kernel on the previous one
 * (Event::wait, runtime.hpp:61, blocks the host and is cg_b200_event_sync above). */
int cg_b200_stream_wait_event(void* stream, void* event);
/* Seconds between two recorded events (Event::elapsed_sec_since, runtime.hpp:62). */
int cg_b200_event_elapsed_sec(void* earlier, void* later, double* seconds);

/* ---- fused elementwise chain ------------------------------------------------------
 * Replaces what TensorToCodegenLowering emits for elementwise ops (one un-looped
 * VectorLoad/Add|Mul/VectorStore per op, src/lowering/tensor_to_codegen.cpp:60-135)
 * and the straight-line ld/st PTX made from it (src/backend/ptx/ptx_emitter.cpp:60-232).
 * One launch evaluates a whole chain of Tensor-IR elementwise ops
 * (src/ir/ops.cpp:277-420) per output element.
 *
 * The chain is a postfix program over a value stack of depth <= 4. Arithmetic is fp32;
 * ADD/SUB/MUL are separately rounded (never contracted into FMA), so chains of
 * add/mul/max are bit-exact with the reference's x86 vaddps/vmulps/vmaxps kernels
 * (benchmarks/benchmark_multithread.py:54-124). With 16-bit storage types and
 * round_each_op != 0 every op result is rounded to the storage type, as if each op had
 * produced a tensor of that type. */
enum cg_b200_eltwise_op {
    CG_B200_EW_INPUT = 0,   /* push inputs[arg][index]                          */
    CG_B200_EW_IMM = 1,     /* push imm                                         */
    CG_B200_EW_ADD = 2,     /* pop b, pop a, push a+b                           */
    CG_B200_EW_SUB = 3,
    CG_B200_EW_MUL = 4,
    CG_B200_EW_DIV = 5,
    CG_B200_EW_MAX = 6,     /* x86 maxps order: a > b ? a : b                   */
    CG_B200_EW_MIN = 7,     /* x86 minps order: a < b ? a : b                   */
    CG_B200_EW_NEG = 8,
    CG_B200_EW_ABS = 9,
    CG_B200_EW_RELU = 10,   /* x > 0 ? x : +0                                   */
    CG_B200_EW_GELU_TANH = 11, /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
    CG_B200_EW_TANH = 12,
    CG_B200_EW_SIGMOID = 13,
    CG_B200_EW_EXP = 14,
    CG_B200_EW_LOG = 15,
    CG_B200_EW_SQRT = 16,
    CG_B200_EW_RSQRT = 17,
    CG_B200_EW_OP_COUNT = 18
};

/* How input i is indexed for flat output index e (row-major, NumPy right-aligned
 * broadcast, src/shape/inference.cpp:11-31). */
enum cg_b200_bcast {
    CG_B200_BC_FULL = 0,    /* [n]            -> in[e]                    */
    CG_B200_BC_SCALAR = 1,  /* [1]            -> in[0]                    */
    CG_B200_BC_ROW = 2,     /* [inner]        -> in[e % inner]            */
    CG_B200_BC_COL = 3      /* [n/inner, 1]   -> in[e / inner]            */
};

#define CG_B200_EW_MAX_INSTR 16
#define CG_B200_EW_MAX_INPUTS 8
#define CG_B200_EW_MAX_STACK 4

typedef struct cg_b200_eltwise_instr {
    int32_t op;    /* cg_b200_eltwise_op */
    int32_t arg;   /* input index for EW_INPUT, else 0 */
    float   imm;   /* value for EW_IMM, else 0 */
} cg_b200_eltwise_instr;

typedef struct cg_b200_eltwise_desc {
    int32_t dtype;                               /* storage type of all inputs and the output */
    int32_t n_instr;
    cg_b200_eltwise_instr prog[CG_B200_EW_MAX_INSTR];
    int32_t bcast[CG_B200_EW_MAX_INPUTS];        /* cg_b200_bcast per input */
    int64_t inner;                               /* period for BC_ROW / BC_COL (>=1) */
    int32_t round_each_op;                       /* 16-bit storage only */
    int32_t reserved;
} cg_b200_eltwise_desc;

/* Checks a program without touching a device: stack discipline, op codes, input
 * indices. Returns CG_B200_OK or CG_B200_ERR_INVALID_ARG. */
int cg_b200_eltwise_validate(const cg_b200_eltwise_desc* desc, int n_inputs);
/* out[e] = program(inputs..., e) for e in [0, n). BC_FULL inputs and `out` must be
 * aligned to the element size; 16-byte alignment selects the 128-bit path. n == 0 is a
 * no-op. */
int cg_b200_eltwise(const cg_b200_eltwise_desc* desc, const void* const* inputs,
                    int n_inputs, void* out, size_t n, void* stream);

/* ---- row reductions ---------------------------------------------------------------
 * The reference defines softmax/layernorm as attribute-less ops over the last axis
 * (src/ir/ops.cpp:536-556), lowers them to an "unknown opcode" Const
 * (src/lowering/tensor_to_codegen.cpp:350-356) and emits a comment for Reduce
 * (src/backend/ptx/ptx_emitter.cpp:136-142). Definitions: max-subtracted softmax
 * (include/cg/egraph/rewrite_rules.hpp:96-101); layernorm = mean, variance, normalise,
 * scale + shift (src/analysis/arithmetic_intensity.cpp:138-146).
 * in/out are [rows, cols] row-major contiguous; math is fp32; `in == out` is allowed. */
int cg_b200_softmax(int dtype, const void* in, void* out, int64_t rows, int64_t cols,
                    void* stream);
/* gamma/beta: [cols] of `dtype`, or NULL for 1 / 0. Variance is the biased (1/cols)
 * centred variance. */
int cg_b200_layernorm(int dtype, const void* in, const void* gamma, const void* beta,
                      float eps, void* out, int64_t rows, int64_t cols, void* stream);
/* layernorm(softmax(in)) in one pass over HBM; the softmax result is rounded to `dtype`
 * before the layernorm, exactly as the two-kernel sequence would produce it. */
int cg_b200_softmax_layernorm(int dtype, const void* in, const void* gamma,
                              const void* beta, float eps, void* out, int64_t rows,
                              int64_t cols, void* stream);

/* ---- reductions over a run of adjacent axes -----------------------------------------
 * Replaces the reduce lowering (VectorLoad, Reduce, VectorStore, src/lowering/tensor_to_codegen.cpp:332;
 * CGOpcode::Reduce is a comment in the PTX emitter, src/backend/ptx/ptx_emitter.cpp:136-142). Semantics
 * follow OP_REDUCE_SUM / _MAX / _MEAN (src/ir/ops.cpp:74-102, 417-436): the reduced axes of a row-major
 * tensor, when adjacent, make it a [outer, reduce, inner] box; out is [outer, inner] (keep_dims changes
 * the result's shape only). Accumulation in fp32, one rounding to `dtype`; mean = sum / reduce; max
 * ignores NaN operands (fmaxf). outer == 0 or inner == 0: no-op; reduce == 0: CG_B200_ERR_INVALID_ARG. */
enum cg_b200_reduce_op { CG_B200_REDUCE_SUM = 0, CG_B200_REDUCE_MAX = 1, CG_B200_REDUCE_MEAN = 2 };
int cg_b200_reduce(int dtype, int op, const void* in, void* out, int64_t outer, int64_t reduce,
                   int64_t inner, void* stream);

/* ---- GEMM with fused epilogue -----------------------------------------------------
 * Replaces the matmul lowering (3 Const, 2 shared VectorLoad, K/k_tile FMA,
 * src/lowering/tensor_to_codegen.cpp:137-210) and the mma.sync skeleton
 * (src/backend/tensor_core/ptx_mma.cpp:115-258). Semantics follow OP_MATMUL
 * (src/ir/ops.cpp, [.., M, K] x [.., K, N], batch dims broadcast; here batch strides
 * in elements, 0 = broadcast). C = epilogue(A x B). */
enum cg_b200_epilogue {
    CG_B200_EPI_NONE = 0,
    CG_B200_EPI_BIAS = 1,            /* + bias[n]                        */
    CG_B200_EPI_BIAS_RELU = 2,
    CG_B200_EPI_BIAS_GELU_TANH = 3,
    CG_B200_EPI_BIAS_RESIDUAL = 4,   /* + bias[n] + residual[m, n]       */
    CG_B200_EPI_RESIDUAL = 5,        /* + residual[m, n]                 */
    CG_B200_EPI_SCALE = 6,           /* * alpha                          */
    CG_B200_EPI_RELU = 7,            /* relu(A x B), no bias             */
    CG_B200_EPI_GELU_TANH = 8        /* gelu_tanh(A x B), no bias        */
};

enum cg_b200_compute {
    CG_B200_COMPUTE_DEFAULT = 0,     /* bf16/f16: native kind::f16; f32: 3xTF32 split */
    CG_B200_COMPUTE_TF32X3 = 1,      /* f32 inputs: hi*hi + hi*lo + lo*hi              */
    CG_B200_COMPUTE_TF32 = 2         /* f32 inputs: single TF32 pass (relaxed numerics) */
};

typedef struct cg_b200_gemm_desc {
    int64_t M, N, K;
    int64_t batch;                   /* >= 1 */
    int64_t lda, ldb, ldc;           /* row strides in elements (A [M,K], B [K,N] or [N,K] if b_transposed, C [M,N]) */
    int64_t batch_stride_a, batch_stride_b, batch_stride_c; /* elements; 0 = broadcast (A, B only) */
    int32_t in_dtype;                /* A and B */
    int32_t out_dtype;               /* C, bias, residual */
    int32_t compute;                 /* cg_b200_compute */
    int32_t epilogue;                /* cg_b200_epilogue */
    int32_t b_transposed;            /* 0: B is [K, N] row-major; 1: B is stored [N, K] row-major */
    float   alpha;                   /* EPI_SCALE factor */
    /* Optional second batch level (e.g. heads inside sequences). With batch_inner > 1 the batch
     * index b in [0, batch) splits as outer = b / batch_inner, inner = b % batch_inner and operand X
     * of GEMM b starts at outer * batch_stride_x + inner * inner_stride_x (elements). batch_inner
     * must divide batch; 0 or 1 = single level. */
    int64_t batch_inner;
    int64_t inner_stride_a, inner_stride_b, inner_stride_c;
} cg_b200_gemm_desc;

/* Bytes of device scratch cg_b200_gemm may need for this problem (0 for 16-bit inputs). fp32 inputs are
 * split into tf32 hi / lo parts: inside the kernel, with no scratch, when A and B can be read in place
 * (16-byte aligned bases, row and batch strides multiples of 16 bytes); operands that are only 4-byte
 * aligned are rewritten into the workspace by a pre-pass first, and CG_B200_ERR_WORKSPACE is returned
 * when it is missing or too small. Both ways give the same bits. */
int cg_b200_gemm_workspace_bytes(const cg_b200_gemm_desc* desc, size_t* bytes);
/* 16-bit A, B: 16-byte aligned base pointers; strides multiples of 16 bytes. C: always so. `bias` is [N],
 * `residual` is [M, N] with row stride ldc (and batch_stride_c), both of out_dtype. The C tiles of
 * different batches must not overlap: batch_stride_c >= M * ldc, or column blocks side by side
 * (batch_stride_c >= N and batch * batch_stride_c <= ldc). */
int cg_b200_gemm(const cg_b200_gemm_desc* desc, const void* A, const void* B,
                 const void* bias, const void* residual, void* C, void* workspace,
                 size_t workspace_bytes, void* stream);
/* The same GEMM with the tile choice made by the caller instead of the library's heuristic: what a
 * BenchmarkFn handed to the reference's autotuner times, one call per candidate schedule
 * (include/cg/autotuner/bayesian_optimizer.hpp:79-96; Runtime::autotune_and_cache,
 * src/runtime/runtime.cpp:287-312, and MatmulPipeline::run, src/pipeline/matmul_pipeline.cpp:261-323,
 * take such a function and today receive a stub). Every field 0 = library default. Results do not
 * depend on the choice (the K order of the accumulation is the same in every variant).
 * CG_B200_ERR_UNSUPPORTED for a combination no kernel has: CTA pairs with fp32 inputs or with a
 * 64-wide tile, a 256-wide tile for the 3xTF32 path. */
typedef struct cg_b200_gemm_tuning {
    int32_t tile_n;      /* 0, 64, 128 or 256 output columns per tile                          */
    int32_t cta_pair;    /* 0 = default, 1 = one CTA per 128-row tile, 2 = CTA pair, 256 rows   */
    int32_t tail_split;  /* 0 = default, 1 = off, 2 = on: last partial wave as half-width units */
    int32_t reserved;    /* 0 */
} cg_b200_gemm_tuning;
int cg_b200_gemm_tuned(const cg_b200_gemm_desc* desc, const cg_b200_gemm_tuning* tuning, const void* A,
                       const void* B, const void* bias, const void* residual, void* C, void* workspace,
                       size_t workspace_bytes, void* stream);
/* Reads and clears the error word written by a bounded device-side wait that ran out
 * (0 = none). Synchronises `stream`. */
int cg_b200_last_device_error(void* stream, uint32_t* word);

/* ---- fused attention ---------------------------------------------------------------------
 * O[b, h] = softmax(Q[b, h] K[b, h]^T * scale) V[b, h] over the last axis, no mask: the pattern
 * the reference annotates as "attention" (src/optimization/graph/graph_pattern.cpp:61-85) and
 * never executes; as separate ops it is matmul, softmax, matmul (src/ir/ops.cpp). Scores and
 * probabilities stay on chip in fp32 (probabilities enter the second product rounded to
 * `dtype`), so results differ from the three-op sequence by its intermediate roundings only.
 * Q/O are [batch, heads, seq_q, head_dim], K/V [batch, heads, seq_kv, head_dim], each given by a
 * base pointer and row / head / batch strides in elements, so heads may be column blocks of a
 * packed [rows, 3 * d_model] projection. head_dim must be 64, dtype bf16 or f16, scale > 0;
 * bases 16-byte aligned, strides multiples of 8 elements. */
typedef struct cg_b200_attention_desc {
    int32_t dtype;
    int32_t head_dim;
    int64_t batch, heads, seq_q, seq_kv;
    int64_t ldq, ldk, ldv, ldo;                                        /* row strides */
    int64_t head_stride_q, head_stride_k, head_stride_v, head_stride_o;
    int64_t batch_stride_q, batch_stride_k, batch_stride_v, batch_stride_o;
    float   scale;
    int32_t reserved;
} cg_b200_attention_desc;
int cg_b200_attention(const cg_b200_attention_desc* desc, const void* Q, const void* K, const void* V,
                      void* O, void* stream);

/* fp32 GEMM for callers that cannot allocate device memory (no counterpart in the reference).
 * Who that is: code that runs where an allocation is not allowed or not possible - a launch
 * routine that is handed only tensors and a stream (the shape of BoundExecutable::launch,
 * include/cg/runtime/runtime.hpp:84-88, which carries no allocator), a service whose device
 * memory was given out in full to its own pools at start-up, or a latency-critical loop that
 * must not hit the implicit device synchronisation of cudaMalloc/cudaFree. cg_b200_gemm needs
 * a caller-provided workspace for fp32 inputs it cannot read in place (see above); this entry
 * point takes operands of any 4-byte alignment and keeps that scratch in a
 * fixed array of CG_B200_GEMM_F32_STATIC_SCRATCH_BYTES inside the library, held by every GPU
 * that loads the library until the process exits. It calls no allocating routine and always runs
 * the pre-pass form.
 *  - in_dtype must be fp32 (other types need no scratch: use cg_b200_gemm); problems whose
 *    workspace (cg_b200_gemm_workspace_bytes) exceeds the array return CG_B200_ERR_WORKSPACE.
 *  - dev_error_word: optional caller-owned device uint32 (zeroed by the caller) that receives a
 *    non-zero code if a bounded device-side wait runs out; may be NULL.
 *  - The first call on each device resolves the array's device address (set-up work); make it
 *    before any stream capture starts on that device.
 *  - All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *    (different streams without ordering) race on it. Calls on one stream are safe. The array
 *    keeps the previous call's bytes; each call overwrites everything it later reads. */
#define CG_B200_GEMM_F32_STATIC_SCRATCH_BYTES (16u << 20)
int cg_b200_gemm_f32_static(const cg_b200_gemm_desc* desc, const void* A, const void* B,
                            const void* bias, const void* residual, void* C,
                            uint32_t* dev_error_word, void* stream);

/* ---- final all-gather for M- / batch-sharded outputs ------------------------------
 * The reference has no collective (its only parallel runtime is the std::thread fan-out
 * in include/cg/backend/parallel_executor.hpp:49-92). One communicator per process,
 * one process per GPU. host_unique_id is CG_B200_COMM_ID_BYTES made by rank 0 and
 * shipped to the other ranks by the caller. */
#define CG_B200_COMM_ID_BYTES 128
int cg_b200_comm_unique_id(void* host_unique_id);
int cg_b200_comm_init_rank(void** comm, int world, int rank, const void* host_unique_id);
/* buf holds world * shard_bytes; rank r's shard already sits at buf + r * shard_bytes. */
int cg_b200_allgather_inplace(void* comm, void* buf, size_t shard_bytes, void* stream);
/* Stream-ordered barrier over the communicator: work enqueued after it on `stream` starts only
 * once every rank's stream has reached its own call. */
int cg_b200_comm_barrier(void* comm, void* stream);
int cg_b200_comm_destroy(void* comm);

/* ---- GEMM fused with the all-gather of its output ---------------------------------------------
 * The M-sharded GEMM and the collective that follows it as ONE kernel: rank `rank` of `world`
 * computes its desc->M rows and its epilogue stores every tile into rows [rank*M, (rank+1)*M) of
 * the full [world*M, N] buffer - the local one (C_full) and, through peer mappings over NVLink,
 * every other rank's (peer_C[r], r != rank; entry `rank` is ignored). The stores are whole row
 * segments spread over the kernel's run time, so the transfer overlaps the math tile by tile;
 * plain peer stores only (no multicast). When the kernel and a cg_b200_comm_barrier after it have
 * completed on a rank, that rank's buffer holds all world*M rows. bias is [N]; residual, if
 * used, is this rank's [M, N] block (row stride ldc). batch must be 1, world <= 8.
 * Peer pointers come from cg_b200_ipc_export on the owning process (of memory allocated with
 * cg_b200_malloc) and cg_b200_ipc_open here. No counterpart in the reference (it has no
 * multi-device execution). */
#define CG_B200_IPC_HANDLE_BYTES 64
int cg_b200_ipc_export(const void* dev_ptr, void* host_handle);
int cg_b200_ipc_open(const void* host_handle, void** peer_ptr);
int cg_b200_ipc_close(void* peer_ptr);
/* Stream-ordered barrier through flags in peer memory (a few microseconds; the NCCL barrier above
 * costs a small collective). flag_buffers[r] is rank r's flag buffer (at least 8 * world bytes,
 * zeroed once before the first barrier; entry `rank` is the local one, the others are peer
 * mappings). Every rank must call the barrier the same number of times. A peer that does not arrive
 * within 2 s is reported through cg_b200_last_device_error (code 0x500 + rank) and the wait ends. */
int cg_b200_peer_barrier_create(void** barrier, void* const* flag_buffers, int world, int rank);
int cg_b200_peer_barrier(void* barrier, void* stream);
/* Replaces the 2 s limit of later barriers on this handle (1 ns .. 60 s). When the limit runs out the
 * kernel returns, the stream stays usable and the error word holds 0x500 + the missing rank. */
int cg_b200_peer_barrier_set_timeout(void* barrier, uint64_t nanoseconds);
int cg_b200_peer_barrier_destroy(void* barrier);
int cg_b200_gemm_allgather(const cg_b200_gemm_desc* desc, const void* A, const void* B,
                           const void* bias, const void* residual, void* C_full,
                           void* const* peer_C, int world, int rank, void* workspace,
                           size_t workspace_bytes, void* stream);
/* The same with the tile choice open to the caller (`tuning`, may be NULL) and the barrier folded into the
 * kernel (`barrier` from cg_b200_peer_barrier_create, may be NULL): the last CTA to finish publishes
 * this rank's epoch and waits for the peers', so the call stands for cg_b200_gemm_allgather followed by
 * cg_b200_peer_barrier without the second launch. Counts as one barrier call on the handle. */
int cg_b200_gemm_allgather_sync(const cg_b200_gemm_desc* desc, const cg_b200_gemm_tuning* tuning,
                                const void* A, const void* B, const void* bias, const void* residual,
                                void* C_full, void* const* peer_C, int world, int rank, void* barrier,
                                void* workspace, size_t workspace_bytes, void* stream);
/* Copies `bytes` (a multiple of 16) from `src` to peer_dst[r] for every r != rank (entry `rank` is
 * ignored): each 16-byte packet is read once and stored to all peers over NVLink by one kernel whose
 * grid is small enough to run beside a compute kernel on another stream. With `barrier` (may be NULL)
 * the kernel ends in the flag barrier, as above; everything pushed earlier on the same stream is then
 * visible to the peers as well. For results that are gathered while later work still computes. */
int cg_b200_peer_push(const void* src, void* const* peer_dst, int world, int rank, size_t bytes,
                      void* barrier, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* CG_B200_H */
