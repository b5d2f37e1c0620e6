// gemm_sm100.cu - C = epilogue(A x B) on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Stands where the reference lowers OP_MATMUL to 3 Const, 2 shared VectorLoad and K/k_tile
// FMA instructions on one thread's registers (src/lowering/tensor_to_codegen.cpp:137-210)
// and where its tensor-core text generator prints an mma.sync m16n8k16 skeleton with the
// global->shared copies elided (src/backend/tensor_core/ptx_mma.cpp:115-258). Neither is
// executable. The only matmul the reference runs is the scalar x86 FMA loop of
// benchmarks/benchmark.py:326-438; parity is defined against that accumulation.
//
// Two tile shapes share one kernel template (kCta):
//   kCta = 2  a cluster of two CTAs on two SMs computes one 256 x BN tile with cta_group::2
//             MMAs issued by the even CTA: each CTA stages its own 128 rows of A and its own half
//             of B's N range, so every byte of the tile's operands is fetched from L2 once per
//             pair (no TMA multicast is used anywhere); each CTA's TMEM holds its 128 rows of the
//             accumulator and its own epilogue warps drain them
//   kCta = 1  one CTA computes a 128 x BN tile (small problems, fp32 split)
// Structure (one CTA per SM, persistent over output tiles, 320 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A and B k-blocks (128 bytes of K
//               per row, 128-byte swizzle) into a ring of shared-memory stages
//   warp 1      TMEM allocator + single-thread tcgen05.mma issuer; tcgen05.commit releases
//               a stage / publishes an accumulator through mbarriers
//   warps 2-9   epilogue: tcgen05.ld of the fp32 accumulator (one TMEM lane = one row; a warp may
//               only touch the lane quarter (warp id mod 4), so two warps share each quarter and
//               split the tile's columns), bias / activation / residual in registers, packed
//               stores to C
// Two accumulators of BN columns live in TMEM so the epilogue of tile i overlaps the
// main loop of tile i+1. fp32 inputs use kind::tf32 on a hi/lo split prepared by a
// pre-pass (3 MMAs per k-step: lo*hi, hi*lo, hi*hi).
//
// Tensor-core bound: 2*M*N*K flop per problem. Every device-side wait is bounded; when a
// wait runs out the kernel records an error word, stops waiting everywhere, drains its
// copies, frees TMEM and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "tc_sm100.cuh"

namespace cgb {

constexpr int kBM = 128;            // rows per tile = TMEM lanes
constexpr int kRowBytes = 128;      // bytes of K per row per stage (one swizzle span)
constexpr int kUmmaKBytes = 32;     // bytes of K one tcgen05.mma consumes per row
constexpr int kThreads = 320;
constexpr int kEpilogueWarps = 8;
constexpr int kConvertWarps = 8;            // fp32 operands split inside the kernel: warps 10-17
constexpr int kMaxOpStages = 4;             // operand stages the split warps fill ahead of the tensor cores (at most)
constexpr int kThreadsConv = kThreads + 32 * kConvertWarps;
constexpr int kEpilogueStagingBytes = kEpilogueWarps * 4096;   // 32 rows x 128 bytes per epilogue warp
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 224 * 1024;
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    long long M, N, K, batch;
    long long ldc;
    long long c_stride_in, c_stride_out;   // elements between GEMMs of the inner / outer batch level
    long long batch_in;                    // GEMMs per outer batch step (>= 1)
    const void* bias;
    const void* residual;
    void* C;
    // Fused all-gather: every output tile is also stored into the same position of up to 7 peer
    // buffers (other GPUs' copies of C, mapped into this process), at `dst_row_offset` elements from
    // their base as in the local C. n_peer == 0 for a plain GEMM.
    void* peer[7];
    int n_peer;
    long long dst_row_offset;
    int epilogue;
    float alpha;
    int b_mn_major;       // 1: B is [K, N] row-major (N contiguous); 0: B is [N, K]
    int a_in, a_out, b_in, b_out;          // 0: the operand is broadcast along that batch level
    int tiles_m, tiles_n;
    long long num_tiles;
    int num_kb;
    uint32_t idesc;
    // Tail balancing (CTA pairs only): work units [0, full_units) are whole tiles; the rest are
    // half-width tiles (two per remaining tile), so that a last partial wave of r <= slots/2 tiles
    // becomes 2r half-cost units spread over the machine. num_tiles counts units.
    long long full_units;
    uint32_t idesc_half;   // instruction descriptor with N = BN / 2
    int tail_split;        // host side only: 0 = library default, 1 = off, 2 = on (cg_b200_gemm_tuning)
    uint32_t* err_word;
    // Barrier folded into the kernel's tail (fused all-gather only; bar_flags == nullptr: none): every CTA
    // counts itself on bar_done after its peer stores, the last one publishes this rank's epoch to the
    // peers' flag buffers and waits, bounded, for theirs.
    unsigned long long* const* bar_flags;
    unsigned int* bar_done;
    unsigned long long bar_epoch, bar_limit_ns;
    int bar_world, bar_rank;
};

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename OutT>
__device__ __forceinline__ float gelu_epilogue(float x) {
    if constexpr (sizeof(OutT) == 4) {
        return gelu_tanh_f32(x);  // fp32 results keep the accurate tanh
    } else {
        const float k0 = 0.7978845608028654f, k1 = 0.044715f;
        const float u = k0 * (x + k1 * x * x * x);
        return 0.5f * x * (1.0f + tanh_fast(u));
    }
}

// Two values at a time for 16-bit results: six packed fp32x2 instructions and two MUFU.TANH per pair
// instead of about nine scalar ones per value. The last tile's epilogue is not hidden behind a main loop.
__device__ __forceinline__ float2 gelu_pair_fast(float2 x) {
    const float2 x2 = __fmul2_rn(x, x);
    const float2 inner = __ffma2_rn(x2, make_float2(0.044715f, 0.044715f), make_float2(1.0f, 1.0f));
    const float2 u = __fmul2_rn(__fmul2_rn(x, make_float2(0.7978845608028654f, 0.7978845608028654f)), inner);
    const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
    return __ffma2_rn(h, make_float2(tanh_fast(u.x), tanh_fast(u.y)), h);
}

// hi = x with the low 13 mantissa bits cleared (exactly a tf32 value), lo = (x - hi) cleared the same way
__device__ __forceinline__ void tf32_split(float x, float& h, float& l) {
    h = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    l = __uint_as_float(__float_as_uint(x - h) & 0xffffe000u);
}

// The split as the tensor cores see it. A tf32 operand is read by its upper 19 bits, the 13 low mantissa bits
// are ignored, so x itself stands for hi and (x - hi) for lo without clearing either; two values per
// instruction (packed fp32 subtract).
__device__ __forceinline__ void tf32_lo_pair(float x0, float x1, float& l0, float& l1) {
    const uint32_t h0 = __float_as_uint(x0) & 0xffffe000u, h1 = __float_as_uint(x1) & 0xffffe000u;
    uint64_t d;
    asm("{\n\t.reg .b64 a, b;\n\t"
        "mov.b64 a, {%1, %2};\n\t"
        "mov.b64 b, {%3, %4};\n\t"
        "sub.rn.f32x2 %0, a, b;\n\t}"
        : "=l"(d)
        : "r"(__float_as_uint(x0)), "r"(__float_as_uint(x1)), "r"(h0), "r"(h1));
    l0 = __uint_as_float((uint32_t)d);
    l1 = __uint_as_float((uint32_t)(d >> 32));
}
__device__ __forceinline__ float4 tf32_lo4(const float4& x) {
    float4 l;
    tf32_lo_pair(x.x, x.y, l.x, l.y);
    tf32_lo_pair(x.z, x.w, l.z, l.w);
    return l;
}

struct TileCoord {
    int b, m0, n0;
    int width;   // columns of this unit: bn, or bn / 2 for a tail half
};
__device__ __forceinline__ TileCoord decode_tile(long long unit, const GemmParams& p, int bm, int bn) {
    const long long per_batch = (long long)p.tiles_m * p.tiles_n;
    long long tile = unit;
    int n_off = 0;
    TileCoord t;
    t.width = bn;
    if (unit >= p.full_units) {
        const long long h = unit - p.full_units;
        tile = p.full_units + (h >> 1);
        t.width = bn >> 1;
        n_off = (int)(h & 1) * (bn >> 1);
    }
    t.b = (int)(tile / per_batch);
    const int r = (int)(tile - (long long)t.b * per_batch);
    t.m0 = (r / p.tiles_n) * bm;
    t.n0 = (r % p.tiles_n) * bn + n_off;
    return t;
}

// kCopies: operand copies per stage (1, or 2 = hi and lo halves of the fp32 split)
// BNL: rows (N) of B staged by one CTA = BN / kCta
// kConv: the in-kernel fp32 split. Two rings then: a deep one of RAW stages the copy engine fills (A and B as
// they lie in memory, 128 bytes of K per row), and a short one of OPERAND stages the split warps write and the
// tensor cores read: hi and lo parts of B in shared memory, hi and lo parts of A in tensor memory (64 columns
// per stage behind the two accumulators), so that A costs no shared-memory bandwidth when the products run.
template <int kCopies, int BNL, bool kConv = false>
struct StageLayout {
    static constexpr int kABytes = kBM * kRowBytes;      // 16 KiB
    static constexpr int kBBytes = BNL * kRowBytes;
    static constexpr int kStageBytes = (kConv ? 1 : kCopies) * (kABytes + kBBytes);
    // narrow tiles: the split warps take two k-blocks per trip (one wait for the tensor-memory stores, one proxy
    // fence and one round of arrivals for both), which wants an even number of operand stages
    static constexpr int kConvBatch = BNL <= 64 ? 2 : 1;
    static constexpr int kOpStages = kConv ? (kConvBatch == 2 ? 4 : 3) : 0;
    static constexpr int kOpBytes = kConv ? 2 * kBBytes : 0;
    static constexpr int kStagesFit = (kSmemBudget - kEpilogueStagingBytes - kOpStages * kOpBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit > kMaxStages ? kMaxStages : kStagesFit;
    static constexpr int kMainBytes = kStages * kStageBytes + kOpStages * kOpBytes;
    static constexpr int kDynSmem = kMainBytes + kEpilogueStagingBytes + 1024;   // + alignment slack
    static_assert(kStages >= 2, "at least a double buffer");
};

// kConv (fp32 3xTF32 only): the operands are read in place by TMA and split into their tf32 hi and lo parts
// by eight extra warps inside the kernel, stage by stage, instead of by a pre-pass into a workspace: one
// launch, no scratch memory, and half the operand traffic from L2 (the lo part never travels).
template <int kCta, bool kTF32, bool kSplit, int BN, typename OutT, bool kConv = false>
__global__ void __launch_bounds__(kConv ? kThreadsConv : kThreads, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_lo,
                  const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b_lo,
                  const __grid_constant__ GemmParams p) {
    static_assert(!kConv || (kTF32 && kSplit && kCta == 1), "the in-kernel split is the fp32 3xTF32 path on one CTA");
    constexpr int kCopies = kSplit ? 2 : 1;
    constexpr int kLoadCopies = kConv ? 1 : kCopies;   // copies that arrive by TMA
    constexpr int kPasses = kSplit ? 3 : 1;   // tcgen05.mma passes per k-step
    constexpr int BNL = BN / kCta;             // B rows this CTA stages
    constexpr int kTileM = kBM * kCta;
    using L = StageLayout<kCopies, BNL, kConv>;
    constexpr int kStages = L::kStages;
    constexpr int kElem = kTF32 ? 4 : 2;
    constexpr int kBKElems = kRowBytes / kElem;         // K elements per stage
    constexpr int kKSteps = kRowBytes / kUmmaKBytes;     // tcgen05.mma per stage per pass
    constexpr int kBBoxCols = kRowBytes / kElem;         // N elements per B box when B is N-contiguous
    constexpr int kBBoxBytes = kBKElems * kRowBytes;     // bytes of one such box

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages];
    __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ __align__(8) uint64_t bar_conv[kMaxOpStages];       // kConv: an operand stage's hi / lo parts are written
    __shared__ __align__(8) uint64_t bar_op_empty[kMaxOpStages];   // kConv: the tensor cores are through with an operand stage
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = kCta == 2 ? cluster_ctarank() : 0u;
    const long long tile_first = kCta == 2 ? (long long)(blockIdx.x >> 1) : (long long)blockIdx.x;
    const long long tile_step = kCta == 2 ? (long long)(gridDim.x >> 1) : (long long)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), kConv ? kConvertWarps : 1);   // kConv: released by the split warps
        }
        for (int a = 0; a < kMaxOpStages; ++a) {
            mbar_init(smem_u32(&bar_conv[a]), kConvertWarps);
            mbar_init(smem_u32(&bar_op_empty[a]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), kEpilogueWarps * kCta);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (kCta == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kCta == 2) cluster_sync_all();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Programmatic dependent launch: everything above (barriers, TMEM) touched no global memory and
    // may overlap the tail of the previous kernel in the stream; from here on operands are read and
    // C is written, so wait for the previous grid to complete and flush. Letting the next grid's
    // CTAs start their own prologue as soon as SMs free up hides its launch latency behind this
    // grid's last wave.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (long long tile = tile_first; ok && tile < p.num_tiles; tile += tile_step) {
                TileCoord t = decode_tile(tile, p, kTileM, BN);
                const int bnl = t.width / kCta;   // B rows this CTA stages for this unit
                const bool half = t.width != BN;
                t.m0 += (int)cta_rank * kBM;      // this CTA's rows of A
                t.n0 += (int)cta_rank * bnl;      // this CTA's part of B's N range
                const int b_in = (int)(t.b % p.batch_in), b_out = (int)(t.b / p.batch_in);
                const int za = p.a_in ? b_in : 0, wa = p.a_out ? b_out : 0;
                const int zb = p.b_in ? b_in : 0, wb = p.b_out ? b_out : 0;
                const uint32_t stage_tx = (uint32_t)(kCta * kLoadCopies * (L::kABytes + bnl * kRowBytes));
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.err_word, 0x100u + stage)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    // the even CTA's barrier collects the bytes of both CTAs
                    if (cta_rank == 0) mbar_expect_tx(full, stage_tx);
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + kLoadCopies * L::kABytes;
                    const int k0 = kb * kBKElems;
#pragma unroll
                    for (int ps = 0; ps < kLoadCopies; ++ps) {
                        const CUtensorMap* ma = ps == 0 ? &tm_a : &tm_a_lo;
                        const CUtensorMap* mb = ps == 0 ? &tm_b : &tm_b_lo;
                        // K-contiguous B, tail half: without the fp32 split the second B map is free and
                        // holds the half-height box
                        const CUtensorMap* mb_k = (half && !kSplit) ? &tm_b_lo : mb;
                        tma_load_4d<kCta>(sa + ps * L::kABytes, ma, full, k0, t.m0, za, wa);
                        if constexpr (kConv) {
                            if (p.b_mn_major) {   // [K, N] as stored: one box of 32 K-rows x BNL columns, no swizzle
                                tma_load_4d<kCta>(sb, mb, full, t.n0, k0, zb, wb);
                                continue;
                            }
                        }
                        if (p.b_mn_major) {
#pragma unroll
                            for (int j = 0; j < BNL / kBBoxCols; ++j)
                                if (j < bnl / kBBoxCols)
                                    tma_load_4d<kCta>(sb + ps * L::kBBytes + j * kBBoxBytes, mb, full, t.n0 + j * kBBoxCols, k0, zb, wb);
                        } else {
                            tma_load_4d<kCta>(sb + ps * L::kBBytes, mb_k, full, k0, t.n0, zb, wb);
                        }
                    }
                    ++issued;
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Let copies already in flight land before the CTA can exit: wait (bounded, ignoring the
                // abort flag) on the full barrier of every stage that may still have one outstanding.
                volatile uint32_t never = 0;
                const long long back = issued < kStages ? issued : kStages;
                int s = stage;
                uint32_t ph = phase;
                for (long long i = 0; i < back; ++i) {
                    if (--s < 0) {
                        s = kStages - 1;
                        ph ^= 1u;
                    }
                    // (the odd CTA of a pair signals the even CTA's barrier: its own never completes and this
                    // simply waits out the limit, which is the point of the drain)
                    mbar_wait(smem_u32(&bar_full[s]), ph, &never, nullptr, 0, 20000000ull);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop converged and waits; one elected lane issues. Under a divergent
        // "if (lane == 0)" the compiler keeps descriptors and addresses in per-thread registers and moves
        // them to the uniform file before every tcgen05.mma, which costs more than the instruction itself.
        if (cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const uint32_t a_lbo = 16, a_sbo = 1024;
            const bool b_mn = p.b_mn_major && !kConv;   // the in-kernel split always produces K-contiguous B tiles
            const uint32_t b_lbo = b_mn ? (uint32_t)kBBoxBytes : 16u, b_sbo = 1024;
            // bytes to advance the B descriptor per tcgen05.mma: one 32-byte K slice inside the swizzle
            // span when K is contiguous, kUmmaK rows of 128 bytes when N is contiguous
            const uint32_t b_kstep = b_mn ? (uint32_t)(kUmmaKBytes / kElem) * kRowBytes : (uint32_t)kUmmaKBytes;
            for (long long tile = tile_first; ok && tile < p.num_tiles; tile += tile_step) {
                bool w = mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, &abort_flag, p.err_word, 0x200u + acc);
                if (!__all_sync(0xffffffffu, w)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                const uint32_t idesc = tile >= p.full_units ? p.idesc_half : p.idesc;
                uint32_t first = 0;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    // (kConv: `stage` walks the double buffer of operand stages)
                    w = mbar_wait(smem_u32(kConv ? &bar_conv[stage] : &bar_full[stage]), phase, &abort_flag, p.err_word, 0x300u + stage);
                    if (!__all_sync(0xffffffffu, w)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = kConv ? smem_base + kStages * L::kStageBytes + stage * L::kOpBytes
                                              : sa + kCopies * L::kABytes;
                    if constexpr (kConv) {
                        if (elect_one()) {
                            // A from tensor memory: one 32-bit column per tf32 value, 8 columns per product
                            const uint32_t ta = tmem_base + (uint32_t)(2 * BN + stage * 64);
#pragma unroll
                            for (int ps = 0; ps < 3; ++ps) {   // (lo, hi), (hi, lo), (hi, hi)
                                const int ia = ps == 0 ? 1 : 0, ib = ps == 1 ? 1 : 0;
                                const uint64_t db = make_smem_desc(sb + ib * L::kBBytes, b_lbo, b_sbo);
#pragma unroll
                                for (int k = 0; k < kKSteps; ++k)
                                    umma_ts_tf32(tmem_d, ta + (uint32_t)(ia * 32 + k * 8), db + (uint64_t)((k * kUmmaKBytes) >> 4),
                                                 idesc, (ps | k | (int)first) ? 1u : 0u);
                            }
                            tc_commit<kCta>(smem_u32(&bar_op_empty[stage]));
                        }
                    } else if (elect_one()) {
                        // passes: (lo, hi), (hi, lo), (hi, hi) for the split; (hi, hi) alone otherwise
#pragma unroll
                        for (int ps = 0; ps < kPasses; ++ps) {
                            const int ia = (kPasses == 3 && ps == 0) ? 1 : 0;
                            const int ib = (kPasses == 3 && ps == 1) ? 1 : 0;
                            const uint64_t da = make_smem_desc(sa + ia * L::kABytes, a_lbo, a_sbo);
                            const uint64_t db = make_smem_desc(sb + ib * L::kBBytes, b_lbo, b_sbo);
#pragma unroll
                            for (int k = 0; k < kKSteps; ++k) {
                                umma<kTF32, kCta>(tmem_d, da + (uint64_t)((k * kUmmaKBytes) >> 4),
                                                  db + (uint64_t)((k * b_kstep) >> 4), idesc, (ps | k | (int)first) ? 1u : 0u);
                            }
                        }
                        tc_commit<kCta>(smem_u32(&bar_empty[stage]));
                    }
                    __syncwarp();
                    first = 1;
                    if (++stage == (kConv ? L::kOpStages : kStages)) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (elect_one()) tc_commit<kCta>(smem_u32(&bar_acc_full[acc]));
                __syncwarp();
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else if (kConv && warp >= 2 + kEpilogueWarps) {
        // ---------------- operand split (warps 10..17) ----------------
        // Each raw stage holds fp32 A and B as they lie in memory. Into the next operand stage go
        // hi = x with the low 13 mantissa bits cleared (exactly a tf32 value) and lo = (x - hi) cleared the
        // same way: A's into tensor memory (a warp reaches the 32 lanes of its id mod 4: one row of the tile
        // per thread, the two warps of a quarter take 16 of the 32 K columns each), B's into shared memory.
        if constexpr (kConv) {
            static_assert(2 * BN + L::kOpStages * 64 <= (int)kTmemCols && L::kOpStages <= kMaxOpStages, "accumulators and A stages fit tensor memory");
            const int t = (int)threadIdx.x - 32 * (2 + kEpilogueWarps);
            const int khalf = (warp - (2 + kEpilogueWarps)) >> 2;
            const int m = (warp & 3) * 32 + lane;
            const uint32_t a_tmem = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(2 * BN + khalf * 16);
            int stage = 0, ostage = 0;         // raw ring and operand ring positions
            uint32_t phase = 0, ophase = 0;
            uint8_t* const base = smem_raw + (smem_base - smem_u32(smem_raw));
            // this CTA's k-blocks, over all of its tiles: the split does not care where a tile ends
            const long long my_tiles = tile_first < p.num_tiles ? (p.num_tiles - tile_first + tile_step - 1) / tile_step : 0;
            const long long total_kb = my_tiles * p.num_kb;
            constexpr int kBatch = L::kConvBatch;
            for (long long i = 0; i < total_kb; i += kBatch) {
                const int nb = total_kb - i < kBatch ? (int)(total_kb - i) : kBatch;
                int st[kBatch], os[kBatch];
                bool w = true;
#pragma unroll
                for (int j = 0; j < kBatch; ++j) {
                    st[j] = stage;
                    os[j] = ostage;
                    if (j < nb) {
                        if (w) w = mbar_wait_poll(smem_u32(&bar_full[stage]), phase, &abort_flag, p.err_word, 0x700u + stage);
                        if (w) w = mbar_wait_poll(smem_u32(&bar_op_empty[ostage]), ophase ^ 1u, &abort_flag, p.err_word, 0x710u + ostage);
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        if (++ostage == L::kOpStages) {
                            ostage = 0;
                            ophase ^= 1u;
                        }
                    }
                }
                if (!__all_sync(0xffffffffu, w)) break;
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < kBatch; ++j) {
                    if (j >= nb) break;
                    const uint8_t* const raw_a = base + st[j] * L::kStageBytes;
                    const uint8_t* const raw_b = raw_a + L::kABytes;
                    uint8_t* const b_hi = base + kStages * L::kStageBytes + os[j] * L::kOpBytes;
                    uint8_t* const b_lo = b_hi + L::kBBytes;
                    {
                        // row m of the tile: 16-byte chunk c sits at position c ^ (m & 7) of its 128 bytes
                        float4 x[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            x[c] = *reinterpret_cast<const float4*>(raw_a + m * kRowBytes + (((khalf * 4 + c) ^ (m & 7)) << 4));
                        uint32_t h[16], l[16];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float4 lo = tf32_lo4(x[c]);
                            h[4 * c + 0] = __float_as_uint(x[c].x); l[4 * c + 0] = __float_as_uint(lo.x);
                            h[4 * c + 1] = __float_as_uint(x[c].y); l[4 * c + 1] = __float_as_uint(lo.y);
                            h[4 * c + 2] = __float_as_uint(x[c].z); l[4 * c + 2] = __float_as_uint(lo.z);
                            h[4 * c + 3] = __float_as_uint(x[c].w); l[4 * c + 3] = __float_as_uint(lo.w);
                        }
                        tmem_st16(a_tmem + (uint32_t)(os[j] * 64), h);
                        tmem_st16(a_tmem + (uint32_t)(os[j] * 64 + 32), l);
                    }
                    if (!p.b_mn_major) {
                        // same offsets in and out, so the swizzle the copy engine applied carries over
#pragma unroll
                        for (int off = t * 16; off < L::kBBytes; off += 32 * kConvertWarps * 16) {
                            const float4 x = *reinterpret_cast<const float4*>(raw_b + off);
                            *reinterpret_cast<float4*>(b_hi + off) = x;
                            *reinterpret_cast<float4*>(b_lo + off) = tf32_lo4(x);
                        }
                    } else {
                        // B arrived [32 K-rows][BNL columns]; the tensor cores want rows of N with K contiguous
                        // (128 bytes per row, 16-byte chunk c of row n at position c ^ (n & 7), the layout the copy
                        // engine's 128-byte swizzle gives a K-contiguous tile). One chunk = 4 consecutive K of one n.
                        const float* raw = reinterpret_cast<const float*>(raw_b);
#pragma unroll
                        for (int q = t; q < BNL * 8; q += 32 * kConvertWarps) {
                            const int n = q % BNL, c = q / BNL;
                            const float4 x = make_float4(raw[(4 * c + 0) * BNL + n], raw[(4 * c + 1) * BNL + n],
                                                         raw[(4 * c + 2) * BNL + n], raw[(4 * c + 3) * BNL + n]);
                            const int off = n * kRowBytes + ((c ^ (n & 7)) << 4);
                            *reinterpret_cast<float4*>(b_hi + off) = x;
                            *reinterpret_cast<float4*>(b_lo + off) = tf32_lo4(x);
                        }
                    }
                }
                tmem_wait_st();
                // the tensor cores read shared memory through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        if (j < nb) {
                            mbar_arrive(smem_u32(&bar_conv[os[j]]));    // operands ready
                            mbar_arrive(smem_u32(&bar_empty[st[j]]));   // raw stage free for the next load
                        }
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9; TMEM lane quarter = warp id mod 4) ----------------
        const int q = warp & 3;
        const int col_half = (warp - 2) >> 2;   // warps 2-5 take the first half of the columns, 6-9 the second
        const int row_in_tile = q * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        OutT* Cbase = static_cast<OutT*>(p.C);
        const OutT* Rbase = static_cast<const OutT*>(p.residual);
        const OutT* bias = static_cast<const OutT*>(p.bias);
        const int epi = p.epilogue;
        const bool has_bias = epi == CG_B200_EPI_BIAS || epi == CG_B200_EPI_BIAS_RELU ||
                              epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_BIAS_RESIDUAL;
        const bool has_res = epi == CG_B200_EPI_BIAS_RESIDUAL || epi == CG_B200_EPI_RESIDUAL;
        const bool bias_vec = has_bias && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
        constexpr int kPack = 16 / sizeof(OutT);  // elements per 16-byte store
        constexpr int kRowPieces = 32 / kPack;    // 16-byte pieces per row of a 32-column chunk
        constexpr int kSub = 8 / kRowPieces;      // chunks per 128-byte staging row (2 for 16-bit outputs)
        uint8_t* const stg = smem_raw + (smem_base - smem_u32(smem_raw)) + L::kMainBytes + (warp - 2) * 4096;
        for (long long tile = tile_first; tile < p.num_tiles; tile += tile_step) {
            bool ok = mbar_wait(smem_u32(&bar_acc_full[acc]), acc_phase, &abort_flag, p.err_word, 0x400u + acc,
                                2000000000ull, 200);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const TileCoord t = decode_tile(tile, p, kTileM, BN);
            const long long m = (long long)t.m0 + (long long)cta_rank * kBM + row_in_tile;
            const bool row_ok = m < p.M;
            const long long row_off = (long long)(t.b % p.batch_in) * p.c_stride_in + (long long)(t.b / p.batch_in) * p.c_stride_out + m * p.ldc;
            const int c_lo = col_half * (t.width >> 1), c_hi = c_lo + (t.width >> 1);
            int staged = 0;            // 32-column chunks waiting in the staging rows
            long long staged_n0 = 0;   // first column of the staged data
            const long long m_base = (long long)t.m0 + (long long)cta_rank * kBM + q * 32;
            const long long tile_off = row_off - m * p.ldc + p.dst_row_offset;   // batch part of the offset
            auto flush = [&]() {
                if (staged == 0) return;
                __syncwarp();
                const int sh = staged * kRowPieces == 8 ? 3 : 2;   // pieces per row present: 8 or 4
                const int total = 32 << sh;
                for (int idx = lane; idx < total; idx += 32) {
                    const int r = idx >> sh, c = idx & ((1 << sh) - 1);
                    const int4 val = *reinterpret_cast<const int4*>(stg + ((r * 8 + (c ^ (r & 7))) << 4));
                    if (m_base + r < p.M) {
                        const long long off = tile_off + (m_base + r) * p.ldc + staged_n0 + c * kPack;
                        *reinterpret_cast<int4*>(Cbase + off) = val;
                        for (int d = 0; d < p.n_peer; ++d)
                            *reinterpret_cast<int4*>(static_cast<OutT*>(p.peer[d]) + off) = val;
                    }
                }
                __syncwarp();   // the staging rows are free again
                staged = 0;
            };
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                float v[32];
                __syncwarp();  // lanes that skipped stores rejoin before the warp-wide TMEM load
                if (p.num_kb > 0) {
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                }
                const long long n0 = (long long)t.n0 + c0;
                if (n0 >= p.N) continue;
                const bool full = n0 + 32 <= p.N;
                if (epi == CG_B200_EPI_SCALE) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
                }
                if (has_bias) {
                    if (full && bias_vec) {
#pragma unroll
                        for (int g = 0; g < 32 / kPack; ++g) {
                            Vec16<OutT> bv = ld_keep(bias + n0 + g * kPack);
#pragma unroll
                            for (int j = 0; j < kPack; ++j) v[g * kPack + j] += Elem<OutT>::to_f32(bv.v[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + j < p.N) v[j] += Elem<OutT>::to_f32(bias[n0 + j]);
                    }
                }
                if (epi == CG_B200_EPI_BIAS_RELU || epi == CG_B200_EPI_RELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.0f ? v[j] : 0.0f;
                } else if (epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_GELU_TANH) {
                    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = gelu_epilogue<OutT>(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float2 r = gelu_pair_fast(make_float2(v[j], v[j + 1]));
                            v[j] = r.x;
                            v[j + 1] = r.y;
                        }
                    }
                }
                if (full) {
                    if (has_res && row_ok) {
                        const OutT* rrow = Rbase + row_off + n0;
#pragma unroll
                        for (int g = 0; g < 32 / kPack; ++g) {
                            Vec16<OutT> rv = ld_stream(rrow + g * kPack);
#pragma unroll
                            for (int j = 0; j < kPack; ++j) v[g * kPack + j] += Elem<OutT>::to_f32(rv.v[j]);
                        }
                    }
                    // Transpose through shared memory so that global (and peer) stores are whole row
                    // segments: lane = row writes its 16-byte pieces into a 128-byte staging row (two
                    // 32-column chunks side by side for 16-bit outputs), flush() then moves the pieces out
                    // in linear order, 128 contiguous bytes of a row per 8 lanes. Piece c of row r sits at
                    // slot c ^ (r & 7): conflict-free in both directions.
                    if (staged == 0) staged_n0 = n0;
#pragma unroll
                    for (int g = 0; g < kRowPieces; ++g) {
                        Vec16<OutT> o;
#pragma unroll
                        for (int j = 0; j < kPack; ++j) o.v[j] = Elem<OutT>::from_f32(v[g * kPack + j]);
                        const int c = staged * kRowPieces + g;
                        *reinterpret_cast<int4*>(stg + ((lane * 8 + (c ^ (lane & 7))) << 4)) = *reinterpret_cast<const int4*>(&o);
                    }
                    ++staged;
                    if (staged == kSub || c0 + 32 >= c_hi) flush();
                } else {
                    flush();   // a staged full chunk goes out before the ragged one
                    if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + j < p.N) {
                            float r = v[j];
                            if (has_res) r += Elem<OutT>::to_f32(Rbase[row_off + n0 + j]);
                            const OutT o = Elem<OutT>::from_f32(r);
                            const long long off = row_off + p.dst_row_offset + n0 + j;
                            Cbase[off] = o;
                            for (int d = 0; d < p.n_peer; ++d) static_cast<OutT*>(p.peer[d])[off] = o;
                        }
                    }
                }
            }
            flush();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                // the issuer waits on the even CTA's barrier for the epilogue warps of both CTAs
                if (cta_rank == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
                else mbar_arrive_remote(smem_u32(&bar_acc_empty[acc]), 0);
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (p.bar_flags) __threadfence_system();   // this thread's peer stores, before the CTA counts itself done
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if constexpr (kCta == 2) cluster_sync_all();   // neither CTA leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kCta == 1)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (p.bar_flags) {
        // The flag barrier of the fused all-gather, without a launch of its own: the last CTA of the grid
        // to get here knows that every other CTA's peer stores are fenced, and speaks for the rank.
        __shared__ bool last_cta;
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(p.bar_done, 1u);
            last_cta = prev == gridDim.x - 1;
            if (last_cta) *p.bar_done = 0;   // every CTA has counted itself: ready for the next launch
        }
        __syncthreads();
        if (last_cta) {
            __threadfence_system();
            const int r = (int)threadIdx.x;
            if (r < p.bar_world && r != p.bar_rank)
                peer_flag_exchange(p.bar_flags, p.bar_rank, r, p.bar_epoch, p.bar_limit_ns, p.err_word);
        }
    }
}

// fp32 operands are rewritten into a K-contiguous workspace before the GEMM: hi = x with the low
// 13 mantissa bits cleared (exactly a tf32 value) and, for the 3xTF32 split, lo = (x - hi) cleared
// the same way (lo == nullptr skips it). rows x cols, source row stride ld_src, destination row
// stride ld_dst >= cols (the pad columns are written as zero).

// Both operands in ONE launch (the whole fp32 GEMM of 1024^3 takes 40 us, a launch a tenth of that):
// blocks [0, a_blocks) split A row-wise; the others handle B, row-wise when it is stored [N, K], through
// 32 x 32 shared-memory tiles when it is [K, N] and has to be transposed. The GEMM behind it is
// launched as a programmatic dependent, so its CTAs may set up while this grid drains.
struct SplitOperand {
    const float* src;
    float *hi, *lo;
    long long rows, cols, ld_src, ld_dst, batch, bs_src, bs_dst;
};

__device__ __forceinline__ void tf32_split_rows(const SplitOperand& o, long long first, long long stride) {
    // four columns per thread where rows, batches and bases are 16-byte tiled (ld_dst always is)
    const bool vec = ((o.ld_src | o.bs_src | o.bs_dst | o.ld_dst) & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(o.src) | reinterpret_cast<uintptr_t>(o.hi) |
                       reinterpret_cast<uintptr_t>(o.lo)) & 15) == 0;
    if (vec) {
        const long long q = o.ld_dst >> 2;
        const long long per = o.rows * q;
        const long long total = per * o.batch;
        for (long long i = first; i < total; i += stride) {
            const long long b = i / per;
            const long long r = (i - b * per) / q;
            const long long c = (i - b * per - r * q) << 2;
            const float* sp = o.src + b * o.bs_src + r * o.ld_src + c;
            float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (c + 3 < o.cols) {
                x = *reinterpret_cast<const float4*>(sp);
            } else {   // the last, partly padded group of a row
                if (c < o.cols) x.x = sp[0];
                if (c + 1 < o.cols) x.y = sp[1];
                if (c + 2 < o.cols) x.z = sp[2];
            }
            float4 h, l;
            tf32_split(x.x, h.x, l.x);
            tf32_split(x.y, h.y, l.y);
            tf32_split(x.z, h.z, l.z);
            tf32_split(x.w, h.w, l.w);
            const long long d = b * o.bs_dst + r * o.ld_dst + c;
            *reinterpret_cast<float4*>(o.hi + d) = h;
            if (o.lo) *reinterpret_cast<float4*>(o.lo + d) = l;
        }
        return;
    }
    const long long per = o.rows * o.ld_dst;
    const long long total = per * o.batch;
    for (long long i = first; i < total; i += stride) {
        const long long b = i / per;
        const long long r = (i - b * per) / o.ld_dst;
        const long long c = i - b * per - r * o.ld_dst;
        float x = 0.0f;
        if (c < o.cols) x = o.src[b * o.bs_src + r * o.ld_src + c];
        float h, l;
        tf32_split(x, h, l);
        o.hi[b * o.bs_dst + r * o.ld_dst + c] = h;
        if (o.lo) o.lo[b * o.bs_dst + r * o.ld_dst + c] = l;
    }
}

// `bo` describes B as stored: [rows = K, cols = N]; the destination is [N, ld_dst >= K].
__global__ void __launch_bounds__(256)
tf32_split_operands_kernel(const SplitOperand ao, const SplitOperand bo, int a_blocks, int b_transpose, int tiles_x,
                           int tiles_y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float tile[32][33];
    if ((int)blockIdx.x < a_blocks) {
        tf32_split_rows(ao, (long long)blockIdx.x * 256 + threadIdx.x, (long long)a_blocks * 256);
        return;
    }
    const long long blk = (long long)blockIdx.x - a_blocks;
    if (!b_transpose) {
        const long long b_blocks = (long long)gridDim.x - a_blocks;
        tf32_split_rows(bo, blk * 256 + threadIdx.x, b_blocks * 256);
        return;
    }
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long per_batch = (long long)tiles_x * tiles_y;
    const long long b = blk / per_batch;
    const long long t = blk - b * per_batch;
    const long long c0 = (t % tiles_x) * 32, r0 = (t / tiles_x) * 32;
    for (int j = ty; j < 32; j += 8) {
        const long long r = r0 + j, c = c0 + tx;
        tile[j][tx] = (r < bo.rows && c < bo.cols) ? bo.src[b * bo.bs_src + r * bo.ld_src + c] : 0.0f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const long long c = c0 + j, r = r0 + tx;   // destination row = source column
        if (c < bo.cols && r < bo.ld_dst) {
            float h, l;
            tf32_split(tile[tx][j], h, l);
            bo.hi[b * bo.bs_dst + c * bo.ld_dst + r] = h;
            if (bo.lo) bo.lo[b * bo.bs_dst + c * bo.ld_dst + r] = l;
        }
    }
}

// ---- host side --------------------------------------------------------------------------------------
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    });
    return fn;
}

// Two batch levels of one operand: counts (1 = broadcast or unused) and strides in elements.
struct BatchDims {
    uint64_t n_in = 1, n_out = 1;
    uint64_t s_in = 0, s_out = 0;
};

// 4-D map {inner, rows, batch_in, batch_out}; box {box_inner, box_rows, 1, 1}; 128-byte swizzle; OOB
// reads give zero. A level with count 1 is never stepped, so its stride only has to be encodable.
static int make_map(CUtensorMap* map, const void* base, int dtype, uint64_t inner, uint64_t rows, const BatchDims& bd,
                    uint64_t ld_elems, uint32_t box_inner, uint32_t box_rows, bool swizzle = true) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) return CG_B200_ERR_CUDA;
    const uint64_t esz = dtype_bytes(dtype);
    CUtensorMapDataType dt = dtype == CG_B200_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                  : (dtype == CG_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const uint64_t fallback = rows * ld_elems * esz;   // any 16-byte multiple serves a count-1 level
    cuuint64_t dims[4] = {inner, rows, bd.n_in, bd.n_out};
    cuuint64_t strides[3] = {ld_elems * esz, bd.n_in > 1 ? bd.s_in * esz : fallback, bd.n_out > 1 ? bd.s_out * esz : fallback};
    cuuint32_t box[4] = {box_inner, box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        note_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return CG_B200_ERR_CUDA;
    }
    return CG_B200_OK;
}

static uint32_t make_idesc(int in_dtype, bool tf32, bool b_mn_major, int bm, int bn) {
    uint32_t d = 0;
    d |= 1u << 4;                                                   // accumulator format: F32
    const uint32_t fmt = tf32 ? 2u : (in_dtype == CG_B200_BF16 ? 1u : 0u);
    d |= fmt << 7;                                                  // A format
    d |= fmt << 10;                                                 // B format
    d |= 0u << 15;                                                  // A: K-major
    d |= (b_mn_major ? 1u : 0u) << 16;                              // B: MN-major when N is contiguous
    d |= (uint32_t)(bn >> 3) << 17;                                 // N / 8
    d |= (uint32_t)(bm >> 4) << 24;                                 // M / 16 (256 for a CTA pair)
    return d;
}

// fp32 inputs always go through the workspace: `copies` arrays (hi, or hi and lo) of A as [M, ldk]
// and of B as [N, ldk], K contiguous, ldk = K rounded up to 4 elements (16 bytes).
struct Fp32Plan {
    bool active;
    int copies;
    long long ldk;
    long long a_elems, b_elems;   // per copy
    size_t bytes;
};

static inline long long round_up(long long x, long long a) { return (x + a - 1) / a * a; }

static Fp32Plan plan_fp32(const cg_b200_gemm_desc* d) {
    Fp32Plan s{};
    s.active = d->in_dtype == CG_B200_F32;
    if (!s.active) return s;
    s.copies = d->compute == CG_B200_COMPUTE_TF32 ? 1 : 2;
    s.ldk = round_up(d->K > 0 ? d->K : 1, 4);
    const long long a_batches = (d->batch_stride_a == 0 || d->batch == 1) ? 1 : d->batch;
    const long long b_batches = (d->batch_stride_b == 0 || d->batch == 1) ? 1 : d->batch;
    s.a_elems = round_up(a_batches * d->M * s.ldk, 64);
    s.b_elems = round_up(b_batches * d->N * s.ldk, 64);
    s.bytes = (size_t)(s.copies * (s.a_elems + s.b_elems)) * sizeof(float);
    return s;
}

static int validate_desc(const cg_b200_gemm_desc* d) {
    if (!d) return CG_B200_ERR_NULL_POINTER;
    if (!dtype_ok(d->in_dtype) || !dtype_ok(d->out_dtype)) return CG_B200_ERR_INVALID_ARG;
    if (d->M < 0 || d->N < 0 || d->K < 0 || d->batch < 1) return CG_B200_ERR_INVALID_ARG;
    if (d->epilogue < CG_B200_EPI_NONE || d->epilogue > CG_B200_EPI_GELU_TANH) return CG_B200_ERR_INVALID_ARG;
    if (d->compute < CG_B200_COMPUTE_DEFAULT || d->compute > CG_B200_COMPUTE_TF32) return CG_B200_ERR_INVALID_ARG;
    if (d->in_dtype != CG_B200_F32 && d->compute != CG_B200_COMPUTE_DEFAULT) return CG_B200_ERR_INVALID_ARG;
    if (d->in_dtype == CG_B200_F32 && d->out_dtype != CG_B200_F32) return CG_B200_ERR_UNSUPPORTED;
    if (d->lda < d->K || d->ldc < d->N) return CG_B200_ERR_INVALID_ARG;
    if (d->ldb < (d->b_transposed ? d->K : d->N)) return CG_B200_ERR_INVALID_ARG;
    if (d->batch_stride_a < 0 || d->batch_stride_b < 0 || d->batch_stride_c < 0) return CG_B200_ERR_INVALID_ARG;
    if (d->batch_inner < 0 || (d->batch_inner > 1 && d->batch % d->batch_inner != 0)) return CG_B200_ERR_INVALID_ARG;
    if (d->batch_inner > 1 && (d->inner_stride_a < 0 || d->inner_stride_b < 0 || d->inner_stride_c <= 0))
        return CG_B200_ERR_INVALID_ARG;
    // outputs of different batches must not overlap: one after another, or side by side inside the rows
    // (column blocks, e.g. the heads of an attention output)
    if (d->batch_inner <= 1 && d->batch > 1 && d->batch_stride_c < d->M * d->ldc &&
        !(d->batch_stride_c >= d->N && d->batch * d->batch_stride_c <= d->ldc))
        return CG_B200_ERR_INVALID_ARG;
    if (d->M > 0x7fffffffLL || d->N > 0x7fffffffLL || d->K > 0x7fffffffLL || d->batch > 0x7fffffffLL)
        return CG_B200_ERR_UNSUPPORTED;
    return CG_B200_OK;
}

// CG_B200_GEMM_PDL=0 turns programmatic dependent launch off (a test and tuning knob).
static bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("CG_B200_GEMM_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

// CG_B200_GEMM_TAIL=0 turns the half-width tail units off (a test and tuning knob).
static bool tail_split_enabled() {
    static const bool on = [] {
        const char* e = getenv("CG_B200_GEMM_TAIL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <int kCta, bool kTF32, bool kSplit, int BN, typename OutT, bool kConv = false>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& ta_lo, const CUtensorMap& tb,
                          const CUtensorMap& tb_lo, GemmParams& p, cudaStream_t s) {
    using L = StageLayout<kSplit ? 2 : 1, BN / kCta, kConv>;
    auto kern = gemm_sm100_kernel<kCta, kTF32, kSplit, BN, OutT, kConv>;
    // the attribute is per device; setting it again is cheap
    CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynSmem));
    const int elem = kTF32 ? 4 : 2;
    p.tiles_m = (int)((p.M + kBM * kCta - 1) / (kBM * kCta));
    p.tiles_n = (int)((p.N + BN - 1) / BN);
    p.num_tiles = (long long)p.tiles_m * p.tiles_n * p.batch;
    p.num_kb = (int)((p.K + (kRowBytes / elem) - 1) / (kRowBytes / elem));
    // persistent: one CTA (or CTA pair) per SM (or SM pair), never more CTAs than tiles
    const long long slots = sm_count() / kCta;
    p.full_units = p.num_tiles;
    const bool tail = p.tail_split == 0 ? tail_split_enabled() : p.tail_split == 2;
    if (kCta == 2 && BN == 256 && !kSplit && tail) {
        // a last partial wave of r <= slots / 2 tiles runs as 2r half-width units instead
        const long long r = p.num_tiles % slots;
        if (r > 0 && 2 * r <= slots) {
            p.full_units = p.num_tiles - r;
            p.num_tiles = p.full_units + 2 * r;
        }
    }
    const int groups = (int)(p.num_tiles < slots ? p.num_tiles : slots);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(groups * kCta), 1, 1);
    cfg.blockDim = dim3(kConv ? kThreadsConv : kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCta;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    CGB_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, ta_lo, tb, tb_lo, p));
    return CG_B200_OK;
}

template <int kCta, bool kTF32, bool kSplit, typename OutT>
static int launch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& ta_lo, const CUtensorMap& tb,
                     const CUtensorMap& tb_lo, GemmParams& p, cudaStream_t s) {
    if constexpr (kCta == 2) {
        if (bn == 128) return launch_variant<2, kTF32, kSplit, 128, OutT>(ta, ta_lo, tb, tb_lo, p, s);
        return launch_variant<2, kTF32, kSplit, 256, OutT>(ta, ta_lo, tb, tb_lo, p, s);
    } else if constexpr (kSplit) {
        if (bn == 64) return launch_variant<1, kTF32, true, 64, OutT>(ta, ta_lo, tb, tb_lo, p, s);
        return launch_variant<1, kTF32, true, 128, OutT>(ta, ta_lo, tb, tb_lo, p, s);
    } else {
        if (bn == 64) return launch_variant<1, kTF32, false, 64, OutT>(ta, ta_lo, tb, tb_lo, p, s);
        if (bn == 128) return launch_variant<1, kTF32, false, 128, OutT>(ta, ta_lo, tb, tb_lo, p, s);
        return launch_variant<1, kTF32, false, 256, OutT>(ta, ta_lo, tb, tb_lo, p, s);
    }
}

// CG_B200_GEMM_PAIR=0 in the environment turns the CTA-pair variant off (a test and tuning knob).
static bool pair_enabled() {
    static const bool on = [] {
        const char* e = getenv("CG_B200_GEMM_PAIR");
        return !(e && e[0] == '0');
    }();
    return on;
}

static int choose_bn(const cg_b200_gemm_desc* d, bool split) {
    if (split) {
        // 3xTF32: 128 x 128 tiles, or 128 x 64 when the wider tiles would leave half of the SMs idle
        const long long tiles = ((d->M + kBM - 1) / kBM) * ((d->N + 127) / 128) * d->batch;
        return (d->N <= 64 || 2 * tiles <= sm_count()) ? 64 : 128;
    }
    if (d->N <= 64) return 64;
    if (d->N <= 128) return 128;
    return 256;
}

}  // namespace cgb

using namespace cgb;

extern "C" int cg_b200_gemm_workspace_bytes(const cg_b200_gemm_desc* desc, size_t* bytes) {
    if (!bytes) return CG_B200_ERR_NULL_POINTER;
    *bytes = 0;
    int st = validate_desc(desc);
    if (st) return st;
    *bytes = plan_fp32(desc).bytes;
    return CG_B200_OK;
}

// Shared body of the GEMM entry points. `shared_err_word`: report bounded-wait timeouts through
// the library's per-device error word (allocated on first use); otherwise through `err_word`
// (may be null).
struct PeerSet {
    void* const* peer_c = nullptr;   // `world` pointers to the peers' full C buffers (entry `rank` is skipped)
    int world = 1, rank = 0;
    PeerBarrier* barrier = nullptr;  // folded into the kernel's tail when given
};

static int gemm_run(const cg_b200_gemm_desc* desc, const void* A, const void* B, const void* bias,
                    const void* residual, void* C, void* workspace, size_t workspace_bytes, void* stream,
                    bool shared_err_word, uint32_t* err_word, const PeerSet* peers = nullptr,
                    const cg_b200_gemm_tuning* tuning = nullptr, bool use_workspace_split = false) {
    int st = validate_desc(desc);
    if (st) return st;
    if (tuning) {
        const cg_b200_gemm_tuning& t = *tuning;
        if ((t.tile_n != 0 && t.tile_n != 64 && t.tile_n != 128 && t.tile_n != 256) || t.cta_pair < 0 || t.cta_pair > 2 ||
            t.tail_split < 0 || t.tail_split > 2 || t.reserved != 0)
            return CG_B200_ERR_INVALID_ARG;
    }
    const cg_b200_gemm_desc& d = *desc;
    if (d.M == 0 || d.N == 0) return CG_B200_OK;
    if (!C || (d.K > 0 && (!A || !B))) return CG_B200_ERR_NULL_POINTER;   // K == 0: A and B are empty
    const int epi = d.epilogue;
    const bool need_bias = epi == CG_B200_EPI_BIAS || epi == CG_B200_EPI_BIAS_RELU ||
                           epi == CG_B200_EPI_BIAS_GELU_TANH || epi == CG_B200_EPI_BIAS_RESIDUAL;
    const bool need_res = epi == CG_B200_EPI_BIAS_RESIDUAL || epi == CG_B200_EPI_RESIDUAL;
    if (need_bias && !bias) return CG_B200_ERR_NULL_POINTER;
    if (need_res && !residual) return CG_B200_ERR_NULL_POINTER;
    const size_t in_sz = dtype_bytes(d.in_dtype), out_sz = dtype_bytes(d.out_dtype);
    const Fp32Plan sp = plan_fp32(desc);
    // fp32, 3xTF32: when TMA can read A and B where they lie (16-byte aligned bases and strides) the hi / lo
    // split happens inside the GEMM kernel and no workspace is touched; otherwise a pre-pass rewrites the
    // operands into the workspace first. use_workspace_split forces the pre-pass (the entry point whose
    // scratch is the library's own array exists to exercise exactly that path).
    const bool in_kernel_split =
        sp.active && sp.copies == 2 && !use_workspace_split && d.K > 0 && aligned_to(A, 16) && aligned_to(B, 16) &&
        (d.lda * 4) % 16 == 0 && (d.ldb * 4) % 16 == 0 && (d.batch_stride_a * 4) % 16 == 0 && (d.batch_stride_b * 4) % 16 == 0;
    // C rows are written with 16-byte stores
    if (!aligned_to(C, 16) || (d.ldc * out_sz) % 16 || (d.batch_stride_c * out_sz) % 16) return CG_B200_ERR_MISALIGNED;
    if (d.batch_inner > 1 && (d.inner_stride_c * out_sz) % 16) return CG_B200_ERR_MISALIGNED;
    if (need_res && !aligned_to(residual, 16)) return CG_B200_ERR_MISALIGNED;
    if (need_bias && !aligned_to(bias, out_sz)) return CG_B200_ERR_MISALIGNED;
    if (!sp.active) {
        // TMA reads A and B in place: 16-byte aligned bases and strides
        if (d.K > 0 && (!aligned_to(A, 16) || !aligned_to(B, 16))) return CG_B200_ERR_MISALIGNED;
        if ((d.lda * in_sz) % 16 || (d.ldb * in_sz) % 16) return CG_B200_ERR_MISALIGNED;
        if ((d.batch_stride_a * in_sz) % 16 || (d.batch_stride_b * in_sz) % 16) return CG_B200_ERR_MISALIGNED;
        if (d.batch_inner > 1 && ((d.inner_stride_a * in_sz) % 16 || (d.inner_stride_b * in_sz) % 16))
            return CG_B200_ERR_MISALIGNED;
    } else {
        if (d.batch_inner > 1) return CG_B200_ERR_UNSUPPORTED;   // fp32 operands: one batch level only
        if (!aligned_to(A, 4) || !aligned_to(B, 4)) return CG_B200_ERR_MISALIGNED;
        if (!in_kernel_split) {
            if (!workspace || workspace_bytes < sp.bytes) return CG_B200_ERR_WORKSPACE;
            if (!aligned_to(workspace, 256)) return CG_B200_ERR_MISALIGNED;
        }
    }
    st = require_sm100();
    if (st) return st;
    cudaStream_t s = (cudaStream_t)stream;

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = d.M; p.N = d.N; p.K = d.K; p.batch = d.batch;
    p.ldc = d.ldc;
    // One batch level is the inner level with a single outer step.
    const bool two = d.batch_inner > 1;
    p.batch_in = two ? d.batch_inner : d.batch;
    const long long n_out = d.batch / p.batch_in;
    p.c_stride_in = two ? d.inner_stride_c : d.batch_stride_c;
    p.c_stride_out = two ? d.batch_stride_c : 0;
    p.bias = bias; p.residual = residual; p.C = C;
    if (peers && peers->world > 1) {
        // C is the base of the full [world * M, N] buffer: this rank's rows start `rank * M` rows in,
        // in the local buffer and in every peer's
        p.dst_row_offset = (long long)peers->rank * d.M * d.ldc;
        for (int r = 0; r < peers->world; ++r)
            if (r != peers->rank) p.peer[p.n_peer++] = peers->peer_c[r];
        if (PeerBarrier* b = peers->barrier) {
            p.bar_flags = reinterpret_cast<unsigned long long* const*>(b->table_dev);
            p.bar_done = b->done_counter;
            p.bar_epoch = b->epoch;
            p.bar_limit_ns = b->wait_limit_ns;
            p.bar_world = b->world;
            p.bar_rank = b->rank;
        }
    }
    p.epilogue = epi; p.alpha = d.alpha;
    p.b_mn_major = (d.b_transposed || (sp.active && !in_kernel_split)) ? 0 : 1;   // the fp32 workspace copy of B is K-contiguous
    const long long a_s_in = two ? d.inner_stride_a : d.batch_stride_a, a_s_out = two ? d.batch_stride_a : 0;
    const long long b_s_in = two ? d.inner_stride_b : d.batch_stride_b, b_s_out = two ? d.batch_stride_b : 0;
    p.a_in = a_s_in != 0 && p.batch_in > 1;
    p.a_out = a_s_out != 0 && n_out > 1;
    p.b_in = b_s_in != 0 && p.batch_in > 1;
    p.b_out = b_s_out != 0 && n_out > 1;
    p.err_word = shared_err_word ? device_error_word() : err_word;

    const bool tf32 = d.in_dtype == CG_B200_F32;
    const bool split = sp.active && sp.copies == 2;
    int bn = choose_bn(desc, split);
    // CTA pairs (256 x 256 tiles) for 16-bit inputs once the problem spans more than one such tile row
    int cta = (!tf32 && bn == 256 && d.M > kBM && pair_enabled()) ? 2 : 1;
    // (Halving the tile width when few 256 x 256 tiles exist - a small shard of a sharded GEMM - was
    // measured slower than leaving SM pairs idle: 512 x 4096 x 4096 takes 24.7 us with 32 full tiles and
    // 27.0 us with 64 half-width ones. The narrower tile stays available through cg_b200_gemm_tuned.)
    p.tail_split = 0;
    if (tuning) {
        // an autotuner's choice replaces the heuristic above; combinations the kernels do not have are refused
        const cg_b200_gemm_tuning& t = *tuning;
        if (t.cta_pair == 2 && tf32) return CG_B200_ERR_UNSUPPORTED;          // pairs: 16-bit inputs only
        if (t.cta_pair != 0) cta = t.cta_pair;
        else if (t.tile_n == 64) cta = 1;                                     // a 64-wide tile exists for one CTA only
        if (t.tile_n != 0) {
            if (split && t.tile_n == 256) return CG_B200_ERR_UNSUPPORTED;     // the 3xTF32 kernel: 64 or 128 wide
            bn = t.tile_n;
        } else if (cta == 2 && bn < 128) {
            bn = 128;
        }
        if (cta == 2 && bn == 64) return CG_B200_ERR_UNSUPPORTED;             // a pair's tile is 128 or 256 wide
        p.tail_split = t.tail_split;
    }
    const bool b_desc_mn = p.b_mn_major != 0 && !in_kernel_split;   // the in-kernel split hands the tensor cores K-contiguous B tiles
    p.idesc = make_idesc(d.in_dtype, tf32, b_desc_mn, kBM * cta, bn);
    p.idesc_half = make_idesc(d.in_dtype, tf32, b_desc_mn, kBM * cta, bn / 2);
    const uint32_t box_k = (uint32_t)(kRowBytes / in_sz);

    // with K == 0 no load is ever issued; the maps only need an encodable base address
    const void* a_hi = d.K > 0 ? A : C;
    const void* a_lo = a_hi;
    const void* b_hi = d.K > 0 ? B : C;
    const void* b_lo = b_hi;
    long long lda = d.lda, ldb = d.ldb;
    BatchDims bda, bdb;
    bda.n_in = p.a_in ? (uint64_t)p.batch_in : 1; bda.s_in = (uint64_t)a_s_in;
    bda.n_out = p.a_out ? (uint64_t)n_out : 1;    bda.s_out = (uint64_t)a_s_out;
    bdb.n_in = p.b_in ? (uint64_t)p.batch_in : 1; bdb.s_in = (uint64_t)b_s_in;
    bdb.n_out = p.b_out ? (uint64_t)n_out : 1;    bdb.s_out = (uint64_t)b_s_out;
    if (sp.active && !in_kernel_split) {
        float* w = static_cast<float*>(workspace);
        float* wa_hi = w;
        float* wa_lo = sp.copies == 2 ? w + sp.a_elems : nullptr;
        float* wb_hi = w + sp.copies * sp.a_elems;
        float* wb_lo = sp.copies == 2 ? wb_hi + sp.b_elems : nullptr;
        const long long a_batches = p.a_in ? d.batch : 1, b_batches = p.b_in ? d.batch : 1;
        if (d.K > 0) {
            const long long row_blocks = (long long)sm_count() * 4;
            const SplitOperand ao = {static_cast<const float*>(A), wa_hi, wa_lo, d.M, d.K, d.lda, sp.ldk, a_batches,
                                     d.batch_stride_a, d.M * sp.ldk};
            SplitOperand bo;
            long long b_blocks, tiles_x = 0, tiles_y = 0;
            if (d.b_transposed) {   // [N, K]: same row-wise rewrite as A
                bo = {static_cast<const float*>(B), wb_hi, wb_lo, d.N, d.K, d.ldb, sp.ldk, b_batches, d.batch_stride_b,
                      d.N * sp.ldk};
                b_blocks = row_blocks;
            } else {                // [K, N]: transposed into [N, ldk]
                bo = {static_cast<const float*>(B), wb_hi, wb_lo, d.K, d.N, d.ldb, sp.ldk, b_batches, d.batch_stride_b,
                      d.N * sp.ldk};
                tiles_x = (d.N + 31) / 32;
                tiles_y = (sp.ldk + 31) / 32;
                b_blocks = tiles_x * tiles_y * b_batches;
            }
            if (row_blocks + b_blocks > 0x7fffffffLL || tiles_x > 0x7fffffffLL || tiles_y > 0x7fffffffLL)
                return CG_B200_ERR_UNSUPPORTED;
            tf32_split_operands_kernel<<<(unsigned)(row_blocks + b_blocks), 256, 0, s>>>(
                ao, bo, (int)row_blocks, d.b_transposed ? 0 : 1, (int)tiles_x, (int)tiles_y);
            CGB_CUDA(cudaGetLastError());
        }
        a_hi = wa_hi; a_lo = wa_lo ? wa_lo : wa_hi; b_hi = wb_hi; b_lo = wb_lo ? wb_lo : wb_hi;
        lda = sp.ldk; ldb = sp.ldk;
        bda.s_in = (uint64_t)(d.M * sp.ldk);   // the workspace copies are dense, one batch level
        bdb.s_in = (uint64_t)(d.N * sp.ldk);
    }
    // K == 0: no k-blocks, the maps are never dereferenced but must still encode
    const uint64_t k_dim = d.K > 0 ? (uint64_t)d.K : 1;

    alignas(64) CUtensorMap ta, ta_lo, tb, tb_lo;
    st = make_map(&ta, a_hi, d.in_dtype, k_dim, d.M, bda, lda, box_k, kBM);
    if (st) return st;
    st = make_map(&ta_lo, a_lo, d.in_dtype, k_dim, d.M, bda, lda, box_k, kBM);
    if (st) return st;
    if (p.b_mn_major && in_kernel_split) {
        // [K, N] fp32 read as it lies: one unswizzled box of 32 K-rows x (tile width) columns per stage
        st = make_map(&tb, b_hi, d.in_dtype, d.N, k_dim, bdb, ldb, (uint32_t)bn, box_k, /*swizzle=*/false);
        if (st) return st;
        st = make_map(&tb_lo, b_lo, d.in_dtype, d.N, k_dim, bdb, ldb, (uint32_t)bn, box_k, false);
    } else if (p.b_mn_major) {
        st = make_map(&tb, b_hi, d.in_dtype, d.N, k_dim, bdb, ldb, box_k, box_k);
        if (st) return st;
        st = make_map(&tb_lo, b_lo, d.in_dtype, d.N, k_dim, bdb, ldb, box_k, box_k);
    } else {
        st = make_map(&tb, b_hi, d.in_dtype, k_dim, d.N, bdb, ldb, box_k, (uint32_t)(bn / cta));
        if (st) return st;
        // pairs without the fp32 split: the second map stages the half-height box of a tail unit
        const uint32_t lo_rows = (cta == 2 && !sp.active) ? (uint32_t)(bn / cta / 2) : (uint32_t)(bn / cta);
        st = make_map(&tb_lo, b_lo, d.in_dtype, k_dim, d.N, bdb, ldb, box_k, lo_rows);
    }
    if (st) return st;

    if (tf32) {
        if (in_kernel_split) {
            if (bn == 64) return launch_variant<1, true, true, 64, float, true>(ta, ta_lo, tb, tb_lo, p, s);
            return launch_variant<1, true, true, 128, float, true>(ta, ta_lo, tb, tb_lo, p, s);
        }
        if (sp.copies == 2) return launch_bn<1, true, true, float>(bn, ta, ta_lo, tb, tb_lo, p, s);
        return launch_bn<1, true, false, float>(bn, ta, ta_lo, tb, tb_lo, p, s);
    }
    if (cta == 2) {
        switch (d.out_dtype) {
            case CG_B200_BF16: return launch_bn<2, false, false, __nv_bfloat16>(bn, ta, ta_lo, tb, tb_lo, p, s);
            case CG_B200_F16: return launch_bn<2, false, false, __half>(bn, ta, ta_lo, tb, tb_lo, p, s);
            default: return launch_bn<2, false, false, float>(bn, ta, ta_lo, tb, tb_lo, p, s);
        }
    }
    switch (d.out_dtype) {
        case CG_B200_BF16: return launch_bn<1, false, false, __nv_bfloat16>(bn, ta, ta_lo, tb, tb_lo, p, s);
        case CG_B200_F16: return launch_bn<1, false, false, __half>(bn, ta, ta_lo, tb, tb_lo, p, s);
        default: return launch_bn<1, false, false, float>(bn, ta, ta_lo, tb, tb_lo, p, s);
    }
}

extern "C" int cg_b200_gemm(const cg_b200_gemm_desc* desc, const void* A, const void* B, const void* bias,
                            const void* residual, void* C, void* workspace, size_t workspace_bytes, void* stream) {
    return gemm_run(desc, A, B, bias, residual, C, workspace, workspace_bytes, stream, true, nullptr);
}

extern "C" int cg_b200_gemm_tuned(const cg_b200_gemm_desc* desc, const cg_b200_gemm_tuning* tuning, const void* A,
                                  const void* B, const void* bias, const void* residual, void* C, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    return gemm_run(desc, A, B, bias, residual, C, workspace, workspace_bytes, stream, true, nullptr, nullptr, tuning);
}

// ---- fp32 GEMM for callers that cannot allocate -----------------------------------------------------
// The scratch of the fp32 path (the tf32 hi/lo copies of A and B) lives in this file-scope device
// array instead of a caller-provided workspace. Every device that loads the library holds these
// bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[CG_B200_GEMM_F32_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch per device. In host code the array's name is only a handle
// for the runtime, never a pointer a kernel could use; cudaGetSymbolAddress turns it into one, for
// the device that is current at the time of the call.
static void* g_static_scratch_addr[64];
static std::mutex g_static_scratch_mu;

static int static_scratch_for_current_device(void** out) {
    int dev = -1;
    CGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CG_B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lk(g_static_scratch_mu);
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        CGB_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return CG_B200_OK;
}

extern "C" int cg_b200_gemm_f32_static(const cg_b200_gemm_desc* desc, const void* A, const void* B,
                                       const void* bias, const void* residual, void* C,
                                       uint32_t* dev_error_word, void* stream) {
    int st = validate_desc(desc);
    if (st) return st;
    if (desc->in_dtype != CG_B200_F32) return CG_B200_ERR_UNSUPPORTED;   // only the fp32 path needs scratch
    const Fp32Plan plan = plan_fp32(desc);
    if (plan.bytes > (size_t)CG_B200_GEMM_F32_STATIC_SCRATCH_BYTES) return CG_B200_ERR_WORKSPACE;
    if (dev_error_word && !aligned_to(dev_error_word, 4)) return CG_B200_ERR_MISALIGNED;
    if (desc->M == 0 || desc->N == 0) return CG_B200_OK;
    st = require_sm100();
    if (st) return st;
    void* scratch = nullptr;
    st = static_scratch_for_current_device(&scratch);
    if (st) return st;
    // The split pre-pass rewrites every scratch byte the GEMM reads (pad columns included), so
    // nothing left over from an earlier call can leak into this one.
    return gemm_run(desc, A, B, bias, residual, C, scratch, (size_t)CG_B200_GEMM_F32_STATIC_SCRATCH_BYTES, stream,
                    false, dev_error_word, nullptr, nullptr, /*use_workspace_split=*/true);
}

// ---- GEMM fused with the all-gather of its M-sharded output ------------------------------------------
extern "C" int cg_b200_gemm_allgather(const cg_b200_gemm_desc* desc, const void* A, const void* B, const void* bias,
                                      const void* residual, void* C_full, void* const* peer_C, int world, int rank,
                                      void* workspace, size_t workspace_bytes, void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CG_B200_ERR_INVALID_ARG;
    if (!desc) return CG_B200_ERR_NULL_POINTER;
    if (desc->batch != 1) return CG_B200_ERR_UNSUPPORTED;   // the shards are row blocks of one matrix
    if (world > 1) {
        if (!peer_C) return CG_B200_ERR_NULL_POINTER;
        for (int r = 0; r < world; ++r)
            if (r != rank && (!peer_C[r] || !aligned_to(peer_C[r], 16))) return peer_C[r] ? CG_B200_ERR_MISALIGNED : CG_B200_ERR_NULL_POINTER;
    }
    PeerSet ps;
    ps.peer_c = peer_C;
    ps.world = world;
    ps.rank = rank;
    return gemm_run(desc, A, B, bias, residual, C_full, workspace, workspace_bytes, stream, true, nullptr, &ps);
}

extern "C" int cg_b200_gemm_allgather_sync(const cg_b200_gemm_desc* desc, const cg_b200_gemm_tuning* tuning, const void* A,
                                           const void* B, const void* bias, const void* residual, void* C_full,
                                           void* const* peer_C, int world, int rank, void* barrier, void* workspace,
                                           size_t workspace_bytes, void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CG_B200_ERR_INVALID_ARG;
    if (!desc) return CG_B200_ERR_NULL_POINTER;
    if (desc->batch != 1) return CG_B200_ERR_UNSUPPORTED;
    PeerBarrier* b = static_cast<PeerBarrier*>(barrier);
    if (b && (b->world != world || b->rank != rank)) return CG_B200_ERR_INVALID_ARG;
    if (world > 1) {
        if (!peer_C) return CG_B200_ERR_NULL_POINTER;
        for (int r = 0; r < world; ++r)
            if (r != rank && (!peer_C[r] || !aligned_to(peer_C[r], 16))) return peer_C[r] ? CG_B200_ERR_MISALIGNED : CG_B200_ERR_NULL_POINTER;
    }
    if (desc->M == 0 || desc->N == 0) {
        // nothing to compute, but the other ranks still wait for this one at the barrier
        return b ? cg_b200_peer_barrier(barrier, stream) : CG_B200_OK;
    }
    PeerSet ps;
    ps.peer_c = peer_C;
    ps.world = world;
    ps.rank = rank;
    if (b && world > 1) {
        ++b->epoch;
        ps.barrier = b;
    }
    const int st = gemm_run(desc, A, B, bias, residual, C_full, workspace, workspace_bytes, stream, true, nullptr, &ps, tuning);
    if (st != CG_B200_OK && b && world > 1) --b->epoch;   // nothing was launched
    return st;
}
