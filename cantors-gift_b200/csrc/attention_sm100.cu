// attention_sm100.cu - softmax(Q K^T * scale) V per head in one kernel (tcgen05 + TMEM).
//
// The reference only annotates this pattern (pattern:"attention",
// src/optimization/graph/graph_pattern.cpp:61-85) and executes nothing; unfused it is three ops of
// the path - matmul, softmax, matmul (src/ir/ops.cpp) - whose [B, H, S, S] intermediate makes three
// trips through HBM. Here the scores never leave the SM.
//
// A work unit is (batch, head, 256 query rows = two query tiles); persistent CTAs of 384 threads, one per
// SM, take units blockIdx.x, blockIdx.x + gridDim.x, ... and carry the whole pipeline - K/V ring, score
// buffers, barrier phases - across units, so the loads and the first scores of the next unit are under
// way while the softmax groups finish the current one (no fill and drain per unit; the Q tiles are
// double-buffered for that). Both query tiles meet each
// K/V tile while it is in shared memory, which halves the K/V traffic from L2 - the first limit of a
// one-tile CTA at head_dim 64. Query tile g (0 or 1) owns a score buffer S_g (128 TMEM columns), a
// probability buffer P_g (64 columns: two 16-bit keys per column) and an output accumulator O_g (64):
//   warp 8     TMA: the two Q tiles of a unit, then K and V tiles of 128 key rows through a 5-stage ring
//   warps 9,10 one issuing warp per query tile. For key tile j of its tile g the warp issues
//              S_g = Q_g K_j^T (128 x 128 x 64) as soon as the softmax group has taken the previous scores
//              out of S_g, i.e. while the group is still computing on them, and O_g += P_g V_j
//              (128 x 64 x 128, P_g read from TMEM) when the group has written P_g. The two warps share
//              nothing but the in-order tensor pipe, so neither waits for the other query tile's softmax,
//              and each runs a short loop (two waits, twelve MMAs, three commits per key tile): with one
//              warp issuing for both tiles in item order, that warp's own instruction stream - waits,
//              fences, address arithmetic, about 2400 cycles per item - set the pace of the whole kernel.
//              The loop runs converged and one elected lane issues, which keeps descriptors and addresses
//              in uniform registers.
//   warps 0-3  softmax group 0: query tile 0;  warps 4-7  softmax group 1: query tile 1 (two whole
//              warpgroups, which take the registers the third one gives up: 216 per thread).
//              One thread per query row, so no exchange between threads: the row's 128 scores are read
//              from TMEM once into registers (S_g is free again from that moment), row max,
//              p = 2^(s - m), row sum, and P is written as bf16/f16 pairs into P_g once the previous
//              product has read it. m is a reference
//              maximum that follows the running maximum only when that has grown by more than 2^8, so
//              the output accumulator in tensor memory is rescaled (O *= 2^(m_old - m_new), by the row's
//              own thread) only on those rare occasions instead of on every key tile. The two warps that
//              share a scheduler belong to different groups, i.e. to different key tiles in different
//              phases: one runs its exponentials while the other loads, reduces or waits.
// Q, K, V are read in place from strided buffers (head = 64 contiguous columns of a row), so the
// packed [rows, 3*d_model] output of a QKV projection needs no reshuffle. head_dim is 64.
// The exponentials are the bound at this head size (one MUFU.EX2 per score).
// Every wait is bounded as in the GEMM kernel; on timeout an error word is set and the CTA leaves.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tc_sm100.cuh"

namespace cgb {

constexpr int kAttnBM = 128;          // query rows per tile = TMEM lanes
constexpr int kAttnQRows = 2 * kAttnBM;   // query rows per CTA
constexpr int kAttnBN = 128;          // key rows per step
constexpr int kAttnD = 64;            // head dim: 128 bytes of bf16 = one swizzle span
constexpr int kAttnKVStages = 5;
constexpr int kAttnThreads = 384;        // three warpgroups: softmax group 0, softmax group 1, {TMA, two MMA warps, one idle warp}
constexpr int kAttnTmaWarp = 8, kAttnMmaWarp = 9;   // MMA warps: 9 (query tile 0) and 10 (query tile 1)
// Registers per thread after the warpgroups re-divide the register file. The kernel is launched with
// 168 per thread (65536 / 384, rounded down to a multiple of 8); an increase waits in hardware, without
// a time limit, until that many registers are free, so the new shares must fit in what the launch
// allocated: 2 x 128 x 216 + 128 x 72 = 64512 = 384 x 168.
constexpr int kAttnLaunchRegs = 168, kAttnSoftmaxRegs = 216, kAttnIssueRegs = 72;
static_assert(2 * 128 * kAttnSoftmaxRegs + 128 * kAttnIssueRegs <= kAttnThreads * kAttnLaunchRegs,
              "the re-divided register shares exceed the launch allocation: setmaxnreg.inc would never return");
constexpr int kAttnTileBytes = 128 * 128;                 // a 128-row x 128-byte tile (Q, K or V)
constexpr int kAttnSmem = 2 * 2 * kAttnTileBytes + kAttnKVStages * 2 * kAttnTileBytes + 1024;
constexpr uint32_t kAttnTmemCols = 512;
constexpr uint32_t kAttnSCol = 0;     // two score buffers (one per query tile) of 128 columns
constexpr uint32_t kAttnPCol = 256;   // two probability buffers of 64 columns (two 16-bit keys per column)
constexpr uint32_t kAttnTCol = 384;   // two output accumulators of 64 columns

struct AttnParams {
    long long S_q, S_kv;
    int H;
    long long B;
    long long ldo, o_stride_h, o_stride_b;
    void* O;
    float scale_log2e;
    int q_tiles, kv_tiles;
    long long units;   // B * H * q_tiles
    uint32_t idesc_s, idesc_t;
    uint32_t* err_word;
};

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {   // two values rounded to T in one word, a in the low half
    if constexpr (Elem<T>::dtype == CG_B200_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {   // one instruction on sm_100
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q_full[2], bar_q_empty[2];
    __shared__ __align__(8) uint64_t bar_kv_full[kAttnKVStages], bar_kv_empty[kAttnKVStages];
    __shared__ __align__(8) uint64_t bar_s_full[2], bar_s_free[2], bar_p_full[2], bar_t_full[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t s_q = smem_base;
    const uint32_t s_kv = s_q + 2 * 2 * kAttnTileBytes;   // after two Q buffers; stage s: K at +s*2T, V at +s*2T + T
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // unit -> (batch, head, query rows): query tile fastest, so that the CTAs running at one time work on
    // few heads and share their K, V in L2
    struct Unit { int q0, h, b; };
    auto decode = [&](long long unit) {   // unit < 2^31 (checked on the host): 32-bit divisions
        Unit u;
        const uint32_t un = (uint32_t)unit, qt = (uint32_t)p.q_tiles, hh = (uint32_t)p.H;
        const uint32_t rest = un / qt;
        u.q0 = (int)(un - rest * qt) * kAttnQRows;
        u.b = (int)(rest / hh);
        u.h = (int)(rest - (uint32_t)u.b * hh);
        return u;
    };
    const int n_tiles = p.kv_tiles;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bar_q_full[i]), 1);
            mbar_init(smem_u32(&bar_q_empty[i]), 2);   // one commit per MMA warp: both query tiles are through with Q
        }
        for (int s = 0; s < kAttnKVStages; ++s) {
            mbar_init(smem_u32(&bar_kv_full[s]), 1);
            mbar_init(smem_u32(&bar_kv_empty[s]), 2);  // one commit per MMA warp
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bar_s_full[i]), 1);
            mbar_init(smem_u32(&bar_s_free[i]), 4);    // one arrival per warp of the group
            mbar_init(smem_u32(&bar_p_full[i]), 4);
            mbar_init(smem_u32(&bar_t_full[i]), 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kAttnMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kAttnTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // Registers follow the work: the softmax warpgroups hold a row of 128 scores per thread, the third
    // warpgroup only issues copies and MMAs. Each role re-sizes its warpgroup's share of the register file
    // as it enters its branch (see kAttnSoftmaxRegs / kAttnIssueRegs).
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kAttnIssueRegs));   // one instruction for the whole third warpgroup
    if (warp == kAttnTmaWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t k = 0;          // units this CTA has started
            int st = 0;              // K/V ring position and the parity of its current round
            uint32_t st_phase = 0;
            bool ok = true;
            for (long long unit = blockIdx.x; ok && unit < p.units; unit += gridDim.x, ++k) {
                const Unit u = decode(unit);
                const int qb = (int)(k & 1u);
                if (!mbar_wait(smem_u32(&bar_q_empty[qb]), ((k >> 1) & 1u) ^ 1u, &abort_flag, p.err_word, 0x608u + qb)) break;
                const uint32_t qfull = smem_u32(&bar_q_full[qb]);
                mbar_expect_tx(qfull, 2 * kAttnTileBytes);   // rows past S_q arrive as zeros
                tma_load_4d<1>(s_q + qb * 2 * kAttnTileBytes, &tm_q, qfull, 0, u.q0, u.h, u.b);
                tma_load_4d<1>(s_q + qb * 2 * kAttnTileBytes + kAttnTileBytes, &tm_q, qfull, 0, u.q0 + kAttnBM, u.h, u.b);
                for (int j = 0; j < n_tiles; ++j) {
                    if (!mbar_wait(smem_u32(&bar_kv_empty[st]), st_phase ^ 1u, &abort_flag, p.err_word, 0x600u + st)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bar_kv_full[st]);
                    mbar_expect_tx(full, 2 * kAttnTileBytes);
                    tma_load_4d<1>(s_kv + st * 2 * kAttnTileBytes, &tm_k, full, 0, j * kAttnBN, u.h, u.b);
                    tma_load_4d<1>(s_kv + st * 2 * kAttnTileBytes + kAttnTileBytes, &tm_v, full, 0, j * kAttnBN, u.h, u.b);
                    if (++st == kAttnKVStages) {
                        st = 0;
                        st_phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == kAttnMmaWarp || warp == kAttnMmaWarp + 1) {
        // ---------------- MMA issuer of query tile g ----------------
        // The whole warp runs the loop and waits; one elected lane issues (see elect_one()). Key tiles are
        // numbered through all units of this CTA: n = k * n_tiles + j. In program order:
        //   S(0); for every n: [ S(n+1) once the group has read S(n) ]; T(n) once the group has written P(n).
        const int g = warp - kAttnMmaWarp;
        const uint32_t my_units = (uint32_t)p.units > blockIdx.x ? ((uint32_t)p.units - 1u - blockIdx.x) / gridDim.x + 1u : 0u;
        const uint32_t total = my_units * (uint32_t)n_tiles;   // < 2^31: units is, and a CTA's share times the key tiles of one head stays far below
        const uint32_t tmem_s = tmem_base + kAttnSCol + (uint32_t)(g * kAttnBN);
        const uint32_t tmem_p = tmem_base + kAttnPCol + (uint32_t)(g * kAttnD);
        const uint32_t tmem_t = tmem_base + kAttnTCol + (uint32_t)(g * kAttnD);
        // position of the next S: key tile within its unit, unit count, K/V ring stage and its parity
        int sj = 0, s_st = 0;
        uint32_t sk = 0, s_st_phase = 0;
        // position of the next T
        int tj = 0, t_st = 0;
        bool ok = true;
        auto issue_s = [&]() -> bool {   // S of the key tile at the "s" position; advances it
            bool w = true;
            if (sj == 0) w = mbar_wait_poll(smem_u32(&bar_q_full[sk & 1u]), (sk >> 1) & 1u, &abort_flag, p.err_word, 0x610u + g);
            if (w) w = mbar_wait_poll(smem_u32(&bar_kv_full[s_st]), s_st_phase, &abort_flag, p.err_word, 0x640u + s_st);
            if (!__all_sync(0xffffffffu, w)) return false;
            tc_fence_after();
            const uint32_t qa = s_q + (sk & 1u) * 2 * kAttnTileBytes + g * kAttnTileBytes;
            const uint32_t kb = s_kv + s_st * 2 * kAttnTileBytes;
            const bool last = sj == n_tiles - 1;
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // 16 of the 64 head dims per MMA
                    const uint64_t da = make_smem_desc(qa + k * 32, 16, 1024);
                    const uint64_t db = make_smem_desc(kb + k * 32, 16, 1024);
                    umma<false, 1>(tmem_s, da, db, p.idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit<1>(smem_u32(&bar_s_full[g]));
                if (last) tc_commit<1>(smem_u32(&bar_q_empty[sk & 1u]));   // this query tile's last read of the Q buffer
            }
            __syncwarp();
            if (++s_st == kAttnKVStages) { s_st = 0; s_st_phase ^= 1u; }
            if (last) { sj = 0; ++sk; } else ++sj;
            return true;
        };
        if (total > 0) ok = issue_s();
        for (uint32_t n = 0; ok && n < total; ++n) {
            if (n + 1 < total) {
                // the group has the scores of tile n in registers: S_g may be overwritten
                bool w = mbar_wait_poll(smem_u32(&bar_s_free[g]), n & 1u, &abort_flag, p.err_word, 0x630u + g);
                if (!__all_sync(0xffffffffu, w)) break;
                if (!issue_s()) break;
            }
            // P(n) is written (and, for a unit's first tile, the group has taken the previous unit's output out
            // of its accumulator)
            bool ready = mbar_wait_poll(smem_u32(&bar_p_full[g]), n & 1u, &abort_flag, p.err_word, 0x620u + g);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            // O_g += P V_j: A = P in tensor memory, B = V_j ([key, d] with d contiguous: MN-major)
            const uint32_t vb = s_kv + t_st * 2 * kAttnTileBytes + kAttnTileBytes;
            const uint32_t first = tj == 0 ? 0u : 1u;   // the unit's first product starts O
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {   // 16 keys per MMA: 8 columns of P
                    const uint64_t db = make_smem_desc(vb + k * 2048, kAttnTileBytes, 1024);
                    umma_ts(tmem_t, tmem_p + k * 8, db, p.idesc_t, (k > 0) ? 1u : first);
                }
                tc_commit<1>(smem_u32(&bar_t_full[g]));
                tc_commit<1>(smem_u32(&bar_kv_empty[t_st]));   // this query tile is through with the stage
            }
            __syncwarp();
            if (++t_st == kAttnKVStages) t_st = 0;
            if (++tj == n_tiles) tj = 0;
        }
    }   // (warp 11 has no role)
    } else {
        // ---------------- softmax; the output accumulates in tensor memory ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kAttnSoftmaxRegs));
        // One thread per query row. The whole row of 128 scores is held in registers (one pass over
        // tensor memory), p = 2^(s * scale * log2e - m) with m the row's REFERENCE maximum: it follows the
        // true running maximum only when that has grown by more than 2^8 since m was last set, so P stays
        // below 256 (exact in bf16 / f16 range, the row sum is fp32) and the output accumulator O - which
        // the tensor cores add every P V product into, in tensor memory - has to be rescaled only on those
        // rare occasions. A rescale is decided per warp (the tensor-memory loads and stores are warp-wide):
        // O_row *= 2^(m_old - m_new), l *= the same, after the group's previous P V has completed.
        constexpr int kKeys = kAttnBN, kCols = kAttnD;
        constexpr float kGrowth = 8.0f;       // log2 of the largest P that is tolerated before m moves
        const int q = warp & 3;               // TMEM lane quarter this warp may access
        const int g = warp >> 2;              // group = query tile = warpgroup
        const int row = q * 32 + lane;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_base + kAttnTCol + (uint32_t)(g * kAttnD);
        float m, l;
        bool ok = true;
        const uint32_t s_addr = tmem_base + lane_base + kAttnSCol + (uint32_t)(g * kAttnBN);
        const uint32_t p_addr = tmem_base + lane_base + kAttnPCol + (uint32_t)(g * kAttnD);
        uint32_t tcount = 0;      // key tiles this group has finished, over all units
        auto wait_pv = [&](uint32_t use) -> bool {   // the group's P V product number `use` has completed
            bool w = mbar_wait_poll(smem_u32(&bar_t_full[g]), use & 1u, &abort_flag, p.err_word, 0x660u + g);
            w = __all_sync(0xffffffffu, w);
            if (w) tc_fence_after();
            return w;
        };
        for (long long unit = blockIdx.x; ok && unit < p.units; unit += gridDim.x) {
            const Unit u = decode(unit);
            m = -INFINITY;
            l = 0.0f;
            for (int j = 0; ok && j < n_tiles; ++j) {
                bool ready = mbar_wait_poll(smem_u32(&bar_s_full[g]), tcount & 1u, &abort_flag, p.err_word, 0x670u + g);
                ready = __all_sync(0xffffffffu, ready);
                if (!ready) { ok = false; break; }
                tc_fence_after();
                const long long kv0 = (long long)j * kAttnBN;
                const bool ragged = kv0 + kKeys > p.S_kv;   // keys past S_kv are zero-filled rows of K
                float s[kKeys / 32][32];
#pragma unroll
                for (int c = 0; c < kKeys / 32; ++c) tmem_ld32_issue(s_addr + c * 32, s[c]);
                tmem_ld_wait();
                // the scores are in registers: the next key tile's scores may be written over them
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_s_free[g]));
                if (ragged) {   // only the last key tile: mask the zero-filled keys
#pragma unroll
                    for (int c = 0; c < kKeys / 32; ++c) {
                        const int valid = (int)(p.S_kv - kv0) - c * 32;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i >= valid) s[c][i] = -INFINITY;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;   // four chains
#pragma unroll
                for (int c = 0; c < kKeys / 32; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        mx0 = fmax3(mx0, s[c][i], s[c][i + 1]);
                        mx1 = fmax3(mx1, s[c][i + 2], s[c][i + 3]);
                        mx2 = fmax3(mx2, s[c][i + 4], s[c][i + 5]);
                        mx3 = fmax3(mx3, s[c][i + 6], s[c][i + 7]);
                    }
                }
                // finite: a tile holds at least one key
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2e;
                bool pv_seen = j == 0;   // the group's previous P V is known to be complete (a unit's first item: waited at the end of the last unit)
                if (j == 0) {
                    m = mx;   // nothing accumulated yet: the first P V of the unit overwrites O
                } else if (__any_sync(0xffffffffu, mx > m + kGrowth)) {
                    // some row of this warp outgrew its reference maximum: bring O and l of the whole warp to the
                    // rows' current maxima (factor 1 for rows that did not grow)
                    ok = wait_pv(tcount - 1u);
                    if (!ok) break;
                    pv_seen = true;
                    const float m_new = fmaxf(m, mx);
                    const float alpha = ex2_approx(m - m_new);
                    const float2 a2 = make_float2(alpha, alpha);
                    // 32 columns at a time: the row of scores stays in registers meanwhile
#pragma unroll 1
                    for (int c = 0; c < kCols / 32; ++c) {
                        float o[32];
                        tmem_ld32(o_addr + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float2 r = __fmul2_rn(make_float2(o[i], o[i + 1]), a2);
                            o[i] = r.x;
                            o[i + 1] = r.y;
                        }
                        tmem_st32(o_addr + c * 32, reinterpret_cast<const uint32_t(&)[32]>(o));
                    }
                    l *= alpha;
                    m = m_new;
                }
                // P_g is rewritten below: the group's previous product, which reads it, must have run. (It was
                // issued when all four warps had announced the previous P, a key tile's worth of work ago, so by
                // now it has normally long finished. The same wait keeps a fast warp from announcing its part of
                // this tile's P while a slower warp has not yet announced the previous one.)
                if (!pv_seen) {
                    ok = wait_pv(tcount - 1u);
                    if (!ok) break;
                }
                // p = 2^(s * scale * log2e - m), two keys per instruction where the ISA allows it (fp32x2 fma /
                // add, packed convert), two keys per column of P_g.
                float2 l2 = make_float2(0.0f, 0.0f);
                const float2 sc2 = make_float2(p.scale_log2e, p.scale_log2e), nm2 = make_float2(-m, -m);
#pragma unroll
                for (int c = 0; c < kKeys / 32; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 t = __ffma2_rn(make_float2(s[c][i], s[c][i + 1]), sc2, nm2);
                        const float2 ex = make_float2(ex2_approx(t.x), ex2_approx(t.y));   // 2^-inf = 0 for masked keys
                        l2 = __fadd2_rn(l2, ex);
                        pk[i >> 1] = pack_pair<T>(ex.x, ex.y);
                    }
                    tmem_st16(p_addr + c * 16, pk);   // keys 32c .. 32c+31 of this row
                }
                // P (and a rescaled O) are complete in tensor memory
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_p_full[g]));
                l += l2.x + l2.y;
                ++tcount;
            }
            // the unit's output: O / l, once the last P V has landed
            if (ok && n_tiles > 0) ok = wait_pv(tcount - 1u);
            if (!ok) break;
            float o[kCols / 32][32];
#pragma unroll
            for (int c = 0; c < kCols / 32; ++c) tmem_ld32_issue(o_addr + c * 32, o[c]);
            tmem_ld_wait();
            tc_fence_before();   // the loads are done before the group's next P arrival lets O be overwritten
            const long long qrow = (long long)u.q0 + g * kAttnBM + row;
            if (qrow < p.S_q) {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                T* orow = static_cast<T*>(p.O) + (long long)u.b * p.o_stride_b + (long long)u.h * p.o_stride_h + qrow * p.ldo;
#pragma unroll
                for (int gi = 0; gi < kCols / 8; ++gi) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) e[i] = o[gi >> 2][(gi & 3) * 8 + i] * inv;
                    const Vec16<T> o8 = pack16<T>(e);
                    *reinterpret_cast<int4*>(orow + gi * 8) = *reinterpret_cast<const int4*>(&o8);
                }
            }
        }   // units
    }

    if (abort_flag) {
        // a wait ran out: give copies that may still be in flight time to land before the CTA's shared
        // memory is released
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kAttnMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAttnTmemCols) : "memory");
    }
}

static int make_head_map(CUtensorMap* map, const void* base, int dtype, long long rows, int H, long long B, long long ld,
                         long long stride_h, long long stride_b) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) return CG_B200_ERR_CUDA;
    const cuuint64_t esz = 2;
    cuuint64_t dims[4] = {(cuuint64_t)kAttnD, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t fallback = (cuuint64_t)rows * ld * esz;
    cuuint64_t strides[3] = {(cuuint64_t)ld * esz, H > 1 ? (cuuint64_t)stride_h * esz : fallback,
                             B > 1 ? (cuuint64_t)stride_b * esz : fallback};
    cuuint32_t box[4] = {(cuuint32_t)kAttnD, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, dtype == CG_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        note_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (attention)");
        return CG_B200_ERR_CUDA;
    }
    return CG_B200_OK;
}

static uint32_t attn_idesc(int dtype, bool b_mn_major, int n) {
    uint32_t d = 0;
    d |= 1u << 4;                                            // fp32 accumulator
    const uint32_t fmt = dtype == CG_B200_BF16 ? 1u : 0u;
    d |= fmt << 7;
    d |= fmt << 10;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(kAttnBM >> 4) << 24;
    return d;
}

}  // namespace cgb

using namespace cgb;

extern "C" int cg_b200_attention(const cg_b200_attention_desc* desc, const void* Q, const void* K, const void* V,
                                 void* O, void* stream) {
    if (!desc) return CG_B200_ERR_NULL_POINTER;
    const cg_b200_attention_desc& d = *desc;
    if (d.dtype != CG_B200_BF16 && d.dtype != CG_B200_F16) return CG_B200_ERR_UNSUPPORTED;
    if (d.head_dim != kAttnD) return CG_B200_ERR_UNSUPPORTED;
    if (d.batch < 0 || d.heads < 1 || d.seq_q < 0 || d.seq_kv < 0) return CG_B200_ERR_INVALID_ARG;
    if (d.batch > 0x7fffffffLL || d.heads > 65535 || d.seq_q > 0x7fffffffLL || d.seq_kv > 0x7fffffffLL) return CG_B200_ERR_UNSUPPORTED;
    if (d.ldq < kAttnD || d.ldk < kAttnD || d.ldv < kAttnD || d.ldo < kAttnD) return CG_B200_ERR_INVALID_ARG;
    if (d.batch == 0 || d.seq_q == 0) return CG_B200_OK;
    if (d.seq_kv == 0 || !(d.scale > 0.0f)) return CG_B200_ERR_INVALID_ARG;   // softmax over an empty set; the row max assumes scale > 0
    if (!Q || !K || !V || !O) return CG_B200_ERR_NULL_POINTER;
    const long long strides[] = {d.ldq, d.ldk, d.ldv, d.ldo, d.head_stride_q, d.head_stride_k, d.head_stride_v, d.head_stride_o,
                                 d.batch_stride_q, d.batch_stride_k, d.batch_stride_v, d.batch_stride_o};
    for (long long s : strides)
        if (s < 0 || (s * 2) % 16) return s < 0 ? CG_B200_ERR_INVALID_ARG : CG_B200_ERR_MISALIGNED;
    if (!aligned_to(Q, 16) || !aligned_to(K, 16) || !aligned_to(V, 16) || !aligned_to(O, 16)) return CG_B200_ERR_MISALIGNED;
    int st = require_sm100();
    if (st) return st;

    alignas(64) CUtensorMap tq, tk, tv;
    st = make_head_map(&tq, Q, d.dtype, d.seq_q, (int)d.heads, d.batch, d.ldq, d.head_stride_q, d.batch_stride_q);
    if (st) return st;
    st = make_head_map(&tk, K, d.dtype, d.seq_kv, (int)d.heads, d.batch, d.ldk, d.head_stride_k, d.batch_stride_k);
    if (st) return st;
    st = make_head_map(&tv, V, d.dtype, d.seq_kv, (int)d.heads, d.batch, d.ldv, d.head_stride_v, d.batch_stride_v);
    if (st) return st;

    AttnParams p;
    memset(&p, 0, sizeof(p));
    p.S_q = d.seq_q; p.S_kv = d.seq_kv; p.H = (int)d.heads; p.B = d.batch;
    p.ldo = d.ldo; p.o_stride_h = d.head_stride_o; p.o_stride_b = d.batch_stride_o;
    p.O = O;
    p.scale_log2e = d.scale * 1.4426950408889634f;
    p.q_tiles = (int)((d.seq_q + kAttnQRows - 1) / kAttnQRows);
    p.kv_tiles = (int)((d.seq_kv + kAttnBN - 1) / kAttnBN);
    p.idesc_s = attn_idesc(d.dtype, false, kAttnBN);
    p.idesc_t = attn_idesc(d.dtype, true, kAttnD);
    p.err_word = device_error_word();
    p.units = (long long)p.q_tiles * p.H * p.B;
    if (p.units > 0x7fffffffLL) return CG_B200_ERR_UNSUPPORTED;   // the kernel decodes a unit with 32-bit arithmetic
    const long long grid = p.units < sm_count() ? p.units : sm_count();   // one persistent CTA per SM
    cudaStream_t s = (cudaStream_t)stream;
    if (d.dtype == CG_B200_BF16) {
        auto kern = attention_sm100_kernel<__nv_bfloat16>;
        CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
        kern<<<(unsigned)grid, kAttnThreads, kAttnSmem, s>>>(tq, tk, tv, p);
    } else {
        auto kern = attention_sm100_kernel<__half>;
        CGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
        kern<<<(unsigned)grid, kAttnThreads, kAttnSmem, s>>>(tq, tk, tv, p);
    }
    CGB_CUDA(cudaGetLastError());
    return CG_B200_OK;
}
