// plan.hpp - the launch plan: what a compiled Executable carries in machine_code on the B200 path.
//
// The reference's Executable holds x86 bytes or PTX text (include/cg/backend/backend.hpp:26-43); its
// KernelCache writes machine_code as opaque bytes (src/runtime/runtime.cpp:244-266). The plan rides in
// that field, so cache files keep the reference's format.
//
// One record per fused kernel = one C-ABI call. Buffers are numbered: [0, n_inputs) are the function's
// inputs (block arguments first, then OP_INPUT results, in program order), [n_inputs, n_inputs +
// n_outputs) its outputs in OP_OUTPUT order, the rest are intermediates the bound executable allocates
// from the device's Allocator. A record addresses a buffer by number plus an element offset (a column
// block of a packed projection is the same buffer at another offset).
#pragma once

#include <cstdint>
#include <optional>
#include <vector>

#include "cg_b200.h"

namespace cg::b200 {

struct PlanBuffer {
    std::uint64_t bytes = 0;
    std::int32_t dtype = CG_B200_F32;        // cg_b200_dtype
    std::vector<std::int64_t> shape;
};

struct PlanRecord {
    enum Kind : std::uint32_t { Eltwise = 1, Gemm = 2, Softmax = 3, LayerNorm = 4, SoftmaxLayerNorm = 5, Attention = 6, Reduce = 7 };
    std::uint32_t kind = 0;
    cg_b200_eltwise_desc eltwise{};      // Eltwise
    cg_b200_gemm_desc gemm{};            // Gemm
    cg_b200_gemm_tuning tuning{};        // Gemm: all zero = the library's heuristic
    cg_b200_attention_desc attention{};  // Attention
    std::int32_t row_dtype = 0;          // row reductions
    std::int64_t rows = 0, cols = 0;     // Reduce: outer and reduced extent of the [outer, reduce, inner] box (inner in n)
    std::int32_t reduce_op = 0;          // Reduce: cg_b200_reduce_op
    float eps = 1e-5f;
    std::uint64_t n = 0;                 // Eltwise: elements
    std::int32_t n_inputs = 0;
    // buffer numbers (-1 = unused). Gemm: A, B, bias, residual. Attention: Q, K, V.
    std::int32_t input[CG_B200_EW_MAX_INPUTS] = {-1, -1, -1, -1, -1, -1, -1, -1};
    std::int64_t input_offset[CG_B200_EW_MAX_INPUTS] = {0, 0, 0, 0, 0, 0, 0, 0};   // elements from the buffer's start
    std::int32_t output = -1;
    std::int64_t output_offset = 0;
};

struct LaunchPlan {
    static constexpr std::uint32_t kMagic = 0x32304243;   // "CB02"
    std::uint32_t n_inputs = 0, n_outputs = 0;
    std::vector<PlanBuffer> buffers;
    std::vector<PlanRecord> records;
    std::uint64_t workspace_bytes = 0;   // max over records (scratch of the fp32 GEMM)

    std::vector<std::uint8_t> serialize() const;
    // Empty when the bytes are not a launch plan of this version, or name a buffer out of range
    // (the bytes may come from a cache file).
    static std::optional<LaunchPlan> deserialize(const std::vector<std::uint8_t>& bytes);
};

}  // namespace cg::b200
