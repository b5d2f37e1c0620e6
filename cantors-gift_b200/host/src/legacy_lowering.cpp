// legacy_lowering.cpp - the reference's own Tensor-IR lowering, reachable under another name.
//
// The build compiles the reference's src/lowering/tensor_to_codegen.cpp, from where it lies, with the
// class renamed to LegacyTensorToCodegenLowering; this file sees the header under the same rename and
// forwards to it. The replacement lowering calls these to keep the generic instruction stream (vector
// loads, FMA per k-tile, barrier) that the reference's PTX emitter and its tests read, in front of the
// fused B200 kernel nodes.
#define TensorToCodegenLowering LegacyTensorToCodegenLowering
#include "cg/lowering/tensor_to_codegen.hpp"
#undef TensorToCodegenLowering

namespace cg::b200 {

void legacy_lower_function(const LoweringOptions& opts, const Function& f, CGFunction& out, const Schedule& schedule) {
    LegacyTensorToCodegenLowering legacy(opts);
    legacy.lower_function(f, out, schedule);
}

}  // namespace cg::b200
