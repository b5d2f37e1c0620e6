// nvidia_backend.cpp - cg::NvidiaBackend::{compile, emit_text} for the B200 path.
//
// Takes the place of the reference's src/backend/nvidia_backend.cpp:7-27, which concatenates PTX text
// per function and pushes {name, 0} entry points. Both of those stay: ptx_text still comes from the
// reference's own PTXEmitter (lower_to_ptx) over the generic instructions, so everything that reads
// that text keeps working, and emit_text returns it. What is new: the fused kernel nodes the lowering
// put into the CGModule ("b200.record" attributes) are decoded into a launch plan that is stored in
// Executable::machine_code, with the launch geometry of the heaviest kernel in threads_per_block /
// shared_mem_bytes. A module without such nodes compiles exactly as before (empty machine_code).
#include "cg/backend/nvidia_backend.hpp"

#include <cstring>

#include "cg/b200/b200.hpp"
#include "cg/b200/plan.hpp"
#include "cg/backend/lowering.hpp"

namespace cg {
namespace {

// PTX for the generic part of a function, from the reference's own emitter. Two kinds of instruction are
// kept away from it: the plan-carrying nodes, which are not of its vocabulary, and the result-less Const
// placeholders the generic lowering leaves for ops it does not know (softmax, layernorm, slice, alloc
// notes; src/lowering/tensor_to_codegen.cpp:271-292, :350-356) - the emitter reads results[0] of every
// Const (src/backend/ptx/ptx_emitter.cpp:218-219) and would run off the end of an empty list. Their
// comments are listed after the kernel text instead.
std::string generic_ptx(const CGFunction& fn, const std::string& sm_target) {
    CGFunction generic = fn;
    generic.instructions.clear();
    std::string notes, kernels;
    for (const CGInstruction& inst : fn.instructions) {
        if (auto k = inst.attributes.get("b200.kernel")) {
            kernels += "//   cg_b200_" + k->str + "  " + inst.comment + "\n";
        } else if (inst.opcode == CGOpcode::Const && inst.results.empty()) {
            if (!inst.comment.empty()) notes += "// " + inst.comment + "\n";
        } else {
            generic.instructions.push_back(inst);
        }
    }
    std::string text = lower_to_ptx(generic, fn.name, sm_target);
    text += notes;
    if (!kernels.empty())
        text += "// B200 launch plan of " + fn.name + " (precompiled sm_100a kernels, one C-ABI call each):\n" + kernels;
    return text;
}

bool decode_record(const CGInstruction& inst, b200::PlanRecord& r) {
    auto rec = inst.attributes.get("b200.record");
    if (!rec || rec->kind != AttrKind::String || rec->str.size() != sizeof(b200::PlanRecord)) return false;
    std::memcpy(&r, rec->str.data(), sizeof(r));
    return true;
}

}  // namespace

std::unique_ptr<Executable> NvidiaBackend::compile(const CGModule& module) {
    auto exe = std::make_unique<Executable>();
    exe->target_device = DeviceId::cuda();
    if (sm_target_.rfind("sm_100", 0) == 0) target_info_.hardware = b200::hardware_model();

    b200::LaunchPlan plan;
    bool have_plan = false;
    for (const CGFunction& fn : module.functions) {
        exe->ptx_text += generic_ptx(fn, sm_target_) + "\n";
        exe->entrypoints.push_back({fn.name, 0});
        if (have_plan) continue;   // one plan per Executable: the first function that carries nodes
        for (const CGInstruction& inst : fn.instructions) {
            b200::PlanRecord r;
            if (!decode_record(inst, r)) continue;
            if (!have_plan) {
                // the first node also carries the buffer table
                auto bytes = inst.attributes.get("b200.buffer_bytes");
                auto dtypes = inst.attributes.get("b200.buffer_dtypes");
                auto n_in = inst.attributes.get("b200.n_inputs");
                auto n_out = inst.attributes.get("b200.n_outputs");
                if (!bytes || !dtypes || !n_in || !n_out || bytes->ints.size() != dtypes->ints.size()) break;
                for (usize i = 0; i < bytes->ints.size(); ++i) {
                    b200::PlanBuffer b;
                    b.bytes = static_cast<u64>(bytes->ints[i]);
                    b.dtype = static_cast<std::int32_t>(dtypes->ints[i]);
                    if (auto shape = inst.attributes.get("b200.buffer_shape." + std::to_string(i))) b.shape = shape->ints;
                    plan.buffers.push_back(std::move(b));
                }
                plan.n_inputs = static_cast<u32>(n_in->integer);
                plan.n_outputs = static_cast<u32>(n_out->integer);
                if (auto ws = inst.attributes.get("b200.workspace_bytes")) plan.workspace_bytes = static_cast<u64>(ws->integer);
                exe->name = fn.name;
                have_plan = true;
            }
            plan.records.push_back(r);
            // launch geometry of the kernels: GEMM and attention run 320 threads per CTA with the whole
            // shared memory, elementwise 256, row reductions 128
            if (r.kind == b200::PlanRecord::Gemm || r.kind == b200::PlanRecord::Attention) {
                exe->threads_per_block = 320;
                exe->shared_mem_bytes = 225 * 1024;
            } else if (exe->threads_per_block == 0) {
                exe->threads_per_block = r.kind == b200::PlanRecord::Eltwise ? 256 : 128;
            }
        }
    }
    if (have_plan) exe->machine_code = plan.serialize();
    return exe;
}

std::optional<std::string> NvidiaBackend::emit_text(const CGModule& module) {
    std::string out;
    for (const CGFunction& fn : module.functions) out += generic_ptx(fn, sm_target_) + "\n";
    return out;
}

}  // namespace cg
