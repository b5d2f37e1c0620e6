// backend.cpp - LaunchPlan (de)serialisation and the NvidiaBackend that fills an Executable.
//
// The reference's NvidiaBackend::compile concatenates PTX text and pushes {name, 0} entrypoints
// (src/backend/nvidia_backend.cpp:7-18). Here compile() decodes the fused nodes the planner put
// into the CGModule and stores the launch plan in Executable::machine_code: opaque bytes, so the
// reference's KernelCache file format (src/runtime/runtime.cpp:162-173) carries it unchanged.
// ptx_text stays a listing for people and for structural checks (.version / .target / .entry).
#include <cstring>
#include <sstream>

#include "cg/b200_host.hpp"

namespace cg {
namespace {

template <typename T>
void put(std::vector<u8>& out, const T& v) {
    const u8* p = reinterpret_cast<const u8*>(&v);
    out.insert(out.end(), p, p + sizeof(T));
}
template <typename T>
bool get(const std::vector<u8>& in, usize& off, T& v) {
    if (off + sizeof(T) > in.size()) return false;
    std::memcpy(&v, in.data() + off, sizeof(T));
    off += sizeof(T);
    return true;
}
constexpr u32 kPlanVersion = 1;

}  // namespace

std::vector<u8> LaunchPlan::serialize() const {
    std::vector<u8> out;
    put(out, kMagic);
    put(out, kPlanVersion);
    put(out, static_cast<u32>(sizeof(PlanRecord)));
    put(out, n_inputs);
    put(out, n_outputs);
    put(out, workspace_bytes);
    put(out, static_cast<u32>(buffers.size()));
    for (const PlanBuffer& b : buffers) {
        put(out, b.bytes);
        put(out, static_cast<u32>(b.dtype));
        put(out, static_cast<u32>(b.shape.size()));
        for (i64 d : b.shape) put(out, d);
    }
    put(out, static_cast<u32>(records.size()));
    for (const PlanRecord& r : records) put(out, r);
    return out;
}

std::optional<LaunchPlan> LaunchPlan::deserialize(const std::vector<u8>& in) {
    LaunchPlan p;
    usize off = 0;
    u32 magic = 0, version = 0, rec_size = 0, nb = 0, nr = 0;
    if (!get(in, off, magic) || magic != kMagic) return std::nullopt;
    if (!get(in, off, version) || version != kPlanVersion) return std::nullopt;
    if (!get(in, off, rec_size) || rec_size != sizeof(PlanRecord)) return std::nullopt;
    if (!get(in, off, p.n_inputs) || !get(in, off, p.n_outputs) || !get(in, off, p.workspace_bytes)) return std::nullopt;
    if (!get(in, off, nb) || nb > (1u << 20)) return std::nullopt;
    for (u32 i = 0; i < nb; ++i) {
        PlanBuffer b;
        u32 dt = 0, rank = 0;
        if (!get(in, off, b.bytes) || !get(in, off, dt) || !get(in, off, rank) || rank > 16) return std::nullopt;
        b.dtype = static_cast<DType>(dt);
        for (u32 k = 0; k < rank; ++k) {
            i64 d = 0;
            if (!get(in, off, d)) return std::nullopt;
            b.shape.push_back(d);
        }
        p.buffers.push_back(std::move(b));
    }
    if (!get(in, off, nr) || nr > (1u << 20)) return std::nullopt;
    for (u32 i = 0; i < nr; ++i) {
        PlanRecord r;
        if (!get(in, off, r)) return std::nullopt;
        // every buffer index must be in range: the bytes may come from a cache file
        auto ok = [&](i32 b) { return b >= -1 && b < static_cast<i32>(nb); };
        for (i32 b : r.input)
            if (!ok(b)) return std::nullopt;
        if (r.output < 0 || !ok(r.output)) return std::nullopt;
        if (r.kind < PlanRecord::Eltwise || r.kind > PlanRecord::SoftmaxLayerNorm) return std::nullopt;
        p.records.push_back(r);
    }
    if (off != in.size() || p.n_inputs + p.n_outputs > nb) return std::nullopt;
    return p;
}

double HardwareModel::peak_flops(DType dt) const {
    auto it = tensor_core_flops_per_sec.find(static_cast<u8>(dt));
    if (it != tensor_core_flops_per_sec.end()) return it->second;
    auto jt = flops_per_sec.find(static_cast<u8>(dt));
    return jt != flops_per_sec.end() ? jt->second : 0.0;
}

HardwareModel HardwareModel::b200() {
    HardwareModel h;
    h.name = "nvidia_b200";
    h.num_sms = 148;
    h.shared_mem_per_block = 227 * 1024;
    h.l2_bytes = 126ull << 20;
    h.hbm_bytes = 180ull << 30;
    h.tmem_bytes_per_sm = 256 * 1024;
    h.memory_bandwidth = 7.7e12;
    h.flops_per_sec[static_cast<u8>(DType::F32)] = 75e12;
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::BF16)] = 2.25e15;   // dense
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::F16)] = 2.25e15;
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::F32)] = 1.1e15 / 3;  // tf32, three passes
    return h;
}

NvidiaBackend::NvidiaBackend(std::string sm_target) : sm_target_(std::move(sm_target)) {
    target_info_.name = "nvidia_" + sm_target_;
    target_info_.device = DeviceId::cuda();
    target_info_.hardware = HardwareModel::b200();
    cg_b200_props props;
    int count = 0;
    if (cg_b200_device_count(&count) == CG_B200_OK && count > 0 && cg_b200_device_props(0, &props) == CG_B200_OK) {
        target_info_.hardware.num_sms = static_cast<u32>(props.sm_count);
        target_info_.hardware.shared_mem_per_block = static_cast<u64>(props.max_smem_per_block);
        target_info_.hardware.l2_bytes = static_cast<u64>(props.l2_bytes);
        target_info_.hardware.hbm_bytes = props.hbm_bytes;
        target_info_.hardware.tmem_bytes_per_sm = props.tmem_bytes_per_sm;
    }
    target_info_.supported_vector_dtypes = {DType::F32, DType::BF16, DType::F16};
    target_info_.max_vector_width_bytes = 16;
    target_info_.tensor_core_tiles = {{256, 256, 16}, {128, 256, 16}, {128, 128, 8}};
}

static const std::string* blob_of(const CGInstruction& inst, const char* key) {
    auto it = inst.attributes.find(key);
    if (it == inst.attributes.end()) return nullptr;
    return std::get_if<std::string>(&it->second);
}

std::optional<std::string> NvidiaBackend::emit_text(const CGModule& module) {
    std::ostringstream os;
    os << "//\n// cg_b200 launch listing (kernels are precompiled sm_100a code in libcg_b200.so)\n//\n";
    os << ".version 8.7\n.target " << sm_target_ << "\n.address_size 64\n";
    for (const CGFunction& fn : module.functions) {
        os << "\n.visible .entry " << fn.name << "(";
        for (usize i = 0; i < fn.args.size(); ++i) os << (i ? ", " : "") << ".param .u64 " << fn.name << "_param_" << i;
        os << ")\n{\n";
        for (const CGInstruction& inst : fn.instructions) {
            const std::string* kern = blob_of(inst, "b200.kernel");
            if (kern) {
                os << "    // call cg_b200_" << *kern;
                if (const std::string* rec = blob_of(inst, "b200.record"); rec && rec->size() == sizeof(PlanRecord)) {
                    PlanRecord r;
                    std::memcpy(&r, rec->data(), sizeof(r));
                    if (r.kind == PlanRecord::Gemm)
                        os << "  M=" << r.gemm.M << " N=" << r.gemm.N << " K=" << r.gemm.K << " batch=" << r.gemm.batch
                           << " epilogue=" << r.gemm.epilogue << "  (tcgen05.mma, TMEM accumulator)";
                    else if (r.kind == PlanRecord::Eltwise)
                        os << "  n=" << r.n << " instrs=" << r.eltwise.n_instr << " inputs=" << r.n_inputs;
                    else
                        os << "  rows=" << r.rows << " cols=" << r.cols;
                }
                os << "\n";
            } else {
                os << "    // " << (inst.comment.empty() ? "codegen op" : inst.comment) << " (no fused kernel: not executable)\n";
            }
        }
        os << "    ret;\n}\n";
    }
    return os.str();
}

std::unique_ptr<Executable> NvidiaBackend::compile(const CGModule& module) {
    auto exe = std::make_unique<Executable>();
    exe->target_device = target_info_.device;
    exe->ptx_text = *emit_text(module);
    exe->threads_per_block = 0;
    LaunchPlan plan;
    bool have_plan = false;
    for (const CGFunction& fn : module.functions) {
        if (exe->name.empty()) exe->name = fn.name;
        exe->entrypoints.push_back({fn.name, 0});
        if (have_plan) continue;   // one plan per Executable: the first function with fused nodes
        for (const CGInstruction& inst : fn.instructions) {
            const std::string* rec = blob_of(inst, "b200.record");
            if (!rec || rec->size() != sizeof(PlanRecord)) continue;
            if (!have_plan) {
                auto bytes = inst.attributes.find("b200.buffer_bytes");
                auto dts = inst.attributes.find("b200.buffer_dtypes");
                auto nin = inst.attributes.find("b200.n_inputs");
                auto nout = inst.attributes.find("b200.n_outputs");
                auto ws = inst.attributes.find("b200.workspace_bytes");
                if (bytes == inst.attributes.end() || dts == inst.attributes.end() || nin == inst.attributes.end() ||
                    nout == inst.attributes.end())
                    break;   // malformed: leave the plan empty, bind() will refuse it
                const auto& bv = std::get<std::vector<i64>>(bytes->second);
                const auto& dv = std::get<std::vector<i64>>(dts->second);
                for (usize i = 0; i < bv.size() && i < dv.size(); ++i) {
                    PlanBuffer b;
                    b.bytes = static_cast<u64>(bv[i]);
                    b.dtype = static_cast<DType>(dv[i]);
                    plan.buffers.push_back(b);
                }
                plan.n_inputs = static_cast<u32>(std::get<i64>(nin->second));
                plan.n_outputs = static_cast<u32>(std::get<i64>(nout->second));
                if (ws != inst.attributes.end()) plan.workspace_bytes = static_cast<u64>(std::get<i64>(ws->second));
                have_plan = true;
            }
            PlanRecord r;
            std::memcpy(&r, rec->data(), sizeof(r));
            plan.records.push_back(r);
            if (r.kind == PlanRecord::Gemm) {
                exe->threads_per_block = 320;
                exe->shared_mem_bytes = 225 * 1024;
            } else if (exe->threads_per_block == 0) {
                exe->threads_per_block = r.kind == PlanRecord::Eltwise ? 256 : 128;
            }
        }
    }
    if (have_plan) exe->machine_code = plan.serialize();
    return exe;
}

}  // namespace cg
