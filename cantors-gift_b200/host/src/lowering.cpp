// lowering.cpp - the kernel planner: Tensor IR -> one Codegen-IR node per fused B200 kernel.
//
// Replaces the per-op emitters of the reference's TensorToCodegenLowering
// (src/lowering/tensor_to_codegen.cpp:33-368). Grouping rules:
//   gemm      matmul, plus a single-use tail  + bias[N]  (relu | gelu)?  (+ residual)?  |  * scalar
//   row op    softmax, layernorm, or layernorm(softmax(x)) when the softmax has no other use
//   eltwise   maximal trees of elementwise ops whose inner values have exactly one use, cut where
//             the C ABI's limits (16 instructions, 8 inputs, stack depth 4) would be exceeded
// Every kernel result that another kernel or an output reads is materialised in a plan buffer.
#include <algorithm>
#include <cstring>
#include <stdexcept>

#include "cg/b200_host.hpp"

namespace cg {
namespace {

bool is_unary(Opcode o) {
    return o == OP_NEG || o == OP_RELU || o == OP_GELU || o == OP_SIGMOID || o == OP_TANH || o == OP_EXP ||
           o == OP_LOG || o == OP_SQRT;
}
bool is_binary(Opcode o) { return o == OP_ADD || o == OP_SUB || o == OP_MUL || o == OP_DIV; }
bool is_eltwise(Opcode o) { return is_unary(o) || is_binary(o); }

int ew_op(Opcode o) {
    switch (o) {
        case OP_ADD: return CG_B200_EW_ADD;
        case OP_SUB: return CG_B200_EW_SUB;
        case OP_MUL: return CG_B200_EW_MUL;
        case OP_DIV: return CG_B200_EW_DIV;
        case OP_NEG: return CG_B200_EW_NEG;
        case OP_RELU: return CG_B200_EW_RELU;
        case OP_GELU: return CG_B200_EW_GELU_TANH;   // tanh form (include/cg/egraph/rewrite_rules.hpp:96-101)
        case OP_SIGMOID: return CG_B200_EW_SIGMOID;
        case OP_TANH: return CG_B200_EW_TANH;
        case OP_EXP: return CG_B200_EW_EXP;
        case OP_LOG: return CG_B200_EW_LOG;
        default: return CG_B200_EW_SQRT;
    }
}

int abi_dtype(DType dt) {
    switch (dt) {
        case DType::F16: return CG_B200_F16;
        case DType::BF16: return CG_B200_BF16;
        case DType::F32: return CG_B200_F32;
        default: return -1;
    }
}

struct Fail : std::runtime_error {
    int status;
    Fail(int st, const std::string& m) : std::runtime_error(m), status(st) {}
};

struct Planner {
    const Function& f;
    const LoweringOptions& opts;
    std::vector<int> uses;            // number of reads of each op's result
    std::vector<int> single_user;     // the reader when uses == 1, else 0
    std::vector<char> root;           // result is materialised by a kernel
    std::vector<char> absorbed;       // op lives inside another kernel (gemm tail, fused softmax)
    std::vector<int> buffer_of;       // plan buffer of a materialised value (-1 = none)
    LaunchPlan plan;
    struct Kernel {
        u32 at;                       // id of the op whose result the kernel produces
        PlanRecord rec;
        std::string name;
    };
    std::vector<Kernel> kernels;

    Planner(const Function& fn, const LoweringOptions& o) : f(fn), opts(o) {
        const usize n = f.ops.size();
        uses.assign(n, 0);
        single_user.assign(n, 0);
        root.assign(n, 0);
        absorbed.assign(n, 0);
        buffer_of.assign(n, -1);
    }

    // reshape is a view: follow it to the op that owns the storage
    u32 source(Value v) const {
        u32 id = v.id;
        while (f.ops[id].opcode == OP_RESHAPE) id = f.ops[id].operands[0].id;
        return id;
    }

    bool scalar_const(u32 id, float* value) const {
        const Operation& op = f.ops[id];
        if (op.opcode != OP_CONSTANT || num_elements(op.shape) != 1) return false;
        if (auto it = op.attributes.find("value"); it != op.attributes.end()) {
            if (auto* d = std::get_if<double>(&it->second)) { *value = static_cast<float>(*d); return true; }
        }
        if (op.dtype == DType::F32 && op.constant_bytes.size() == 4) {
            std::memcpy(value, op.constant_bytes.data(), 4);
            return true;
        }
        return false;
    }

    void check_markers() const {
        for (const Operation& op : f.ops) {
            if (op.opcode == OP_FUSE || op.attributes.count("fused_chain") || op.attributes.count("fused_with"))
                throw Fail(CG_B200_ERR_FUSED_IR,
                           "IR carries fusion markers (fused_chain / fused_with / fuse op): the producer chain is "
                           "lost, run the planner on pre-fusion IR");
        }
    }

    void count_uses() {
        for (u32 i = 1; i < f.ops.size(); ++i)
            for (Value v : f.ops[i].operands) {
                const u32 s = source(v);
                if (f.ops[i].opcode == OP_RESHAPE) continue;   // counted at the reshape's own readers
                ++uses[s];
                single_user[s] = static_cast<int>(i);
            }
        for (u32 i = 1; i < f.ops.size(); ++i)
            if (uses[i] != 1) single_user[i] = 0;
    }

    int new_buffer(const Operation& op) {
        PlanBuffer b;
        b.dtype = op.dtype;
        b.shape = op.shape;
        b.bytes = static_cast<u64>(num_elements(op.shape)) * dtype_size(op.dtype);
        plan.buffers.push_back(b);
        return static_cast<int>(plan.buffers.size() - 1);
    }

    int buffer_for_read(u32 id) {
        if (buffer_of[id] < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "internal: value read before it is materialised");
        return buffer_of[id];
    }

    // ---- gemm ----------------------------------------------------------------------------------
    void plan_gemm(u32 id) {
        const Operation& mm = f.ops[id];
        const Operation& a = f.ops[mm.operands[0].id];
        const Operation& b = f.ops[mm.operands[1].id];
        const int in_dt = abi_dtype(a.dtype);
        if (in_dt < 0 || a.dtype != b.dtype) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: operand dtypes must be one of f16/bf16/f32 and equal");
        const i64 M = a.shape[a.shape.size() - 2], K = a.shape[a.shape.size() - 1], N = b.shape[b.shape.size() - 1];
        const i64 batch = num_elements(mm.shape) / (M * N);
        const i64 a_batch = num_elements(a.shape) / (M * K), b_batch = num_elements(b.shape) / (K * N);
        if ((a_batch != batch && a_batch != 1) || (b_batch != batch && b_batch != 1))
            throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: partial batch broadcast is not supported");
        PlanRecord r;
        r.kind = PlanRecord::Gemm;
        cg_b200_gemm_desc& d = r.gemm;
        d.M = M; d.N = N; d.K = K; d.batch = batch;
        d.lda = K; d.ldb = N; d.ldc = N;
        d.batch_stride_a = a_batch == 1 ? 0 : M * K;
        d.batch_stride_b = b_batch == 1 ? 0 : K * N;
        d.batch_stride_c = M * N;
        d.in_dtype = in_dt;
        d.compute = CG_B200_COMPUTE_DEFAULT;
        d.epilogue = CG_B200_EPI_NONE;
        d.alpha = 1.0f;
        r.input[0] = buffer_for_read(source(mm.operands[0]));
        r.input[1] = buffer_for_read(source(mm.operands[1]));
        r.n_inputs = 2;

        // absorb a single-use tail into the epilogue
        u32 last = id;
        auto next_user = [&](u32 cur) -> u32 { return single_user[cur] > 0 ? static_cast<u32>(single_user[cur]) : 0u; };
        auto other_operand = [&](const Operation& op, u32 cur) -> u32 {
            return source(op.operands[0]) == cur ? source(op.operands[1]) : source(op.operands[0]);
        };
        u32 u = next_user(last);
        float sc = 0.0f;
        if (u && f.ops[u].opcode == OP_MUL && f.ops[u].shape == mm.shape && scalar_const(other_operand(f.ops[u], last), &sc)) {
            d.epilogue = CG_B200_EPI_SCALE;
            d.alpha = sc;
            absorbed[u] = 1;
            last = u;
        } else if (u && f.ops[u].opcode == OP_ADD && f.ops[u].shape == mm.shape) {
            const u32 o = other_operand(f.ops[u], last);
            const Shape& os = f.ops[o].shape;
            const bool is_bias = num_elements(os) == N && !os.empty() && os.back() == N && buffer_of[o] >= 0 &&
                                 f.ops[o].dtype == mm.dtype;
            const bool is_res = os == mm.shape && buffer_of[o] >= 0 && f.ops[o].dtype == mm.dtype;
            if (is_bias) {
                d.epilogue = CG_B200_EPI_BIAS;
                r.input[2] = buffer_of[o];
                absorbed[u] = 1;
                last = u;
                u32 u2 = next_user(last);
                if (u2 && (f.ops[u2].opcode == OP_RELU || f.ops[u2].opcode == OP_GELU)) {
                    d.epilogue = f.ops[u2].opcode == OP_RELU ? CG_B200_EPI_BIAS_RELU : CG_B200_EPI_BIAS_GELU_TANH;
                    absorbed[u2] = 1;
                    last = u2;
                } else if (u2 && f.ops[u2].opcode == OP_ADD && f.ops[u2].shape == mm.shape) {
                    const u32 o2 = other_operand(f.ops[u2], last);
                    if (f.ops[o2].shape == mm.shape && buffer_of[o2] >= 0 && f.ops[o2].dtype == mm.dtype) {
                        d.epilogue = CG_B200_EPI_BIAS_RESIDUAL;
                        r.input[3] = buffer_of[o2];
                        absorbed[u2] = 1;
                        last = u2;
                    }
                }
            } else if (is_res) {
                d.epilogue = CG_B200_EPI_RESIDUAL;
                r.input[3] = buffer_of[o];
                absorbed[u] = 1;
                last = u;
            }
        }
        const int out_dt = abi_dtype(f.ops[last].dtype);
        if (out_dt < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: unsupported result dtype");
        d.out_dtype = out_dt;
        if (id != last) absorbed[id] = 1;
        finish_kernel(last, r, "gemm");
    }

    // ---- row reductions --------------------------------------------------------------------------
    void plan_row(u32 id) {
        const Operation& op = f.ops[id];
        if (absorbed[id]) return;
        PlanRecord r;
        const int dt = abi_dtype(op.dtype);
        if (dt < 0 || op.shape.empty()) throw Fail(CG_B200_ERR_UNSUPPORTED, "softmax/layernorm: unsupported type");
        r.row_dtype = dt;
        r.cols = op.shape.back();
        r.rows = num_elements(op.shape) / (r.cols ? r.cols : 1);
        r.eps = opts.layernorm_eps;
        r.n_inputs = 1;
        u32 last = id;
        if (op.opcode == OP_SOFTMAX) {
            r.kind = PlanRecord::Softmax;
            const u32 u = single_user[id] > 0 ? static_cast<u32>(single_user[id]) : 0u;
            if (opts.fuse_softmax_layernorm && u && f.ops[u].opcode == OP_LAYERNORM) {
                r.kind = PlanRecord::SoftmaxLayerNorm;
                absorbed[u] = 1;      // the layernorm op is produced by this kernel
                absorbed[id] = 1;
                last = u;
            }
        } else {
            r.kind = PlanRecord::LayerNorm;
        }
        r.input[0] = buffer_for_read(source(op.operands[0]));
        finish_kernel(last, r, r.kind == PlanRecord::Softmax ? "softmax" : (r.kind == PlanRecord::LayerNorm ? "layernorm" : "softmax_layernorm"));
    }

    // ---- elementwise trees -------------------------------------------------------------------------
    struct EwBuild {
        cg_b200_eltwise_desc d{};
        std::vector<u32> inputs;      // source op ids
        i64 n = 0;
        i64 inner = 0;                // 0 = not fixed yet
        const Shape* out_shape = nullptr;
    };

    int classify(const EwBuild& b, const Shape& s, i64* inner) const {
        const i64 ne = num_elements(s);
        if (ne == b.n && ne != 1) return CG_B200_BC_FULL;
        if (ne == 1) return CG_B200_BC_SCALAR;
        const Shape& os = *b.out_shape;
        // trailing dims equal -> row vector of period ne
        Shape trimmed = s;
        while (trimmed.size() > 1 && trimmed.front() == 1) trimmed.erase(trimmed.begin());
        if (trimmed.size() <= os.size() && std::equal(trimmed.rbegin(), trimmed.rend(), os.rbegin())) {
            *inner = ne;
            return CG_B200_BC_ROW;
        }
        // [..., 1] against [..., C] -> column vector
        if (s.size() == os.size() && !s.empty() && s.back() == 1 && std::equal(s.begin(), s.end() - 1, os.begin())) {
            *inner = os.back();
            return CG_B200_BC_COL;
        }
        return -1;
    }

    // depth of the subtree if inlined; -1 if it cannot be inlined (limits)
    bool can_inline(u32 id, u32 parent) const {
        const Operation& op = f.ops[id];
        return is_eltwise(op.opcode) && !root[id] && !absorbed[id] && uses[id] == 1 &&
               static_cast<u32>(single_user[id]) == parent && op.shape == f.ops[parent].shape &&
               op.dtype == f.ops[parent].dtype;
    }

    // Appends code that leaves the value of `id` on the stack. Returns the stack depth it needs.
    // `reserve`: instructions the callers still have to append after this value (their own ops and
    // at least one instruction per operand not generated yet).
    int gen(EwBuild& b, u32 id, u32 parent, bool is_root, int reserve = 0) {
        const Operation& op = f.ops[id];
        float imm = 0.0f;
        if (!is_root && scalar_const(id, &imm)) {
            if (b.d.n_instr + 1 + reserve > CG_B200_EW_MAX_INSTR) throw Fail(CG_B200_ERR_UNSUPPORTED, "cut");
            b.d.prog[b.d.n_instr++] = {CG_B200_EW_IMM, 0, imm};
            return 1;
        }
        if (is_root || can_inline(id, parent)) {
            // try to inline; on overflow fall back to reading it as an input (caller handles by marking root)
            const int save_n = b.d.n_instr;
            const usize save_in = b.inputs.size();
            const i64 save_inner = b.inner;
            try {
                int depth;
                if (is_binary(op.opcode)) {
                    const int da = gen(b, source(op.operands[0]), id, false, reserve + 2);
                    const int db = gen(b, source(op.operands[1]), id, false, reserve + 1);
                    depth = std::max(da, 1 + db);
                } else {
                    depth = gen(b, source(op.operands[0]), id, false, reserve + 1);
                }
                if (depth > CG_B200_EW_MAX_STACK) throw Fail(CG_B200_ERR_UNSUPPORTED, "cut");
                b.d.prog[b.d.n_instr++] = {ew_op(op.opcode), 0, 0.0f};
                return depth;
            } catch (const Fail& e) {
                if (is_root || std::string(e.what()) != "cut") throw;
                b.d.n_instr = save_n;
                b.inputs.resize(save_in);
                b.inner = save_inner;
                pending_roots.push_back(id);   // materialise this subtree on its own
            }
        }
        // read as an input
        if (op.dtype != f.ops[parent].dtype && !(op.opcode == OP_CONSTANT))
            throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: mixed operand dtypes");
        i64 inner = 0;
        const int kind = classify(b, op.shape, &inner);
        if (kind < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: unsupported broadcast");
        if (kind == CG_B200_BC_ROW || kind == CG_B200_BC_COL) {
            if (b.inner != 0 && b.inner != inner) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: two broadcast periods in one chain");
            b.inner = inner;
        }
        int slot = -1;
        for (usize i = 0; i < b.inputs.size(); ++i)
            if (b.inputs[i] == id && b.d.bcast[i] == kind) slot = static_cast<int>(i);
        if (slot < 0) {
            if (b.inputs.size() >= CG_B200_EW_MAX_INPUTS) throw Fail(CG_B200_ERR_UNSUPPORTED, "cut");
            slot = static_cast<int>(b.inputs.size());
            b.inputs.push_back(id);
            b.d.bcast[slot] = kind;
        }
        if (b.d.n_instr + 1 + reserve > CG_B200_EW_MAX_INSTR) throw Fail(CG_B200_ERR_UNSUPPORTED, "cut");
        b.d.prog[b.d.n_instr++] = {CG_B200_EW_INPUT, slot, 0.0f};
        return 1;
    }

    std::vector<u32> pending_roots;

    // Builds the program of root `id`; inputs may not be materialised yet (resolved in emit order).
    struct EwKernel {
        u32 at;
        EwBuild b;
    };
    std::vector<EwKernel> ew_kernels;

    void build_eltwise(u32 id) {
        EwBuild b;
        const Operation& op = f.ops[id];
        const int dt = abi_dtype(op.dtype);
        if (dt < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: unsupported dtype");
        b.d.dtype = dt;
        b.d.round_each_op = dt != CG_B200_F32;   // every Tensor-IR op result is a tensor of that type
        b.n = num_elements(op.shape);
        b.out_shape = &op.shape;
        gen(b, id, id, true);
        b.d.inner = b.inner > 0 ? b.inner : 1;
        ew_kernels.push_back({id, b});
    }

    void finish_kernel(u32 at, PlanRecord r, const std::string& name) {
        r.output = buffer_of[at] >= 0 ? buffer_of[at] : (buffer_of[at] = new_buffer(f.ops[at]));
        kernels.push_back({at, r, name});
    }

    LaunchPlan run() {
        check_markers();
        count_uses();
        // inputs and outputs first: fixed buffer numbering
        for (u32 i = 1; i < f.ops.size(); ++i)
            if (f.ops[i].opcode == OP_INPUT) { buffer_of[i] = new_buffer(f.ops[i]); ++plan.n_inputs; }
        for (u32 i = 1; i < f.ops.size(); ++i)
            if (f.ops[i].opcode == OP_OUTPUT) {
                const u32 s = source(f.ops[i].operands[0]);
                if (f.ops[s].opcode == OP_INPUT || buffer_of[s] >= 0)
                    throw Fail(CG_B200_ERR_UNSUPPORTED, "output: a value may be output once and must be computed");
                buffer_of[s] = new_buffer(f.ops[s]);
                ++plan.n_outputs;
            }
        // which elementwise ops must be materialised: read by a non-elementwise op, read more than once,
        // read through a broadcast, or an output
        for (u32 i = 1; i < f.ops.size(); ++i) {
            const Operation& op = f.ops[i];
            if (!is_eltwise(op.opcode)) continue;
            const u32 u = single_user[i] > 0 ? static_cast<u32>(single_user[i]) : 0u;
            if (uses[i] != 1 || buffer_of[i] >= 0 || !is_eltwise(f.ops[u].opcode) || f.ops[u].shape != op.shape ||
                f.ops[u].dtype != op.dtype)
                root[i] = 1;
        }
        // kernels in program order; gemm tails and fused softmax mark what they absorb before the
        // elementwise pass looks at those ops
        for (u32 i = 1; i < f.ops.size(); ++i) {
            const Operation& op = f.ops[i];
            switch (op.opcode) {
                case OP_INPUT: case OP_OUTPUT: case OP_RESHAPE: break;
                case OP_CONSTANT: {
                    float v;
                    if (!scalar_const(i, &v)) throw Fail(CG_B200_ERR_UNSUPPORTED, "only scalar constants are supported");
                    break;
                }
                case OP_MATMUL: plan_gemm(i); break;
                case OP_SOFTMAX: case OP_LAYERNORM: plan_row(i); break;
                default:
                    if (!is_eltwise(op.opcode)) throw Fail(CG_B200_ERR_UNSUPPORTED, "opcode " + std::to_string(op.opcode) + " has no B200 kernel");
                    if (absorbed[i] || !root[i]) break;
                    emit_eltwise_root(i);
            }
        }
        for (const Kernel& k : kernels) {
            plan.records.push_back(k.rec);
            if (k.rec.kind == PlanRecord::Gemm && k.rec.gemm.in_dtype == CG_B200_F32) {
                const i64 ldk = (k.rec.gemm.K + 3) / 4 * 4;
                auto r64 = [](i64 x) { return (x + 63) / 64 * 64; };
                const i64 ab = k.rec.gemm.batch_stride_a == 0 ? 1 : k.rec.gemm.batch, bb = k.rec.gemm.batch_stride_b == 0 ? 1 : k.rec.gemm.batch;
                const u64 ws = static_cast<u64>(2 * (r64(ab * k.rec.gemm.M * ldk) + r64(bb * k.rec.gemm.N * ldk))) * 4;
                plan.workspace_bytes = std::max(plan.workspace_bytes, ws);
            }
        }
        return plan;
    }

    // A root may spill sub-trees that exceed the ABI limits: those become roots of their own and are
    // emitted first (they only depend on earlier values).
    void emit_eltwise_root(u32 id) {
        pending_roots.clear();
        build_eltwise(id);
        EwKernel k = ew_kernels.back();
        ew_kernels.pop_back();
        const std::vector<u32> spill = pending_roots;
        for (u32 s : spill) {
            if (buffer_of[s] < 0) { root[s] = 1; emit_eltwise_root(s); }
        }
        PlanRecord r;
        r.kind = PlanRecord::Eltwise;
        r.eltwise = k.b.d;
        r.n = static_cast<u64>(k.b.n);
        r.n_inputs = static_cast<i32>(k.b.inputs.size());
        for (usize i = 0; i < k.b.inputs.size(); ++i) r.input[i] = buffer_for_read(k.b.inputs[i]);
        finish_kernel(id, r, "eltwise");
    }
};

std::string record_blob(const PlanRecord& r) {
    return std::string(reinterpret_cast<const char*>(&r), sizeof(PlanRecord));
}

}  // namespace

CGModule TensorToCodegenLowering::lower(const Module& m, const Schedule& schedule) {
    status_ = CG_B200_OK;
    message_.clear();
    CGModule out;
    const std::optional<cg_b200_gemm_tuning> tuning = gemm_tuning_from_schedule(schedule);
    if (!tuning) {
        status_ = CG_B200_ERR_UNSUPPORTED;
        message_ = "schedule: the GEMM kernels have no such tile";
        return out;
    }
    try {
        for (const Function& fn : m.functions) {
            Planner p(fn, opts_);
            const LaunchPlan plan = p.run();
            for (auto& ker : p.kernels)
                if (ker.rec.kind == PlanRecord::Gemm) ker.rec.tuning = *tuning;
            CGFunction& cf = out.create_function(fn.name);
            for (u32 i = 0; i < plan.n_inputs + plan.n_outputs; ++i) {
                CGValue v = cf.allocate(plan.buffers[i].dtype, 1);
                v.name = (i < plan.n_inputs ? "in" : "out") + std::to_string(i < plan.n_inputs ? i : i - plan.n_inputs);
                cf.args.push_back(v);   // outputs are arguments too: a launch needs somewhere to write
            }
            std::vector<i64> buffer_bytes, buffer_dtypes;
            for (const PlanBuffer& b : plan.buffers) {
                buffer_bytes.push_back(static_cast<i64>(b.bytes));
                buffer_dtypes.push_back(static_cast<i64>(b.dtype));
            }
            for (usize k = 0; k < p.kernels.size(); ++k) {
                const auto& ker = p.kernels[k];
                CGInstruction inst;
                inst.opcode = ker.rec.kind == PlanRecord::Gemm ? CGOpcode::FMA
                              : (ker.rec.kind == PlanRecord::Eltwise ? CGOpcode::Add : CGOpcode::Reduce);
                inst.attributes["b200.kernel"] = ker.name;
                inst.attributes["b200.record"] = record_blob(ker.rec);
                if (k == 0) {
                    inst.attributes["b200.buffer_bytes"] = buffer_bytes;
                    inst.attributes["b200.buffer_dtypes"] = buffer_dtypes;
                    inst.attributes["b200.n_inputs"] = static_cast<i64>(plan.n_inputs);
                    inst.attributes["b200.n_outputs"] = static_cast<i64>(plan.n_outputs);
                    inst.attributes["b200.workspace_bytes"] = static_cast<i64>(plan.workspace_bytes);
                }
                inst.comment = "cg_b200 " + ker.name;
                cf.emit(std::move(inst));
            }
        }
    } catch (const Fail& e) {
        status_ = e.status;
        message_ = e.what();
        return CGModule{};
    }
    return out;
}

}  // namespace cg
