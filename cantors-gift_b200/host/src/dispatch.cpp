// dispatch.cpp - cg::VendorDispatcher with kernels that can run.
//
// Takes the place of the reference's src/vendor/dispatch.cpp. There, the registry holds four
// descriptor kernels (cuBLAS / cuDNN / rocBLAS / oneDNN) whose runtimes are constants and whose
// execute() is the base class's "return false" (include/cg/vendor/dispatch.hpp:61). The descriptors
// stay, with the same names, opcodes, dtype sets and estimates - code and tests that ask for "the best
// matmul kernel" keep getting the cuBLAS descriptor - and the cg_b200 kernels are registered beside
// them as candidates whose execute() launches real work.
//
// VendorKernel::execute(const Operation&, void* stream) carries no tensors, so the pointers ride on
// the operation itself: integer attributes "b200.in0", "b200.in1", ... and "b200.out0" hold device
// addresses (cg::b200::bind_pointers in cg/b200/vendor.hpp sets them). `stream` is a cudaStream_t.
// The cg_b200 kernels report no runtime estimate (the interface gives estimated_runtime() no operation
// to size it by), so find_best prefers a descriptor that has one and falls back to them for the ops
// only they support (softmax, layernorm, the elementwise ops).
#include "cg/vendor/dispatch.hpp"

#include <limits>

#include "cg/b200/vendor.hpp"
#include "cg/ir/ops.hpp"
#include "cg_b200.h"

namespace cg {
namespace {

// One class for all descriptor-only kernels: what a vendor library would support if it were loaded.
class Descriptor final : public VendorKernel {
public:
    Descriptor(VendorKind v, std::string n, Opcode opc, std::vector<DType> dtypes, double seconds)
        : vendor_(v), name_(std::move(n)), opcode_(opc), dtypes_(std::move(dtypes)), seconds_(seconds) {}
    VendorKind vendor() const override { return vendor_; }
    std::string name() const override { return name_; }
    Opcode opcode() const override { return opcode_; }
    bool supports(const Operation& op) const override {
        if (op.opcode != opcode_ || op.operands.size() != 2) return false;
        auto first = op.operands[0].as_tensor();
        if (!first) return false;
        if (opcode_ == OP_MATMUL && vendor_ == VendorKind::cuBLAS && !op.operands[1].as_tensor()) return false;
        for (DType dt : dtypes_)
            if (first->dtype == dt) return true;
        return false;
    }
    std::optional<double> estimated_runtime() const override { return seconds_; }

private:
    VendorKind vendor_;
    std::string name_;
    Opcode opcode_;
    std::vector<DType> dtypes_;
    double seconds_;
};

int abi_dtype(DType dt) { return dt == DType::F16 ? CG_B200_F16 : dt == DType::BF16 ? CG_B200_BF16 : dt == DType::F32 ? CG_B200_F32 : -1; }

bool static_dims(const TensorType& t, std::vector<i64>& out) {
    out.clear();
    for (const auto& d : t.shape) {
        if (!d->is_constant()) return false;
        out.push_back(d->value);
    }
    return true;
}

void* pointer_attr(const Operation& op, const std::string& key) {
    auto a = op.attributes.get(key);
    return a && a->kind == AttrKind::Integer ? reinterpret_cast<void*>(static_cast<std::uintptr_t>(a->integer)) : nullptr;
}

// The hand-written tcgen05 GEMM. VendorKind has no entry for this library; CUTLASS, the kind for
// hand-tuned tensor-core kernels, is the closest and is otherwise unused.
class B200Gemm final : public VendorKernel {
public:
    VendorKind vendor() const override { return VendorKind::CUTLASS; }
    std::string name() const override { return "cg_b200_gemm"; }
    Opcode opcode() const override { return OP_MATMUL; }
    bool supports(const Operation& op) const override {
        if (op.opcode != OP_MATMUL || op.operands.size() != 2 || op.results.size() != 1) return false;
        auto a = op.operands[0].as_tensor(), b = op.operands[1].as_tensor();
        return a && b && a->dtype == b->dtype && abi_dtype(a->dtype) >= 0 && a->shape.rank() == 2 && b->shape.rank() == 2;
    }
    bool execute(const Operation& op, void* stream) override {
        if (!supports(op)) return false;
        auto a = op.operands[0].as_tensor(), b = op.operands[1].as_tensor(), c = op.results[0].as_tensor();
        std::vector<i64> as, bs;
        if (!c || !static_dims(*a, as) || !static_dims(*b, bs) || as[1] != bs[0]) return false;
        void *pa = pointer_attr(op, "b200.in0"), *pb = pointer_attr(op, "b200.in1"), *pc = pointer_attr(op, "b200.out0");
        if (!pa || !pb || !pc) return false;
        cg_b200_gemm_desc d{};
        d.M = as[0]; d.K = as[1]; d.N = bs[1]; d.batch = 1;
        d.lda = d.K; d.ldb = d.N; d.ldc = d.N;
        d.batch_stride_a = d.M * d.K; d.batch_stride_b = d.K * d.N; d.batch_stride_c = d.M * d.N;
        d.in_dtype = abi_dtype(a->dtype);
        d.out_dtype = abi_dtype(c->dtype);
        d.alpha = 1.0f;
        if (d.out_dtype < 0) return false;
        size_t ws_bytes = 0;
        if (cg_b200_gemm_workspace_bytes(&d, &ws_bytes) != CG_B200_OK) return false;
        // fp32 operands need scratch for their tf32 split: the caller's, or one allocated for this call
        void* ws = pointer_attr(op, "b200.workspace");
        bool own_ws = false;
        if (ws_bytes && !ws) {
            if (cg_b200_malloc(&ws, ws_bytes) != CG_B200_OK) return false;
            own_ws = true;
        }
        const int st = cg_b200_gemm(&d, pa, pb, nullptr, nullptr, pc, ws, ws_bytes, stream);
        if (own_ws) {
            cg_b200_stream_sync(stream);   // the kernel reads the scratch until it has finished
            cg_b200_free(ws);
        }
        return st == CG_B200_OK;
    }
};

class B200Row final : public VendorKernel {
public:
    explicit B200Row(Opcode opc) : opc_(opc) {}
    VendorKind vendor() const override { return VendorKind::CUTLASS; }
    std::string name() const override { return opc_ == OP_SOFTMAX ? "cg_b200_softmax" : "cg_b200_layernorm"; }
    Opcode opcode() const override { return opc_; }
    bool supports(const Operation& op) const override {
        if (op.opcode != opc_ || op.operands.size() != 1) return false;
        auto x = op.operands[0].as_tensor();
        return x && abi_dtype(x->dtype) >= 0 && x->shape.rank() >= 1;
    }
    bool execute(const Operation& op, void* stream) override {
        if (!supports(op)) return false;
        auto x = op.operands[0].as_tensor();
        std::vector<i64> s;
        if (!static_dims(*x, s)) return false;
        void *in = pointer_attr(op, "b200.in0"), *out = pointer_attr(op, "b200.out0");
        if (!in || !out) return false;
        const i64 cols = s.back();
        i64 rows = 1;
        for (usize i = 0; i + 1 < s.size(); ++i) rows *= s[i];
        const int dt = abi_dtype(x->dtype);
        const int st = opc_ == OP_SOFTMAX ? cg_b200_softmax(dt, in, out, rows, cols, stream)
                                          : cg_b200_layernorm(dt, in, nullptr, nullptr, 1e-5f, out, rows, cols, stream);
        return st == CG_B200_OK;
    }

private:
    Opcode opc_;
};

// reduce_sum / reduce_max / reduce_mean over adjacent axes (the [outer, reduce, inner] box of cg_b200_reduce).
class B200Reduce final : public VendorKernel {
public:
    explicit B200Reduce(Opcode opc) : opc_(opc) {}
    VendorKind vendor() const override { return VendorKind::CUTLASS; }
    std::string name() const override {
        return opc_ == OP_REDUCE_SUM ? "cg_b200_reduce_sum" : (opc_ == OP_REDUCE_MAX ? "cg_b200_reduce_max" : "cg_b200_reduce_mean");
    }
    Opcode opcode() const override { return opc_; }
    bool supports(const Operation& op) const override {
        i64 box[3];
        return op.opcode == opc_ && box_of(op, box);
    }
    bool execute(const Operation& op, void* stream) override {
        i64 box[3];
        if (op.opcode != opc_ || !box_of(op, box)) return false;
        void *in = pointer_attr(op, "b200.in0"), *out = pointer_attr(op, "b200.out0");
        if (!in || !out) return false;
        const int rop = opc_ == OP_REDUCE_SUM ? CG_B200_REDUCE_SUM : (opc_ == OP_REDUCE_MAX ? CG_B200_REDUCE_MAX : CG_B200_REDUCE_MEAN);
        return cg_b200_reduce(abi_dtype(op.operands[0].as_tensor()->dtype), rop, in, out, box[0], box[1], box[2], stream) == CG_B200_OK;
    }

private:
    static bool box_of(const Operation& op, i64 (&box)[3]) {
        if (op.operands.size() != 1) return false;
        auto x = op.operands[0].as_tensor();
        auto axes = op.attributes.get("axes");
        std::vector<i64> s;
        if (!x || abi_dtype(x->dtype) < 0 || !axes || axes->ints.empty() || !static_dims(*x, s)) return false;
        const i64 rank = static_cast<i64>(s.size());
        i64 lo = rank, hi = -1;
        std::vector<char> seen(s.size(), 0);
        usize distinct = 0;
        for (i64 a : axes->ints) {
            if (a < 0) a += rank;
            if (a < 0 || a >= rank) return false;
            if (!seen[static_cast<usize>(a)]) { seen[static_cast<usize>(a)] = 1; ++distinct; }
            lo = std::min(lo, a);
            hi = std::max(hi, a);
        }
        if (hi - lo + 1 != static_cast<i64>(distinct)) return false;   // not a run of adjacent axes
        box[0] = box[1] = box[2] = 1;
        for (i64 i = 0; i < rank; ++i) box[i < lo ? 0 : (i > hi ? 2 : 1)] *= s[static_cast<usize>(i)];
        return box[1] > 0;
    }
    Opcode opc_;
};

// One elementwise op over whole tensors of one shape (broadcasts go through the planner).
class B200Eltwise final : public VendorKernel {
public:
    B200Eltwise(Opcode opc, int ew, int arity) : opc_(opc), ew_(ew), arity_(arity) {}
    VendorKind vendor() const override { return VendorKind::CUTLASS; }
    std::string name() const override {
        const OpInfo* info = OpRegistry::instance().lookup(opc_);
        return "cg_b200_eltwise_" + (info ? info->name : std::to_string(opc_));
    }
    Opcode opcode() const override { return opc_; }
    bool supports(const Operation& op) const override {
        if (op.opcode != opc_ || static_cast<int>(op.operands.size()) != arity_ || op.results.size() != 1) return false;
        auto r = op.results[0].as_tensor();
        if (!r || abi_dtype(r->dtype) < 0) return false;
        for (const Value& v : op.operands) {
            auto t = v.as_tensor();
            if (!t || t->dtype != r->dtype || !(t->shape == r->shape)) return false;
        }
        return true;
    }
    bool execute(const Operation& op, void* stream) override {
        if (!supports(op)) return false;
        auto r = op.results[0].as_tensor();
        std::vector<i64> s;
        if (!static_dims(*r, s)) return false;
        size_t n = 1;
        for (i64 d : s) n *= static_cast<size_t>(d);
        const void* in[2] = {pointer_attr(op, "b200.in0"), arity_ == 2 ? pointer_attr(op, "b200.in1") : nullptr};
        void* out = pointer_attr(op, "b200.out0");
        if (!in[0] || (arity_ == 2 && !in[1]) || !out) return false;
        cg_b200_eltwise_desc d{};
        d.dtype = abi_dtype(r->dtype);
        d.inner = 1;
        d.round_each_op = d.dtype != CG_B200_F32;
        for (int i = 0; i < arity_; ++i) d.prog[d.n_instr++] = {CG_B200_EW_INPUT, i, 0.0f};
        d.prog[d.n_instr++] = {ew_, 0, 0.0f};
        return cg_b200_eltwise(&d, in, arity_, out, n, stream) == CG_B200_OK;
    }

private:
    Opcode opc_;
    int ew_, arity_;
};

}  // namespace

namespace b200 {
void bind_pointers(Operation& op, const std::vector<void*>& inputs, void* output, void* workspace) {
    auto as_attr = [](void* p) { return Attribute::make_integer(static_cast<i64>(reinterpret_cast<std::uintptr_t>(p))); };
    for (usize i = 0; i < inputs.size(); ++i) op.attributes.set("b200.in" + std::to_string(i), as_attr(inputs[i]));
    op.attributes.set("b200.out0", as_attr(output));
    if (workspace) op.attributes.set("b200.workspace", as_attr(workspace));
}

VendorKernel* find_executable(const Operation& op) {
    for (const auto& k : VendorDispatcher::instance().kernels())
        if (k->vendor() == VendorKind::CUTLASS && k->supports(op)) return k.get();
    return nullptr;
}
}  // namespace b200

VendorDispatcher::VendorDispatcher() {
    // the four descriptors of the reference (src/vendor/dispatch.cpp:52-133), as a table
    const std::vector<DType> f3 = {DType::F32, DType::F16, DType::BF16};
    register_kernel(std::make_unique<Descriptor>(VendorKind::cuBLAS, "cublas_matmul", OP_MATMUL,
                                                 std::vector<DType>{DType::F32, DType::F16, DType::BF16, DType::F64, DType::I8}, 1e-5));
    register_kernel(std::make_unique<Descriptor>(VendorKind::cuDNN, "cudnn_conv2d", OP_CONV2D, f3, 5e-5));
    register_kernel(std::make_unique<Descriptor>(VendorKind::rocBLAS, "rocblas_matmul", OP_MATMUL, f3, 1.2e-5));
    register_kernel(std::make_unique<Descriptor>(VendorKind::oneDNN, "onednn_matmul", OP_MATMUL, std::vector<DType>{DType::F32}, 2e-5));
    // kernels that execute
    register_kernel(std::make_unique<B200Gemm>());
    register_kernel(std::make_unique<B200Row>(OP_SOFTMAX));
    register_kernel(std::make_unique<B200Row>(OP_LAYERNORM));
    for (Opcode opc : {OP_REDUCE_SUM, OP_REDUCE_MAX, OP_REDUCE_MEAN}) register_kernel(std::make_unique<B200Reduce>(opc));
    const struct { Opcode opc; int ew; int arity; } ops[] = {
        {OP_ADD, CG_B200_EW_ADD, 2}, {OP_SUB, CG_B200_EW_SUB, 2}, {OP_MUL, CG_B200_EW_MUL, 2}, {OP_DIV, CG_B200_EW_DIV, 2},
        {OP_NEG, CG_B200_EW_NEG, 1}, {OP_RELU, CG_B200_EW_RELU, 1}, {OP_GELU, CG_B200_EW_GELU_TANH, 1},
        {OP_SIGMOID, CG_B200_EW_SIGMOID, 1}, {OP_TANH, CG_B200_EW_TANH, 1}, {OP_EXP, CG_B200_EW_EXP, 1},
        {OP_LOG, CG_B200_EW_LOG, 1}, {OP_SQRT, CG_B200_EW_SQRT, 1}};
    for (const auto& o : ops) register_kernel(std::make_unique<B200Eltwise>(o.opc, o.ew, o.arity));
}

VendorDispatcher& VendorDispatcher::instance() {
    static VendorDispatcher d;
    return d;
}

void VendorDispatcher::register_kernel(std::unique_ptr<VendorKernel> kernel) {
    if (kernel) kernels_.push_back(std::move(kernel));
}

// The cheapest estimate among the kernels that support `op`; kernels without an estimate are taken
// only when none has one (the first such kernel in registration order).
VendorKernel* VendorDispatcher::find_best(const Operation& op) const {
    VendorKernel* best = nullptr;
    VendorKernel* unrated = nullptr;
    double best_t = std::numeric_limits<double>::infinity();
    for (const auto& k : kernels_) {
        if (!k->supports(op)) continue;
        const std::optional<double> t = k->estimated_runtime();
        if (t && *t < best_t) {
            best_t = *t;
            best = k.get();
        } else if (!t && !unrated) {
            unrated = k.get();
        }
    }
    return best ? best : unrated;
}

bool VendorDispatcher::has_vendor(VendorKind kind) const {
    for (const auto& k : kernels_)
        if (k->vendor() == kind) return true;
    return false;
}

}  // namespace cg
