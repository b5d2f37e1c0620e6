// tensor_to_codegen.cpp - cg::TensorToCodegenLowering::{lower, lower_function} for the B200 path:
// the kernel planner.
//
// Takes the place of the reference's src/lowering/tensor_to_codegen.cpp:33-368, which emits one
// un-looped vector instruction group per Tensor-IR op. That generic stream is still produced, by the
// reference's own code (cg::b200::legacy_lower_function), because its PTX emitter and tests read it.
// Behind it this lowering appends ONE CGInstruction per fused B200 kernel (opcode FMA = GEMM or
// attention, Add = elementwise chain, Reduce = row reduction) whose attributes carry the kernel's name
// and its serialised launch record ("b200.kernel", "b200.record"); the first node also carries the
// buffer table. NvidiaBackend::compile turns those nodes into the Executable's launch plan.
//
// Grouping rules (pre-fusion Tensor IR):
//   attention  matmul(q, k^T) -> (mul by a scalar)? -> softmax -> matmul(p, v), every inner value read
//              once, head_dim 64, 16-bit: one cg_b200_attention node. Other head sizes or fp32 are not
//              guessed at: they stay three kernels.
//   gemm       matmul plus a single-use tail  (+ bias[N])? (relu | gelu)? (+ residual)?  |  * scalar.
//              A transposed operand (transpose of the last two axes), a column block (slice of the
//              last axis), a head split (reshape + transpose [0,2,1,3]) are read in place through
//              row / batch strides; nothing is copied.
//   row op     softmax, layernorm, or layernorm(softmax(x)) when the softmax has no other reader
//   eltwise    maximal trees of elementwise ops whose inner values are read once, cut where the C
//              ABI's limits (16 instructions, 8 inputs, stack depth 4) would be exceeded
// A GEMM or attention result that is only read through "merge heads" (transpose [0,2,1,3] + reshape)
// is written in the merged layout directly.
// IR that carries the reference's lossy fusion markers (fused_chain / fused_with attributes, OP_FUSE;
// src/optimization/fusion/fusion.cpp:415-441) cannot be executed faithfully: no nodes are attached and
// cg::b200::last_lowering_status() reports CG_B200_ERR_FUSED_IR. The same holds, with
// CG_B200_ERR_UNSUPPORTED, for graphs with ops that have no B200 kernel: the generic stream is all the
// backend then gets, exactly what the reference produced.
#include "cg/lowering/tensor_to_codegen.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>

#include "cg/b200/b200.hpp"
#include "cg/b200/plan.hpp"
#include "cg/ir/ops.hpp"

namespace cg {
namespace b200 {
void legacy_lower_function(const LoweringOptions& opts, const Function& f, CGFunction& out, const Schedule& schedule);
}

namespace {

thread_local int t_status = CG_B200_OK;
thread_local std::string t_message;

using b200::LaunchPlan;
using b200::PlanBuffer;
using b200::PlanRecord;
using Dims = std::vector<i64>;

struct Fail : std::runtime_error {
    int status;
    Fail(int st, const std::string& m) : std::runtime_error(m), status(st) {}
};
struct Cut {};   // an elementwise tree hit a limit of the C ABI: the subtree becomes a kernel of its own

bool is_unary(Opcode o) {
    return o == OP_NEG || o == OP_RELU || o == OP_GELU || o == OP_SIGMOID || o == OP_TANH || o == OP_EXP ||
           o == OP_LOG || o == OP_SQRT;
}
bool is_binary(Opcode o) { return o == OP_ADD || o == OP_SUB || o == OP_MUL || o == OP_DIV; }
bool is_eltwise(Opcode o) { return is_unary(o) || is_binary(o); }
bool is_view(Opcode o) { return o == OP_RESHAPE || o == OP_TRANSPOSE || o == OP_SLICE || o == OP_COPY || o == OP_BROADCAST; }

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

std::string op_name(Opcode o) {
    const OpInfo* info = OpRegistry::instance().lookup(o);
    return info ? info->name : "opcode " + std::to_string(o);
}

int abi_dtype(DType dt) {
    switch (dt) {
        case DType::F16: return CG_B200_F16;
        case DType::BF16: return CG_B200_BF16;
        case DType::F32: return CG_B200_F32;
        default: return -1;
    }
}

i64 count(const Dims& s) {
    i64 n = 1;
    for (i64 d : s) n *= d;
    return n;
}

Dims canonical_strides(const Dims& shape) {
    Dims st(shape.size(), 1);
    for (usize i = shape.size(); i-- > 1;) st[i - 1] = st[i] * shape[i];
    return st;
}

// ---- the function as the planner sees it ---------------------------------------------------------------
struct Node {
    Opcode op = OP_INVALID;
    std::vector<int> in;
    Dims shape;
    DType dtype = DType::F32;
    const Operation* src = nullptr;   // null for block arguments
};

// A strided window into the storage of `root` (a node that owns memory), in elements.
struct View {
    int root = 0;
    i64 offset = 0;
    Dims shape, stride;
};

bool contiguous(const View& v) {
    i64 expect = 1;
    for (usize i = v.shape.size(); i-- > 0;) {
        if (v.shape[i] == 1) continue;
        if (v.stride[i] != expect) return false;
        expect *= v.shape[i];
    }
    return true;
}

// New shape over the same memory without a copy, when the strides allow it: dimensions are matched in
// groups of equal element count, and a group of old dimensions can be re-split only if it is itself
// contiguous.
bool reshape_view(const View& v, const Dims& to, View& out) {
    out = v;
    out.shape = to;
    out.stride.assign(to.size(), 0);
    if (count(v.shape) != count(to)) return false;
    if (count(to) == 0) {
        out.stride = canonical_strides(to);
        return true;
    }
    Dims os, ost;   // old dims without the 1s
    for (usize i = 0; i < v.shape.size(); ++i)
        if (v.shape[i] != 1) {
            os.push_back(v.shape[i]);
            ost.push_back(v.stride[i]);
        }
    usize oi = 0, ni = 0;
    while (ni < to.size()) {
        if (to[ni] == 1) {
            out.stride[ni] = 1;
            ++ni;
            continue;
        }
        if (oi >= os.size()) return false;
        // grow both sides until the products agree
        usize oj = oi + 1, nj = ni + 1;
        i64 op = os[oi], np = to[ni];
        while (op != np) {
            if (op < np) {
                if (oj >= os.size()) return false;
                op *= os[oj++];
            } else {
                while (nj < to.size() && to[nj] == 1) out.stride[nj++] = 1;
                if (nj >= to.size()) return false;
                np *= to[nj++];
            }
        }
        for (usize k = oi; k + 1 < oj; ++k)
            if (ost[k] != ost[k + 1] * os[k + 1]) return false;   // the old group is not one block of memory
        i64 st = ost[oj - 1];
        for (usize k = nj; k-- > ni;) {
            out.stride[k] = st;
            st *= to[k];
        }
        oi = oj;
        ni = nj;
    }
    return oi == os.size();
}

struct Planner {
    const Function& f;
    const LoweringOptions& opts;
    std::vector<Node> nodes;                    // nodes[0] is unused so that 0 means "none"
    std::unordered_map<ValueId, int> node_of;
    std::vector<int> uses, single_user;         // readers of a storage owner (through any views)
    std::vector<char> root, absorbed;
    std::vector<int> buffer_of;                 // plan buffer of a storage owner, -1 = none
    std::vector<int> emit_at;                   // for a GEMM / attention head: the node whose visit emits it
    std::vector<View> views;
    std::vector<char> view_done;
    LaunchPlan plan;
    struct Kernel {
        PlanRecord rec;
        std::string name, note;
    };
    std::vector<Kernel> kernels;

    Planner(const Function& fn, const LoweringOptions& o) : f(fn), opts(o) {}

    // ---- extraction -------------------------------------------------------------------------------------
    static Dims static_shape(const Value& v, DType* dt) {
        auto t = v.as_tensor();
        if (!t) throw Fail(CG_B200_ERR_UNSUPPORTED, "non-tensor value");
        Dims s;
        for (const auto& d : t->shape) {
            if (!d->is_constant()) throw Fail(CG_B200_ERR_UNSUPPORTED, "symbolic shapes have no B200 kernel");
            s.push_back(d->value);
        }
        *dt = t->dtype;
        return s;
    }

    void extract() {
        nodes.emplace_back();
        for (const Value& a : f.args()) {
            Node n;
            n.op = OP_INPUT;
            n.shape = static_shape(a, &n.dtype);
            node_of[a.id()] = static_cast<int>(nodes.size());
            nodes.push_back(std::move(n));
        }
        for (const Operation& op : *f.entry()) {
            if (op.opcode == OP_FUSE || op.attributes.has("fused_chain") || op.attributes.has("fused_with"))
                throw Fail(CG_B200_ERR_FUSED_IR,
                           "IR carries fusion markers (fused_chain / fused_with / fuse op): the producer chain is lost, "
                           "lower pre-fusion IR");
            if (op.opcode == OP_RETURN || op.opcode == OP_ALLOC || op.opcode == OP_FREE || op.opcode == OP_REUSE) continue;
            Node n;
            n.op = op.opcode;
            n.src = &op;
            for (const Value& v : op.operands) {
                auto it = node_of.find(v.id());
                if (it == node_of.end()) throw Fail(CG_B200_ERR_UNSUPPORTED, "operand defined outside the function body");
                n.in.push_back(it->second);
            }
            if (op.opcode == OP_OUTPUT) {
                if (n.in.size() != 1) throw Fail(CG_B200_ERR_UNSUPPORTED, "output takes one value");
            } else {
                if (op.results.size() != 1) throw Fail(CG_B200_ERR_UNSUPPORTED, "ops with several results have no B200 kernel");
                n.shape = static_shape(op.results[0], &n.dtype);
                node_of[op.results[0].id()] = static_cast<int>(nodes.size());
            }
            nodes.push_back(std::move(n));
        }
        const usize n = nodes.size();
        uses.assign(n, 0);
        single_user.assign(n, 0);
        root.assign(n, 0);
        absorbed.assign(n, 0);
        buffer_of.assign(n, -1);
        emit_at.assign(n, 0);
        views.assign(n, View{});
        view_done.assign(n, 0);
    }

    // ---- views --------------------------------------------------------------------------------------------
    const View& view(int id) {
        if (view_done[id]) return views[id];
        const Node& nd = nodes[id];
        View v;
        if (!is_view(nd.op)) {
            v.root = id;
            v.shape = nd.shape;
            v.stride = canonical_strides(nd.shape);
        } else {
            const View& in = view(nd.in[0]);
            switch (nd.op) {
                case OP_COPY: v = in; break;
                case OP_RESHAPE:
                    if (!reshape_view(in, nd.shape, v))
                        throw Fail(CG_B200_ERR_UNSUPPORTED, "reshape of a strided view would need a copy");
                    break;
                case OP_TRANSPOSE: {
                    auto perm = nd.src->attributes.get("perm");
                    if (!perm || perm->ints.size() != in.shape.size()) throw Fail(CG_B200_ERR_UNSUPPORTED, "transpose without a full perm");
                    v = in;
                    for (usize i = 0; i < perm->ints.size(); ++i) {
                        const i64 p = perm->ints[i];
                        if (p < 0 || p >= static_cast<i64>(in.shape.size())) throw Fail(CG_B200_ERR_INVALID_ARG, "transpose: bad perm");
                        v.shape[i] = in.shape[static_cast<usize>(p)];
                        v.stride[i] = in.stride[static_cast<usize>(p)];
                    }
                    break;
                }
                case OP_SLICE: {
                    auto b = nd.src->attributes.get("begins"), e = nd.src->attributes.get("ends");
                    if (!b || !e || b->ints.size() != in.shape.size() || e->ints.size() != in.shape.size())
                        throw Fail(CG_B200_ERR_UNSUPPORTED, "slice needs begins and ends for every axis");
                    v = in;
                    for (usize i = 0; i < in.shape.size(); ++i) {
                        if (b->ints[i] < 0 || e->ints[i] > in.shape[i] || b->ints[i] > e->ints[i])
                            throw Fail(CG_B200_ERR_INVALID_ARG, "slice out of range");
                        v.offset += b->ints[i] * in.stride[i];
                        v.shape[i] = e->ints[i] - b->ints[i];
                    }
                    break;
                }
                default: {   // OP_BROADCAST: right-aligned, stride 0 along broadcast axes
                    v.root = in.root;
                    v.offset = in.offset;
                    v.shape = nd.shape;
                    v.stride.assign(nd.shape.size(), 0);
                    const usize lead = nd.shape.size() - in.shape.size();
                    for (usize i = 0; i < in.shape.size(); ++i)
                        v.stride[lead + i] = in.shape[i] == 1 ? 0 : in.stride[i];
                }
            }
            if (v.shape != nd.shape) throw Fail(CG_B200_ERR_UNSUPPORTED, "view shape disagrees with the op's result type");
        }
        views[id] = std::move(v);
        view_done[id] = 1;
        return views[id];
    }
    int owner(int id) { return view(id).root; }
    // the whole of its owner's storage in the owner's own order (a reshape at most)
    bool plain(int id) {
        const View& v = view(id);
        return v.offset == 0 && contiguous(v) && count(v.shape) == count(nodes[v.root].shape);
    }

    bool scalar_const(int id, float* value) {
        const Node& nd = nodes[id];
        if (nd.op != OP_CONSTANT || count(nd.shape) != 1) return false;
        auto bytes = nd.src->attributes.get("bytes");
        if (!bytes || bytes->kind != AttrKind::String) return false;
        const std::string& b = bytes->str;
        if (nd.dtype == DType::F32 && b.size() >= 4) {
            std::memcpy(value, b.data(), 4);
            return true;
        }
        if ((nd.dtype == DType::BF16 || nd.dtype == DType::F16) && b.size() >= 2) {
            std::uint16_t h;
            std::memcpy(&h, b.data(), 2);
            std::uint32_t w;
            if (nd.dtype == DType::BF16) {
                w = static_cast<std::uint32_t>(h) << 16;
            } else {   // f16 -> f32 (normal numbers and zero; a scale factor is nothing else)
                const std::uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
                if (exp == 0 || exp == 31) return man == 0 && exp == 0 ? (*value = 0.0f, true) : false;
                w = sign | ((exp + 112) << 23) | (man << 13);
            }
            std::memcpy(value, &w, 4);
            return true;
        }
        return false;
    }

    void count_uses() {
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i) {
            if (is_view(nodes[i].op)) continue;   // a view's readers count at its owner
            for (int in : nodes[i].in) {
                const int s = owner(in);
                ++uses[s];
                single_user[s] = i;
            }
        }
        for (usize i = 1; i < nodes.size(); ++i)
            if (uses[i] != 1) single_user[i] = 0;
    }
    int next_user(int id) const { return single_user[id]; }

    int new_buffer(int id) {
        PlanBuffer b;
        b.dtype = abi_dtype(nodes[id].dtype);
        if (b.dtype < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "only f16 / bf16 / f32 tensors have B200 kernels");
        b.shape = nodes[id].shape;
        b.bytes = static_cast<u64>(count(nodes[id].shape)) * dtype_size(nodes[id].dtype);
        plan.buffers.push_back(std::move(b));
        return static_cast<int>(plan.buffers.size() - 1);
    }
    int buffer_for(int owner_id) {
        if (buffer_of[owner_id] < 0) buffer_of[owner_id] = new_buffer(owner_id);
        return buffer_of[owner_id];
    }
    // an operand that must be one contiguous block: buffer + element offset
    void contiguous_operand(int id, std::int32_t* buf, std::int64_t* off, const char* what) {
        const View& v = view(id);
        if (!contiguous(v)) throw Fail(CG_B200_ERR_UNSUPPORTED, std::string(what) + ": operand is a strided view (would need a copy)");
        *buf = buffer_for(v.root);
        *off = v.offset;
    }

    // ---- "merge heads": a [B, H, S, d] matmul result whose only reader is transpose [0,2,1,3] ------------------
    // The transpose node then owns the storage, in its own canonical [B, S, H, d] order, and the matmul
    // (GEMM or attention) writes into it through row / head / batch strides. Decided on the graph's
    // structure before any view is resolved, because every later view depends on who owns the memory.
    void adopt_merged_layouts() {
        std::vector<int> readers(nodes.size(), 0), last_reader(nodes.size(), 0);
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i)
            for (int in : nodes[i].in) {
                ++readers[static_cast<usize>(in)];
                last_reader[static_cast<usize>(in)] = i;
            }
        for (int p = 1; p < static_cast<int>(nodes.size()); ++p) {
            if (nodes[p].op != OP_MATMUL || nodes[p].shape.size() != 4 || readers[static_cast<usize>(p)] != 1) continue;
            const int t = last_reader[static_cast<usize>(p)];
            if (nodes[t].op != OP_TRANSPOSE) continue;
            auto perm = nodes[t].src->attributes.get("perm");
            if (!perm || perm->ints != std::vector<i64>{0, 2, 1, 3}) continue;
            View tv;
            tv.root = t;
            tv.shape = nodes[t].shape;
            tv.stride = canonical_strides(nodes[t].shape);
            View pv;
            pv.root = t;
            pv.shape = nodes[p].shape;   // [B, H, S, d] over [B, S, H, d]
            pv.stride = {tv.stride[0], tv.stride[2], tv.stride[1], tv.stride[3]};
            views[static_cast<usize>(t)] = std::move(tv);
            views[static_cast<usize>(p)] = std::move(pv);
            view_done[static_cast<usize>(t)] = view_done[static_cast<usize>(p)] = 1;
        }
    }

    // ---- batch dimensions of a matmul-like op --------------------------------------------------------------
    struct Batch {
        i64 n_out = 1, n_in = 1;                 // outer x inner GEMMs (one level: n_in == total, n_out == 1)
        i64 a_out = 0, a_in = 0, b_out = 0, b_in = 0, c_out = 0, c_in = 0;
        bool two = false;
    };
    // strides of `v` (whose last two axes are the matrix) along the output's batch axes; 0 = broadcast
    static Dims batch_strides(const View& v, usize out_batch_rank) {
        Dims st(out_batch_rank, 0);
        const usize own = v.shape.size() - 2;
        if (own > out_batch_rank) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul operand has more batch axes than the result");
        for (usize i = 0; i < own; ++i) st[out_batch_rank - own + i] = v.shape[i] == 1 ? 0 : v.stride[i];
        return st;
    }
    static Batch collapse(Dims sizes, Dims sa, Dims sb, Dims sc) {
        // drop size-1 axes, merge neighbours that step like one axis in all three operands
        Dims n, a, b, c;
        for (usize i = 0; i < sizes.size(); ++i) {
            if (sizes[i] == 1) continue;
            if (!n.empty() && a.back() == sa[i] * sizes[i] && b.back() == sb[i] * sizes[i] && c.back() == sc[i] * sizes[i]) {
                n.back() *= sizes[i];
                a.back() = sa[i];
                b.back() = sb[i];
                c.back() = sc[i];
            } else {
                n.push_back(sizes[i]);
                a.push_back(sa[i]);
                b.push_back(sb[i]);
                c.push_back(sc[i]);
            }
        }
        Batch r;
        if (n.size() > 2) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: more than two independent batch levels");
        if (n.size() == 1) {
            r.n_in = n[0];
            r.a_in = a[0]; r.b_in = b[0]; r.c_in = c[0];
        } else if (n.size() == 2) {
            r.two = true;
            r.n_out = n[0]; r.n_in = n[1];
            r.a_out = a[0]; r.b_out = b[0]; r.c_out = c[0];
            r.a_in = a[1]; r.b_in = b[1]; r.c_in = c[1];
        }
        return r;
    }

    // ---- gemm -----------------------------------------------------------------------------------------------
    struct Tail {
        std::vector<int> chain;   // the ops the epilogue absorbs, in order
        int last = 0, bias = 0, residual = 0;
        int epilogue = CG_B200_EPI_NONE;
        float alpha = 1.0f;
    };
    std::unordered_map<int, Tail> tails;   // matmul node -> what its epilogue absorbs

    int other_operand(int op_id, int cur) {
        const Node& n = nodes[op_id];
        return owner(n.in[0]) == cur ? n.in[1] : n.in[0];
    }

    void match_tail(int id) {
        const Node& mm = nodes[id];
        Tail t;
        t.last = id;
        // a tail op has the GEMM's shape and type and reads the running value as it is (no view in between)
        auto same = [&](int u) {
            if (nodes[u].shape != mm.shape || nodes[u].dtype != mm.dtype) return false;
            for (int in : nodes[u].in)
                if (owner(in) == t.last && in != t.last) return false;
            return true;
        };
        auto is_bias = [&](int o) {
            const View& v = view(o);
            const i64 N = mm.shape.back();
            return count(v.shape) == N && !v.shape.empty() && v.shape.back() == N && contiguous(v) && nodes[v.root].dtype == mm.dtype;
        };
        auto is_residual = [&](int o) { return nodes[o].shape == mm.shape && contiguous(view(o)) && nodes[owner(o)].dtype == mm.dtype; };
        int u = next_user(t.last);
        float sc = 0.0f;
        if (u && nodes[u].op == OP_MUL && same(u) && scalar_const(owner(other_operand(u, t.last)), &sc)) {
            t.epilogue = CG_B200_EPI_SCALE;
            t.alpha = sc;
            t.last = u;
            t.chain.push_back(u);
        } else if (u && (nodes[u].op == OP_RELU || nodes[u].op == OP_GELU) && same(u)) {
            t.epilogue = nodes[u].op == OP_RELU ? CG_B200_EPI_RELU : CG_B200_EPI_GELU_TANH;
            t.last = u;
            t.chain.push_back(u);
        } else if (u && nodes[u].op == OP_ADD && same(u)) {
            const int o = other_operand(u, t.last);
            if (is_bias(o)) {
                t.epilogue = CG_B200_EPI_BIAS;
                t.bias = o;
                t.last = u;
                t.chain.push_back(u);
                const int u2 = next_user(t.last);
                if (u2 && (nodes[u2].op == OP_RELU || nodes[u2].op == OP_GELU) && same(u2)) {
                    t.epilogue = nodes[u2].op == OP_RELU ? CG_B200_EPI_BIAS_RELU : CG_B200_EPI_BIAS_GELU_TANH;
                    t.last = u2;
                    t.chain.push_back(u2);
                } else if (u2 && nodes[u2].op == OP_ADD && same(u2)) {
                    const int o2 = other_operand(u2, t.last);
                    if (is_residual(o2)) {
                        t.epilogue = CG_B200_EPI_BIAS_RESIDUAL;
                        t.residual = o2;
                        t.last = u2;
                        t.chain.push_back(u2);
                    }
                }
            } else if (is_residual(o)) {
                t.epilogue = CG_B200_EPI_RESIDUAL;
                t.residual = o;
                t.last = u;
                t.chain.push_back(u);
            }
        }
        // the tail's ops live inside the GEMM; what it reads from elsewhere must be in memory by the time
        // the kernel runs, so those values are materialised by kernels of their own (never inlined)
        for (int w : t.chain) absorbed[w] = 1;
        if (t.last != id) absorbed[id] = 1;
        for (int o : {t.bias, t.residual})
            if (o && is_eltwise(nodes[owner(o)].op)) root[owner(o)] = 1;
        emit_at[id] = t.last;
        tails[id] = t;
    }

    void plan_gemm(int id) {
        const Node& mm = nodes[id];
        const Tail& t = tails.at(id);
        const View& a = view(mm.in[0]);
        const View& b = view(mm.in[1]);
        const int in_dt = abi_dtype(nodes[a.root].dtype);
        if (in_dt < 0 || nodes[a.root].dtype != nodes[b.root].dtype)
            throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: operand dtypes must be one of f16/bf16/f32 and equal");
        if (a.shape.size() < 2 || b.shape.size() < 2) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: rank < 2");
        const usize ra = a.shape.size(), rb = b.shape.size(), rc = mm.shape.size();
        i64 M = a.shape[ra - 2];
        const i64 K = a.shape[ra - 1], N = b.shape[rb - 1];
        if (b.shape[rb - 2] != K) throw Fail(CG_B200_ERR_INVALID_ARG, "matmul: inner dimensions differ");
        PlanRecord r;
        r.kind = PlanRecord::Gemm;
        cg_b200_gemm_desc& d = r.gemm;
        // A: K must be contiguous
        if (K != 1 && a.stride[ra - 1] != 1) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: A is not K-contiguous (transposed A)");
        d.lda = M == 1 ? K : a.stride[ra - 2];
        if (N == 1 || b.stride[rb - 1] == 1) {
            d.b_transposed = 0;
            d.ldb = K == 1 ? N : b.stride[rb - 2];
        } else if (K == 1 || b.stride[rb - 2] == 1) {
            d.b_transposed = 1;
            d.ldb = N == 1 ? K : b.stride[rb - 1];
        } else {
            throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: B has no contiguous axis");
        }
        // where the result goes: its own canonical storage, or the merged-heads layout of its reader
        const int out_node = t.last;
        const View& c = view(out_node);
        const usize nb = rc - 2;
        Dims sizes(mm.shape.begin(), mm.shape.begin() + static_cast<std::ptrdiff_t>(nb));
        Dims sa = batch_strides(a, nb), sb = batch_strides(b, nb);
        Dims sc(c.stride.begin(), c.stride.begin() + static_cast<std::ptrdiff_t>(nb));
        d.ldc = M == 1 ? N : c.stride[rc - 2];
        // rows of a batch that simply continue (A and C contiguous across the batch, B shared) are one taller matrix
        Batch bt = collapse(sizes, sa, sb, sc);
        if (!bt.two && bt.n_in > 1 && bt.b_in == 0 && bt.a_in == M * d.lda && bt.c_in == M * d.ldc) {
            M *= bt.n_in;
            bt = Batch{};
        }
        d.M = M; d.N = N; d.K = K;
        d.batch = bt.n_out * bt.n_in;
        if (bt.two) {
            d.batch_inner = bt.n_in;
            d.batch_stride_a = bt.a_out; d.batch_stride_b = bt.b_out; d.batch_stride_c = bt.c_out;
            d.inner_stride_a = bt.a_in; d.inner_stride_b = bt.b_in; d.inner_stride_c = bt.c_in;
        } else {
            d.batch_stride_a = bt.a_in; d.batch_stride_b = bt.b_in;
            d.batch_stride_c = d.batch > 1 ? bt.c_in : M * d.ldc;
        }
        d.in_dtype = in_dt;
        d.compute = CG_B200_COMPUTE_DEFAULT;
        d.epilogue = t.epilogue;
        d.alpha = t.alpha;
        const int out_dt = abi_dtype(nodes[out_node].dtype);
        if (out_dt < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: unsupported result dtype");
        d.out_dtype = out_dt;
        if (in_dt == CG_B200_F32 && bt.two) throw Fail(CG_B200_ERR_UNSUPPORTED, "matmul: fp32 operands take one batch level");
        r.input[0] = buffer_for(a.root); r.input_offset[0] = a.offset;
        r.input[1] = buffer_for(b.root); r.input_offset[1] = b.offset;
        r.n_inputs = 2;
        if (t.bias) contiguous_operand(t.bias, &r.input[2], &r.input_offset[2], "bias");
        if (t.residual) {
            // the residual is read with C's strides: it must be laid out like C
            const View& rv = view(t.residual);
            if (rv.stride != c.stride && !(contiguous(rv) && contiguous(c)))
                throw Fail(CG_B200_ERR_UNSUPPORTED, "residual is laid out differently from the result");
            r.input[3] = buffer_for(rv.root);
            r.input_offset[3] = rv.offset;
        }
        finish_kernel(out_node, r, "gemm",
                      "M=" + std::to_string(M) + " N=" + std::to_string(N) + " K=" + std::to_string(K) + " batch=" +
                          std::to_string(d.batch) + " epilogue=" + std::to_string(d.epilogue) + (d.b_transposed ? " B^T" : ""));
    }

    // ---- attention ----------------------------------------------------------------------------------------------
    struct Attn {
        int scores = 0, scale_op = 0, softmax = 0;
        float scale = 1.0f;
    };
    std::unordered_map<int, Attn> attns;   // second matmul -> the pattern it closes

    void match_attention(int s) {
        // s = matmul(q, k^T); reader chain: (mul by scalar)? -> softmax -> matmul(p, v) with p as operand 0
        if (nodes[s].op != OP_MATMUL || absorbed[s]) return;
        Attn at;
        at.scores = s;
        int cur = s;
        int u = next_user(cur);
        float sc = 1.0f;
        if (u && nodes[u].op == OP_MUL && nodes[u].shape == nodes[s].shape && scalar_const(owner(other_operand(u, cur)), &sc)) {
            at.scale_op = u;
            at.scale = sc;
            cur = u;
            u = next_user(cur);
        }
        if (!u || nodes[u].op != OP_SOFTMAX) return;
        at.softmax = u;
        const int o = next_user(u);
        if (!o || nodes[o].op != OP_MATMUL || owner(nodes[o].in[0]) != u || !plain(nodes[o].in[0])) return;
        const View& q = view(nodes[s].in[0]);
        const View& kt = view(nodes[s].in[1]);
        const View& v = view(nodes[o].in[1]);
        const usize r = q.shape.size();
        if (r < 2 || kt.shape.size() != r || v.shape.size() != r) return;
        const i64 dh = q.shape[r - 1];
        const DType dt = nodes[q.root].dtype;
        // the fused kernel: head_dim 64, 16-bit, positive scale; anything else stays three kernels
        if (dh != 64 || (dt != DType::BF16 && dt != DType::F16) || !(at.scale > 0.0f)) return;
        if (nodes[kt.root].dtype != dt || nodes[v.root].dtype != dt || nodes[o].dtype != dt) return;
        if (v.shape[r - 1] != dh || q.stride[r - 1] != 1 || kt.stride[r - 2] != 1 || v.stride[r - 1] != 1) return;
        absorbed[s] = 1;
        if (at.scale_op) absorbed[at.scale_op] = 1;
        absorbed[u] = 1;
        emit_at[s] = -1;   // never emitted on its own
        attns[o] = at;
    }

    void plan_attention(int o) {
        const Attn& at = attns.at(o);
        const View& q = view(nodes[at.scores].in[0]);
        const View& kt = view(nodes[at.scores].in[1]);
        const View& v = view(nodes[o].in[1]);
        const usize r = q.shape.size();
        PlanRecord rec;
        rec.kind = PlanRecord::Attention;
        cg_b200_attention_desc& d = rec.attention;
        d.dtype = abi_dtype(nodes[q.root].dtype);
        d.head_dim = 64;
        d.seq_q = q.shape[r - 2];
        d.seq_kv = v.shape[r - 2];
        d.ldq = q.stride[r - 2];
        d.ldk = kt.stride[r - 1];   // k^T is [.., d, S_kv]: a key row steps along its last axis
        d.ldv = v.stride[r - 2];
        d.scale = at.scale;
        const View& ov = view(o);   // canonical, or the merged-heads layout of its reader
        d.ldo = ov.stride[r - 2];
        // batch axes -> (batch, heads): K and V share strides per axis, so collapse q/k/o jointly and check v
        const usize nb = r - 2;
        Dims sizes(nodes[o].shape.begin(), nodes[o].shape.begin() + static_cast<std::ptrdiff_t>(nb));
        Dims sq = batch_strides(q, nb), sk = batch_strides(kt, nb), sv = batch_strides(v, nb);
        Dims so(ov.stride.begin(), ov.stride.begin() + static_cast<std::ptrdiff_t>(nb));
        Batch qk = collapse(sizes, sq, sk, so);
        Batch vv = collapse(sizes, sv, sv, so);
        if (qk.two != vv.two || qk.n_in != vv.n_in || qk.n_out != vv.n_out)
            throw Fail(CG_B200_ERR_UNSUPPORTED, "attention: Q/K and V split their batch axes differently");
        d.batch = qk.n_out;
        d.heads = qk.n_in;
        d.head_stride_q = qk.a_in; d.head_stride_k = qk.b_in; d.head_stride_v = vv.a_in; d.head_stride_o = qk.c_in;
        d.batch_stride_q = qk.a_out; d.batch_stride_k = qk.b_out; d.batch_stride_v = vv.a_out; d.batch_stride_o = qk.c_out;
        rec.input[0] = buffer_for(q.root); rec.input_offset[0] = q.offset;
        rec.input[1] = buffer_for(kt.root); rec.input_offset[1] = kt.offset;
        rec.input[2] = buffer_for(v.root); rec.input_offset[2] = v.offset;
        rec.n_inputs = 3;
        finish_kernel(o, rec, "attention",
                      "batch=" + std::to_string(d.batch) + " heads=" + std::to_string(d.heads) + " seq_q=" + std::to_string(d.seq_q) +
                          " seq_kv=" + std::to_string(d.seq_kv) + " head_dim=64");
    }

    // ---- row reductions --------------------------------------------------------------------------------------
    void plan_row(int id) {
        const Node& nd = nodes[id];
        if (absorbed[id]) return;
        PlanRecord r;
        const int dt = abi_dtype(nd.dtype);
        if (dt < 0 || nd.shape.empty()) throw Fail(CG_B200_ERR_UNSUPPORTED, "softmax/layernorm: unsupported type");
        r.row_dtype = dt;
        r.cols = nd.shape.back();
        r.rows = r.cols ? count(nd.shape) / r.cols : 0;
        r.eps = 1e-5f;   // the op carries no attribute (src/ir/ops.cpp:536-556); 1e-5 is what its benchmarks use
        r.n_inputs = 1;
        int last = id;
        if (nd.op == OP_SOFTMAX) {
            r.kind = PlanRecord::Softmax;
            const int u = next_user(id);
            if (u && nodes[u].op == OP_LAYERNORM && plain(nodes[u].in[0])) {
                r.kind = PlanRecord::SoftmaxLayerNorm;
                absorbed[u] = 1;
                absorbed[id] = 1;
                last = u;
            }
        } else {
            r.kind = PlanRecord::LayerNorm;
        }
        contiguous_operand(nd.in[0], &r.input[0], &r.input_offset[0], "row reduction");
        finish_kernel(last, r, r.kind == PlanRecord::Softmax ? "softmax" : (r.kind == PlanRecord::LayerNorm ? "layernorm" : "softmax_layernorm"),
                      "rows=" + std::to_string(r.rows) + " cols=" + std::to_string(r.cols));
    }

    // ---- reductions over axes --------------------------------------------------------------------------------
    // reduce_sum / reduce_max / reduce_mean (src/ir/ops.cpp:74-102, 417-436): `axes` (negative = from the end),
    // `keep_dims`. A run of adjacent axes of a contiguous operand is a [outer, reduce, inner] box and has a
    // kernel; anything else stays in the generic instruction stream only.
    void plan_reduce(int id) {
        const Node& nd = nodes[id];
        const Node& in = nodes[nd.in[0]];
        const int dt = abi_dtype(nd.dtype);
        auto axes = nd.src ? nd.src->attributes.get("axes") : nullptr;
        if (dt < 0 || !axes || axes->ints.empty()) throw Fail(CG_B200_ERR_UNSUPPORTED, "reduce: unsupported type or no axes");
        const i64 rank = static_cast<i64>(in.shape.size());
        std::vector<i64> ax;
        for (i64 a : axes->ints) {
            if (a < 0) a += rank;
            if (a < 0 || a >= rank) throw Fail(CG_B200_ERR_UNSUPPORTED, "reduce: axis out of range");
            if (std::find(ax.begin(), ax.end(), a) == ax.end()) ax.push_back(a);
        }
        std::sort(ax.begin(), ax.end());
        if (ax.back() - ax.front() + 1 != static_cast<i64>(ax.size()))
            throw Fail(CG_B200_ERR_UNSUPPORTED, "reduce: the reduced axes are not adjacent (no B200 kernel)");
        PlanRecord r;
        r.kind = PlanRecord::Reduce;
        r.row_dtype = dt;
        r.reduce_op = nd.op == OP_REDUCE_SUM ? CG_B200_REDUCE_SUM : (nd.op == OP_REDUCE_MAX ? CG_B200_REDUCE_MAX : CG_B200_REDUCE_MEAN);
        i64 outer = 1, red = 1, inner = 1;
        for (i64 i = 0; i < rank; ++i) (i < ax.front() ? outer : (i > ax.back() ? inner : red)) *= in.shape[static_cast<usize>(i)];
        if (red == 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "reduce: empty reduced extent");
        r.rows = outer;
        r.cols = red;
        r.n = static_cast<u64>(inner);
        r.n_inputs = 1;
        contiguous_operand(nd.in[0], &r.input[0], &r.input_offset[0], "reduce");
        finish_kernel(id, r, "reduce", "outer=" + std::to_string(outer) + " reduce=" + std::to_string(red) + " inner=" + std::to_string(inner));
    }

    // ---- elementwise trees ---------------------------------------------------------------------------------------
    struct EwBuild {
        cg_b200_eltwise_desc d{};
        std::vector<int> inputs;   // operand nodes (possibly views)
        i64 n = 0, inner = 0;
        const Dims* out_shape = nullptr;
    };
    std::vector<int> pending_roots;

    int classify(const EwBuild& b, const Dims& s, i64* inner) const {
        const i64 ne = count(s);
        if (ne == b.n && ne != 1) return CG_B200_BC_FULL;
        if (ne == 1) return CG_B200_BC_SCALAR;
        const Dims& os = *b.out_shape;
        Dims trimmed = s;
        while (trimmed.size() > 1 && trimmed.front() == 1) trimmed.erase(trimmed.begin());
        if (trimmed.size() <= os.size() && std::equal(trimmed.rbegin(), trimmed.rend(), os.rbegin())) {
            *inner = ne;
            return CG_B200_BC_ROW;   // trailing axes equal: a row vector of period ne
        }
        if (s.size() == os.size() && !s.empty() && s.back() == 1 && std::equal(s.begin(), s.end() - 1, os.begin())) {
            *inner = os.back();
            return CG_B200_BC_COL;   // [..., 1] against [..., C]
        }
        return -1;
    }

    bool can_inline(int id, int parent) {
        if (is_view(nodes[id].op)) {
            // a reshape of an inlinable value is still that value
            return nodes[id].op == OP_RESHAPE && plain(id) && can_inline(owner(id), parent) && count(nodes[id].shape) == count(nodes[parent].shape);
        }
        const Node& nd = nodes[id];
        return is_eltwise(nd.op) && !root[id] && !absorbed[id] && uses[id] == 1 && single_user[id] == parent &&
               count(nd.shape) == count(nodes[parent].shape) && nd.dtype == nodes[parent].dtype;
    }

    // Appends code that leaves the value of `id` on the stack; returns the stack depth it needs.
    // `reserve`: instructions the callers still have to append after this value.
    int gen(EwBuild& b, int id, int parent, bool is_root, int reserve = 0) {
        float imm = 0.0f;
        const int own = owner(id);
        if (!is_root && scalar_const(own, &imm)) {
            if (b.d.n_instr + 1 + reserve > CG_B200_EW_MAX_INSTR) throw Cut{};
            b.d.prog[b.d.n_instr++] = {CG_B200_EW_IMM, 0, imm};
            return 1;
        }
        if (is_root || can_inline(id, parent)) {
            const Node& nd = nodes[own];
            const int save_n = b.d.n_instr;
            const usize save_in = b.inputs.size();
            const i64 save_inner = b.inner;
            try {
                int depth;
                if (is_binary(nd.op)) {
                    const int da = gen(b, nd.in[0], own, false, reserve + 2);
                    const int db = gen(b, nd.in[1], own, false, reserve + 1);
                    depth = std::max(da, 1 + db);
                } else {
                    depth = gen(b, nd.in[0], own, false, reserve + 1);
                }
                if (depth > CG_B200_EW_MAX_STACK) throw Cut{};
                b.d.prog[b.d.n_instr++] = {ew_op(nd.op), 0, 0.0f};
                return depth;
            } catch (const Cut&) {
                if (is_root) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: a single op exceeds the kernel's limits");
                b.d.n_instr = save_n;
                b.inputs.resize(save_in);
                b.inner = save_inner;
                pending_roots.push_back(own);   // this subtree becomes a kernel of its own, read as an input
            }
        }
        // read from memory
        const View& v = view(id);
        if (nodes[v.root].dtype != nodes[parent].dtype) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: mixed operand dtypes");
        Dims as_stored = v.shape;
        if (!contiguous(v)) {
            // a pure broadcast of a whole tensor is indexed by the kernel itself
            bool bc = true;
            Dims src;
            i64 expect = 1;
            for (usize i = v.shape.size(); i-- > 0;) {
                if (v.stride[i] == 0 || v.shape[i] == 1) { src.insert(src.begin(), 1); continue; }
                if (v.stride[i] != expect) bc = false;
                expect *= v.shape[i];
                src.insert(src.begin(), v.shape[i]);
            }
            if (!bc) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: operand is a strided view (would need a copy)");
            as_stored = src;
        }
        i64 inner = 0;
        const int kind = classify(b, as_stored, &inner);
        if (kind < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: unsupported broadcast");
        if (kind == CG_B200_BC_ROW || kind == CG_B200_BC_COL) {
            if (b.inner != 0 && b.inner != inner) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: two broadcast periods in one chain");
            b.inner = inner;
        }
        int slot = -1;
        for (usize i = 0; i < b.inputs.size(); ++i)
            if (view(b.inputs[i]).root == v.root && view(b.inputs[i]).offset == v.offset && b.d.bcast[i] == kind) slot = static_cast<int>(i);
        if (slot < 0) {
            if (b.inputs.size() >= CG_B200_EW_MAX_INPUTS) throw Cut{};
            slot = static_cast<int>(b.inputs.size());
            b.inputs.push_back(id);
            b.d.bcast[slot] = kind;
        }
        if (b.d.n_instr + 1 + reserve > CG_B200_EW_MAX_INSTR) throw Cut{};
        b.d.prog[b.d.n_instr++] = {CG_B200_EW_INPUT, slot, 0.0f};
        return 1;
    }

    // A root may spill subtrees that exceed the ABI limits: those become roots of their own and are
    // emitted first (they only depend on earlier values).
    void emit_eltwise_root(int id) {
        const Node& nd = nodes[id];
        EwBuild b;
        const int dt = abi_dtype(nd.dtype);
        if (dt < 0) throw Fail(CG_B200_ERR_UNSUPPORTED, "elementwise: unsupported dtype");
        b.d.dtype = dt;
        b.d.round_each_op = dt != CG_B200_F32;   // every Tensor-IR op result is a tensor of that type
        b.n = count(nd.shape);
        b.out_shape = &nd.shape;
        pending_roots.clear();
        gen(b, id, id, true);
        b.d.inner = b.inner > 0 ? b.inner : 1;
        const std::vector<int> spill = pending_roots;
        for (int s : spill)
            if (!produced(s)) {
                root[s] = 1;
                emit_eltwise_root(s);
            }
        PlanRecord r;
        r.kind = PlanRecord::Eltwise;
        r.eltwise = b.d;
        r.n = static_cast<u64>(b.n);
        r.n_inputs = static_cast<std::int32_t>(b.inputs.size());
        for (usize i = 0; i < b.inputs.size(); ++i) {
            const View& v = view(b.inputs[i]);
            r.input[i] = buffer_for(v.root);
            r.input_offset[i] = v.offset;
        }
        finish_kernel(id, r, "eltwise", "n=" + std::to_string(b.n) + " instrs=" + std::to_string(b.d.n_instr));
    }

    std::vector<char> done;
    bool produced(int owner_id) const { return done[static_cast<usize>(owner_id)] != 0; }

    void finish_kernel(int at, PlanRecord r, const std::string& name, const std::string& note) {
        const View& v = view(at);   // canonical, or the merged-heads layout of its reader
        r.output = buffer_for(v.root);
        r.output_offset = v.offset;
        done[static_cast<usize>(at)] = 1;
        done[static_cast<usize>(v.root)] = 1;
        // every value a kernel reads must have been written by an earlier kernel or be an input
        for (int i = 0; i < CG_B200_EW_MAX_INPUTS; ++i)
            if (r.input[i] >= 0 && (static_cast<usize>(r.input[i]) >= buffer_ready.size() || !buffer_ready[static_cast<usize>(r.input[i])]))
                throw Fail(CG_B200_ERR_UNSUPPORTED, "internal: kernel '" + name + "' reads a buffer no earlier kernel writes");
        if (static_cast<usize>(r.output) >= buffer_ready.size()) buffer_ready.resize(static_cast<usize>(r.output) + 1, 0);
        buffer_ready[static_cast<usize>(r.output)] = 1;
        kernels.push_back({r, name, note});
    }
    std::vector<char> buffer_ready;

    LaunchPlan run() {
        extract();
        done.assign(nodes.size(), 0);
        adopt_merged_layouts();
        count_uses();
        // inputs and outputs first: fixed buffer numbering
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i)
            if (nodes[i].op == OP_INPUT) {
                buffer_for(i);
                done[static_cast<usize>(i)] = 1;
                ++plan.n_inputs;
            }
        buffer_ready.assign(plan.buffers.size(), 1);
        std::vector<int> outs;
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i)
            if (nodes[i].op == OP_OUTPUT) outs.push_back(i);
        // patterns that decide where values live, in dependency order
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i)
            if (nodes[i].op == OP_MATMUL) match_attention(i);
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i) {
            if (nodes[i].op != OP_MATMUL || emit_at[i] == -1) continue;
            if (attns.count(i)) {
                emit_at[i] = i;
                continue;
            }
            match_tail(i);
        }
        for (int o : outs) {
            const int src = nodes[o].in[0];
            if (!plain(src)) throw Fail(CG_B200_ERR_UNSUPPORTED, "output: a view cannot be an output (would need a copy)");
            const int s = owner(src);
            if (nodes[s].op == OP_INPUT || buffer_of[s] >= 0)
                throw Fail(CG_B200_ERR_UNSUPPORTED, "output: a value may be output once and must be computed");
            buffer_for(s);
            ++plan.n_outputs;
        }
        buffer_ready.resize(plan.buffers.size(), 0);
        // which elementwise ops are materialised: read by a non-elementwise op, read more than once, read
        // through a view or a broadcast, or an output
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i) {
            const Node& nd = nodes[i];
            if (!is_eltwise(nd.op) || absorbed[i]) continue;
            const int u = single_user[i];
            if (uses[i] != 1 || buffer_of[i] >= 0 || !is_eltwise(nodes[u].op) || absorbed[u] || count(nodes[u].shape) != count(nd.shape) ||
                nodes[u].dtype != nd.dtype)
                root[i] = 1;
            else {
                // read through a non-trivial view?
                for (int in : nodes[u].in)
                    if (owner(in) == i && !plain(in)) root[i] = 1;
            }
        }
        // kernels in program order. A GEMM is emitted where its absorbed tail ends, so that everything
        // the epilogue reads has been written by then.
        std::vector<std::vector<int>> emit_here(nodes.size());
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i)
            if (nodes[i].op == OP_MATMUL && emit_at[i] > 0) emit_here[static_cast<usize>(emit_at[i])].push_back(i);
        for (int i = 1; i < static_cast<int>(nodes.size()); ++i) {
            const Node& nd = nodes[i];
            for (int g : emit_here[static_cast<usize>(i)]) {
                if (attns.count(g)) plan_attention(g);
                else plan_gemm(g);
            }
            switch (nd.op) {
                case OP_INPUT: case OP_OUTPUT: case OP_MATMUL: break;
                case OP_CONSTANT: {
                    float v;
                    if (!scalar_const(i, &v)) throw Fail(CG_B200_ERR_UNSUPPORTED, "only scalar constants with a value are supported");
                    break;
                }
                case OP_SOFTMAX: case OP_LAYERNORM: plan_row(i); break;
                case OP_REDUCE_SUM: case OP_REDUCE_MAX: case OP_REDUCE_MEAN: plan_reduce(i); break;
                default:
                    if (is_view(nd.op)) break;
                    if (!is_eltwise(nd.op))
                        throw Fail(CG_B200_ERR_UNSUPPORTED, "op '" + op_name(nd.op) + "' has no B200 kernel");
                    if (absorbed[i] || !root[i] || produced(i)) break;
                    emit_eltwise_root(i);
            }
        }
        for (const Kernel& k : kernels) {
            plan.records.push_back(k.rec);
            if (k.rec.kind == PlanRecord::Gemm && k.rec.gemm.in_dtype == CG_B200_F32) {
                // the fp32 GEMM's scratch: hi and lo copies of A and B, K padded to 4 (cg_b200_gemm_workspace_bytes)
                const cg_b200_gemm_desc& g = k.rec.gemm;
                const i64 ldk = ((g.K > 0 ? g.K : 1) + 3) / 4 * 4;
                auto r64 = [](i64 x) { return (x + 63) / 64 * 64; };
                const i64 ab = (g.batch_stride_a == 0 || g.batch == 1) ? 1 : g.batch, bb = (g.batch_stride_b == 0 || g.batch == 1) ? 1 : g.batch;
                const u64 ws = static_cast<u64>(2 * (r64(ab * g.M * ldk) + r64(bb * g.N * ldk))) * 4;
                plan.workspace_bytes = std::max(plan.workspace_bytes, ws);
            }
        }
        return plan;
    }
};

std::string record_blob(const PlanRecord& r) { return std::string(reinterpret_cast<const char*>(&r), sizeof(PlanRecord)); }

void append_plan_nodes(const Function& f, const LoweringOptions& opts, const cg_b200_gemm_tuning& tuning, CGFunction& cf) {
    Planner p(f, opts);
    const LaunchPlan plan = p.run();
    if (p.kernels.empty()) return;
    std::vector<i64> buffer_bytes, buffer_dtypes;
    for (const PlanBuffer& b : plan.buffers) {
        buffer_bytes.push_back(static_cast<i64>(b.bytes));
        buffer_dtypes.push_back(static_cast<i64>(b.dtype));
    }
    for (usize k = 0; k < p.kernels.size(); ++k) {
        auto& ker = p.kernels[k];
        if (ker.rec.kind == PlanRecord::Gemm) ker.rec.tuning = tuning;
        CGInstruction inst;
        inst.opcode = (ker.rec.kind == PlanRecord::Gemm || ker.rec.kind == PlanRecord::Attention)
                          ? CGOpcode::FMA
                          : (ker.rec.kind == PlanRecord::Eltwise ? CGOpcode::Add : CGOpcode::Reduce);
        inst.attributes.set("b200.kernel", Attribute::make_string(ker.name));
        inst.attributes.set("b200.record", Attribute::make_string(record_blob(ker.rec)));
        if (k == 0) {
            inst.attributes.set("b200.buffer_bytes", Attribute::make_int_array(buffer_bytes));
            inst.attributes.set("b200.buffer_dtypes", Attribute::make_int_array(buffer_dtypes));
            for (usize i = 0; i < plan.buffers.size(); ++i)
                inst.attributes.set("b200.buffer_shape." + std::to_string(i), Attribute::make_int_array(plan.buffers[i].shape));
            inst.attributes.set("b200.n_inputs", Attribute::make_integer(plan.n_inputs));
            inst.attributes.set("b200.n_outputs", Attribute::make_integer(plan.n_outputs));
            inst.attributes.set("b200.workspace_bytes", Attribute::make_integer(static_cast<i64>(plan.workspace_bytes)));
        }
        inst.comment = ker.note;
        cf.emit(std::move(inst));
    }
}

}  // namespace

namespace b200 {
int last_lowering_status() { return t_status; }
const std::string& last_lowering_message() { return t_message; }

std::optional<cg_b200_gemm_tuning> gemm_tuning_from_schedule(const Schedule& s) {
    cg_b200_gemm_tuning t{};
    for (const Transform& x : s.transforms()) {
        if (x.kind != TransformKind::Tile) continue;
        if (x.dim == "m") {
            if (x.factor == 128) t.cta_pair = 1;
            else if (x.factor == 256) t.cta_pair = 2;
            else if (x.factor != 0) return std::nullopt;
        } else if (x.dim == "n") {
            if (x.factor == 64 || x.factor == 128 || x.factor == 256) t.tile_n = static_cast<int32_t>(x.factor);
            else if (x.factor != 0) return std::nullopt;
        }
    }
    if (t.cta_pair == 2 && t.tile_n == 64) return std::nullopt;   // a CTA pair's tile is 128 or 256 wide
    return t;
}

std::optional<cg_b200_gemm_desc> first_gemm_desc(const Module& m) {
    try {
        for (const auto& fn : m.functions()) {
            LoweringOptions opts;
            Planner p(*fn, opts);
            p.run();
            for (const auto& k : p.kernels)
                if (k.rec.kind == PlanRecord::Gemm) return k.rec.gemm;
        }
    } catch (const Fail&) {
    }
    return std::nullopt;
}
}  // namespace b200

void TensorToCodegenLowering::lower_function(const Function& f, CGFunction& out, const Schedule& schedule) {
    // the generic stream first, produced by the reference's own lowering
    b200::legacy_lower_function(opts_, f, out, schedule);
    const std::optional<cg_b200_gemm_tuning> tuning = b200::gemm_tuning_from_schedule(schedule);
    if (!tuning) {
        t_status = CG_B200_ERR_UNSUPPORTED;
        t_message = "schedule: the GEMM kernels have no such tile";
        return;
    }
    try {
        append_plan_nodes(f, opts_, *tuning, out);
    } catch (const Fail& e) {
        t_status = e.status;
        t_message = f.name() + ": " + e.what();
    } catch (const std::exception& e) {
        t_status = CG_B200_ERR_INVALID_ARG;
        t_message = f.name() + ": " + e.what();
    }
}

CGModule TensorToCodegenLowering::lower(const Module& m, const Schedule& schedule) {
    t_status = CG_B200_OK;
    t_message.clear();
    CGModule out;
    for (const auto& f : m.functions()) {
        CGFunction& cf = out.create_function(f->name());
        lower_function(*f, cf, schedule);
    }
    return out;
}

}  // namespace cg
