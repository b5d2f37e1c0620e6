// ir.cpp - dtype helpers and the Builder of the Tensor-IR stand-in.
// Shape rules follow the reference: right-aligned NumPy broadcast for elementwise ops
// (src/shape/inference.cpp:11-31), result dtype = promote(a, b) (include/cg/core/dtype.hpp:137-150),
// matmul [.., M, K] x [.., K, N] with broadcast batch dims (src/shape/inference.cpp:168-198),
// softmax / layernorm keep the input type (src/ir/ops.cpp:536-556).
#include <cstring>
#include <stdexcept>

#include "cg/b200_host.hpp"

namespace cg {

usize dtype_size(DType dt) {
    switch (dt) {
        case DType::BOOL: case DType::I8: case DType::U8: return 1;
        case DType::F16: case DType::BF16: case DType::I16: case DType::U16: return 2;
        case DType::F32: case DType::I32: case DType::U32: return 4;
        case DType::CF32: case DType::F64: case DType::I64: case DType::U64: case DType::INDEX: return 8;
        case DType::CF64: return 16;
    }
    return 0;
}

static bool is_float(DType dt) {
    return dt == DType::F16 || dt == DType::BF16 || dt == DType::F32 || dt == DType::F64 || dt == DType::CF32 ||
           dt == DType::CF64;
}
static bool is_signed(DType dt) {
    return is_float(dt) || dt == DType::I8 || dt == DType::I16 || dt == DType::I32 || dt == DType::I64 || dt == DType::INDEX;
}

DType promote(DType a, DType b) {
    if (a == b) return a;
    if (is_float(a) && !is_float(b)) return a;
    if (is_float(b) && !is_float(a)) return b;
    if (is_float(a) && is_float(b)) return dtype_size(a) >= dtype_size(b) ? a : b;
    if (dtype_size(a) != dtype_size(b)) return dtype_size(a) > dtype_size(b) ? a : b;
    return is_signed(a) ? a : b;
}

i64 num_elements(const Shape& s) {
    i64 n = 1;
    for (i64 d : s) n *= d;
    return n;
}

static Shape broadcast_shapes(const Shape& a, const Shape& b) {
    const usize r = a.size() > b.size() ? a.size() : b.size();
    Shape out(r, 1);
    for (usize i = 0; i < r; ++i) {
        const i64 da = i < r - a.size() ? 1 : a[i - (r - a.size())];
        const i64 db = i < r - b.size() ? 1 : b[i - (r - b.size())];
        if (da != db && da != 1 && db != 1) throw std::invalid_argument("elementwise: shapes do not broadcast");
        out[i] = da == 1 ? db : da;
    }
    return out;
}

Value Builder::emit(Operation op) {
    fn_->ops.push_back(std::move(op));
    return Value{static_cast<u32>(fn_->ops.size() - 1)};
}

Value Builder::input_tensor(Shape shape, DType dt) {
    Operation op;
    op.opcode = OP_INPUT;
    op.shape = std::move(shape);
    op.dtype = dt;
    return emit(std::move(op));
}

Value Builder::constant_tensor(Shape shape, DType dt, std::vector<u8> bytes) {
    Operation op;
    op.opcode = OP_CONSTANT;
    op.shape = std::move(shape);
    op.dtype = dt;
    op.constant_bytes = std::move(bytes);
    return emit(std::move(op));
}

Value Builder::constant_scalar(float v, DType dt) {
    std::vector<u8> bytes(sizeof(float));
    std::memcpy(bytes.data(), &v, sizeof(float));
    Operation op;
    op.opcode = OP_CONSTANT;
    op.dtype = dt;
    op.constant_bytes = std::move(bytes);
    op.attributes["value"] = static_cast<double>(v);
    return emit(std::move(op));
}

void Builder::output_tensor(Value v) {
    if (!v.valid()) throw std::invalid_argument("output: invalid value");
    Operation op;
    op.opcode = OP_OUTPUT;
    op.operands = {v};
    op.shape = fn_->def(v).shape;
    op.dtype = fn_->def(v).dtype;
    emit(std::move(op));
}

Value Builder::binary(Opcode opc, Value a, Value b) {
    if (!a.valid() || !b.valid()) throw std::invalid_argument("binary op: invalid operand");
    Operation op;
    op.opcode = opc;
    op.operands = {a, b};
    op.shape = broadcast_shapes(fn_->def(a).shape, fn_->def(b).shape);
    op.dtype = promote(fn_->def(a).dtype, fn_->def(b).dtype);
    return emit(std::move(op));
}

Value Builder::unary(Opcode opc, Value a) {
    if (!a.valid()) throw std::invalid_argument("unary op: invalid operand");
    Operation op;
    op.opcode = opc;
    op.operands = {a};
    op.shape = fn_->def(a).shape;
    op.dtype = fn_->def(a).dtype;
    return emit(std::move(op));
}

Value Builder::add(Value a, Value b) { return binary(OP_ADD, a, b); }
Value Builder::sub(Value a, Value b) { return binary(OP_SUB, a, b); }
Value Builder::mul(Value a, Value b) { return binary(OP_MUL, a, b); }
Value Builder::div(Value a, Value b) { return binary(OP_DIV, a, b); }
Value Builder::neg(Value a) { return unary(OP_NEG, a); }
Value Builder::relu(Value a) { return unary(OP_RELU, a); }
Value Builder::gelu(Value a) { return unary(OP_GELU, a); }
Value Builder::exp(Value a) { return unary(OP_EXP, a); }
Value Builder::sqrt(Value a) { return unary(OP_SQRT, a); }
Value Builder::sigmoid(Value a) { return unary(OP_SIGMOID, a); }
Value Builder::tanh(Value a) { return unary(OP_TANH, a); }
Value Builder::log(Value a) { return unary(OP_LOG, a); }
Value Builder::softmax(Value a) { return unary(OP_SOFTMAX, a); }
Value Builder::layernorm(Value a) { return unary(OP_LAYERNORM, a); }

Value Builder::matmul(Value a, Value b) {
    if (!a.valid() || !b.valid()) throw std::invalid_argument("matmul: invalid operand");
    const Shape& sa = fn_->def(a).shape;
    const Shape& sb = fn_->def(b).shape;
    if (sa.size() < 2 || sb.size() < 2) throw std::invalid_argument("matmul: rank must be >= 2");
    if (sa[sa.size() - 1] != sb[sb.size() - 2]) throw std::invalid_argument("matmul: inner dimensions differ");
    Shape batch = broadcast_shapes(Shape(sa.begin(), sa.end() - 2), Shape(sb.begin(), sb.end() - 2));
    batch.push_back(sa[sa.size() - 2]);
    batch.push_back(sb[sb.size() - 1]);
    Operation op;
    op.opcode = OP_MATMUL;
    op.operands = {a, b};
    op.shape = std::move(batch);
    op.dtype = promote(fn_->def(a).dtype, fn_->def(b).dtype);
    return emit(std::move(op));
}

Value Builder::reshape(Value a, std::vector<i64> target_shape) {
    if (!a.valid()) throw std::invalid_argument("reshape: invalid operand");
    if (num_elements(target_shape) != num_elements(fn_->def(a).shape))
        throw std::invalid_argument("reshape: element count differs");
    Operation op;
    op.opcode = OP_RESHAPE;
    op.operands = {a};
    op.shape = std::move(target_shape);
    op.dtype = fn_->def(a).dtype;
    return emit(std::move(op));
}

}  // namespace cg
