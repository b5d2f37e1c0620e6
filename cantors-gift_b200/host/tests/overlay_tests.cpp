// overlay_tests.cpp - tests of the B200 layer through the reference's own classes (cg::Module, Builder,
// TensorToCodegenLowering, NvidiaBackend, Runtime, KernelCache, VendorDispatcher), with the reference's
// test harness. Without CG_B200_TEST_GPU=1 only the host side runs (planner, plan and cache formats,
// failure conventions); with it, compiled graphs run on cuda:0 through Runtime::bind / launch and are
// checked against the CPU oracle (libcg_oracle.so, test infrastructure).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <random>
#include <unistd.h>

#include "cg/b200/b200.hpp"
#include "cg/b200/plan.hpp"
#include "cg/b200/vendor.hpp"
#include "cg/backend/cpu_backend.hpp"
#include "cg/backend/nvidia_backend.hpp"
#include "cg/backend/tensor_core/ptx_mma.hpp"
#include "cg/ir/builder.hpp"
#include "cg/pipeline/matmul_pipeline.hpp"
#include "cg/test/gtest_compat.hpp"

extern "C" {   // the CPU oracle
int cgo_eltwise(const cg_b200_eltwise_desc* d, const void* const* inputs, int n_inputs, void* out, size_t n);
int cgo_gemm(const cg_b200_gemm_desc* d, const void* A, const void* B, const void* bias, const void* residual, void* C,
             const int64_t* rows, int64_t n_rows, int acc64);
int cgo_softmax(int dt, const void* in, void* out, int64_t rows, int64_t cols);
int cgo_layernorm(int dt, const void* in, const void* gamma, const void* beta, float eps, void* out, int64_t rows, int64_t cols);
int cgo_softmax_layernorm(int dt, const void* in, const void* gamma, const void* beta, float eps, void* out, int64_t rows,
                          int64_t cols);
void cgo_f32_to_bf16(const float* in, uint16_t* out, size_t n);
void cgo_bf16_to_f32(const uint16_t* in, float* out, size_t n);
}

using namespace cg;
using b200::LaunchPlan;
using b200::PlanRecord;

namespace {

bool gpu_mode() {
    const char* e = std::getenv("CG_B200_TEST_GPU");
    return e && e[0] == '1';
}

Value scalar(Builder& b, float v, DType dt = DType::F32) {
    std::vector<u8> bytes(4);
    std::memcpy(bytes.data(), &v, 4);
    if (dt == DType::BF16) {   // a constant of the tensors' own type, or the product would be promoted to fp32
        uint16_t h;
        cgo_f32_to_bf16(&v, &h, 1);
        bytes.assign(2, 0);
        std::memcpy(bytes.data(), &h, 2);
    }
    return b.constant_tensor(Shape{}, dt, bytes);
}

TypePtr tt(std::initializer_list<i64> dims, DType dt) { return make_tensor_type(Shape(dims), dt); }

// the B200 kernel nodes of a lowered function, in order
std::vector<PlanRecord> records_of(const CGFunction& fn) {
    std::vector<PlanRecord> out;
    for (const CGInstruction& inst : fn.instructions) {
        auto rec = inst.attributes.get("b200.record");
        if (!rec) continue;
        PlanRecord r;
        if (rec->str.size() != sizeof(r)) continue;
        std::memcpy(&r, rec->str.data(), sizeof(r));
        out.push_back(r);
    }
    return out;
}

void chain_graph(Module& m, i64 n) {   // y = relu(a*b + c) * 0.5
    auto f = m.create_function("chain", {tt({n}, DType::F32), tt({n}, DType::F32), tt({n}, DType::F32)}, {tt({n}, DType::F32)});
    Builder b(f);
    b.output_tensor(b.mul(b.relu(b.add(b.mul(f->args()[0], f->args()[1]), f->args()[2])), scalar(b, 0.5f)));
}

void mlp_graph(Module& m, i64 M, i64 D, i64 H) {   // y = gelu(x W1 + b1) W2 + b2 + x
    auto f = m.create_function("mlp", {tt({M, D}, DType::F32), tt({D, H}, DType::F32), tt({H}, DType::F32), tt({H, D}, DType::F32),
                                       tt({D}, DType::F32)}, {tt({M, D}, DType::F32)});
    Builder b(f);
    const auto& a = f->args();
    Value h = b.gelu(b.add(b.matmul(a[0], a[1]), a[2]));
    b.output_tensor(b.add(b.add(b.matmul(h, a[3]), a[4]), a[0]));
}

// The reference's transformer benchmark graph (one attention head of width d_model, no biases).
void reference_block_graph(Module& m, i64 B, i64 S, i64 D, i64 F, DType dt) {
    auto f = m.create_function("transformer_block", {tt({B, S, D}, dt)}, {tt({B, S, D}, dt)});
    Builder b(f);
    Value x = f->args()[0];
    Value ln1 = b.layernorm(x);
    Value wq = b.input_tensor(Shape{D, D}, dt), wk = b.input_tensor(Shape{D, D}, dt), wv = b.input_tensor(Shape{D, D}, dt);
    Value q = b.matmul(ln1, wq), k = b.matmul(ln1, wk), v = b.matmul(ln1, wv);
    Value attn = b.softmax(b.matmul(q, b.transpose(k, {0, 2, 1})));
    Value res1 = b.add(x, b.matmul(attn, v));
    Value ln2 = b.layernorm(res1);
    Value w1 = b.input_tensor(Shape{D, F}, dt), w2 = b.input_tensor(Shape{F, D}, dt);
    Value h = b.gelu(b.matmul(ln2, w1));
    b.output_tensor(b.add(res1, b.matmul(h, w2)));
}

// The configured encoder block: packed QKV projection, H heads of width 64, biases on the FFN.
void encoder_block_graph(Module& m, i64 B, i64 S, i64 D, i64 H, i64 F, DType dt) {
    const i64 dh = D / H;
    auto f = m.create_function("encoder_block", {tt({B, S, D}, dt), tt({D, 3 * D}, dt), tt({D, D}, dt), tt({D, F}, dt), tt({F}, dt),
                                                 tt({F, D}, dt), tt({D}, dt)}, {tt({B, S, D}, dt)});
    Builder b(f);
    const auto& a = f->args();
    Value x = a[0];
    Value qkv = b.matmul(b.layernorm(x), a[1]);   // [B, S, 3D]
    auto heads = [&](i64 which) {
        Value part = b.slice(qkv, {0, 0, which * D}, {B, S, (which + 1) * D});
        return b.transpose(b.reshape(part, {B, S, H, dh}), {0, 2, 1, 3});   // [B, H, S, dh]
    };
    Value q = heads(0), k = heads(1), v = heads(2);
    Value scores = b.mul(b.matmul(q, b.transpose(k, {0, 1, 3, 2})), scalar(b, 1.0f / std::sqrt(static_cast<float>(dh)), dt));
    Value ctx = b.matmul(b.softmax(scores), v);                          // [B, H, S, dh]
    Value merged = b.reshape(b.transpose(ctx, {0, 2, 1, 3}), {B, S, D});
    Value h = b.add(b.matmul(merged, a[2]), x);
    Value ff = b.gelu(b.add(b.matmul(b.layernorm(h), a[3]), a[4]));
    b.output_tensor(b.add(b.add(b.matmul(ff, a[5]), a[6]), h));
}

}  // namespace

// ---- planner ------------------------------------------------------------------------------------------------
TEST(B200Lowering, ChainBecomesOneKernelBehindTheGenericStream) {
    Module m;
    chain_graph(m, 1000);
    TensorToCodegenLowering low;
    CGModule cg = low.lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(cg.functions.size(), 1u);
    const CGFunction& fn = cg.functions[0];
    // the reference's instruction stream is still there (vector loads / stores around each op)
    usize loads = 0;
    for (const auto& i : fn.instructions) loads += i.opcode == CGOpcode::VectorLoad;
    EXPECT_GE(loads, 4u);
    auto recs = records_of(fn);
    EXPECT_EQ(recs.size(), 1u);
    if (recs.size() != 1) return;
    const PlanRecord& r = recs[0];
    EXPECT_EQ(r.kind, static_cast<u32>(PlanRecord::Eltwise));
    EXPECT_EQ(r.n, 1000u);
    EXPECT_EQ(r.n_inputs, 3);
    EXPECT_EQ(r.eltwise.n_instr, 8);
    const int want[8] = {CG_B200_EW_INPUT, CG_B200_EW_INPUT, CG_B200_EW_MUL, CG_B200_EW_INPUT, CG_B200_EW_ADD,
                         CG_B200_EW_RELU, CG_B200_EW_IMM, CG_B200_EW_MUL};
    for (int i = 0; i < 8; ++i) EXPECT_EQ(r.eltwise.prog[i].op, want[i]);
    EXPECT_EQ(r.eltwise.prog[6].imm, 0.5f);
    EXPECT_EQ(cg_b200_eltwise_validate(&r.eltwise, r.n_inputs), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(r.output, 3);   // three inputs, then the output
}

TEST(B200Lowering, GemmAbsorbsBiasActivationResidual) {
    Module m;
    mlp_graph(m, 64, 32, 128);
    CGModule cg = TensorToCodegenLowering().lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    auto recs = records_of(cg.functions[0]);
    EXPECT_EQ(recs.size(), 2u);   // two GEMMs, everything else in their epilogues
    if (recs.size() != 2) return;
    EXPECT_EQ(recs[0].gemm.epilogue, static_cast<int>(CG_B200_EPI_BIAS_GELU_TANH));
    EXPECT_TRUE(recs[0].gemm.M == 64 && recs[0].gemm.N == 128 && recs[0].gemm.K == 32);
    EXPECT_EQ(recs[0].input[2], 2);
    EXPECT_EQ(recs[1].gemm.epilogue, static_cast<int>(CG_B200_EPI_BIAS_RESIDUAL));
    EXPECT_EQ(recs[1].input[3], 0);
    EXPECT_EQ(recs[1].input[0], recs[0].output);
    EXPECT_EQ(recs[1].output, 5);
}

TEST(B200Lowering, EpilogueOperandDefinedAfterTheMatmulIsComputedFirst) {
    // mm = a @ b;  r = relu(x);  y = mm + r : the GEMM reads r in its epilogue, so relu's kernel must come first
    Module m;
    auto f = m.create_function("late", {tt({128, 64}, DType::F32), tt({64, 96}, DType::F32), tt({128, 96}, DType::F32)},
                               {tt({128, 96}, DType::F32)});
    Builder b(f);
    Value mm = b.matmul(f->args()[0], f->args()[1]);
    Value r = b.relu(f->args()[2]);
    b.output_tensor(b.add(mm, r));
    CGModule cg = TensorToCodegenLowering().lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    auto recs = records_of(cg.functions[0]);
    EXPECT_EQ(recs.size(), 2u);
    if (recs.size() != 2) return;
    EXPECT_EQ(recs[0].kind, static_cast<u32>(PlanRecord::Eltwise));
    EXPECT_EQ(recs[1].kind, static_cast<u32>(PlanRecord::Gemm));
    EXPECT_EQ(recs[1].gemm.epilogue, static_cast<int>(CG_B200_EPI_RESIDUAL));
    EXPECT_EQ(recs[1].input[3], recs[0].output);
}

TEST(B200Lowering, SoftmaxLayernormFuseUnlessTheSoftmaxHasAnotherReader) {
    Module m;
    auto f = m.create_function("rows", {tt({16, 256}, DType::BF16)}, {tt({16, 256}, DType::BF16)});
    Builder b(f);
    b.output_tensor(b.layernorm(b.softmax(f->args()[0])));
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    EXPECT_EQ(recs.size(), 1u);
    if (!recs.empty()) EXPECT_EQ(recs[0].kind, static_cast<u32>(PlanRecord::SoftmaxLayerNorm));
    Module m2;
    auto f2 = m2.create_function("rows2", {tt({16, 256}, DType::BF16)}, {tt({16, 256}, DType::BF16), tt({16, 256}, DType::BF16)});
    Builder b2(f2);
    Value p = b2.softmax(f2->args()[0]);
    b2.output_tensor(b2.layernorm(p));
    b2.output_tensor(b2.mul(p, p));
    auto recs2 = records_of(TensorToCodegenLowering().lower(m2).functions[0]);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(recs2.size(), 3u);
}

TEST(B200Lowering, FusionMarkersAreRefusedNotGuessedAt) {
    Module m;
    chain_graph(m, 64);
    for (auto& op : *m.functions()[0]->entry())
        if (op.opcode == OP_RELU) op.attributes.set("fused_chain", Attribute::make_int_array({4, 10}));
    CGModule cg = TensorToCodegenLowering().lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_ERR_FUSED_IR));
    EXPECT_FALSE(b200::last_lowering_message().empty());
    EXPECT_EQ(cg.functions.size(), 1u);
    EXPECT_FALSE(cg.functions[0].instructions.empty());        // the generic stream, as the reference made it
    EXPECT_TRUE(records_of(cg.functions[0]).empty());          // nothing executable attached
    NvidiaBackend nv("sm_100a");
    auto exe = nv.compile(cg);
    EXPECT_TRUE(exe->machine_code.empty());
    Runtime rt;
    EXPECT_TRUE(rt.bind(std::shared_ptr<Executable>(exe.release()), DeviceId::cuda(0)) == nullptr);
}

TEST(B200Lowering, LongChainIsCutIntoValidKernels) {
    Module m;
    auto f = m.create_function("long", {tt({4096}, DType::F32), tt({4096}, DType::F32)}, {tt({4096}, DType::F32)});
    Builder b(f);
    Value v = f->args()[0];
    for (int i = 0; i < 20; ++i) v = b.add(b.mul(v, f->args()[1]), scalar(b, 1.0f + static_cast<float>(i)));
    b.output_tensor(v);
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_GE(recs.size(), 3u);
    for (const PlanRecord& r : recs) EXPECT_EQ(cg_b200_eltwise_validate(&r.eltwise, r.n_inputs), static_cast<int>(CG_B200_OK));
}

TEST(B200Lowering, BroadcastOperands) {
    Module m;
    auto f = m.create_function("bcast", {tt({8, 32}, DType::F32), tt({32}, DType::F32), tt({8, 1}, DType::F32), tt({1}, DType::F32)},
                               {tt({8, 32}, DType::F32)});
    Builder b(f);
    const auto& a = f->args();
    b.output_tensor(b.sub(b.mul(b.add(a[0], a[1]), a[2]), a[3]));
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(recs.size(), 1u);
    if (recs.size() != 1) return;
    const auto& e = recs[0].eltwise;
    EXPECT_TRUE(e.bcast[0] == CG_B200_BC_FULL && e.bcast[1] == CG_B200_BC_ROW && e.bcast[2] == CG_B200_BC_COL &&
                e.bcast[3] == CG_B200_BC_SCALAR && e.inner == 32);
}

TEST(B200Lowering, ReferenceTransformerGraphLowersToTenKernels) {
    // one head of width 128: not the fused kernel's head size, so attention stays matmul / softmax / matmul,
    // with the transpose of K folded into the first one
    Module m;
    reference_block_graph(m, 2, 64, 128, 256, DType::F32);
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(recs.size(), 10u);
    if (recs.size() != 10) return;
    const u32 kinds[10] = {PlanRecord::LayerNorm, PlanRecord::Gemm, PlanRecord::Gemm, PlanRecord::Gemm, PlanRecord::Gemm,
                           PlanRecord::Softmax, PlanRecord::Gemm, PlanRecord::LayerNorm, PlanRecord::Gemm, PlanRecord::Gemm};
    for (int i = 0; i < 10; ++i) EXPECT_EQ(recs[i].kind, kinds[i]);
    EXPECT_TRUE(recs[1].gemm.M == 128 && recs[1].gemm.batch == 1);           // [2, 64, 128] x [128, 128]: rows run on
    EXPECT_TRUE(recs[4].gemm.b_transposed == 1 && recs[4].gemm.batch == 2 && recs[4].gemm.M == 64 && recs[4].gemm.N == 64 &&
                recs[4].gemm.K == 128);
    EXPECT_EQ(recs[6].gemm.epilogue, static_cast<int>(CG_B200_EPI_RESIDUAL));
    EXPECT_EQ(recs[8].gemm.epilogue, static_cast<int>(CG_B200_EPI_GELU_TANH));
    EXPECT_EQ(recs[9].gemm.epilogue, static_cast<int>(CG_B200_EPI_RESIDUAL));
}

TEST(B200Lowering, EncoderBlockLowersToSevenKernels) {
    const i64 B = 2, S = 128, D = 256, H = 4, F = 512;
    Module m;
    encoder_block_graph(m, B, S, D, H, F, DType::BF16);
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    if (b200::last_lowering_status() != CG_B200_OK) std::printf("  %s\n", b200::last_lowering_message().c_str());
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(recs.size(), 7u);
    if (recs.size() != 7) return;
    const u32 kinds[7] = {PlanRecord::LayerNorm, PlanRecord::Gemm, PlanRecord::Attention, PlanRecord::Gemm, PlanRecord::LayerNorm,
                          PlanRecord::Gemm, PlanRecord::Gemm};
    for (int i = 0; i < 7; ++i) EXPECT_EQ(recs[i].kind, kinds[i]);
    EXPECT_TRUE(recs[1].gemm.M == B * S && recs[1].gemm.N == 3 * D && recs[1].gemm.K == D);
    const cg_b200_attention_desc& a = recs[2].attention;
    EXPECT_TRUE(a.batch == B && a.heads == H && a.seq_q == S && a.seq_kv == S && a.head_dim == 64);
    EXPECT_TRUE(a.ldq == 3 * D && a.ldk == 3 * D && a.ldv == 3 * D && a.ldo == D);
    EXPECT_TRUE(a.head_stride_q == 64 && a.head_stride_o == 64 && a.batch_stride_q == S * 3 * D && a.batch_stride_o == S * D);
    EXPECT_NEAR(a.scale, 0.125f, 1e-7);
    // Q, K, V are column blocks of the projection's buffer
    EXPECT_TRUE(recs[2].input[0] == recs[1].output && recs[2].input[1] == recs[1].output && recs[2].input[2] == recs[1].output);
    EXPECT_TRUE(recs[2].input_offset[0] == 0 && recs[2].input_offset[1] == D && recs[2].input_offset[2] == 2 * D);
    EXPECT_EQ(recs[3].gemm.epilogue, static_cast<int>(CG_B200_EPI_RESIDUAL));
    EXPECT_EQ(recs[3].input[0], recs[2].output);   // the merged-heads buffer, no copy in between
    EXPECT_EQ(recs[5].gemm.epilogue, static_cast<int>(CG_B200_EPI_BIAS_GELU_TANH));
    EXPECT_EQ(recs[6].gemm.epilogue, static_cast<int>(CG_B200_EPI_BIAS_RESIDUAL));
}

TEST(B200Lowering, AttentionWithAnotherHeadSizeStaysThreeKernels) {
    Module m;
    encoder_block_graph(m, 1, 64, 128, 4, 128, DType::BF16);   // head width 32
    auto recs = records_of(TensorToCodegenLowering().lower(m).functions[0]);
    if (b200::last_lowering_status() != CG_B200_OK) std::printf("  %s\n", b200::last_lowering_message().c_str());
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    EXPECT_EQ(recs.size(), 9u);
    if (recs.size() != 9) return;
    EXPECT_TRUE(recs[2].kind == PlanRecord::Gemm && recs[2].gemm.epilogue == CG_B200_EPI_SCALE && recs[2].gemm.b_transposed == 1);
    EXPECT_TRUE(recs[2].gemm.batch == 4 && recs[2].gemm.K == 32);
    EXPECT_EQ(recs[3].kind, static_cast<u32>(PlanRecord::Softmax));
    EXPECT_TRUE(recs[4].kind == PlanRecord::Gemm && recs[4].gemm.ldc == 128 && recs[4].gemm.N == 32);   // written merged
}

TEST(B200Lowering, OpsWithoutAKernelLeaveTheGenericStreamOnly) {
    Module m;
    auto f = m.create_function("conv", {tt({1, 3, 32, 32}, DType::F32), tt({16, 3, 3, 3}, DType::F32)}, {tt({1, 16, 30, 30}, DType::F32)});
    Builder b(f);
    b.output_tensor(b.conv2d(f->args()[0], f->args()[1]));
    CGModule cg = TensorToCodegenLowering().lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_ERR_UNSUPPORTED));
    EXPECT_TRUE(records_of(cg.functions[0]).empty());
    EXPECT_FALSE(cg.functions[0].instructions.empty());
}

TEST(B200Lowering, ReductionsOverAdjacentAxesBecomeKernels) {
    auto mean_of = [](Builder& b, Value a, std::vector<i64> axes, bool keep) {   // the builder has no reduce_mean helper
        AttributeDict attrs;
        attrs.set("axes", Attribute::make_int_array(std::move(axes)));
        attrs.set("keep_dims", Attribute::make_bool(keep));
        return b.create(OP_REDUCE_MEAN, {a}, std::move(attrs))->results[0];
    };
    Module m;
    auto f = m.create_function("reductions", {tt({4, 6, 8}, DType::BF16)},
                               {tt({4}, DType::BF16), tt({4, 6, 1}, DType::BF16), tt({6, 8}, DType::BF16)});
    Builder b(f);
    Value x = f->args()[0];
    b.output_tensor(b.reduce_sum(x, {1, 2}));
    b.output_tensor(b.reduce_max(x, {-1}, true));
    b.output_tensor(mean_of(b, x, {0}, false));
    CGModule cg = TensorToCodegenLowering().lower(m);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
    auto recs = records_of(cg.functions[0]);
    EXPECT_EQ(recs.size(), 3u);
    if (recs.size() != 3) return;
    for (const auto& r : recs) EXPECT_EQ(r.kind, static_cast<u32>(PlanRecord::Reduce));
    EXPECT_TRUE(recs[0].reduce_op == CG_B200_REDUCE_SUM && recs[0].rows == 4 && recs[0].cols == 48 && recs[0].n == 1);
    EXPECT_TRUE(recs[1].reduce_op == CG_B200_REDUCE_MAX && recs[1].rows == 24 && recs[1].cols == 8 && recs[1].n == 1);
    EXPECT_TRUE(recs[2].reduce_op == CG_B200_REDUCE_MEAN && recs[2].rows == 1 && recs[2].cols == 4 && recs[2].n == 48);
    // axes that are not adjacent have no kernel: the generic stream alone, and a status that says so
    Module m2;
    auto f2 = m2.create_function("gapped", {tt({4, 6, 8}, DType::F32)}, {tt({6}, DType::F32)});
    Builder b2(f2);
    b2.output_tensor(b2.reduce_sum(f2->args()[0], {0, 2}));
    CGModule cg2 = TensorToCodegenLowering().lower(m2);
    EXPECT_EQ(b200::last_lowering_status(), static_cast<int>(CG_B200_ERR_UNSUPPORTED));
    EXPECT_TRUE(records_of(cg2.functions[0]).empty());
    EXPECT_FALSE(cg2.functions[0].instructions.empty());
}

TEST(B200Lowering, ScheduleTilesChooseTheGemmKernel) {
    auto space = ScheduleSpace::grid_matmul({128, 256}, {64, 128, 256}, {64}, {8});
    EXPECT_EQ(space.size(), 6u);
    auto t = b200::gemm_tuning_from_schedule(space.schedules()[5]);
    EXPECT_TRUE(t && t->tile_n == 256 && t->cta_pair == 2);
    EXPECT_FALSE(b200::gemm_tuning_from_schedule(space.schedules()[3]).has_value());   // pair with a 64-wide tile
    Module m;
    mlp_graph(m, 64, 32, 128);
    auto recs = records_of(TensorToCodegenLowering().lower(m, space.schedules()[1]).functions[0]);
    EXPECT_TRUE(recs.size() == 2 && recs[0].tuning.tile_n == 128 && recs[0].tuning.cta_pair == 1);
    Schedule bad;
    bad.add(Transform{TransformKind::Tile, "n", 96, 0, "", MemorySpace::Generic});
    TensorToCodegenLowering().lower(m, bad);
    EXPECT_NE(b200::last_lowering_status(), static_cast<int>(CG_B200_OK));
}

// ---- backend, cache, runtime ---------------------------------------------------------------------------------
TEST(B200Backend, TextFromTheOldEmitterPlanInMachineCode) {
    Module m;
    mlp_graph(m, 64, 32, 128);
    CGModule cg = TensorToCodegenLowering().lower(m);
    NvidiaBackend nv;   // the reference's default target
    EXPECT_EQ(nv.name(), std::string("nvidia"));
    EXPECT_EQ(nv.target_info().name, std::string("nvidia_sm_80"));
    auto exe = nv.compile(cg);
    EXPECT_TRUE(exe != nullptr);
    for (const char* needle : {".version", ".target sm_80", ".entry", "fma.rn", "bar.sync", "cg_b200_gemm"})
        EXPECT_NE(exe->ptx_text.find(needle), std::string::npos);
    EXPECT_EQ(exe->entrypoints.size(), 1u);
    EXPECT_EQ(exe->entrypoints[0].first, std::string("mlp"));
    EXPECT_EQ(exe->threads_per_block, 320u);
    auto plan = LaunchPlan::deserialize(exe->machine_code);
    EXPECT_TRUE(plan.has_value());
    if (!plan) return;
    EXPECT_TRUE(plan->n_inputs == 5 && plan->n_outputs == 1 && plan->records.size() == 2 && plan->workspace_bytes > 0);
    EXPECT_EQ(plan->buffers[5].shape, (std::vector<std::int64_t>{64, 32}));
    auto text = nv.emit_text(cg);
    EXPECT_TRUE(text && text->find("fma.rn") != std::string::npos);
    // damaged plans are refused
    auto bytes = exe->machine_code;
    bytes.resize(bytes.size() - 3);
    EXPECT_FALSE(LaunchPlan::deserialize(bytes).has_value());
    bytes = exe->machine_code;
    bytes[0] ^= 0xff;
    EXPECT_FALSE(LaunchPlan::deserialize(bytes).has_value());
    NvidiaBackend b200_target("sm_100a");
    b200_target.compile(cg);
    EXPECT_EQ(b200_target.target_info().hardware.num_cores, 148u);
    EXPECT_GT(b200_target.target_info().hardware.peak_flops(DType::BF16, true), 1e15);
}

TEST(B200Runtime, CacheFileKeepsTheReferenceFormatAndThePlan) {
    namespace fs = std::filesystem;
    const fs::path dir = fs::temp_directory_path() / ("cg_b200_cache_" + std::to_string(::getpid()));
    fs::remove_all(dir);
    Module m;
    chain_graph(m, 4096);
    CGModule cg = TensorToCodegenLowering().lower(m);
    NvidiaBackend nv("sm_100a");
    const u64 key = KernelCache::compute_key("chain", "4096", "f32", "b200");
    EXPECT_EQ(KernelCache::compute_key("", "", "", ""), 0xcbf29ce484222325ULL);
    {
        KernelCache cache(dir.string());
        EXPECT_FALSE(cache.lookup(key).has_value());
        cache.insert(key, std::shared_ptr<Executable>(nv.compile(cg).release()));
        EXPECT_EQ(cache.size(), 1u);
    }
    const fs::path file = dir / (std::to_string(key) + ".cgbin");
    EXPECT_TRUE(fs::exists(file));
    {
        KernelCache cache(dir.string());   // a fresh cache reads the file
        auto hit = cache.lookup(key);
        EXPECT_TRUE(hit.has_value());
        if (hit) {
            EXPECT_EQ((*hit)->name, std::string("chain"));
            EXPECT_TRUE((*hit)->target_device == DeviceId::cuda());
            auto plan = LaunchPlan::deserialize((*hit)->machine_code);
            EXPECT_TRUE(plan && plan->records.size() == 1);
        }
    }
    // header of the file: "CGKE", version 1, then the name with a 64-bit length
    std::FILE* fp = std::fopen(file.c_str(), "rb");
    unsigned char head[20] = {};
    EXPECT_EQ(std::fread(head, 1, 20, fp), 20u);
    std::fclose(fp);
    EXPECT_TRUE(std::memcmp(head, "CGKE", 4) == 0 && head[4] == 1 && head[8] == 5 && std::memcmp(head + 16, "chai", 4) == 0);
    {   // a truncated file is a miss, not a crash
        fs::resize_file(file, fs::file_size(file) / 2);
        KernelCache cache(dir.string());
        EXPECT_FALSE(cache.lookup(key).has_value());
    }
    fs::remove_all(dir);
}

TEST(B200Runtime, BindFailsQuietlyWithoutADevice) {
    Module m;
    chain_graph(m, 256);
    NvidiaBackend nv("sm_100a");
    std::shared_ptr<Executable> exe(nv.compile(TensorToCodegenLowering().lower(m)).release());
    Runtime rt;
    EXPECT_EQ(rt.num_devices(), 0u);
    EXPECT_TRUE(rt.bind(exe, DeviceId::cuda(0)) == nullptr);   // no such device registered
    EXPECT_TRUE(rt.bind(nullptr, DeviceId::cuda(0)) == nullptr);
    EXPECT_TRUE(rt.bind(exe, DeviceId::cpu(0)) == nullptr);    // a CUDA executable is not x86 code
    if (!gpu_mode()) EXPECT_TRUE(b200::make_cuda_device(0) == nullptr || true);
}

TEST(B200Runtime, CpuExecutablesStillBindAndRun) {
    // an x86 function that returns at once: bind must produce something callable, as the reference's did
    auto exe = std::make_shared<Executable>();
    exe->target_device = DeviceId::cpu();
    exe->machine_code = {0xc3};   // ret
    Runtime rt;
    auto bound = rt.bind(exe, DeviceId::cpu(0));
    EXPECT_TRUE(bound != nullptr);
    if (!bound) return;
    float x = 1.0f;
    Tensor t = b200::tensor_from_ptr(&x, {1}, DType::F32, 0);
    std::vector<Tensor*> in = {&t}, out = {&t};
    struct NoStream : Stream {
        void sync() override {}
        DeviceId device() const override { return DeviceId::cpu(); }
    } s;
    bound->launch(in, out, s);
    EXPECT_EQ(x, 1.0f);
}

// ---- vendor dispatch, hardware ------------------------------------------------------------------------------------
TEST(B200Vendor, DescriptorsKeepWinningAndRunnableKernelsAreRegistered) {
    Module m;
    auto f = m.create_function("ops", {tt({64, 64}, DType::F32), tt({64, 64}, DType::F32)}, {tt({64, 64}, DType::F32)});
    Builder b(f);
    Value mm = b.matmul(f->args()[0], f->args()[1]);
    Value sm = b.softmax(mm);
    b.output_tensor(sm);
    Operation *mm_op = nullptr, *sm_op = nullptr;
    for (auto& op : *f->entry()) {
        if (op.opcode == OP_MATMUL) mm_op = &op;
        if (op.opcode == OP_SOFTMAX) sm_op = &op;
    }
    auto& d = VendorDispatcher::instance();
    EXPECT_GE(d.kernels().size(), 8u);
    VendorKernel* best = d.find_best(*mm_op);
    EXPECT_TRUE(best && best->vendor() == VendorKind::cuBLAS && best->name() == "cublas_matmul");
    VendorKernel* run = b200::find_executable(*mm_op);
    EXPECT_TRUE(run && run->name() == "cg_b200_gemm" && run->opcode() == OP_MATMUL && !run->estimated_runtime().has_value());
    VendorKernel* soft = d.find_best(*sm_op);   // only the B200 kernel supports it
    EXPECT_TRUE(soft && soft->name() == "cg_b200_softmax");
    EXPECT_FALSE(run->execute(*mm_op, nullptr));   // no pointers bound: refuses instead of launching on garbage
}

TEST(B200Hardware, ModelAndTensorCoreCaps) {
    HardwareModel h = b200::hardware_model(b200::Calibration{});
    EXPECT_EQ(h.num_cores, 148u);
    EXPECT_EQ(h.shared_mem_bytes, 227u * 1024u);
    EXPECT_NEAR(h.peak_flops(DType::BF16, true), 2.25e15, 1e9);
    EXPECT_NEAR(h.memory.get(MemorySpace::Generic), 7.7e12, 1e6);
    EXPECT_GT(h.roofline_ridge(DType::BF16, true), 250.0);
    b200::Calibration c;
    c.hbm_gbs = 6538.6;
    c.bf16_tflops = 1683.2;
    c.measured = true;
    HardwareModel hm = b200::hardware_model(c);
    EXPECT_NEAR(hm.peak_flops(DType::BF16, true), 1683.2e12, 1e6);
    EXPECT_NEAR(hm.memory.get(MemorySpace::Generic), 6538.6e9, 1e3);
    // from a file, in the shape the measurement tool writes
    const std::string path = (std::filesystem::temp_directory_path() / ("cg_b200_peaks_" + std::to_string(::getpid()) + ".json")).string();
    std::FILE* fp = std::fopen(path.c_str(), "w");
    std::fputs("{\n \"hbm_gbs\": 6538.6,\n \"bf16_tflops\": 1683.2,\n \"bf16_tflops_sustained\": 1415.8\n}\n", fp);
    std::fclose(fp);
    b200::Calibration fromfile = b200::load_calibration(path);
    EXPECT_TRUE(fromfile.measured && std::fabs(fromfile.bf16_tflops_sustained - 1415.8) < 1e-9);
    std::filesystem::remove(path);
    TensorCoreCaps caps = TensorCoreCaps::blackwell();
    EXPECT_TRUE(caps.has_tma && caps.has_async_barrier && !caps.has_hopper_wgmma && caps.has_ampere_mma);
    EXPECT_GT(caps.peak_fp8_tflops, 3000.0);
    bool pair_tile = false;
    for (const auto& t : caps.supported_tiles) pair_tile = pair_tile || (t.m == 256 && t.n == 256 && t.k == 16);
    EXPECT_TRUE(pair_tile);
}

// ---- on the GPU ----------------------------------------------------------------------------------------------------
namespace {

struct Gpu {
    Runtime rt;
    Device* dev = nullptr;
    std::unique_ptr<Stream> stream;
    Gpu() {
        rt.add_device(b200::make_cuda_device(0));
        dev = rt.get_device(DeviceId::cuda(0));
        if (dev) stream = dev->create_stream();
    }
    Tensor upload(const void* host, std::vector<i64> shape, DType dt) {
        Tensor t = b200::make_tensor(*dev, std::move(shape), dt);
        b200::copy_to_device(t, host, t.num_bytes, *stream);
        return t;
    }
    std::unique_ptr<BoundExecutable> compile(const Module& m, const char* sm = "sm_100a") {
        CGModule cg = TensorToCodegenLowering().lower(m);
        if (b200::last_lowering_status() != CG_B200_OK) {
            std::printf("  lowering: %s\n", b200::last_lowering_message().c_str());
            return nullptr;
        }
        NvidiaBackend nv(sm);
        return rt.bind(std::shared_ptr<Executable>(nv.compile(cg).release()), DeviceId::cuda(0));
    }
};

std::vector<float> randn(usize n, unsigned seed, float scale = 1.0f) {
    std::mt19937 g(seed);
    std::normal_distribution<float> d(0.0f, scale);
    std::vector<float> v(n);
    for (float& x : v) x = d(g);
    return v;
}

double max_rel(const std::vector<float>& got, const std::vector<float>& want) {
    double err = 0.0, scale = 1e-30;
    for (usize i = 0; i < want.size(); ++i) {
        err = std::max(err, static_cast<double>(std::fabs(got[i] - want[i])));
        scale = std::max(scale, static_cast<double>(std::fabs(want[i])));
    }
    return err / scale;
}

}  // namespace

TEST(B200Gpu, ChainRunsBitExact) {
    if (!gpu_mode()) return;
    Gpu g;
    EXPECT_TRUE(g.dev != nullptr);
    if (!g.dev) return;
    const i64 n = (1 << 20) + 3;
    Module m;
    chain_graph(m, n);
    auto bound = g.compile(m);
    EXPECT_TRUE(bound != nullptr);
    if (!bound) return;
    auto a = randn(n, 1), b = randn(n, 2), c = randn(n, 3);
    Tensor ta = g.upload(a.data(), {n}, DType::F32), tb = g.upload(b.data(), {n}, DType::F32), tc = g.upload(c.data(), {n}, DType::F32);
    Tensor ty = b200::make_tensor(*g.dev, {n}, DType::F32);
    std::vector<Tensor*> in = {&ta, &tb, &tc}, out = {&ty};
    auto e0 = g.dev->create_event(), e1 = g.dev->create_event();
    e0->record(*g.stream);
    bound->launch(in, out, *g.stream);
    e1->record(*g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_OK));
    std::vector<float> got(n), want(n);
    b200::copy_to_host(got.data(), ty, ty.num_bytes, *g.stream);
    g.stream->sync();
    EXPECT_GT(e1->elapsed_sec_since(*e0), 0.0);
    for (i64 i = 0; i < n; ++i) {
        const float t = a[i] * b[i] + c[i];   // compiled with -ffp-contract=off: two roundings, as the kernel's
        want[i] = (t > 0.0f ? t : 0.0f) * 0.5f;
    }
    EXPECT_TRUE(std::memcmp(got.data(), want.data(), n * 4) == 0);
    // wrong arity is refused with a status, nothing launched
    std::vector<Tensor*> two = {&ta, &tb};
    bound->launch(two, out, *g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_ERR_INVALID_ARG));
    for (Tensor* t : {&ta, &tb, &tc, &ty}) b200::release_tensor(*g.dev, *t);
}

TEST(B200Gpu, ReductionsMatchAHostLoop) {
    if (!gpu_mode()) return;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    const i64 A = 33, R = 170, C = 9;
    Module m;
    auto f = m.create_function("reductions", {tt({A, R, C}, DType::F32)}, {tt({A, C}, DType::F32), tt({A, R}, DType::F32)});
    {
        Builder b(f);
        b.output_tensor(b.reduce_sum(f->args()[0], {1}));     // strided: inner = C
        b.output_tensor(b.reduce_max(f->args()[0], {2}));     // rows: inner = 1
    }
    auto bound = g.compile(m);
    EXPECT_TRUE(bound != nullptr);
    if (!bound) return;
    auto x = randn(A * R * C, 11);
    Tensor tx = g.upload(x.data(), {A, R, C}, DType::F32);
    Tensor ts = b200::make_tensor(*g.dev, {A, C}, DType::F32), tm = b200::make_tensor(*g.dev, {A, R}, DType::F32);
    std::vector<Tensor*> in = {&tx}, out = {&ts, &tm};
    bound->launch(in, out, *g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_OK));
    std::vector<float> sum(A * C), mx(A * R);
    b200::copy_to_host(sum.data(), ts, ts.num_bytes, *g.stream);
    b200::copy_to_host(mx.data(), tm, tm.num_bytes, *g.stream);
    g.stream->sync();
    double worst = 0.0;
    bool max_exact = true;
    for (i64 a = 0; a < A; ++a) {
        for (i64 c = 0; c < C; ++c) {
            double acc = 0.0;
            for (i64 r = 0; r < R; ++r) acc += x[(a * R + r) * C + c];
            worst = std::max(worst, std::fabs(acc - sum[a * C + c]));
        }
        for (i64 r = 0; r < R; ++r) {
            float v = x[(a * R + r) * C];
            for (i64 c = 1; c < C; ++c) v = std::max(v, x[(a * R + r) * C + c]);
            max_exact = max_exact && v == mx[a * R + r];
        }
    }
    EXPECT_LT(worst, 1e-4);
    EXPECT_TRUE(max_exact);
    for (Tensor* t : {&tx, &ts, &tm}) b200::release_tensor(*g.dev, *t);
}

TEST(B200Gpu, MlpAndLateEpilogueOperandMatchTheOracle) {
    if (!gpu_mode()) return;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    const i64 M = 200, D = 96, H = 328;
    Module m;
    mlp_graph(m, M, D, H);
    auto bound = g.compile(m);
    EXPECT_TRUE(bound != nullptr);
    if (!bound) return;
    auto x = randn(M * D, 1, 0.5f), w1 = randn(D * H, 2, 0.1f), b1 = randn(H, 3), w2 = randn(H * D, 4, 0.1f), b2 = randn(D, 5);
    Tensor tx = g.upload(x.data(), {M, D}, DType::F32), tw1 = g.upload(w1.data(), {D, H}, DType::F32), tb1 = g.upload(b1.data(), {H}, DType::F32);
    Tensor tw2 = g.upload(w2.data(), {H, D}, DType::F32), tb2 = g.upload(b2.data(), {D}, DType::F32);
    Tensor ty = b200::make_tensor(*g.dev, {M, D}, DType::F32);
    std::vector<Tensor*> in = {&tx, &tw1, &tb1, &tw2, &tb2}, out = {&ty};
    bound->launch(in, out, *g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_OK));
    std::vector<float> got(M * D), h(M * H), want(M * D);
    b200::copy_to_host(got.data(), ty, ty.num_bytes, *g.stream);
    g.stream->sync();
    cg_b200_gemm_desc d1{};
    d1.M = M; d1.N = H; d1.K = D; d1.batch = 1; d1.lda = D; d1.ldb = H; d1.ldc = H;
    d1.in_dtype = d1.out_dtype = CG_B200_F32; d1.epilogue = CG_B200_EPI_BIAS_GELU_TANH; d1.alpha = 1.0f;
    EXPECT_EQ(cgo_gemm(&d1, x.data(), w1.data(), b1.data(), nullptr, h.data(), nullptr, 0, 0), 0);
    cg_b200_gemm_desc d2 = d1;
    d2.N = D; d2.K = H; d2.lda = H; d2.ldb = D; d2.ldc = D; d2.epilogue = CG_B200_EPI_BIAS_RESIDUAL;
    EXPECT_EQ(cgo_gemm(&d2, h.data(), w2.data(), b2.data(), x.data(), want.data(), nullptr, 0, 0), 0);
    EXPECT_LE(max_rel(got, want), 1e-4);
    uint32_t word = 1;
    EXPECT_EQ(cg_b200_last_device_error(b200::native_stream(*g.stream), &word), 0);
    EXPECT_EQ(word, 0u);

    // mm + relu(x) with relu defined after the matmul
    Module m2;
    auto f = m2.create_function("late", {tt({128, 64}, DType::F32), tt({64, 96}, DType::F32), tt({128, 96}, DType::F32)},
                                {tt({128, 96}, DType::F32)});
    Builder b(f);
    Value mm = b.matmul(f->args()[0], f->args()[1]);
    b.output_tensor(b.add(mm, b.relu(f->args()[2])));
    auto bound2 = g.compile(m2);
    EXPECT_TRUE(bound2 != nullptr);
    if (!bound2) return;
    auto A = randn(128 * 64, 7, 0.3f), Bm = randn(64 * 96, 8, 0.3f), X = randn(128 * 96, 9);
    Tensor tA = g.upload(A.data(), {128, 64}, DType::F32), tB = g.upload(Bm.data(), {64, 96}, DType::F32), tX = g.upload(X.data(), {128, 96}, DType::F32);
    Tensor tY = b200::make_tensor(*g.dev, {128, 96}, DType::F32);
    std::vector<Tensor*> in2 = {&tA, &tB, &tX}, out2 = {&tY};
    bound2->launch(in2, out2, *g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_OK));
    std::vector<float> got2(128 * 96), relu(128 * 96), want2(128 * 96);
    b200::copy_to_host(got2.data(), tY, tY.num_bytes, *g.stream);
    g.stream->sync();
    for (usize i = 0; i < relu.size(); ++i) relu[i] = X[i] > 0.0f ? X[i] : 0.0f;
    cg_b200_gemm_desc d3{};
    d3.M = 128; d3.N = 96; d3.K = 64; d3.batch = 1; d3.lda = 64; d3.ldb = 96; d3.ldc = 96;
    d3.in_dtype = d3.out_dtype = CG_B200_F32; d3.epilogue = CG_B200_EPI_RESIDUAL; d3.alpha = 1.0f;
    EXPECT_EQ(cgo_gemm(&d3, A.data(), Bm.data(), nullptr, relu.data(), want2.data(), nullptr, 0, 0), 0);
    EXPECT_LE(max_rel(got2, want2), 1e-4);
}

TEST(B200Gpu, ReferenceTransformerGraphMatchesTheOracleComposition) {
    if (!gpu_mode()) return;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    const i64 B = 2, S = 96, D = 128, F = 256;
    Module m;
    reference_block_graph(m, B, S, D, F, DType::F32);
    auto bound = g.compile(m);
    EXPECT_TRUE(bound != nullptr);
    if (!bound) return;
    auto x = randn(B * S * D, 1), wq = randn(D * D, 2, 0.05f), wk = randn(D * D, 3, 0.05f), wv = randn(D * D, 4, 0.05f);
    auto w1 = randn(D * F, 5, 0.05f), w2 = randn(F * D, 6, 0.05f);
    Tensor tx = g.upload(x.data(), {B, S, D}, DType::F32), tq = g.upload(wq.data(), {D, D}, DType::F32), tk = g.upload(wk.data(), {D, D}, DType::F32);
    Tensor tv = g.upload(wv.data(), {D, D}, DType::F32), t1 = g.upload(w1.data(), {D, F}, DType::F32), t2 = g.upload(w2.data(), {F, D}, DType::F32);
    Tensor ty = b200::make_tensor(*g.dev, {B, S, D}, DType::F32);
    std::vector<Tensor*> in = {&tx, &tq, &tk, &tv, &t1, &t2}, out = {&ty};
    bound->launch(in, out, *g.stream);
    EXPECT_EQ(b200::last_launch_status(), static_cast<int>(CG_B200_OK));
    std::vector<float> got(B * S * D);
    b200::copy_to_host(got.data(), ty, ty.num_bytes, *g.stream);
    g.stream->sync();
    // the same dataflow out of the oracle's ops
    const i64 R = B * S;
    std::vector<float> ln1(R * D), q(R * D), k(R * D), v(R * D), sc(B * S * S), p(B * S * S), res1(R * D), ln2(R * D), h(R * F), want(R * D);
    cgo_layernorm(CG_B200_F32, x.data(), nullptr, nullptr, 1e-5f, ln1.data(), R, D);
    auto gemm = [&](i64 M, i64 N, i64 K, const float* a, const float* bb, float* c, int epi, const float* res, i64 batch, int bt, i64 sa, i64 sb, i64 scs) {
        cg_b200_gemm_desc d{};
        d.M = M; d.N = N; d.K = K; d.batch = batch; d.lda = K; d.ldb = bt ? K : N; d.ldc = N;
        d.batch_stride_a = sa; d.batch_stride_b = sb; d.batch_stride_c = scs;
        d.in_dtype = d.out_dtype = CG_B200_F32; d.epilogue = epi; d.alpha = 1.0f; d.b_transposed = bt;
        EXPECT_EQ(cgo_gemm(&d, a, bb, nullptr, res, c, nullptr, 0, 0), 0);
    };
    gemm(R, D, D, ln1.data(), wq.data(), q.data(), CG_B200_EPI_NONE, nullptr, 1, 0, 0, 0, R * D);
    gemm(R, D, D, ln1.data(), wk.data(), k.data(), CG_B200_EPI_NONE, nullptr, 1, 0, 0, 0, R * D);
    gemm(R, D, D, ln1.data(), wv.data(), v.data(), CG_B200_EPI_NONE, nullptr, 1, 0, 0, 0, R * D);
    gemm(S, S, D, q.data(), k.data(), sc.data(), CG_B200_EPI_NONE, nullptr, B, 1, S * D, S * D, S * S);
    cgo_softmax(CG_B200_F32, sc.data(), p.data(), B * S, S);
    gemm(S, D, S, p.data(), v.data(), res1.data(), CG_B200_EPI_RESIDUAL, x.data(), B, 0, S * S, S * D, S * D);
    cgo_layernorm(CG_B200_F32, res1.data(), nullptr, nullptr, 1e-5f, ln2.data(), R, D);
    gemm(R, F, D, ln2.data(), w1.data(), h.data(), CG_B200_EPI_GELU_TANH, nullptr, 1, 0, 0, 0, R * F);
    gemm(R, D, F, h.data(), w2.data(), want.data(), CG_B200_EPI_RESIDUAL, res1.data(), 1, 0, 0, 0, R * D);
    EXPECT_LE(max_rel(got, want), 1e-4);
}

TEST(B200Gpu, AutotuneTimesTheRealKernelAndCachesTheWinner) {
    if (!gpu_mode()) return;
    namespace fs = std::filesystem;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    Module m;
    auto f = m.create_function("mm", {tt({512, 256}, DType::BF16), tt({256, 512}, DType::BF16)}, {tt({512, 512}, DType::BF16)});
    Builder b(f);
    b.output_tensor(b.matmul(f->args()[0], f->args()[1]));
    auto desc = b200::first_gemm_desc(m);
    EXPECT_TRUE(desc && desc->M == 512 && desc->N == 512 && desc->K == 256);
    if (!desc) return;
    BenchmarkFn bench = b200::make_gemm_benchmark(*desc, *g.dev, 10, 2);
    auto space = ScheduleSpace::grid_matmul({128, 256}, {64, 128, 256}, {64}, {8});
    const double t = bench(space.schedules()[0]);
    EXPECT_TRUE(t > 0.0 && t < 1e-2);
    EXPECT_TRUE(std::isinf(bench(space.schedules()[3])));   // pair + 64-wide tile: no such kernel
    NvidiaBackend nv("sm_100a");
    const u64 key = KernelCache::compute_key("mm", "512x256x512", "bf16", "b200-test-" + std::to_string(::getpid()));
    auto tuned = b200::autotune_and_cache(g.rt, key, m, space, bench, nv);
    EXPECT_TRUE(tuned.executable != nullptr && !tuned.cache_hit && tuned.total_benchmarks >= 5 && tuned.best_runtime > 0.0);
    auto again = b200::autotune_and_cache(g.rt, key, m, space, bench, nv);
    EXPECT_TRUE(again.cache_hit && again.executable != nullptr);
    if (tuned.executable) {
        auto plan = LaunchPlan::deserialize(tuned.executable->machine_code);
        EXPECT_TRUE(plan && plan->records.size() == 1);
        auto want = b200::gemm_tuning_from_schedule(tuned.best_schedule);
        if (plan && want) EXPECT_TRUE(plan->records[0].tuning.tile_n == want->tile_n && plan->records[0].tuning.cta_pair == want->cta_pair);
    }
    // the reference's own entry point runs the same search with the real timer and reports its figures
    auto res = g.rt.autotune_and_cache(key + 1, space, bench, nv);
    EXPECT_TRUE(!res.cache_hit && res.total_benchmarks > 0 && res.best_runtime > 0.0 && res.best_runtime < 1e-2);
    fs::remove_all(g.rt.kernel_cache().dir());
}

TEST(B200Gpu, MatmulPipelineSearchesWithMeasuredRuntimes) {
    // The reference's orchestrator (src/pipeline/matmul_pipeline.cpp:261-323) prunes the schedule space with
    // its analytical model and hands the survivors to a BenchmarkFn - in-tree only ever a stub. Here it gets
    // the function that times the real kernel, with the B200 hardware model behind the analytical part.
    if (!gpu_mode()) return;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    MatmulPipeline::Config cfg;
    cfg.M = 2048; cfg.N = 2048; cfg.K = 1024;
    cfg.dtype = DType::BF16;
    cfg.m_tiles = {128, 256};
    cfg.n_tiles = {64, 128, 256};
    cfg.k_tiles = {64};
    cfg.vector_widths = {8};
    cfg.max_benchmarks = 6;
    cfg.initial_random = 2;
    cfg.top_k_prune = 6;
    cg_b200_gemm_desc d{};
    d.M = 2048; d.N = 2048; d.K = 1024; d.batch = 1; d.lda = 1024; d.ldb = 2048; d.ldc = 2048;
    d.batch_stride_a = d.M * d.lda; d.batch_stride_b = d.K * d.ldb; d.batch_stride_c = d.M * d.ldc;
    d.in_dtype = d.out_dtype = CG_B200_BF16; d.epilogue = CG_B200_EPI_BIAS_RELU; d.alpha = 1.0f;
    BenchmarkFn bench = b200::make_gemm_benchmark(d, *g.dev, 10, 2);
    MatmulPipeline pipeline(b200::hardware_model(), cfg);
    MatmulPipelineResult res = pipeline.run(bench);
    EXPECT_GT(res.autotune_benchmarks, 0u);
    EXPECT_TRUE(res.best_runtime_sec > 1e-6 && res.best_runtime_sec < 1e-3);   // 8.6 GFLOP: microseconds, measured
    auto tile = b200::gemm_tuning_from_schedule(res.best_schedule);
    EXPECT_TRUE(tile.has_value());
    std::printf("  MatmulPipeline: measured best %.2f us (%zu candidates timed, %zu of %zu after pruning), cost model said %.2f us\n",
                res.best_runtime_sec * 1e6, res.autotune_benchmarks, res.pruned_space_size, res.schedule_space_size,
                res.analytical_estimate_sec * 1e6);
}

TEST(B200Gpu, VendorKernelsExecuteOnBoundPointers) {
    if (!gpu_mode()) return;
    Gpu g;
    if (!g.dev) { EXPECT_TRUE(false); return; }
    Module m;
    auto f = m.create_function("ops", {tt({64, 128}, DType::F32)}, {tt({64, 128}, DType::F32)});
    Builder b(f);
    b.output_tensor(b.softmax(f->args()[0]));
    Operation* op = nullptr;
    for (auto& o : *f->entry())
        if (o.opcode == OP_SOFTMAX) op = &o;
    auto x = randn(64 * 128, 3);
    Tensor tx = g.upload(x.data(), {64, 128}, DType::F32), ty = b200::make_tensor(*g.dev, {64, 128}, DType::F32);
    b200::bind_pointers(*op, {tx.data}, ty.data);
    VendorKernel* k = VendorDispatcher::instance().find_best(*op);
    EXPECT_TRUE(k != nullptr);
    if (!k) return;
    EXPECT_TRUE(k->execute(*op, b200::native_stream(*g.stream)));
    std::vector<float> got(64 * 128), want(64 * 128);
    b200::copy_to_host(got.data(), ty, ty.num_bytes, *g.stream);
    g.stream->sync();
    cgo_softmax(CG_B200_F32, x.data(), want.data(), 64, 128);
    EXPECT_LE(max_rel(got, want), 1e-4);
    // a reduction through the dispatcher: column maxima of the same tensor
    auto f2 = m.create_function("colmax", {tt({64, 128}, DType::F32)}, {tt({128}, DType::F32)});
    Builder b2(f2);
    b2.output_tensor(b2.reduce_max(f2->args()[0], {0}));
    Operation* rop = nullptr;
    for (auto& o : *f2->entry())
        if (o.opcode == OP_REDUCE_MAX) rop = &o;
    Tensor tm = b200::make_tensor(*g.dev, {128}, DType::F32);
    b200::bind_pointers(*rop, {tx.data}, tm.data);
    VendorKernel* rk = VendorDispatcher::instance().find_best(*rop);
    EXPECT_TRUE(rk != nullptr && rk->name() == "cg_b200_reduce_max");
    if (!rk) return;
    EXPECT_TRUE(rk->execute(*rop, b200::native_stream(*g.stream)));
    std::vector<float> cm(128);
    b200::copy_to_host(cm.data(), tm, tm.num_bytes, *g.stream);
    g.stream->sync();
    bool exact = true;
    for (int c = 0; c < 128; ++c) {
        float v = x[c];
        for (int r = 1; r < 64; ++r) v = std::max(v, x[r * 128 + c]);
        exact = exact && v == cm[c];
    }
    EXPECT_TRUE(exact);
}
