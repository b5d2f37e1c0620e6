// host_tests.cpp - tests of the C++ host layer. `host_tests cpu` needs no GPU (planner, plan and
// cache formats, failure conventions); `host_tests gpu` runs compiled graphs on cuda:0 through
// Runtime / BoundExecutable and checks them against the CPU oracle (libcg_oracle.so).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <random>
#include <string>
#include <unistd.h>
#include <vector>

#include "cg/b200_host.hpp"

extern "C" {   // the CPU oracle (test infrastructure)
int cgo_eltwise(const cg_b200_eltwise_desc* d, const void* const* inputs, int n_inputs, void* out, size_t n);
int cgo_gemm(const cg_b200_gemm_desc* d, const void* A, const void* B, const void* bias, const void* residual, void* C,
             const int64_t* rows, int64_t n_rows, int acc64);
void cgo_f32_to_bf16(const float* in, uint16_t* out, size_t n);
void cgo_bf16_to_f32(const uint16_t* in, float* out, size_t n);
int cgo_softmax_layernorm(int dt, const void* in, const void* gamma, const void* beta, float eps, void* out,
                          int64_t rows, int64_t cols);
}

using namespace cg;

static int g_failed = 0, g_checks = 0;
#define CHECK(cond)                                                                   \
    do {                                                                              \
        ++g_checks;                                                                   \
        if (!(cond)) { ++g_failed; std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

static PlanRecord record_of(const CGInstruction& inst) {
    PlanRecord r;
    const auto& blob = std::get<std::string>(inst.attributes.at("b200.record"));
    std::memcpy(&r, blob.data(), sizeof(r));
    return r;
}

static Module chain_module(i64 n) {   // y = relu(a*b + c) * 0.5
    Module m;
    Function& f = m.create_function("chain");
    Builder b(&f);
    Value a = b.input_tensor({n}, DType::F32), bb = b.input_tensor({n}, DType::F32), c = b.input_tensor({n}, DType::F32);
    b.output_tensor(b.mul(b.relu(b.add(b.mul(a, bb), c)), b.constant_scalar(0.5f, DType::F32)));
    return m;
}

static Module mlp_module(i64 M, i64 D, i64 H) {   // y = gelu(x W1 + b1) W2 + b2 + x
    Module m;
    Function& f = m.create_function("mlp");
    Builder b(&f);
    Value x = b.input_tensor({M, D}, DType::F32), w1 = b.input_tensor({D, H}, DType::F32), b1 = b.input_tensor({H}, DType::F32);
    Value w2 = b.input_tensor({H, D}, DType::F32), b2 = b.input_tensor({D}, DType::F32);
    Value h = b.gelu(b.add(b.matmul(x, w1), b1));
    b.output_tensor(b.add(b.add(b.matmul(h, w2), b2), x));
    return m;
}

static void test_planner() {
    TensorToCodegenLowering low;
    {
        CGModule cg = low.lower(chain_module(1000));
        CHECK(low.status() == CG_B200_OK);
        CHECK(cg.functions.size() == 1 && cg.functions[0].instructions.size() == 1);
        const CGInstruction& inst = cg.functions[0].instructions[0];
        CHECK(inst.opcode == CGOpcode::Add);
        CHECK(std::get<std::string>(inst.attributes.at("b200.kernel")) == "eltwise");
        PlanRecord r = record_of(inst);
        CHECK(r.kind == PlanRecord::Eltwise && r.n == 1000 && r.n_inputs == 3 && r.eltwise.n_instr == 8);
        const int want[8] = {CG_B200_EW_INPUT, CG_B200_EW_INPUT, CG_B200_EW_MUL, CG_B200_EW_INPUT, CG_B200_EW_ADD,
                             CG_B200_EW_RELU, CG_B200_EW_IMM, CG_B200_EW_MUL};
        for (int i = 0; i < 8; ++i) CHECK(r.eltwise.prog[i].op == want[i]);
        CHECK(r.eltwise.prog[6].imm == 0.5f);
        CHECK(cg_b200_eltwise_validate(&r.eltwise, r.n_inputs) == CG_B200_OK);
        CHECK(cg.functions[0].args.size() == 4);   // three inputs and the output
    }
    {
        CGModule cg = low.lower(mlp_module(64, 32, 128));
        CHECK(low.status() == CG_B200_OK);
        CHECK(cg.functions[0].instructions.size() == 2);   // two GEMMs, everything else in their epilogues
        PlanRecord g1 = record_of(cg.functions[0].instructions[0]), g2 = record_of(cg.functions[0].instructions[1]);
        CHECK(g1.kind == PlanRecord::Gemm && g1.gemm.epilogue == CG_B200_EPI_BIAS_GELU_TANH);
        CHECK(g1.gemm.M == 64 && g1.gemm.N == 128 && g1.gemm.K == 32 && g1.input[2] == 2);
        CHECK(g2.kind == PlanRecord::Gemm && g2.gemm.epilogue == CG_B200_EPI_BIAS_RESIDUAL && g2.input[3] == 0);
        CHECK(g2.input[0] == g1.output && g2.output == 5);   // 5 inputs, output is buffer 5
    }
    {   // layernorm(softmax(x)) fuses; a second reader of the softmax splits it
        Module m;
        Function& f = m.create_function("rows");
        Builder b(&f);
        Value x = b.input_tensor({16, 256}, DType::BF16);
        b.output_tensor(b.layernorm(b.softmax(x)));
        CGModule cg = low.lower(m);
        CHECK(cg.functions[0].instructions.size() == 1);
        CHECK(record_of(cg.functions[0].instructions[0]).kind == PlanRecord::SoftmaxLayerNorm);
        CHECK(cg.functions[0].instructions[0].opcode == CGOpcode::Reduce);
        Module m2;
        Function& f2 = m2.create_function("rows2");
        Builder b2(&f2);
        Value x2 = b2.input_tensor({16, 256}, DType::BF16);
        Value p = b2.softmax(x2);
        b2.output_tensor(b2.layernorm(p));
        b2.output_tensor(b2.mul(p, p));
        CGModule cg2 = low.lower(m2);
        CHECK(low.status() == CG_B200_OK && cg2.functions[0].instructions.size() == 3);
    }
    {   // the reference's lossy fusion markers are refused, never guessed at
        Module m = chain_module(64);
        m.functions[0].ops[4].attributes["fused_chain"] = std::vector<i64>{4, 10};
        CGModule cg = low.lower(m);
        CHECK(low.status() == CG_B200_ERR_FUSED_IR && cg.functions.empty() && !low.message().empty());
    }
    {   // a chain longer than the ABI allows is cut into several valid kernels
        Module m;
        Function& f = m.create_function("long");
        Builder b(&f);
        Value x = b.input_tensor({4096}, DType::F32), y = b.input_tensor({4096}, DType::F32);
        Value v = x;
        for (int i = 0; i < 20; ++i) v = b.add(b.mul(v, y), b.constant_scalar(1.0f + i, DType::F32));
        b.output_tensor(v);
        CGModule cg = low.lower(m);
        CHECK(low.status() == CG_B200_OK);
        CHECK(cg.functions.size() == 1 && cg.functions[0].instructions.size() >= 3);
        for (const CGInstruction& inst : cg.functions[0].instructions) {
            PlanRecord r = record_of(inst);
            CHECK(cg_b200_eltwise_validate(&r.eltwise, r.n_inputs) == CG_B200_OK);
        }
    }
    {   // broadcast operands: row vector, column vector, scalar tensor
        Module m;
        Function& f = m.create_function("bcast");
        Builder b(&f);
        Value x = b.input_tensor({8, 32}, DType::F32), r = b.input_tensor({32}, DType::F32);
        Value c = b.input_tensor({8, 1}, DType::F32), s = b.input_tensor({1}, DType::F32);
        b.output_tensor(b.sub(b.mul(b.add(x, r), c), s));
        CGModule cg = low.lower(m);
        CHECK(low.status() == CG_B200_OK && cg.functions[0].instructions.size() == 1);
        PlanRecord rec = record_of(cg.functions[0].instructions[0]);
        CHECK(rec.eltwise.bcast[0] == CG_B200_BC_FULL && rec.eltwise.bcast[1] == CG_B200_BC_ROW &&
              rec.eltwise.bcast[2] == CG_B200_BC_COL && rec.eltwise.bcast[3] == CG_B200_BC_SCALAR && rec.eltwise.inner == 32);
    }
    {   // type inference failures throw, as the reference's Builder::create does
        Module m;
        Function& f = m.create_function("bad");
        Builder b(&f);
        bool threw = false;
        try { b.matmul(b.input_tensor({4, 5}, DType::F32), b.input_tensor({6, 7}, DType::F32)); } catch (const std::invalid_argument&) { threw = true; }
        CHECK(threw);
    }
}

static void test_backend_and_cache() {
    TensorToCodegenLowering low;
    NvidiaBackend backend;   // default target sm_100a
    CHECK(backend.name() == "nvidia");
    CHECK(backend.target_info().device.kind == DeviceId::Kind::CUDA);
    CHECK(backend.target_info().hardware.peak_flops(DType::F16) > 0);
    CHECK(backend.target_info().hardware.num_sms == 148);
    CHECK(backend.target_info().supports_tensor_core(DType::BF16));
    CGModule cg = low.lower(mlp_module(64, 32, 128));
    auto exe = backend.compile(cg);
    CHECK(exe && exe->name == "mlp" && exe->entrypoints.size() == 1 && exe->entrypoints[0].first == "mlp");
    for (const char* tok : {".version", ".target sm_100a", ".entry mlp", "cg_b200_gemm"})
        CHECK(exe->ptx_text.find(tok) != std::string::npos);
    CHECK(backend.emit_text(cg)->find("mlp") != std::string::npos);
    CHECK(exe->threads_per_block == 320 && exe->shared_mem_bytes > 0);
    auto plan = LaunchPlan::deserialize(exe->machine_code);
    CHECK(plan && plan->n_inputs == 5 && plan->n_outputs == 1 && plan->records.size() == 2 && plan->buffers.size() == 7);
    CHECK(plan->workspace_bytes > 0);   // fp32 GEMMs need the split workspace
    CHECK(plan->serialize() == exe->machine_code);
    // damaged plans are refused
    std::vector<u8> bad = exe->machine_code;
    bad[0] ^= 0xff;
    CHECK(!LaunchPlan::deserialize(bad));
    bad = exe->machine_code;
    bad.pop_back();
    CHECK(!LaunchPlan::deserialize(bad));
    CHECK(!LaunchPlan::deserialize({}));
    // a module without fused nodes compiles to a listing with no plan: bind must refuse it
    CGModule plain;
    CGFunction& pf = plain.create_function("plain");
    CGInstruction fma;
    fma.opcode = CGOpcode::FMA;
    pf.emit(fma);
    auto pexe = backend.compile(plain);
    CHECK(pexe && pexe->machine_code.empty() && pexe->ptx_text.find(".entry plain") != std::string::npos);

    // KernelCache: FNV-1a key and the .cgbin round trip through a fresh cache object
    CHECK(KernelCache::compute_key("", "", "", "") == 0xcbf29ce484222325ULL);
    CHECK(KernelCache::compute_key("a", "", "", "") == 0xaf63dc4c8601ec8cULL);
    CHECK(KernelCache::compute_key("ab", "", "", "") == KernelCache::compute_key("a", "b", "", ""));
    namespace fs = std::filesystem;
    const fs::path dir = fs::temp_directory_path() / ("cg_b200_cache_test_" + std::to_string(::getpid()));
    fs::remove_all(dir);
    {
        Runtime rt(dir.string());
        CHECK(rt.num_devices() == 0);
        const u64 key = KernelCache::compute_key("mlp", "64x32x128", "f32", backend.target_info().name);
        auto r1 = rt.compile_and_cache(key, cg, backend);
        CHECK(r1.executable && !r1.cache_hit);
        auto r2 = rt.compile_and_cache(key, cg, backend);
        CHECK(r2.cache_hit && r2.executable == r1.executable);
        CHECK(fs::exists(dir / (std::to_string(key) + ".cgbin")));
        Runtime rt2(dir.string());   // cold memory cache: must come from disk
        auto hit = rt2.kernel_cache().lookup(key);
        CHECK(hit && (*hit)->machine_code == r1.executable->machine_code && (*hit)->ptx_text == r1.executable->ptx_text);
        CHECK(hit && (*hit)->entrypoints == r1.executable->entrypoints && (*hit)->threads_per_block == 320);
        CHECK(hit && (*hit)->target_device == DeviceId::cuda());
        CHECK(!rt2.kernel_cache().lookup(key + 1));
        // bind fails (null) without a registered device, and for a CPU device id
        CHECK(rt.bind(r1.executable, DeviceId::cuda(0)) == nullptr);
        CHECK(rt.bind(r1.executable, DeviceId::cpu(0)) == nullptr);
        CHECK(rt.bind(nullptr, DeviceId::cuda(0)) == nullptr);
    }
    fs::remove_all(dir);

    VendorDispatcher& vd = VendorDispatcher::instance();
    CHECK(vd.has_vendor("cublas") && vd.has_vendor("cg_b200") && !vd.has_vendor("rocblas"));
    Module m = mlp_module(64, 32, 128);
    const Function& f = m.functions[0];
    // find_best = minimum estimated runtime among supporting kernels, as in the reference: the
    // cuBLAS stub claims a constant 10 us, so the roofline estimate of cg_b200_gemm wins below that
    // and loses above it (only cg_b200 kernels can execute)
    for (const Operation& op : f.ops)
        if (op.opcode == OP_MATMUL) {
            const VendorKernel* k = vd.find_best(op, f);
            CHECK(k && k->name() == "cg_b200_gemm");
        }
    Operation big;
    big.opcode = OP_MATMUL;
    big.shape = {8192, 8192};
    big.dtype = DType::BF16;
    CHECK(vd.find_best(big, f) && vd.find_best(big, f)->vendor() == "cublas");
    Operation ln;
    ln.opcode = OP_LAYERNORM;
    ln.shape = {128, 1024};
    ln.dtype = DType::BF16;
    const VendorKernel* k = vd.find_best(ln, f);
    CHECK(k && k->name() == "cg_b200_layernorm");
}

// ---- schedules and the autotuner's interface (no GPU: the benchmark function is a table) ------------------
static void test_autotune_host_logic() {
    const ScheduleSpace space = ScheduleSpace::grid_matmul({128, 256}, {64, 128, 256}, {64}, {8});
    CHECK(space.size() == 6);
    CHECK(space.schedules()[0].transforms().size() == 8);   // as src/schedule/schedule.cpp:74-82 builds them
    CHECK(space.schedules()[0] == space.schedules()[0] && !(space.schedules()[0] == space.schedules()[1]));
    CHECK(space.schedules()[0].hash() != space.schedules()[1].hash());
    // tiles -> kernel variant
    auto t0 = gemm_tuning_from_schedule(space.schedules()[0]);   // m 128, n 64
    CHECK(t0 && t0->cta_pair == 1 && t0->tile_n == 64 && t0->tail_split == 0);
    auto t5 = gemm_tuning_from_schedule(space.schedules()[5]);   // m 256, n 256
    CHECK(t5 && t5->cta_pair == 2 && t5->tile_n == 256);
    CHECK(!gemm_tuning_from_schedule(space.schedules()[3]));     // m 256, n 64: no such kernel
    auto none = gemm_tuning_from_schedule(Schedule{});
    CHECK(none && none->cta_pair == 0 && none->tile_n == 0);     // empty schedule = the library's heuristic
    Schedule odd;
    odd.add({TransformKind::Tile, "n", 96, 0, ""});
    CHECK(!gemm_tuning_from_schedule(odd));
    // the search keeps the fastest candidate and skips those that cannot run
    const double inf = std::numeric_limits<double>::infinity();
    const double table[6] = {5e-6, 3e-6, 4e-6, inf, 2e-6, 2.5e-6};
    int calls = 0;
    BenchmarkFn fake = [&](const Schedule& s) {
        ++calls;
        for (usize i = 0; i < space.size(); ++i)
            if (space.schedules()[i] == s) return table[i];
        return inf;
    };
    const AutotuneResult r = bayesian_autotune(space, fake);
    CHECK(r.total_benchmarks == 6 && calls == 6 && r.runtime_history.size() == 6);
    CHECK(r.best_runtime == 2e-6 && r.best_schedule == space.schedules()[4]);
    CHECK(bayesian_autotune(space, fake, 2).total_benchmarks == 2);
    // Runtime::autotune_and_cache: the winner's tiles reach the plan record, and the second call is a cache hit
    const auto dir = std::filesystem::temp_directory_path() / "cg_b200_autotune_cache_test";
    std::filesystem::remove_all(dir);
    Runtime rt(dir.string());
    NvidiaBackend backend;
    TensorToCodegenLowering low;
    Module m;
    Function& f = m.create_function("mm");
    Builder b(&f);
    const Value a_in = b.input_tensor({512, 256}, DType::BF16);
    const Value b_in = b.input_tensor({256, 384}, DType::BF16);
    b.output_tensor(b.matmul(a_in, b_in));
    auto lower_best = [&](const Schedule& s) { return low.lower(m, s); };
    const u64 key = KernelCache::compute_key("mm", "512x384x256", "bf16", "b200-tuned");
    calls = 0;
    auto first = rt.autotune_and_cache(key, space, fake, backend, lower_best);
    CHECK(!first.cache_hit && first.executable && first.total_benchmarks == 6 && first.best_runtime == 2e-6);
    if (first.executable) {
        auto plan = LaunchPlan::deserialize(first.executable->machine_code);
        CHECK(plan && plan->records.size() == 1 && plan->records[0].kind == PlanRecord::Gemm);
        if (plan && !plan->records.empty()) CHECK(plan->records[0].tuning.cta_pair == 2 && plan->records[0].tuning.tile_n == 128);
    }
    auto second = rt.autotune_and_cache(key, space, fake, backend, lower_best);
    CHECK(second.cache_hit && second.executable && calls == 6);   // no further measurements
    if (second.executable) {
        auto plan = LaunchPlan::deserialize(second.executable->machine_code);
        CHECK(plan && plan->records.size() == 1 && plan->records[0].tuning.tile_n == 128);
    }
    // a schedule with a tile the kernels do not have is refused by the lowering
    CGModule bad = low.lower(m, odd);
    CHECK(low.status() == CG_B200_ERR_UNSUPPORTED && bad.functions.empty());
    std::filesystem::remove_all(dir);
}

static int run_cpu() {
    test_planner();
    test_backend_and_cache();
    test_autotune_host_logic();
    int count = -1;
    if (cg_b200_device_count(&count) != CG_B200_OK) CHECK(make_cuda_device(0) == nullptr);
    std::printf("host_tests cpu: %d checks, %d failed\n", g_checks, g_failed);
    return g_failed ? 1 : 0;
}

// ---- GPU: compiled graphs through Runtime -----------------------------------------------------------------
struct DevTensor {
    Tensor t;
    Device* dev;
    DevTensor(Device* d, Shape shape, DType dt) : dev(d) {
        t.shape = std::move(shape);
        t.dtype = dt;
        t.device = d->id();
        t.num_bytes = static_cast<u64>(num_elements(t.shape)) * dtype_size(dt);
        t.data = d->allocator().allocate(t.num_bytes ? t.num_bytes : 1);
        t.owns_memory = true;
    }
    ~DevTensor() { dev->allocator().deallocate(t.data); }
};

static std::vector<float> randn(usize n, unsigned seed, float scale = 1.0f) {
    std::mt19937 g(seed);
    std::normal_distribution<float> d(0.0f, scale);
    std::vector<float> v(n);
    for (float& x : v) x = d(g);
    return v;
}

static int run_gpu() {
    Runtime rt((std::filesystem::temp_directory_path() / "cg_b200_gpu_cache").string());
    rt.add_device(make_cuda_device(0));
    CHECK(rt.num_devices() == 1);
    if (rt.num_devices() != 1) { std::printf("no sm_100 device\n"); return 1; }
    Device* dev = rt.get_device(DeviceId::cuda(0));
    auto stream = dev->create_stream();
    TensorToCodegenLowering low;
    NvidiaBackend backend;

    {   // cfg2-shaped chain, bit-exact against the oracle
        const i64 n = (1 << 20) + 3;
        Module m = chain_module(n);
        CGModule cg = low.lower(m);
        auto res = rt.compile_and_cache(KernelCache::compute_key("chain", std::to_string(n), "f32", "b200"), cg, backend);
        auto bound = rt.bind(res.executable, DeviceId::cuda(0));
        CHECK(bound != nullptr);
        if (bound) {
            std::vector<float> a = randn(n, 1), b = randn(n, 2), c = randn(n, 3), y(n), want(n);
            DevTensor da(dev, {n}, DType::F32), db(dev, {n}, DType::F32), dc(dev, {n}, DType::F32), dy(dev, {n}, DType::F32);
            copy_to_device(da.t, a.data(), da.t.num_bytes, *stream);
            copy_to_device(db.t, b.data(), db.t.num_bytes, *stream);
            copy_to_device(dc.t, c.data(), dc.t.num_bytes, *stream);
            std::vector<Tensor*> in = {&da.t, &db.t, &dc.t}, out = {&dy.t};
            auto e0 = dev->create_event(), e1 = dev->create_event();
            e0->record(*stream);
            bound->launch(Span<Tensor*>(in), Span<Tensor*>(out), *stream);
            e1->record(*stream);
            CHECK(bound->status() == CG_B200_OK);
            copy_to_host(y.data(), dy.t, dy.t.num_bytes, *stream);
            stream->sync();
            e1->wait();
            CHECK(e1->elapsed_sec_since(*e0) > 0.0);
            PlanRecord r = record_of(cg.functions[0].instructions[0]);
            const void* ins[3] = {a.data(), b.data(), c.data()};
            cgo_eltwise(&r.eltwise, ins, 3, want.data(), n);
            CHECK(std::memcmp(y.data(), want.data(), n * sizeof(float)) == 0);
            // wrong argument counts are reported, not executed
            std::vector<Tensor*> short_in = {&da.t};
            bound->launch(Span<Tensor*>(short_in), Span<Tensor*>(out), *stream);
            CHECK(bound->status() == CG_B200_ERR_INVALID_ARG);
        }
    }
    {   // two fused GEMMs (bias+gelu, bias+residual), fp32 through the 3xTF32 path
        const i64 M = 200, D = 136, H = 264;
        Module m = mlp_module(M, D, H);
        CGModule cg = low.lower(m);
        auto exe = std::shared_ptr<Executable>(backend.compile(cg).release());
        auto bound = rt.bind(exe, DeviceId::cuda(0));
        CHECK(bound != nullptr);
        if (bound) {
            std::vector<float> x = randn(M * D, 4), w1 = randn(D * H, 5, 0.1f), b1 = randn(H, 6), w2 = randn(H * D, 7, 0.1f),
                               b2 = randn(D, 8), y(M * D), h(M * H), want(M * D);
            DevTensor dx(dev, {M, D}, DType::F32), dw1(dev, {D, H}, DType::F32), db1(dev, {H}, DType::F32),
                dw2(dev, {H, D}, DType::F32), db2(dev, {D}, DType::F32), dy(dev, {M, D}, DType::F32);
            copy_to_device(dx.t, x.data(), dx.t.num_bytes, *stream);
            copy_to_device(dw1.t, w1.data(), dw1.t.num_bytes, *stream);
            copy_to_device(db1.t, b1.data(), db1.t.num_bytes, *stream);
            copy_to_device(dw2.t, w2.data(), dw2.t.num_bytes, *stream);
            copy_to_device(db2.t, b2.data(), db2.t.num_bytes, *stream);
            std::vector<Tensor*> in = {&dx.t, &dw1.t, &db1.t, &dw2.t, &db2.t}, out = {&dy.t};
            bound->launch(Span<Tensor*>(in), Span<Tensor*>(out), *stream);
            CHECK(bound->status() == CG_B200_OK);
            copy_to_host(y.data(), dy.t, dy.t.num_bytes, *stream);
            stream->sync();
            PlanRecord g1 = record_of(cg.functions[0].instructions[0]), g2 = record_of(cg.functions[0].instructions[1]);
            cgo_gemm(&g1.gemm, x.data(), w1.data(), b1.data(), nullptr, h.data(), nullptr, 0, 0);
            cgo_gemm(&g2.gemm, h.data(), w2.data(), b2.data(), x.data(), want.data(), nullptr, 0, 0);
            double err = 0, scale = 0;
            for (usize i = 0; i < y.size(); ++i) {
                err = std::fmax(err, std::fabs(static_cast<double>(y[i]) - want[i]));
                scale = std::fmax(scale, std::fabs(static_cast<double>(want[i])));
            }
            std::printf("mlp max-normalised error %.3e\n", err / scale);
            CHECK(err <= 1e-4 * scale);   // fp32 bound of the path
            uint32_t word = 1;
            CHECK(cg_b200_last_device_error(nullptr, &word) == CG_B200_OK && word == 0);
        }
    }
    {   // fused row reduction, fp32
        const i64 R = 77, Ccols = 1000;
        Module m;
        Function& f = m.create_function("rows");
        Builder b(&f);
        b.output_tensor(b.layernorm(b.softmax(b.input_tensor({R, Ccols}, DType::F32))));
        CGModule cg = low.lower(m);
        auto bound = rt.bind(std::shared_ptr<Executable>(backend.compile(cg).release()), DeviceId::cuda(0));
        CHECK(bound != nullptr);
        if (bound) {
            std::vector<float> x = randn(R * Ccols, 9), y(R * Ccols), want(R * Ccols);
            DevTensor dx(dev, {R, Ccols}, DType::F32), dy(dev, {R, Ccols}, DType::F32);
            copy_to_device(dx.t, x.data(), dx.t.num_bytes, *stream);
            std::vector<Tensor*> in = {&dx.t}, out = {&dy.t};
            bound->launch(Span<Tensor*>(in), Span<Tensor*>(out), *stream);
            copy_to_host(y.data(), dy.t, dy.t.num_bytes, *stream);
            stream->sync();
            cgo_softmax_layernorm(CG_B200_F32, x.data(), nullptr, nullptr, 1e-5f, want.data(), R, Ccols);
            double err = 0, scale = 0;
            for (usize i = 0; i < y.size(); ++i) {
                err = std::fmax(err, std::fabs(static_cast<double>(y[i]) - want[i]));
                scale = std::fmax(scale, std::fabs(static_cast<double>(want[i])));
            }
            CHECK(err <= 1e-4 * scale);
        }
    }
    {   // the autotuner's benchmark function on the real kernel, then the tuned executable against the oracle
        const i64 M = 1024, N = 768, K = 512;
        Module m16;
        Function& f16 = m16.create_function("mm16");
        Builder b16(&f16);
        const Value a_in = b16.input_tensor({M, K}, DType::BF16);   // separate statements: argument evaluation
        const Value b_in = b16.input_tensor({K, N}, DType::BF16);   // order would otherwise pick the input order
        b16.output_tensor(b16.matmul(a_in, b_in));
        CGModule cg16 = low.lower(m16);
        CHECK(low.status() == CG_B200_OK);
        const PlanRecord rec = record_of(cg16.functions[0].instructions[0]);
        const ScheduleSpace space = ScheduleSpace::grid_matmul({128, 256}, {64, 128, 256}, {64}, {8});
        BenchmarkFn bench = make_gemm_benchmark(rec.gemm, *dev, 10, 2);
        int finite = 0;
        for (usize i = 0; i < space.size(); ++i) {
            const double t = bench(space.schedules()[i]);
            const bool runnable = gemm_tuning_from_schedule(space.schedules()[i]).has_value();
            CHECK(runnable == std::isfinite(t));
            if (std::isfinite(t)) {
                CHECK(t > 1e-7 && t < 1e-2);   // a 0.8 GFLOP GEMM: microseconds
                ++finite;
                std::printf("  tile m %lld n %lld: %.2f us\n", (long long)space.schedules()[i].transforms()[0].factor,
                            (long long)space.schedules()[i].transforms()[1].factor, t * 1e6);
            }
        }
        CHECK(finite == 5);
        const auto dir = std::filesystem::temp_directory_path() / "cg_b200_autotune_gpu_cache";
        std::filesystem::remove_all(dir);
        Runtime rt2(dir.string());
        rt2.add_device(make_cuda_device(0));
        auto tuned = rt2.autotune_and_cache(KernelCache::compute_key("mm16", "1024x768x512", "bf16", "b200-tuned"), space, bench,
                                            backend, [&](const Schedule& s) { return low.lower(m16, s); });
        CHECK(tuned.executable && !tuned.cache_hit && tuned.total_benchmarks == 6 && std::isfinite(tuned.best_runtime));
        auto bound = rt2.bind(tuned.executable, DeviceId::cuda(0));
        CHECK(bound != nullptr);
        if (bound) {
            // bf16 operands as raw 16-bit words; the oracle multiplies the same words
            std::vector<float> af = randn(M * K, 21), bf = randn(K * N, 22);
            std::vector<uint16_t> a16(M * K), b16w(K * N), y16(M * N), want16(M * N);
            cgo_f32_to_bf16(af.data(), a16.data(), M * K);
            cgo_f32_to_bf16(bf.data(), b16w.data(), K * N);
            DevTensor da(dev, {M, K}, DType::BF16), db(dev, {K, N}, DType::BF16), dy(dev, {M, N}, DType::BF16);
            copy_to_device(da.t, a16.data(), da.t.num_bytes, *stream);
            copy_to_device(db.t, b16w.data(), db.t.num_bytes, *stream);
            std::vector<Tensor*> in = {&da.t, &db.t}, out = {&dy.t};
            bound->launch(Span<Tensor*>(in), Span<Tensor*>(out), *stream);
            if (bound->status() != CG_B200_OK) std::printf("tuned launch status %d (%s)\n", bound->status(), cg_b200_status_string(bound->status()));
            CHECK(bound->status() == CG_B200_OK);
            copy_to_host(y16.data(), dy.t, dy.t.num_bytes, *stream);
            stream->sync();
            cgo_gemm(&rec.gemm, a16.data(), b16w.data(), nullptr, nullptr, want16.data(), nullptr, 0, 0);
            std::vector<float> y(M * N), want(M * N);
            cgo_bf16_to_f32(y16.data(), y.data(), M * N);
            cgo_bf16_to_f32(want16.data(), want.data(), M * N);
            double err = 0, scale = 0;
            for (usize i = 0; i < y.size(); ++i) {
                err = std::fmax(err, std::fabs(static_cast<double>(y[i]) - want[i]));
                scale = std::fmax(scale, std::fabs(static_cast<double>(want[i])));
            }
            std::printf("tuned bf16 gemm max-normalised error %.3e\n", err / scale);
            CHECK(err <= 1e-2 * scale);   // the path's 16-bit bound
        }
        std::filesystem::remove_all(dir);
    }
    {   // a vendor kernel that really executes
        VendorDispatcher& vd = VendorDispatcher::instance();
        Operation op;
        op.opcode = OP_LAYERNORM;
        op.shape = {4, 64};
        op.dtype = DType::F32;
        Function dummy;
        VendorKernel* k = const_cast<VendorKernel*>(vd.find_best(op, dummy));
        std::vector<float> x = randn(256, 10), y(256);
        DevTensor dx(dev, {4, 64}, DType::F32), dy(dev, {4, 64}, DType::F32);
        copy_to_device(dx.t, x.data(), dx.t.num_bytes, *stream);
        std::vector<Tensor*> in = {&dx.t}, out = {&dy.t};
        CHECK(k && k->execute(op, Span<Tensor*>(in), Span<Tensor*>(out), *stream));
        copy_to_host(y.data(), dy.t, dy.t.num_bytes, *stream);
        stream->sync();
        double mean = 0;
        for (int i = 0; i < 64; ++i) mean += y[i];
        CHECK(std::fabs(mean / 64) < 1e-5);
    }
    std::printf("host_tests gpu: %d checks, %d failed\n", g_checks, g_failed);
    return g_failed ? 1 : 0;
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    return mode == "gpu" ? run_gpu() : run_cpu();
}
