// cgc.cpp - the command-line driver with its NVIDIA path executing.
//
// The reference's tool (tools/cgc/cgc.cpp) builds a synthetic relu(A x B + bias) graph, lowers it, and
// for `--backend nvidia --jit-run` prints PTX; its CPU `--jit-run` loads the code and stops short of
// calling it (tools/cgc/cgc.cpp:206-228). This one takes the same flags and, for the NVIDIA backend with
// --jit-run, compiles for sm_100a, binds through Runtime::bind on CUDA device 0, runs the graph on seeded
// inputs, checks sampled outputs against a double-precision host loop and reports the kernel time.
//   cgc --backend nvidia --jit-run [--matmul M,N,K] [--sm-target sm_100a] [--emit ptx] [-o file]
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <random>
#include <string>

#include "cg/b200/b200.hpp"
#include "cg/b200/plan.hpp"
#include "cg/backend/cpu_backend.hpp"
#include "cg/backend/nvidia_backend.hpp"
#include "cg/ir/builder.hpp"
#include "cg/ir/printer.hpp"

using namespace cg;

namespace {

struct Args {
    std::string backend = "cpu", emit = "print", sm = "sm_80", out;
    bool jit_run = false;
    i64 M = 1024, N = 1024, K = 1024;
};

bool parse(int argc, char** argv, Args& a) {
    for (int i = 1; i < argc; ++i) {
        const std::string s = argv[i];
        auto next = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
        if (s == "--backend") a.backend = next();
        else if (s == "--emit") a.emit = next();
        else if (s == "--sm-target") a.sm = next();
        else if (s == "-o") a.out = next();
        else if (s == "--jit-run") a.jit_run = true;
        else if (s == "--matmul") {
            if (std::sscanf(next().c_str(), "%ld,%ld,%ld", &a.M, &a.N, &a.K) != 3) return false;
        } else if (s == "-h" || s == "--help") return false;
    }
    return a.M > 0 && a.N > 0 && a.K > 0;
}

int run_on_gpu(const Args& a, const Module& m, const CGModule& cgm) {
    NvidiaBackend nv(a.sm.rfind("sm_100", 0) == 0 ? a.sm : "sm_100a");   // the kernels exist for sm_100a only
    std::shared_ptr<Executable> exe(nv.compile(cgm).release());
    auto plan = b200::LaunchPlan::deserialize(exe->machine_code);
    if (!plan) {
        std::cerr << "// no launch plan: " << b200::last_lowering_message() << "\n";
        return 2;
    }
    Runtime rt;
    rt.add_device(b200::make_cuda_device(0));
    Device* dev = rt.get_device(DeviceId::cuda(0));
    if (!dev) {
        std::cerr << "// --jit-run: no usable sm_100 device (there is no CPU fallback for the NVIDIA backend)\n";
        return 3;
    }
    auto bound = rt.bind(exe, DeviceId::cuda(0));
    if (!bound) {
        std::cerr << "// bind failed\n";
        return 4;
    }
    auto stream = dev->create_stream();
    std::mt19937 gen(0);
    std::uniform_real_distribution<float> u(-1.0f, 1.0f);
    std::vector<float> A(static_cast<usize>(a.M * a.K)), B(static_cast<usize>(a.K * a.N)), bias(static_cast<usize>(a.M * a.N));
    for (auto* v : {&A, &B, &bias})
        for (float& x : *v) x = u(gen);
    Tensor tA = b200::make_tensor(*dev, {a.M, a.K}, DType::F32), tB = b200::make_tensor(*dev, {a.K, a.N}, DType::F32);
    Tensor tb = b200::make_tensor(*dev, {a.M, a.N}, DType::F32), tC = b200::make_tensor(*dev, {a.M, a.N}, DType::F32);
    b200::copy_to_device(tA, A.data(), tA.num_bytes, *stream);
    b200::copy_to_device(tB, B.data(), tB.num_bytes, *stream);
    b200::copy_to_device(tb, bias.data(), tb.num_bytes, *stream);
    std::vector<Tensor*> in = {&tA, &tB, &tb}, out = {&tC};
    bound->launch(in, out, *stream);   // warm-up
    auto e0 = dev->create_event(), e1 = dev->create_event();
    const int reps = 10;
    e0->record(*stream);
    for (int i = 0; i < reps; ++i) bound->launch(in, out, *stream);
    e1->record(*stream);
    if (b200::last_launch_status() != CG_B200_OK) {
        std::cerr << "// launch failed: " << cg_b200_status_string(b200::last_launch_status()) << "\n";
        return 5;
    }
    std::vector<float> C(static_cast<usize>(a.M * a.N));
    b200::copy_to_host(C.data(), tC, tC.num_bytes, *stream);
    stream->sync();
    const double sec = e1->elapsed_sec_since(*e0) / reps;
    // sampled check against a double-precision loop
    double worst = 0.0, scale = 1e-30;
    std::mt19937 pick(1);
    for (int s = 0; s < 512; ++s) {
        const i64 i = static_cast<i64>(pick() % static_cast<unsigned long>(a.M)), j = static_cast<i64>(pick() % static_cast<unsigned long>(a.N));
        double acc = 0.0;
        for (i64 k = 0; k < a.K; ++k) acc += static_cast<double>(A[static_cast<usize>(i * a.K + k)]) * B[static_cast<usize>(k * a.N + j)];
        acc += bias[static_cast<usize>(i * a.N + j)];
        acc = acc > 0.0 ? acc : 0.0;
        worst = std::max(worst, std::fabs(acc - C[static_cast<usize>(i * a.N + j)]));
        scale = std::max(scale, std::fabs(acc));
    }
    std::cerr << "// JIT: " << plan->records.size() << " kernel(s) on cuda:0, " << sec * 1e6 << " us per run, "
              << 2.0 * static_cast<double>(a.M) * static_cast<double>(a.N) * static_cast<double>(a.K) / sec / 1e12 << " TFLOP/s\n";
    std::cerr << "// JIT: max error of 512 sampled outputs / max|C| = " << worst / scale << (worst / scale <= 1e-4 ? " (ok)" : " (MISMATCH)") << "\n";
    for (Tensor* t : {&tA, &tB, &tb, &tC}) b200::release_tensor(*dev, *t);
    (void)m;
    return worst / scale <= 1e-4 ? 0 : 6;
}

}  // namespace

int main(int argc, char** argv) {
    Args a;
    if (!parse(argc, argv, a)) {
        std::cerr << "usage: cgc [--backend cpu|nvidia] [--emit print|ir|ptx|x86|codegen] [--jit-run] [--sm-target sm_100a]\n"
                     "           [--matmul M,N,K] [-o file]\n";
        return 1;
    }
    // C = relu(A x B + bias), the tool's synthetic graph
    Module m;
    auto f = m.create_function("matmul_relu",
                               {make_tensor_type({a.M, a.K}, DType::F32), make_tensor_type({a.K, a.N}, DType::F32),
                                make_tensor_type({a.M, a.N}, DType::F32)},
                               {make_tensor_type({a.M, a.N}, DType::F32)});
    Builder b(f);
    b.output_tensor(b.relu(b.add(b.matmul(f->args()[0], f->args()[1]), f->args()[2])));

    std::string text;
    int rc = 0;
    if (a.emit == "print" || a.emit == "ir") text = to_string(m);
    if (a.emit == "ptx" || a.emit == "x86" || a.emit == "codegen" || a.jit_run) {
        CGModule cgm = TensorToCodegenLowering().lower(m);
        if (a.emit == "codegen") {
            for (const auto& fn : cgm.functions) {
                text += "; function " + fn.name + " (" + std::to_string(fn.instructions.size()) + " instructions)\n";
                for (const auto& inst : fn.instructions) {
                    auto k = inst.attributes.get("b200.kernel");
                    text += "  op" + std::to_string(static_cast<int>(inst.opcode)) + (k ? "  [cg_b200_" + k->str + "]" : "") +
                            (inst.comment.empty() ? "" : " ; " + inst.comment) + "\n";
                }
            }
        }
        if (a.backend == "nvidia") {
            NvidiaBackend nv(a.sm);
            if (a.emit == "ptx" || a.jit_run) text = nv.compile(cgm)->ptx_text;
            if (a.jit_run) rc = run_on_gpu(a, m, cgm);
        } else if (a.emit == "x86" || a.jit_run) {
            CpuBackend cpu;
            text = cpu.compile(cgm)->disassembly;
        }
    }
    if (a.out.empty()) std::cout << text;
    else std::ofstream(a.out) << text;
    return rc;
}
