// ref_kernels.cpp - driver that assembles and runs the reference's own x86 kernels.
//
// TEST INFRASTRUCTURE ONLY. Linked with the reference's X86Emitter and JITMemory sources
// (src/backend/x86/x86_emitter.cpp, src/backend/jit.cpp, compiled where they lie; see the
// Makefile next to this file) into oracle/_ref/libcg_ref.so. The instruction sequences
// follow the reference's benchmark kernels:
//   - add / relu(a*b), count-parameterised: benchmarks/benchmark_multithread.py:54-124
//   - scalar-FMA triple-loop matmul:       benchmarks/benchmark.py:326-438
//   - relu(a*b+c)*s: the same load/op/store loop with the emitter's vmulps, vaddps, vmaxps
//     (include/cg/backend/x86/x86_emitter.hpp:90-119)
// and the thread fan-out follows ParallelExecutor::execute
// (include/cg/backend/parallel_executor.hpp:49-92): contiguous chunks of 4-float groups,
// one std::thread per chunk, join.
#include "cg/backend/jit.hpp"
#include "cg/backend/x86/x86_emitter.hpp"

#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

using namespace cg;

namespace {

using R = X86Reg;
using V = X86VReg;
constexpr VEXWidth W = VEXWidth::XMM;

void frame_open(X86Emitter& e) {
    e.push(R::RBP);
    e.mov_reg(R::RBP, R::RSP);
}
void frame_close(X86Emitter& e) {
    e.pop(R::RBP);
    e.ret();
}
// xmm <- [base + index]
void load_at(X86Emitter& e, V dst, R base, R index) {
    e.mov_reg(R::RAX, base);
    e.add_reg(R::RAX, index);
    e.vmovups_load(dst, R::RAX, 0, W);
}
void store_at(X86Emitter& e, R base, R index, V src) {
    e.mov_reg(R::RAX, base);
    e.add_reg(R::RAX, index);
    e.vmovups_store(R::RAX, 0, src, W);
}

// void fn(float* a, float* b, float* c, int64_t groups): c = a + b  (mode 0), relu(a*b) (mode 1)
std::vector<u8> build_binary(int mode) {
    X86Emitter e;
    frame_open(e);
    if (mode == 1) e.vxorps(V::XMM2, V::XMM2);
    e.xor_reg(R::R8, R::R8);
    e.mov_imm64(R::R9, 16);
    auto loop = e.label();
    e.mark_label(loop);
    load_at(e, V::XMM0, R::RDI, R::R8);
    load_at(e, V::XMM1, R::RSI, R::R8);
    if (mode == 0) {
        e.vaddps(V::XMM0, V::XMM0, V::XMM1, W);
    } else {
        e.vmulps(V::XMM0, V::XMM0, V::XMM1, W);
        e.vmaxps(V::XMM0, V::XMM0, V::XMM2, W);
    }
    store_at(e, R::RDX, R::R8, V::XMM0);
    e.add_reg(R::R8, R::R9);
    e.dec_reg(R::RCX);
    e.jne(loop);
    frame_close(e);
    return e.take_bytes();
}

// void fn(float* a, float* b, float* c, const float* scale4, float* out, int64_t groups)
//   out = relu(a*b + c) * scale, each op separately rounded
std::vector<u8> build_fma_relu_scale() {
    X86Emitter e;
    frame_open(e);
    e.vxorps(V::XMM2, V::XMM2);
    e.vmovups_load(V::XMM3, R::RCX, 0, W);
    e.xor_reg(R::R10, R::R10);
    e.mov_imm64(R::R11, 16);
    auto loop = e.label();
    e.mark_label(loop);
    load_at(e, V::XMM0, R::RDI, R::R10);
    load_at(e, V::XMM1, R::RSI, R::R10);
    e.vmulps(V::XMM0, V::XMM0, V::XMM1, W);
    load_at(e, V::XMM1, R::RDX, R::R10);
    e.vaddps(V::XMM0, V::XMM0, V::XMM1, W);
    e.vmaxps(V::XMM0, V::XMM0, V::XMM2, W);
    e.vmulps(V::XMM0, V::XMM0, V::XMM3, W);
    store_at(e, R::R8, R::R10, V::XMM0);
    e.add_reg(R::R10, R::R11);
    e.dec_reg(R::R9);
    e.jne(loop);
    frame_close(e);
    return e.take_bytes();
}

// void fn(const float* A, const float* B, float* C): C[m,n] = fma-chain over k ascending
std::vector<u8> build_matmul(int64_t M, int64_t K, int64_t N) {
    X86Emitter e;
    frame_open(e);
    e.push(R::RBX);
    e.mov_imm64(R::R10, static_cast<u64>(K));
    e.mov_imm64(R::R11, static_cast<u64>(N));
    auto elem_addr = [&](R row, R row_len, R col, R base) {
        e.mov_reg(R::RAX, row);
        e.imul_reg(R::RAX, row_len);
        e.add_reg(R::RAX, col);
        e.mov_imm64(R::RBX, 4);
        e.imul_reg(R::RAX, R::RBX);
        e.add_reg(R::RAX, base);
    };
    auto bump_and_loop = [&](R counter, int64_t bound, X86Emitter::LabelId target) {
        e.mov_imm64(R::RBX, 1);
        e.add_reg(counter, R::RBX);
        e.cmp_imm32(counter, static_cast<i32>(bound));
        e.jne(target);
    };
    e.xor_reg(R::RCX, R::RCX);  // m
    auto m_loop = e.label();
    e.mark_label(m_loop);
    e.xor_reg(R::R8, R::R8);  // n
    auto n_loop = e.label();
    e.mark_label(n_loop);
    e.vxorps(V::XMM0, V::XMM0);
    e.xor_reg(R::R9, R::R9);  // k
    auto k_loop = e.label();
    e.mark_label(k_loop);
    elem_addr(R::RCX, R::R10, R::R9, R::RDI);
    e.vmovss_load(V::XMM1, R::RAX, 0);
    elem_addr(R::R9, R::R11, R::R8, R::RSI);
    e.vmovss_load(V::XMM2, R::RAX, 0);
    e.vfmadd231ss(V::XMM0, V::XMM1, V::XMM2);
    bump_and_loop(R::R9, K, k_loop);
    elem_addr(R::RCX, R::R11, R::R8, R::RDX);
    e.vmovss_store(R::RAX, 0, V::XMM0);
    bump_and_loop(R::R8, N, n_loop);
    bump_and_loop(R::RCX, M, m_loop);
    e.pop(R::RBX);
    frame_close(e);
    return e.take_bytes();
}

// Chunking of ParallelExecutor::execute: groups split evenly, the first `extra` chunks get
// one more; each chunk runs on its own std::thread.
template <typename Fn>
void fan_out(uint64_t total_groups, unsigned threads, Fn&& run_chunk) {
    if (threads == 0) threads = std::thread::hardware_concurrency();
    if (threads == 0) threads = 1;
    uint64_t per = total_groups / threads, extra = total_groups % threads, off = 0;
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < threads; ++t) {
        uint64_t chunk = per + (t < extra ? 1 : 0);
        if (chunk == 0) continue;
        pool.emplace_back([=] { run_chunk(off, chunk); });
        off += chunk;
    }
    for (auto& th : pool) th.join();
}

using Fn3 = void (*)(float*, float*, float*, int64_t);
using Fn5 = void (*)(const float*, const float*, const float*, const float*, float*, int64_t);
using FnMM = void (*)(const float*, const float*, float*);

JITMemory& jit_binary(int mode) {
    static JITMemory mem[2];
    if (!mem[mode].valid()) mem[mode].allocate(build_binary(mode));
    return mem[mode];
}
JITMemory& jit_chain() {
    static JITMemory mem;
    if (!mem.valid()) mem.allocate(build_fma_relu_scale());
    return mem;
}

}  // namespace

extern "C" {

// n must be a multiple of 4 (the reference kernels process 4-float groups).
int cgref_binary(int mode, float* a, float* b, float* c, uint64_t n, unsigned threads) {
    if (mode < 0 || mode > 1 || (n % 4) != 0) return 1;
    if (n == 0) return 0;
    auto fn = reinterpret_cast<Fn3>(jit_binary(mode).entry());
    if (!fn) return 2;
    fan_out(n / 4, threads, [=](uint64_t off, uint64_t groups) {
        fn(a + off * 4, b + off * 4, c + off * 4, static_cast<int64_t>(groups));
    });
    return 0;
}

int cgref_fma_relu_scale(const float* a, const float* b, const float* c, float scale, float* out,
                         uint64_t n, unsigned threads) {
    if ((n % 4) != 0) return 1;
    if (n == 0) return 0;
    auto fn = reinterpret_cast<Fn5>(jit_chain().entry());
    if (!fn) return 2;
    alignas(16) const float s4[4] = {scale, scale, scale, scale};
    const float* sp = s4;
    fan_out(n / 4, threads, [=](uint64_t off, uint64_t groups) {
        fn(a + off * 4, b + off * 4, c + off * 4, sp, out + off * 4, static_cast<int64_t>(groups));
    });
    return 0;
}

int cgref_matmul(const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N) {
    if (M <= 0 || K <= 0 || N <= 0) return 1;
    JITMemory mem;
    auto fn = reinterpret_cast<FnMM>(mem.allocate(build_matmul(M, K, N)));
    if (!fn) return 2;
    fn(A, B, C);
    return 0;
}

}  // extern "C"
