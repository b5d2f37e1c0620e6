// hardware.cpp - B200 hardware constants for the cost model and the tensor-core capability table.
//
// The reference's NVIDIA model is A100-class (src/cost/hardware_model.cpp:71-106: 19.5 TF fp32, 312 TF
// tensor cores, 2 TB/s, 108 SMs, 164 KB shared memory) and its TensorCoreCaps::blackwell() is hopper()
// with a larger fp8 number (src/backend/tensor_core/ptx_mma.cpp:293-299) - it still claims wgmma, which
// sm_100 does not have. The build renames that one function in the reference's file and links this
// definition instead.
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "cg/b200/b200.hpp"
#include "cg/backend/tensor_core/ptx_mma.hpp"

namespace cg::b200 {
namespace {

// The number that follows "key": in a flat JSON object; 0 when absent.
double json_number(const std::string& text, const std::string& key) {
    const std::string quoted = "\"" + key + "\"";
    usize at = text.find(quoted);
    if (at == std::string::npos) return 0.0;
    at = text.find(':', at + quoted.size());
    if (at == std::string::npos) return 0.0;
    return std::strtod(text.c_str() + at + 1, nullptr);
}

}  // namespace

Calibration load_calibration(const std::string& json_path) {
    Calibration c;
    std::ifstream in(json_path);
    if (!in) return c;
    std::stringstream ss;
    ss << in.rdbuf();
    const std::string text = ss.str();
    c.hbm_gbs = json_number(text, "hbm_gbs");
    c.bf16_tflops = json_number(text, "bf16_tflops");
    c.bf16_tflops_sustained = json_number(text, "bf16_tflops_sustained");
    c.measured = c.hbm_gbs > 0.0 && c.bf16_tflops > 0.0;
    return c;
}

Calibration calibration_from_env() {
    const char* path = std::getenv("CG_B200_PEAKS_JSON");
    return path ? load_calibration(path) : Calibration{};
}

HardwareModel hardware_model(const Calibration& cal) {
    HardwareModel h;
    h.name = cal.measured ? "nvidia_b200 (measured peaks)" : "nvidia_b200";
    h.device = DeviceId::cuda();
    const double tensor16 = cal.measured ? cal.bf16_tflops * 1e12 : 2.25e15;   // dense bf16 / f16
    const double hbm = cal.measured ? cal.hbm_gbs * 1e9 : 7.7e12;
    // CUDA-core peaks: 148 SMs x 128 fp32 lanes x 2 flop x 1.965 GHz
    const double fp32 = 148.0 * 128.0 * 2.0 * 1.965e9;
    h.compute.flops_per_sec[static_cast<u8>(DType::F32)] = fp32;
    h.compute.flops_per_sec[static_cast<u8>(DType::F16)] = fp32;        // packed half2 math is no faster on sm_100
    h.compute.flops_per_sec[static_cast<u8>(DType::BF16)] = fp32;
    h.compute.flops_per_sec[static_cast<u8>(DType::F64)] = fp32 / 2.0;
    h.compute.flops_per_sec[static_cast<u8>(DType::I32)] = fp32 / 2.0;
    h.memory.bytes_per_sec[static_cast<u8>(MemorySpace::Generic)] = hbm;
    h.memory.bytes_per_sec[static_cast<u8>(MemorySpace::Shared)] = 148.0 * 128.0 * 1.965e9;   // 128 B / clk / SM
    h.shared_mem_bytes = 227 * 1024;
    h.l1_cache_bytes = 256 * 1024;
    h.l2_cache_bytes = 126ull << 20;
    h.constant_mem_bytes = 64 * 1024;
    h.simd_width_bytes = 16;
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::BF16)] = tensor16;
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::F16)] = tensor16;
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::F32)] = tensor16 / 2.0 / 3.0;   // kind::tf32, three passes
    h.tensor_core_flops_per_sec[static_cast<u8>(DType::I8)] = 2.0 * tensor16;
    h.num_cores = 148;
    h.threads_per_core = 2048;
    h.launch_overhead_sec = 2.5e-6;
    h.register_file_per_sm = 65536;
    h.base_regs_per_thread = 32;
    h.max_warps_per_sm = 64;
    h.warp_size = 32;
    h.l2_read_bw = 2.5 * hbm;
    h.l2_hit_rate_estimate = 0.7;      // 126 MB: the operands of every configured GEMM fit
    h.stall_cycles_per_warp = 2.0;
    return h;
}

}  // namespace cg::b200

namespace cg {

// sm_100: tcgen05.mma with tensor-memory accumulators (one CTA: 128 x N x 16 for 16-bit inputs, a CTA
// pair: 256 x N x 16, N up to 256), TMA and mbarriers; mma.sync still compiles; wgmma does not exist.
TensorCoreCaps TensorCoreCaps::blackwell() {
    TensorCoreCaps caps = ampere();
    caps.has_hopper_wgmma = false;
    caps.has_tma = true;
    caps.has_async_barrier = true;
    const b200::Calibration cal = b200::calibration_from_env();
    const double t16 = cal.measured ? cal.bf16_tflops : 2250.0;
    caps.peak_f16_tflops = t16;
    caps.peak_bf16_tflops = t16;
    caps.peak_i8_tflops = 2.0 * t16;
    caps.peak_fp8_tflops = 2.0 * t16;
    caps.supported_tiles.push_back({128, 64, 16});
    caps.supported_tiles.push_back({128, 128, 16});
    caps.supported_tiles.push_back({128, 256, 16});
    caps.supported_tiles.push_back({256, 128, 16});
    caps.supported_tiles.push_back({256, 256, 16});
    caps.supported_tiles.push_back({128, 128, 8});    // kind::tf32
    return caps;
}

}  // namespace cg
