// b200.hpp - what the B200 layer adds to the reference's interfaces.
//
// The layer itself is the implementation of four of the reference's own translation units, compiled
// against the reference's own headers (paths relative to the cantors-gift tree):
//   cg::NvidiaBackend::{compile,emit_text}        include/cg/backend/nvidia_backend.hpp:13-31
//   cg::TensorToCodegenLowering::{lower,lower_function}   include/cg/lowering/tensor_to_codegen.hpp:49-84
//   cg::Runtime, cg::KernelCache                  include/cg/runtime/runtime.hpp:90-157
//   cg::VendorDispatcher + built-in kernels       include/cg/vendor/dispatch.hpp:45-84
// Those classes keep their declarations. What their interfaces have no room for lives here, in
// namespace cg::b200: a CUDA Device to hand to Runtime::add_device, host<->device copies for a Tensor,
// the status of the last lowering / launch, the mapping from a Schedule to a GEMM tile, a BenchmarkFn
// that times the real kernel, and the B200 hardware model.
#pragma once

#include <functional>
#include <memory>
#include <optional>
#include <string>

#include "cg/autotuner/bayesian_optimizer.hpp"
#include "cg/backend/backend.hpp"
#include "cg/cost/hardware_model.hpp"
#include "cg/ir/module.hpp"
#include "cg/lowering/tensor_to_codegen.hpp"
#include "cg/runtime/runtime.hpp"
#include "cg/schedule/schedule.hpp"
#include "cg_b200.h"

namespace cg::b200 {

// ---- devices ---------------------------------------------------------------------------------------
// A cg::Device over the C ABI (allocator, streams, events); nullptr when `index` is not a usable
// compute-capability-10.x device. Runtime::add_device takes it.
std::unique_ptr<Device> make_cuda_device(u32 index);
// The cudaStream_t behind a Stream created by such a device (nullptr for any other Stream).
void* native_stream(Stream& s);
// A Stream object over an existing cudaStream_t (not owned): lets a caller that already has a stream
// (another framework's) pass it to BoundExecutable::launch.
std::unique_ptr<Stream> wrap_stream(void* cuda_stream, u32 device_index);
// Host <-> device copies on a stream of that device (the reference's Tensor has no copy API).
int copy_to_device(Tensor& dst, const void* host_src, u64 bytes, Stream& s);
int copy_to_host(void* host_dst, const Tensor& src, u64 bytes, Stream& s);
// A Tensor of `shape` / `dtype` in memory from `dev`'s allocator (owns_memory = true; free it with
// release_tensor), or over memory the caller owns.
Tensor make_tensor(Device& dev, std::vector<i64> shape, DType dtype);
Tensor tensor_from_ptr(void* device_ptr, std::vector<i64> shape, DType dtype, u32 device_index);
void release_tensor(Device& dev, Tensor& t);

// ---- status ----------------------------------------------------------------------------------------
// The reference's lower() returns a CGModule and launch() returns void; neither can report a failure.
// Status (cg_b200_status) and message of the last lower() / launch() on the calling thread.
int last_lowering_status();
const std::string& last_lowering_message();
int last_launch_status();

// For a batch-sharded or M-sharded executable: makes the GEMM that produces output 0 store its rows
// into every rank's full-size output as its tiles are produced (cg_b200_gemm_allgather). `bound` must
// come from Runtime::bind on a CUDA device; the launch's output tensor 0 is then this rank's full
// buffer and `peer_outputs` holds `world` pointers to every rank's (entry `rank` ignored).
// Returns CG_B200_ERR_UNSUPPORTED when output 0 is not produced by a single-batch GEMM.
int set_output_gather(BoundExecutable& bound, void* const* peer_outputs, int world, int rank);

// ---- schedules and autotuning ------------------------------------------------------------------------
// The reference's lowering accepts a Schedule and ignores it (src/lowering/tensor_to_codegen.cpp:361-366).
// Here Tile transforms on "m" (128 = one CTA, 256 = a CTA pair) and "n" (64 / 128 / 256) choose the
// GEMM kernel's tile; other transforms have no knob and are ignored. Empty: a tile no kernel has.
std::optional<cg_b200_gemm_tuning> gemm_tuning_from_schedule(const Schedule& s);

// The function the reference's autotuner was missing (include/cg/autotuner/bayesian_optimizer.hpp:79:
// in-tree it only ever receives an analytical stub): runs `desc` with the schedule's tile through
// cg_b200_gemm_tuned on zero-filled operands of `device` and returns the mean seconds of `iters`
// launches after `warmup`, timed with events on the device. Infinity for a schedule no kernel has.
BenchmarkFn make_gemm_benchmark(const cg_b200_gemm_desc& desc, Device& device, int iters = 20, int warmup = 3);
// The GEMM descriptor of the first matmul of `m` (what make_gemm_benchmark should time for it).
std::optional<cg_b200_gemm_desc> first_gemm_desc(const Module& m);

// Runtime::autotune_and_cache has no module to compile (src/runtime/runtime.cpp:287-312 says "the
// caller is responsible for compiling it"). This does the whole step: search `space` with the
// reference's bayesian_autotune, lower `m` with the winning schedule, compile, cache under `key`.
struct TunedExecutable {
    std::shared_ptr<Executable> executable;
    Schedule best_schedule;
    double best_runtime = 0.0;
    usize total_benchmarks = 0;
    bool cache_hit = false;
};
TunedExecutable autotune_and_cache(Runtime& rt, u64 key, const Module& m, const ScheduleSpace& space,
                                   const BenchmarkFn& benchmark, MachineBackend& backend);

// ---- hardware model ----------------------------------------------------------------------------------
// HardwareModel::generic_nvidia_gpu() holds A100-class constants (src/cost/hardware_model.cpp:71-106).
// B200: 148 SMs, 227 KiB shared memory per block, 126 MB L2, 256 KiB tensor memory per SM, HBM3e.
// Peaks are the nominal dense figures (2.25 PFLOP/s bf16/f16, 7.7 TB/s) unless a calibration file is
// found: $CG_B200_PEAKS_JSON, a JSON object with "hbm_gbs", "bf16_tflops" and optionally
// "bf16_tflops_sustained" as measured on the machine (copy bandwidth, library GEMM). With it
// AnalyticalCostModelV2 predictions can be set beside measured times.
struct Calibration {
    double hbm_gbs = 0.0, bf16_tflops = 0.0, bf16_tflops_sustained = 0.0;
    bool measured = false;
};
Calibration load_calibration(const std::string& json_path);
Calibration calibration_from_env();
HardwareModel hardware_model(const Calibration& c = calibration_from_env());

}  // namespace cg::b200
