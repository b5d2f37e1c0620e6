// b200_host.hpp - C++ host layer over the cg_b200 C ABI, shaped like the reference's own
// backend / lowering / runtime interfaces so that it can take their place.
//
// Every class below carries the name and members of the reference class it mirrors (cantors-gift,
// paths relative to its root):
//   DType, DeviceId, Shape            include/cg/core/dtype.hpp:14-40, include/cg/ir/type.hpp:38-57
//   Codegen IR (CGOpcode ... CGModule) include/cg/codegen/codegen_ir.hpp:23-107
//   Executable, TargetInfo, MachineBackend, NvidiaBackend
//                                      include/cg/backend/backend.hpp:26-90, backend/nvidia_backend.hpp:13-31
//   TensorToCodegenLowering, LoweringOptions
//                                      include/cg/lowering/tensor_to_codegen.hpp:31-84
//   Tensor, Allocator, Stream, Event, Device, BoundExecutable, KernelCache, Runtime
//                                      include/cg/runtime/runtime.hpp:32-157
//   VendorKernel, VendorDispatcher     include/cg/vendor/dispatch.hpp:24-84
// The Tensor-IR classes (Operation, Function, Module, Builder) are a minimal stand-in for the
// reference's IR (include/cg/ir/*.hpp): only what the kernel planner reads. In a build inside the
// reference tree the planner takes the real cg::Module instead.
//
// No CPU fallback: binding or launching without a usable sm_100 device fails (null / status).
#pragma once

#include <cstdint>
#include <deque>
#include <functional>
#include <limits>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <utility>
#include <variant>
#include <vector>

#include "cg_b200.h"

namespace cg {

using u8 = std::uint8_t;
using u32 = std::uint32_t;
using u64 = std::uint64_t;
using i32 = std::int32_t;
using i64 = std::int64_t;
using usize = std::size_t;

// ---- core ------------------------------------------------------------------------------------------
enum class DType : u8 { F16, BF16, F32, F64, I8, I16, I32, I64, U8, U16, U32, U64, BOOL, INDEX, CF32, CF64 };
usize dtype_size(DType dt);
DType promote(DType a, DType b);

struct DeviceId {
    enum class Kind : u8 { CPU, CUDA, ROCM, METAL };
    Kind kind = Kind::CPU;
    u32 index = 0;
    bool operator==(const DeviceId& o) const { return kind == o.kind && index == o.index; }
    bool operator!=(const DeviceId& o) const { return !(*this == o); }
    static DeviceId cpu(u32 i = 0) { return {Kind::CPU, i}; }
    static DeviceId cuda(u32 i = 0) { return {Kind::CUDA, i}; }
};

using Shape = std::vector<i64>;
i64 num_elements(const Shape& s);

using Attribute = std::variant<i64, double, std::string, std::vector<i64>>;
using AttributeDict = std::map<std::string, Attribute>;

// ---- Tensor IR stand-in ----------------------------------------------------------------------------
using Opcode = u32;
constexpr Opcode OP_CONSTANT = 1, OP_INPUT = 2, OP_OUTPUT = 3, OP_ADD = 4, OP_SUB = 5, OP_MUL = 6, OP_DIV = 7,
                 OP_NEG = 8, OP_RELU = 9, OP_GELU = 10, OP_SIGMOID = 11, OP_TANH = 12, OP_EXP = 13, OP_LOG = 14,
                 OP_SQRT = 15, OP_MATMUL = 16, OP_RESHAPE = 18, OP_SOFTMAX = 29, OP_LAYERNORM = 30, OP_FUSE = 34;

struct Value {
    u32 id = 0;   // index of the defining Operation in its Function (0 = invalid)
    bool valid() const { return id != 0; }
};

struct Operation {
    Opcode opcode = 0;
    std::vector<Value> operands;
    Shape shape;                  // result shape
    DType dtype = DType::F32;     // result dtype
    AttributeDict attributes;
    std::vector<u8> constant_bytes;   // OP_CONSTANT payload (little endian, `dtype`)
};

class Function {
public:
    std::string name;
    std::vector<Operation> ops;   // ops[0] is a placeholder so that Value{0} is invalid
    Function() { ops.emplace_back(); }
    const Operation& def(Value v) const { return ops.at(v.id); }
};

class Module {
public:
    std::deque<Function> functions;   // a deque: create_function must not move the functions handed out before
    Function& create_function(std::string name) {
        functions.emplace_back();
        functions.back().name = std::move(name);
        return functions.back();
    }
};

// Same convenience surface as the reference's Builder (include/cg/ir/builder.hpp:19-83); type
// inference failures throw std::invalid_argument as Builder::create does (src/ir/builder.cpp:47-49).
class Builder {
public:
    explicit Builder(Function* fn) : fn_(fn) {}
    Function* function() const { return fn_; }
    Value input_tensor(Shape shape, DType dt);
    Value constant_tensor(Shape shape, DType dt, std::vector<u8> bytes = {});
    Value constant_scalar(float v, DType dt);   // shape {} constant
    void output_tensor(Value v);
    Value add(Value a, Value b);
    Value sub(Value a, Value b);
    Value mul(Value a, Value b);
    Value div(Value a, Value b);
    Value neg(Value a);
    Value relu(Value a);
    Value gelu(Value a);
    Value exp(Value a);
    Value sqrt(Value a);
    Value sigmoid(Value a);
    Value tanh(Value a);
    Value log(Value a);
    Value matmul(Value a, Value b);
    Value reshape(Value a, std::vector<i64> target_shape);
    Value softmax(Value a);
    Value layernorm(Value a);

private:
    Value emit(Operation op);
    Value binary(Opcode opc, Value a, Value b);
    Value unary(Opcode opc, Value a);
    Function* fn_;
};

// ---- Codegen IR ------------------------------------------------------------------------------------
enum class CGOpcode : u8 {
    Load, Store, VectorLoad, VectorStore, FMA, Add, Mul, Reduce, Barrier, AsyncCopy, Prefetch, Broadcast,
    Shuffle, Cmp, Select, Cast, Const,
};

class CGValue {
public:
    u32 id = 0;
    DType dtype = DType::F32;
    u8 width = 1;
    std::string name;
    bool operator==(const CGValue& o) const { return id == o.id; }
};

class CGInstruction {
public:
    CGOpcode opcode = CGOpcode::Const;
    std::vector<CGValue> operands;
    std::vector<CGValue> results;
    AttributeDict attributes;
    std::string comment;
};

class CGFunction {
public:
    std::string name;
    std::vector<CGInstruction> instructions;
    std::vector<CGValue> args;
    std::vector<CGValue> returns;
    CGValue allocate(DType dt, u8 width = 1) {
        CGValue v;
        v.id = next_id_++;
        v.dtype = dt;
        v.width = width;
        return v;
    }
    void emit(CGInstruction inst) { instructions.push_back(std::move(inst)); }

private:
    u32 next_id_ = 1;
};

class CGModule {
public:
    std::vector<CGFunction> functions;
    CGFunction& create_function(std::string name) {
        functions.emplace_back();
        functions.back().name = std::move(name);
        return functions.back();
    }
};

// ---- launch plan: what a compiled Executable carries in machine_code -----------------------------------
// One record per fused kernel. Buffers are numbered: [0, n_inputs) are the function's inputs in
// OP_INPUT order, [n_inputs, n_inputs + n_outputs) its outputs in OP_OUTPUT order, the rest are
// intermediates the bound executable allocates from the device's Allocator.
struct PlanBuffer {
    u64 bytes = 0;
    DType dtype = DType::F32;
    Shape shape;
};

struct PlanRecord {
    enum Kind : u32 { Eltwise = 1, Gemm = 2, Softmax = 3, LayerNorm = 4, SoftmaxLayerNorm = 5 };
    u32 kind = 0;
    cg_b200_eltwise_desc eltwise{};     // Eltwise
    cg_b200_gemm_desc gemm{};           // Gemm
    cg_b200_gemm_tuning tuning{};       // Gemm: all zero = the library's heuristic
    i32 row_dtype = 0;                  // row reductions
    i64 rows = 0, cols = 0;
    float eps = 1e-5f;
    u64 n = 0;                          // Eltwise: elements
    i32 n_inputs = 0;
    i32 input[CG_B200_EW_MAX_INPUTS] = {-1, -1, -1, -1, -1, -1, -1, -1};   // buffer ids; Gemm: A, B, bias, residual
    i32 output = -1;
};

struct LaunchPlan {
    static constexpr u32 kMagic = 0x31304243;   // "CB01"
    u32 n_inputs = 0, n_outputs = 0;
    std::vector<PlanBuffer> buffers;
    std::vector<PlanRecord> records;
    u64 workspace_bytes = 0;            // max over records (fp32 GEMM scratch)

    std::vector<u8> serialize() const;
    // Empty optional when the bytes are not a launch plan of this version.
    static std::optional<LaunchPlan> deserialize(const std::vector<u8>& bytes);
};

// ---- lowering: Tensor IR -> fused Codegen-IR nodes -----------------------------------------------------
// Mirrors TensorToCodegenLowering(LoweringOptions).lower(module, schedule). The reference emits one
// un-looped vector op per Tensor-IR op (src/lowering/tensor_to_codegen.cpp:306-357); this planner
// groups ops into the three kernel families of the B200 path and emits ONE CGInstruction per
// kernel (opcode FMA = gemm, Add = elementwise chain, Reduce = row reduction) whose attributes
// carry the kernel name and its serialised record ("b200.kernel", "b200.record").
// It takes pre-fusion IR. IR that carries the reference's lossy fusion markers
// (fused_chain / fused_with attributes, OP_FUSE; src/optimization/fusion/fusion.cpp:415-441) cannot be
// executed faithfully: lower() then reports CG_B200_ERR_FUSED_IR and returns an empty module.
struct LoweringOptions {
    u32 m_tile = 256, n_tile = 256, k_tile = 64;   // informational: the tcgen05 tile
    bool use_shared_memory = true;
    bool use_tensor_cores = true;
    bool fuse_softmax_layernorm = true;
    float layernorm_eps = 1e-5f;                    // the op carries no attribute (src/ir/ops.cpp:536-556)
};

// ---- schedules and the autotuner's interface ------------------------------------------------------
// Stand-ins for include/cg/schedule/schedule.hpp:24-84 (the schedule subsystem itself is outside this
// path): a Schedule is a list of transforms, a ScheduleSpace a list of schedules, and grid_matmul
// builds the same Tile m / Tile n / Tile k (+ Vectorize) schedules as src/schedule/schedule.cpp:66-87.
// The reference's lowering accepts a schedule and ignores it (tensor_to_codegen.cpp:361-366); this
// one reads the Tile transforms on "m" and "n" as the GEMM kernel's tile choice.
enum class TransformKind : u8 { Split, Tile, Interchange, Fuse, Vectorize, Parallelize, Unroll, Cache, Pipeline, Prefetch, Bind };

struct Transform {
    TransformKind kind = TransformKind::Tile;
    std::string dim;
    i64 factor = 0;
    i64 factor2 = 0;
    std::string target;
};

class Schedule {
public:
    void add(Transform t) { transforms_.push_back(std::move(t)); }
    const std::vector<Transform>& transforms() const { return transforms_; }
    u64 hash() const;
    bool operator==(const Schedule& o) const;

private:
    std::vector<Transform> transforms_;
};

class ScheduleSpace {
public:
    void add(Schedule s) { schedules_.push_back(std::move(s)); }
    const std::vector<Schedule>& schedules() const { return schedules_; }
    usize size() const { return schedules_.size(); }
    static ScheduleSpace grid_matmul(std::vector<i64> m_tiles, std::vector<i64> n_tiles, std::vector<i64> k_tiles,
                                     std::vector<i64> vector_widths);

private:
    std::vector<Schedule> schedules_;
};

// include/cg/autotuner/bayesian_optimizer.hpp:79-96. A benchmark function returns the measured runtime
// of a schedule in seconds (infinity: cannot run).
using BenchmarkFn = std::function<double(const Schedule&)>;

struct AutotuneResult {
    Schedule best_schedule;
    double best_runtime = std::numeric_limits<double>::infinity();
    std::vector<double> runtime_history;
    usize total_benchmarks = 0;
};

// Same signature as the reference's search. The GEMM kernel's tile space has a dozen points, so this
// one simply measures candidates in order until `max_benchmarks` (a surrogate model has nothing to
// add at that size); `initial_random` is accepted for source compatibility.
AutotuneResult bayesian_autotune(const ScheduleSpace& space, BenchmarkFn benchmark, usize max_benchmarks = 20,
                                 usize initial_random = 3);

// Tile m = 128 -> one CTA per tile, 256 -> CTA pair; Tile n = 64 / 128 / 256 -> tile width. Transforms
// the kernel has no knob for are ignored. Empty optional: a tile the kernels do not have.
std::optional<cg_b200_gemm_tuning> gemm_tuning_from_schedule(const Schedule& s);

class Device;
// The function an autotuner calls per candidate: runs `desc` with the schedule's tiles through
// cg_b200_gemm_tuned on zero-filled operands of `device` and returns the mean seconds of `iters`
// launches after `warmup`, timed with events on the device's stream. Infinity for a schedule that
// maps to no kernel. The operand buffers live as long as the returned function.
BenchmarkFn make_gemm_benchmark(const cg_b200_gemm_desc& desc, Device& device, int iters = 20, int warmup = 3);

class TensorToCodegenLowering {
public:
    explicit TensorToCodegenLowering(LoweringOptions opts = {}) : opts_(opts) {}
    // Tile transforms on "m" / "n" in `schedule` choose the tiles of every GEMM kernel of the module.
    CGModule lower(const Module& m, const Schedule& schedule = {});
    const LoweringOptions& options() const { return opts_; }
    int status() const { return status_; }              // cg_b200_status of the last lower()
    const std::string& message() const { return message_; }

private:
    LoweringOptions opts_;
    int status_ = CG_B200_OK;
    std::string message_;
};

// ---- backend ---------------------------------------------------------------------------------------------
class Executable {
public:
    std::string name;
    DeviceId target_device;
    std::vector<u8> machine_code;   // serialised LaunchPlan
    std::string ptx_text;           // listing for debugging
    std::vector<std::pair<std::string, u64>> entrypoints;
    u64 shared_mem_bytes = 0;
    u64 constant_mem_bytes = 0;
    u32 threads_per_block = 0;
    std::string disassembly;
};

struct HardwareModel {
    std::string name;
    u32 num_sms = 0;
    u64 shared_mem_per_block = 0, l2_bytes = 0, hbm_bytes = 0, tmem_bytes_per_sm = 0;
    double memory_bandwidth = 0;                         // bytes/s
    std::map<u8, double> flops_per_sec;                  // vector pipes, by DType
    std::map<u8, double> tensor_core_flops_per_sec;      // by DType
    double peak_flops(DType dt) const;
    // Nominal B200 figures; filled from the device when one is present.
    static HardwareModel b200();
};

class TargetInfo {
public:
    std::string name;
    DeviceId device;
    HardwareModel hardware;
    std::vector<DType> supported_vector_dtypes;
    u32 max_vector_width_bytes = 16;
    std::vector<std::tuple<u32, u32, u32>> tensor_core_tiles;
    bool supports_tensor_core(DType dt) const { return hardware.tensor_core_flops_per_sec.count(static_cast<u8>(dt)) > 0; }
};

class MachineBackend {
public:
    virtual ~MachineBackend() = default;
    virtual std::string name() const = 0;
    virtual const TargetInfo& target_info() const = 0;
    virtual std::unique_ptr<Executable> compile(const CGModule& module) = 0;
    virtual std::optional<std::string> emit_text(const CGModule&) { return std::nullopt; }
};

class NvidiaBackend : public MachineBackend {
public:
    explicit NvidiaBackend(std::string sm_target = "sm_100a");
    std::string name() const override { return "nvidia"; }
    const TargetInfo& target_info() const override { return target_info_; }
    // machine_code = launch plan decoded from the fused nodes; ptx_text = listing; one entrypoint
    // per function. A module without fused nodes compiles to a listing only (empty plan).
    std::unique_ptr<Executable> compile(const CGModule& module) override;
    std::optional<std::string> emit_text(const CGModule& module) override;

private:
    std::string sm_target_;
    TargetInfo target_info_;
};

// ---- runtime ----------------------------------------------------------------------------------------------
class Tensor {
public:
    Shape shape;
    DType dtype = DType::F32;
    DeviceId device;
    void* data = nullptr;
    u64 num_bytes = 0;
    bool owns_memory = false;
};

class Allocator {
public:
    virtual ~Allocator() = default;
    virtual void* allocate(u64 bytes, u64 alignment = 256) = 0;
    virtual void deallocate(void* p) = 0;
};

class Stream {
public:
    virtual ~Stream() = default;
    virtual void sync() = 0;
    virtual DeviceId device() const = 0;
};

class Event {
public:
    virtual ~Event() = default;
    virtual void record(Stream& s) = 0;
    virtual void wait() = 0;
    virtual double elapsed_sec_since(Event& earlier) = 0;
};

class Device {
public:
    virtual ~Device() = default;
    virtual DeviceId id() const = 0;
    virtual Allocator& allocator() = 0;
    virtual std::unique_ptr<Stream> create_stream() = 0;
    virtual std::unique_ptr<Event> create_event() = 0;
};

// The CUDA device over the C ABI; nullptr when `index` is not a usable sm_100 device.
std::unique_ptr<Device> make_cuda_device(u32 index);
// Host <-> device copies on a stream of that device (the reference's Tensor has no copy API).
int copy_to_device(Tensor& dst, const void* host_src, u64 bytes, Stream& s);
int copy_to_host(void* host_dst, const Tensor& src, u64 bytes, Stream& s);

template <typename T>
class Span {
public:
    Span(T* p, usize n) : p_(p), n_(n) {}
    Span(std::vector<T>& v) : p_(v.data()), n_(v.size()) {}
    T* data() const { return p_; }
    usize size() const { return n_; }
    T& operator[](usize i) const { return p_[i]; }

private:
    T* p_;
    usize n_;
};

class BoundExecutable {
public:
    virtual ~BoundExecutable() = default;
    virtual void launch(Span<Tensor*> inputs, Span<Tensor*> outputs, Stream& stream) = 0;
    virtual int status() const { return CG_B200_OK; }   // status of the last launch (the reference's launch is void)
};

class KernelCache {
public:
    explicit KernelCache(std::string dir) : dir_(std::move(dir)) {}
    std::optional<std::shared_ptr<Executable>> lookup(u64 key);
    void insert(u64 key, std::shared_ptr<Executable> exe);
    static u64 compute_key(const std::string& graph_text, const std::string& shapes, const std::string& dtypes,
                           const std::string& hardware_name);
    const std::string& dir() const { return dir_; }
    usize size() const { return mem_cache_.size(); }

private:
    std::string dir_;
    std::unordered_map<u64, std::shared_ptr<Executable>> mem_cache_;
};

class Runtime {
public:
    explicit Runtime(std::string cache_dir = ".cantors_cache");
    ~Runtime();
    void add_device(std::unique_ptr<Device> d);
    Device* get_device(DeviceId id) const;
    usize num_devices() const { return devices_.size(); }
    KernelCache& kernel_cache() { return cache_; }
    // Null on failure: no such device, or machine_code is not a launch plan.
    std::unique_ptr<BoundExecutable> bind(std::shared_ptr<Executable> exe, DeviceId device);
    struct CompileResult {
        std::shared_ptr<Executable> executable;
        bool cache_hit = false;
    };
    CompileResult compile_and_cache(u64 cache_key, const CGModule& cgm, MachineBackend& backend);
    // src/runtime/runtime.cpp:287-312 runs the search and then leaves compiling to the caller ("the
    // caller would lower the Tensor IR using the best schedule"). Here the caller passes that lowering
    // as `lower_best`, and the executable compiled from the winning schedule is what gets cached.
    struct AutotuneResult {
        std::shared_ptr<Executable> executable;
        bool cache_hit = false;
        double best_runtime = std::numeric_limits<double>::infinity();
        usize total_benchmarks = 0;
        Schedule best_schedule;
    };
    AutotuneResult autotune_and_cache(u64 cache_key, const ScheduleSpace& space, const BenchmarkFn& benchmark,
                                      MachineBackend& backend, const std::function<CGModule(const Schedule&)>& lower_best);

private:
    std::vector<std::unique_ptr<Device>> devices_;
    KernelCache cache_;
};

// ---- vendor dispatch ------------------------------------------------------------------------------------------
class VendorKernel {
public:
    virtual ~VendorKernel() = default;
    virtual std::string name() const = 0;
    virtual std::string vendor() const = 0;
    virtual bool supports(const Operation& op) const = 0;
    virtual double estimated_runtime(const Operation& op) const = 0;   // seconds
    // Runs the op on `stream`; false when this kernel cannot execute (the reference's stubs).
    virtual bool execute(const Operation&, Span<Tensor*>, Span<Tensor*>, Stream&) { return false; }
};

class VendorDispatcher {
public:
    static VendorDispatcher& instance();
    void register_kernel(std::unique_ptr<VendorKernel> k);
    const VendorKernel* find_best(const Operation& op, const Function& fn) const;
    bool has_vendor(const std::string& vendor) const;
    usize size() const { return kernels_.size(); }

private:
    VendorDispatcher();
    std::vector<std::unique_ptr<VendorKernel>> kernels_;
};

}  // namespace cg
