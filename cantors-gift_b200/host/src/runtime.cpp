// runtime.cpp - CUDA Device / Allocator / Stream / Event, the bound executable that walks a launch
// plan, KernelCache and Runtime.
//
// The reference's runtime is host-only (src/runtime/runtime.cpp:15-104): a malloc allocator, a
// no-op stream, an event whose elapsed time is 0, a CPUBoundExecutable that calls JIT-ed code, and
// Runtime::bind returns nullptr for every GPU (:120-129). KernelCache keeps the reference's file
// format byte for byte (:149-267) so cache directories stay interchangeable.
#include <cstring>
#include <filesystem>
#include <fstream>

#include "cg/b200_host.hpp"

namespace cg {
namespace {

class CudaAllocator final : public Allocator {
public:
    explicit CudaAllocator(u32 index) : index_(index) {}
    void* allocate(u64 bytes, u64 /*alignment: device allocations are 256-byte aligned*/) override {
        void* p = nullptr;
        if (cg_b200_set_device(static_cast<int>(index_)) != CG_B200_OK) return nullptr;
        return cg_b200_malloc(&p, bytes) == CG_B200_OK ? p : nullptr;
    }
    void deallocate(void* p) override { cg_b200_free(p); }

private:
    u32 index_;
};

class CudaStream final : public Stream {
public:
    explicit CudaStream(DeviceId d) : dev_(d) {
        cg_b200_set_device(static_cast<int>(d.index));
        cg_b200_stream_create(&s_);
    }
    ~CudaStream() override { cg_b200_stream_destroy(s_); }
    void sync() override { cg_b200_stream_sync(s_); }
    DeviceId device() const override { return dev_; }
    void* handle() const { return s_; }

private:
    DeviceId dev_;
    void* s_ = nullptr;
};

class CudaEvent final : public Event {
public:
    CudaEvent() { cg_b200_event_create(&e_); }
    ~CudaEvent() override { cg_b200_event_destroy(e_); }
    void record(Stream& s) override { cg_b200_event_record(e_, static_cast<CudaStream&>(s).handle()); }
    void wait() override { cg_b200_event_sync(e_); }
    double elapsed_sec_since(Event& earlier) override {
        double sec = 0.0;
        cg_b200_event_elapsed_sec(static_cast<CudaEvent&>(earlier).e_, e_, &sec);
        return sec;
    }

private:
    void* e_ = nullptr;
};

class CudaDevice final : public Device {
public:
    explicit CudaDevice(u32 index) : id_(DeviceId::cuda(index)), alloc_(index) {}
    DeviceId id() const override { return id_; }
    Allocator& allocator() override { return alloc_; }
    std::unique_ptr<Stream> create_stream() override { return std::make_unique<CudaStream>(id_); }
    std::unique_ptr<Event> create_event() override {
        cg_b200_set_device(static_cast<int>(id_.index));
        return std::make_unique<CudaEvent>();
    }

private:
    DeviceId id_;
    CudaAllocator alloc_;
};

// Walks the plan: one C-ABI call per record, asynchronous on the caller's stream.
class CudaBoundExecutable final : public BoundExecutable {
public:
    CudaBoundExecutable(std::shared_ptr<Executable> exe, LaunchPlan plan, Device* dev)
        : exe_(std::move(exe)), plan_(std::move(plan)), dev_(dev) {
        const usize first = plan_.n_inputs + plan_.n_outputs;
        scratch_.assign(plan_.buffers.size(), nullptr);
        for (usize i = first; i < plan_.buffers.size(); ++i) {
            scratch_[i] = dev_->allocator().allocate(plan_.buffers[i].bytes ? plan_.buffers[i].bytes : 1);
            if (!scratch_[i]) ok_ = false;
        }
        if (plan_.workspace_bytes) {
            workspace_ = dev_->allocator().allocate(plan_.workspace_bytes);
            if (!workspace_) ok_ = false;
        }
    }
    ~CudaBoundExecutable() override {
        for (void* p : scratch_)
            if (p) dev_->allocator().deallocate(p);
        if (workspace_) dev_->allocator().deallocate(workspace_);
    }
    bool ok() const { return ok_; }
    int status() const override { return status_; }

    void launch(Span<Tensor*> inputs, Span<Tensor*> outputs, Stream& stream) override {
        status_ = CG_B200_OK;
        if (inputs.size() != plan_.n_inputs || outputs.size() != plan_.n_outputs) {
            status_ = CG_B200_ERR_INVALID_ARG;
            return;
        }
        std::vector<void*> buf(scratch_);
        for (usize i = 0; i < inputs.size(); ++i) {
            if (!inputs[i] || inputs[i]->num_bytes < plan_.buffers[i].bytes) { status_ = CG_B200_ERR_INVALID_ARG; return; }
            buf[i] = inputs[i]->data;
        }
        for (usize i = 0; i < outputs.size(); ++i) {
            const usize b = plan_.n_inputs + i;
            if (!outputs[i] || outputs[i]->num_bytes < plan_.buffers[b].bytes) { status_ = CG_B200_ERR_INVALID_ARG; return; }
            buf[b] = outputs[i]->data;
        }
        void* st = static_cast<CudaStream&>(stream).handle();
        auto at = [&](i32 id) -> void* { return id >= 0 ? buf[static_cast<usize>(id)] : nullptr; };
        for (const PlanRecord& r : plan_.records) {
            int s = CG_B200_OK;
            switch (r.kind) {
                case PlanRecord::Eltwise: {
                    const void* ptrs[CG_B200_EW_MAX_INPUTS] = {};
                    for (i32 k = 0; k < r.n_inputs; ++k) ptrs[k] = at(r.input[k]);
                    s = cg_b200_eltwise(&r.eltwise, ptrs, r.n_inputs, at(r.output), r.n, st);
                    break;
                }
                case PlanRecord::Gemm:
                    s = cg_b200_gemm_tuned(&r.gemm, &r.tuning, at(r.input[0]), at(r.input[1]), at(r.input[2]), at(r.input[3]),
                                           at(r.output), workspace_, plan_.workspace_bytes, st);
                    break;
                case PlanRecord::Softmax:
                    s = cg_b200_softmax(r.row_dtype, at(r.input[0]), at(r.output), r.rows, r.cols, st);
                    break;
                case PlanRecord::LayerNorm:
                    s = cg_b200_layernorm(r.row_dtype, at(r.input[0]), nullptr, nullptr, r.eps, at(r.output), r.rows, r.cols, st);
                    break;
                case PlanRecord::SoftmaxLayerNorm:
                    s = cg_b200_softmax_layernorm(r.row_dtype, at(r.input[0]), nullptr, nullptr, r.eps, at(r.output), r.rows,
                                                  r.cols, st);
                    break;
                default: s = CG_B200_ERR_INVALID_ARG;
            }
            if (s != CG_B200_OK) {   // the reference's launch returns silently on failure; the status is kept
                status_ = s;
                return;
            }
        }
    }

private:
    std::shared_ptr<Executable> exe_;
    LaunchPlan plan_;
    Device* dev_;
    std::vector<void*> scratch_;
    void* workspace_ = nullptr;
    bool ok_ = true;
    int status_ = CG_B200_OK;
};

}  // namespace

std::unique_ptr<Device> make_cuda_device(u32 index) {
    int count = 0;
    if (cg_b200_device_count(&count) != CG_B200_OK || static_cast<int>(index) >= count) return nullptr;
    cg_b200_props props;
    if (cg_b200_device_props(static_cast<int>(index), &props) != CG_B200_OK || props.cc_major != 10) return nullptr;
    return std::make_unique<CudaDevice>(index);
}

int copy_to_device(Tensor& dst, const void* host_src, u64 bytes, Stream& s) {
    if (bytes > dst.num_bytes) return CG_B200_ERR_INVALID_ARG;
    return cg_b200_memcpy_h2d(dst.data, host_src, bytes, static_cast<CudaStream&>(s).handle());
}

int copy_to_host(void* host_dst, const Tensor& src, u64 bytes, Stream& s) {
    if (bytes > src.num_bytes) return CG_B200_ERR_INVALID_ARG;
    return cg_b200_memcpy_d2h(host_dst, src.data, bytes, static_cast<CudaStream&>(s).handle());
}

// ---- KernelCache: the reference's format, field for field --------------------------------------------------
u64 KernelCache::compute_key(const std::string& graph_text, const std::string& shapes, const std::string& dtypes,
                             const std::string& hardware_name) {
    u64 h = 0xcbf29ce484222325ULL;   // FNV-1a, 64 bit
    for (const std::string* s : {&graph_text, &shapes, &dtypes, &hardware_name})
        for (char c : *s) {
            h ^= static_cast<u64>(static_cast<u8>(c));
            h *= 0x100000001b3ULL;
        }
    return h;
}

namespace {
constexpr u32 kCacheMagic = 0x454B4743;   // "CGKE"
struct Reader {
    std::ifstream& in;
    template <typename T> T num() { T v{}; in.read(reinterpret_cast<char*>(&v), sizeof(T)); return v; }
    std::string str() {
        const u64 len = num<u64>();
        if (!in || len > (1ull << 32)) { in.setstate(std::ios::failbit); return {}; }
        std::string s(len, '\0');
        in.read(s.data(), static_cast<std::streamsize>(len));
        return s;
    }
};
struct Writer {
    std::ofstream& out;
    template <typename T> void num(T v) { out.write(reinterpret_cast<const char*>(&v), sizeof(T)); }
    void str(const std::string& s) { num<u64>(s.size()); out.write(s.data(), static_cast<std::streamsize>(s.size())); }
};
}  // namespace

std::optional<std::shared_ptr<Executable>> KernelCache::lookup(u64 key) {
    if (auto it = mem_cache_.find(key); it != mem_cache_.end()) return it->second;
    namespace fs = std::filesystem;
    const fs::path path = fs::path(dir_) / (std::to_string(key) + ".cgbin");
    std::error_code ec;
    if (!fs::exists(path, ec)) return std::nullopt;
    std::ifstream in(path, std::ios::binary);
    if (!in) return std::nullopt;
    Reader r{in};
    if (r.num<u32>() != kCacheMagic || r.num<u32>() != 1) return std::nullopt;
    auto exe = std::make_shared<Executable>();
    exe->name = r.str();
    exe->target_device.kind = static_cast<DeviceId::Kind>(r.num<u64>());
    exe->target_device.index = r.num<u32>();
    const std::string code = r.str();
    exe->machine_code.assign(code.begin(), code.end());
    exe->ptx_text = r.str();
    exe->disassembly = r.str();
    const u64 n_entry = r.num<u64>();
    for (u64 i = 0; in && i < n_entry && i < (1u << 20); ++i) {
        std::string name = r.str();
        const u64 offset = r.num<u64>();
        exe->entrypoints.push_back({std::move(name), offset});
    }
    exe->shared_mem_bytes = r.num<u64>();
    exe->constant_mem_bytes = r.num<u64>();
    exe->threads_per_block = r.num<u32>();
    if (!in) return std::nullopt;   // truncated file
    mem_cache_[key] = exe;
    return exe;
}

void KernelCache::insert(u64 key, std::shared_ptr<Executable> exe) {
    mem_cache_[key] = exe;
    namespace fs = std::filesystem;
    std::error_code ec;
    fs::create_directories(dir_, ec);
    std::ofstream out(fs::path(dir_) / (std::to_string(key) + ".cgbin"), std::ios::binary);
    if (!out) return;
    Writer w{out};
    w.num<u32>(kCacheMagic);
    w.num<u32>(1);
    w.str(exe->name);
    w.num<u64>(static_cast<u64>(exe->target_device.kind));
    w.num<u32>(exe->target_device.index);
    w.str(std::string(exe->machine_code.begin(), exe->machine_code.end()));
    w.str(exe->ptx_text);
    w.str(exe->disassembly);
    w.num<u64>(exe->entrypoints.size());
    for (const auto& [name, offset] : exe->entrypoints) {
        w.str(name);
        w.num<u64>(offset);
    }
    w.num<u64>(exe->shared_mem_bytes);
    w.num<u64>(exe->constant_mem_bytes);
    w.num<u32>(exe->threads_per_block);
}

// ---- Runtime ----------------------------------------------------------------------------------------------------
Runtime::Runtime(std::string cache_dir) : cache_(std::move(cache_dir)) {}
Runtime::~Runtime() = default;

void Runtime::add_device(std::unique_ptr<Device> d) {
    if (d) devices_.push_back(std::move(d));
}

Device* Runtime::get_device(DeviceId id) const {
    for (const auto& d : devices_)
        if (d->id() == id) return d.get();
    return nullptr;
}

std::unique_ptr<BoundExecutable> Runtime::bind(std::shared_ptr<Executable> exe, DeviceId device) {
    if (!exe || device.kind != DeviceId::Kind::CUDA) return nullptr;   // this runtime has no CPU path
    Device* dev = get_device(device);
    if (!dev) return nullptr;
    auto plan = LaunchPlan::deserialize(exe->machine_code);
    if (!plan) return nullptr;
    auto bound = std::make_unique<CudaBoundExecutable>(std::move(exe), std::move(*plan), dev);
    if (!bound->ok()) return nullptr;
    return bound;
}

Runtime::CompileResult Runtime::compile_and_cache(u64 cache_key, const CGModule& cgm, MachineBackend& backend) {
    CompileResult res;
    if (auto hit = cache_.lookup(cache_key)) {
        res.executable = *hit;
        res.cache_hit = true;
        return res;
    }
    res.executable = std::shared_ptr<Executable>(backend.compile(cgm).release());
    if (res.executable) cache_.insert(cache_key, res.executable);
    return res;
}

}  // namespace cg

// ---- schedules and autotuning ---------------------------------------------------------------------------
namespace cg {

static u64 mix(u64 h, u64 v) {   // FNV-1a over 64-bit words
    h ^= v;
    return h * 1099511628211ull;
}

u64 Schedule::hash() const {
    u64 h = 1469598103934665603ull;
    for (const Transform& t : transforms_) {
        h = mix(h, static_cast<u64>(t.kind));
        for (char c : t.dim) h = mix(h, static_cast<u8>(c));
        h = mix(h, static_cast<u64>(t.factor));
        h = mix(h, static_cast<u64>(t.factor2));
        for (char c : t.target) h = mix(h, static_cast<u8>(c));
    }
    return h;
}

bool Schedule::operator==(const Schedule& o) const {
    if (transforms_.size() != o.transforms_.size()) return false;
    for (usize i = 0; i < transforms_.size(); ++i) {
        const Transform &a = transforms_[i], &b = o.transforms_[i];
        if (a.kind != b.kind || a.dim != b.dim || a.factor != b.factor || a.factor2 != b.factor2 || a.target != b.target)
            return false;
    }
    return true;
}

ScheduleSpace ScheduleSpace::grid_matmul(std::vector<i64> m_tiles, std::vector<i64> n_tiles, std::vector<i64> k_tiles,
                                         std::vector<i64> vector_widths) {
    ScheduleSpace space;
    for (i64 m : m_tiles)
        for (i64 n : n_tiles)
            for (i64 k : k_tiles)
                for (i64 v : vector_widths) {
                    Schedule s;
                    s.add({TransformKind::Tile, "m", m, n, ""});
                    s.add({TransformKind::Tile, "n", n, 0, ""});
                    s.add({TransformKind::Tile, "k", k, 0, ""});
                    s.add({TransformKind::Parallelize, "m", 0, 0, ""});
                    s.add({TransformKind::Parallelize, "n", 0, 0, ""});
                    s.add({TransformKind::Vectorize, "n_inner", v, 0, ""});
                    s.add({TransformKind::Cache, "a", 0, 0, "A"});
                    s.add({TransformKind::Cache, "b", 0, 0, "B"});
                    space.add(std::move(s));
                }
    return space;
}

AutotuneResult bayesian_autotune(const ScheduleSpace& space, BenchmarkFn benchmark, usize max_benchmarks, usize initial_random) {
    (void)initial_random;
    AutotuneResult res;
    if (!benchmark) return res;
    for (const Schedule& s : space.schedules()) {
        if (res.total_benchmarks >= max_benchmarks) break;
        const double t = benchmark(s);
        res.runtime_history.push_back(t);
        ++res.total_benchmarks;
        if (t < res.best_runtime) {
            res.best_runtime = t;
            res.best_schedule = s;
        }
    }
    return res;
}

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

namespace {
struct GemmBenchState {
    cg_b200_gemm_desc desc{};
    Device* device = nullptr;
    std::unique_ptr<Stream> stream;
    std::unique_ptr<Event> begin, end;
    void *a = nullptr, *b = nullptr, *c = nullptr, *bias = nullptr, *res = nullptr, *ws = nullptr;
    size_t ws_bytes = 0;
    int iters = 20, warmup = 3;
    bool ok = false;
    ~GemmBenchState() {
        if (!device) return;
        for (void* p : {a, b, c, bias, res, ws})
            if (p) device->allocator().deallocate(p);
    }
};
u64 elem_bytes(int dtype) { return dtype == CG_B200_F32 ? 4 : 2; }
void* stream_handle(Stream& s) { return static_cast<CudaStream&>(s).handle(); }
}  // namespace

BenchmarkFn make_gemm_benchmark(const cg_b200_gemm_desc& desc, Device& device, int iters, int warmup) {
    auto st = std::make_shared<GemmBenchState>();
    st->desc = desc;
    st->device = &device;
    st->iters = iters > 0 ? iters : 1;
    st->warmup = warmup >= 0 ? warmup : 0;
    st->stream = device.create_stream();
    st->begin = device.create_event();
    st->end = device.create_event();
    const cg_b200_gemm_desc& d = st->desc;
    const u64 in = elem_bytes(d.in_dtype), out = elem_bytes(d.out_dtype);
    const i64 b_rows = d.b_transposed ? d.N : d.K;
    const u64 a_bytes = static_cast<u64>((d.batch_stride_a ? d.batch_stride_a * d.batch : d.M * d.lda)) * in;
    const u64 b_bytes = static_cast<u64>((d.batch_stride_b ? d.batch_stride_b * d.batch : b_rows * d.ldb)) * in;
    const u64 c_bytes = static_cast<u64>((d.batch_stride_c ? d.batch_stride_c * d.batch : d.M * d.ldc)) * out;
    auto zeroed = [&](u64 bytes) -> void* {
        void* p = device.allocator().allocate(bytes ? bytes : 16);
        if (p) cg_b200_memset(p, 0, bytes ? bytes : 16, nullptr);
        return p;
    };
    st->a = zeroed(a_bytes);
    st->b = zeroed(b_bytes);
    st->c = zeroed(c_bytes);
    st->bias = zeroed(static_cast<u64>(d.N) * out);
    st->res = zeroed(c_bytes);
    if (cg_b200_gemm_workspace_bytes(&st->desc, &st->ws_bytes) == CG_B200_OK && st->ws_bytes) st->ws = zeroed(st->ws_bytes);
    st->ok = st->stream && st->begin && st->end && st->a && st->b && st->c && st->bias && st->res && (st->ws || !st->ws_bytes);
    cg_b200_stream_sync(nullptr);
    return [st](const Schedule& s) -> double {
        const double never = std::numeric_limits<double>::infinity();
        if (!st->ok) return never;
        const auto tuning = gemm_tuning_from_schedule(s);
        if (!tuning) return never;
        void* h = stream_handle(*st->stream);
        auto once = [&]() {
            return cg_b200_gemm_tuned(&st->desc, &*tuning, st->a, st->b, st->bias, st->res, st->c, st->ws, st->ws_bytes, h);
        };
        for (int i = 0; i < st->warmup + 1; ++i)
            if (once() != CG_B200_OK) return never;   // refused combinations end here
        st->begin->record(*st->stream);
        for (int i = 0; i < st->iters; ++i)
            if (once() != CG_B200_OK) return never;
        st->end->record(*st->stream);
        st->end->wait();
        uint32_t word = 0;
        if (cg_b200_last_device_error(h, &word) != CG_B200_OK || word != 0) return never;
        return st->end->elapsed_sec_since(*st->begin) / st->iters;
    };
}

Runtime::AutotuneResult Runtime::autotune_and_cache(u64 cache_key, const ScheduleSpace& space, const BenchmarkFn& benchmark,
                                                    MachineBackend& backend,
                                                    const std::function<CGModule(const Schedule&)>& lower_best) {
    AutotuneResult res;
    if (auto hit = cache_.lookup(cache_key)) {
        res.executable = *hit;
        res.cache_hit = true;
        return res;
    }
    const cg::AutotuneResult tuned = bayesian_autotune(space, benchmark);
    res.best_runtime = tuned.best_runtime;
    res.total_benchmarks = tuned.total_benchmarks;
    res.best_schedule = tuned.best_schedule;
    if (!(tuned.best_runtime < std::numeric_limits<double>::infinity()) || !lower_best) return res;   // nothing ran
    const CGModule cgm = lower_best(tuned.best_schedule);
    res.executable = std::shared_ptr<Executable>(backend.compile(cgm).release());
    if (res.executable) cache_.insert(cache_key, res.executable);
    return res;
}

}  // namespace cg
