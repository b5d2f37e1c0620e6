// Python surface of the C++ host layer, with the names the reference's module uses for the same things
// (python/bindings.cpp: DType :98, DeviceId :123, Value/Function/Module/Builder :352-534, Schedule and
// ScheduleSpace :764-815, Executable/NvidiaBackend :1040-1087, Runtime/KernelCache/CompileResult
// :1445-1470, LoweringOptions/TensorToCodegenLowering :1512-1530), plus what the reference could not
// offer from Python (runtime.hpp's Device, Tensor, Stream and Runtime::bind are not bound there): a CUDA
// device factory, a Tensor over a raw device pointer, bind() and launch().
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cg/b200_host.hpp"

namespace py = pybind11;
using namespace cg;

namespace {
// Streams are created by a device of the runtime and must not outlive it; the wrapper keeps the runtime alive.
struct PyStream {
    std::shared_ptr<Runtime> rt;
    std::unique_ptr<Stream> s;
};
struct PyBound {
    std::shared_ptr<Runtime> rt;
    std::unique_ptr<BoundExecutable> b;
};
}  // namespace

PYBIND11_MODULE(cg_b200_host, m) {
    m.doc() = "C++ host layer of the B200 execution path (NvidiaBackend, Runtime, lowering) for Python";

    py::enum_<DType>(m, "DType")
        .value("F16", DType::F16).value("BF16", DType::BF16).value("F32", DType::F32).value("F64", DType::F64)
        .value("I32", DType::I32).value("I64", DType::I64);
    py::enum_<DeviceId::Kind>(m, "DeviceKind")
        .value("CPU", DeviceId::Kind::CPU).value("CUDA", DeviceId::Kind::CUDA);
    py::class_<DeviceId>(m, "DeviceId")
        .def(py::init<>())
        .def_readwrite("kind", &DeviceId::kind)
        .def_readwrite("index", &DeviceId::index)
        .def_static("cpu", &DeviceId::cpu, py::arg("index") = 0)
        .def_static("cuda", &DeviceId::cuda, py::arg("index") = 0)
        .def("__eq__", [](const DeviceId& a, const DeviceId& b) { return a == b; });

    // ---- Tensor IR stand-in --------------------------------------------------------------------------
    py::class_<Value>(m, "Value").def_readonly("id", &Value::id).def("valid", &Value::valid);
    py::class_<Function>(m, "Function")
        .def("name", [](const Function& f) { return f.name; })
        .def("num_operations", [](const Function& f) { return f.ops.size() - 1; });
    py::class_<Module>(m, "Module")
        .def(py::init<>())
        .def("create_function", &Module::create_function, py::return_value_policy::reference_internal)
        .def("num_functions", [](const Module& mod) { return mod.functions.size(); });
    py::class_<Builder>(m, "Builder")
        .def(py::init<Function*>(), py::keep_alive<1, 2>())
        .def("input_tensor", &Builder::input_tensor)
        .def("constant_scalar", &Builder::constant_scalar)
        .def("output_tensor", &Builder::output_tensor)
        .def("add", &Builder::add).def("sub", &Builder::sub).def("mul", &Builder::mul).def("div", &Builder::div)
        .def("neg", &Builder::neg).def("relu", &Builder::relu).def("gelu", &Builder::gelu).def("exp", &Builder::exp)
        .def("sqrt", &Builder::sqrt).def("sigmoid", &Builder::sigmoid).def("tanh", &Builder::tanh).def("log", &Builder::log)
        .def("matmul", &Builder::matmul).def("reshape", &Builder::reshape)
        .def("softmax", &Builder::softmax).def("layernorm", &Builder::layernorm);

    // ---- schedules -----------------------------------------------------------------------------------
    py::enum_<TransformKind>(m, "TransformKind")
        .value("Split", TransformKind::Split).value("Tile", TransformKind::Tile)
        .value("Interchange", TransformKind::Interchange).value("Fuse", TransformKind::Fuse)
        .value("Vectorize", TransformKind::Vectorize).value("Parallelize", TransformKind::Parallelize)
        .value("Unroll", TransformKind::Unroll).value("Cache", TransformKind::Cache)
        .value("Pipeline", TransformKind::Pipeline).value("Prefetch", TransformKind::Prefetch)
        .value("Bind", TransformKind::Bind);
    py::class_<Transform>(m, "Transform")
        .def(py::init([](TransformKind k, std::string dim, i64 factor, i64 factor2, std::string target) {
                 return Transform{k, std::move(dim), factor, factor2, std::move(target)};
             }),
             py::arg("kind"), py::arg("dim"), py::arg("factor") = 0, py::arg("factor2") = 0, py::arg("target") = "")
        .def_readwrite("kind", &Transform::kind).def_readwrite("dim", &Transform::dim)
        .def_readwrite("factor", &Transform::factor).def_readwrite("factor2", &Transform::factor2)
        .def_readwrite("target", &Transform::target);
    py::class_<Schedule>(m, "Schedule")
        .def(py::init<>())
        .def("add", &Schedule::add)
        .def("transforms", &Schedule::transforms)
        .def("hash", &Schedule::hash);
    py::class_<ScheduleSpace>(m, "ScheduleSpace")
        .def(py::init<>())
        .def("add", &ScheduleSpace::add)
        .def("schedules", &ScheduleSpace::schedules)
        .def("size", &ScheduleSpace::size)
        .def_static("grid_matmul", &ScheduleSpace::grid_matmul);

    // ---- lowering and backend --------------------------------------------------------------------------
    py::class_<CGModule>(m, "CGModule").def("num_functions", [](const CGModule& c) { return c.functions.size(); });
    py::class_<LoweringOptions>(m, "LoweringOptions")
        .def(py::init<>())
        .def_readwrite("m_tile", &LoweringOptions::m_tile).def_readwrite("n_tile", &LoweringOptions::n_tile)
        .def_readwrite("k_tile", &LoweringOptions::k_tile)
        .def_readwrite("use_shared_memory", &LoweringOptions::use_shared_memory)
        .def_readwrite("use_tensor_cores", &LoweringOptions::use_tensor_cores)
        .def_readwrite("fuse_softmax_layernorm", &LoweringOptions::fuse_softmax_layernorm)
        .def_readwrite("layernorm_eps", &LoweringOptions::layernorm_eps);
    py::class_<TensorToCodegenLowering>(m, "TensorToCodegenLowering")
        .def(py::init<LoweringOptions>(), py::arg("options") = LoweringOptions{})
        .def("lower", &TensorToCodegenLowering::lower, py::arg("module"), py::arg("schedule") = Schedule{})
        .def("options", &TensorToCodegenLowering::options)
        .def("status", &TensorToCodegenLowering::status)
        .def("message", &TensorToCodegenLowering::message);
    py::class_<Executable, std::shared_ptr<Executable>>(m, "Executable")
        .def(py::init<>())
        .def_readwrite("name", &Executable::name)
        .def_readwrite("target_device", &Executable::target_device)
        .def_property("machine_code",
                      [](const Executable& e) { return py::bytes(reinterpret_cast<const char*>(e.machine_code.data()), e.machine_code.size()); },
                      [](Executable& e, const std::string& b) { e.machine_code.assign(b.begin(), b.end()); })
        .def_readwrite("ptx_text", &Executable::ptx_text)
        .def_readwrite("entrypoints", &Executable::entrypoints)
        .def_readwrite("shared_mem_bytes", &Executable::shared_mem_bytes)
        .def_readwrite("constant_mem_bytes", &Executable::constant_mem_bytes)
        .def_readwrite("threads_per_block", &Executable::threads_per_block)
        .def_readwrite("disassembly", &Executable::disassembly);
    py::class_<MachineBackend>(m, "MachineBackend");
    py::class_<NvidiaBackend, MachineBackend>(m, "NvidiaBackend")
        .def(py::init<std::string>(), py::arg("sm_target") = "sm_100a")
        .def("name", &NvidiaBackend::name)
        .def("compile", [](NvidiaBackend& b, const CGModule& c) { return std::shared_ptr<Executable>(b.compile(c).release()); })
        .def("emit_text", &NvidiaBackend::emit_text);

    // ---- runtime ---------------------------------------------------------------------------------------
    py::class_<Tensor>(m, "Tensor")
        .def(py::init<>())
        .def_static("from_ptr",
                    [](std::uintptr_t ptr, Shape shape, DType dt, DeviceId dev) {
                        Tensor t;
                        t.shape = std::move(shape);
                        t.dtype = dt;
                        t.device = dev;
                        t.data = reinterpret_cast<void*>(ptr);
                        t.num_bytes = static_cast<u64>(num_elements(t.shape)) * dtype_size(dt);
                        return t;
                    },
                    py::arg("ptr"), py::arg("shape"), py::arg("dtype"), py::arg("device"),
                    "A tensor over memory the caller owns (a torch tensor's data_ptr(), a cudaMalloc'd buffer)")
        .def_readwrite("shape", &Tensor::shape).def_readwrite("dtype", &Tensor::dtype)
        .def_readwrite("device", &Tensor::device).def_readwrite("num_bytes", &Tensor::num_bytes)
        .def_property_readonly("data", [](const Tensor& t) { return reinterpret_cast<std::uintptr_t>(t.data); });
    py::class_<PyStream>(m, "Stream").def("sync", [](PyStream& s) { s.s->sync(); });
    py::class_<PyBound>(m, "BoundExecutable")
        .def("launch",
             [](PyBound& b, std::vector<Tensor*> in, std::vector<Tensor*> out, PyStream& s) {
                 b.b->launch(Span<Tensor*>(in), Span<Tensor*>(out), *s.s);
             },
             "Asynchronous on `stream`; status() reports what the launch did")
        .def("status", [](PyBound& b) { return b.b->status(); });
    py::class_<KernelCache>(m, "KernelCache")
        .def("size", &KernelCache::size)
        .def("dir", &KernelCache::dir)
        .def_static("compute_key", &KernelCache::compute_key);
    py::class_<Runtime::CompileResult>(m, "CompileResult")
        .def_readonly("executable", &Runtime::CompileResult::executable)
        .def_readonly("cache_hit", &Runtime::CompileResult::cache_hit);
    py::class_<Runtime, std::shared_ptr<Runtime>>(m, "Runtime")
        .def(py::init<std::string>(), py::arg("cache_dir") = ".cantors_cache")
        .def("add_cuda_device",
             [](Runtime& rt, u32 index) {
                 auto d = make_cuda_device(index);
                 if (!d) return false;
                 rt.add_device(std::move(d));
                 return true;
             },
             py::arg("index") = 0, "Adds the CUDA device `index`; False when it is not a usable sm_100 device")
        .def("num_devices", &Runtime::num_devices)
        .def("kernel_cache", &Runtime::kernel_cache, py::return_value_policy::reference_internal)
        .def("create_stream",
             [](std::shared_ptr<Runtime> rt, DeviceId id) -> std::unique_ptr<PyStream> {
                 Device* d = rt->get_device(id);
                 if (!d) return nullptr;
                 return std::unique_ptr<PyStream>(new PyStream{rt, d->create_stream()});
             })
        .def("bind",
             [](std::shared_ptr<Runtime> rt, std::shared_ptr<Executable> exe, DeviceId id) -> std::unique_ptr<PyBound> {
                 auto b = rt->bind(std::move(exe), id);
                 if (!b) return nullptr;   // None, as Runtime::bind returns nullptr on failure
                 return std::unique_ptr<PyBound>(new PyBound{rt, std::move(b)});
             })
        .def("compile_and_cache", &Runtime::compile_and_cache);
    m.def("gemm_tuning_from_schedule", [](const Schedule& s) -> py::object {
        auto t = gemm_tuning_from_schedule(s);
        if (!t) return py::none();
        return py::make_tuple(t->tile_n, t->cta_pair, t->tail_split);
    });
}
