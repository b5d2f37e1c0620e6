// b200_bindings.cpp - Python module cg_b200_ext: what the reference's python/bindings.cpp does not bind.
//
// That file (compiled unmodified against this layer) exposes Module / Builder / TensorToCodegenLowering /
// NvidiaBackend / Executable / Runtime / KernelCache, but Runtime.add_device takes a unique_ptr<Device>
// no Python class can supply, and Runtime::bind, Tensor, Stream and BoundExecutable are not bound at all
// (python/bindings.cpp:1445-1470), so a compiled graph could not be run from Python even if a GPU path
// existed. This module adds exactly those pieces. It shares the reference module's registered types
// (import cantors_gift first): functions here take its Runtime, Executable, Module and Schedule objects.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cg/b200/b200.hpp"
#include "cg/b200/plan.hpp"
#include "cg/backend/nvidia_backend.hpp"

namespace py = pybind11;
using namespace cg;

namespace {

// A bound executable together with what keeps it valid.
struct Bound {
    std::unique_ptr<BoundExecutable> exe;
    u32 device_index = 0;
};

struct StreamHandle {
    std::unique_ptr<Stream> s;
};

std::vector<i64> dims_of(const Tensor& t) {
    std::vector<i64> d;
    for (const auto& x : t.shape) d.push_back(x->value);
    return d;
}

}  // namespace

PYBIND11_MODULE(cg_b200_ext, m) {
    m.doc() = "CUDA devices, tensors, bind and launch for the cantors_gift module on B200";
    py::module_::import("cantors_gift");   // the shared type registrations

    py::class_<Tensor>(m, "Tensor")
        .def_property_readonly("shape", &dims_of)
        .def_readonly("dtype", &Tensor::dtype)
        .def_readonly("num_bytes", &Tensor::num_bytes)
        .def_readonly("owns_memory", &Tensor::owns_memory)
        .def_property_readonly("data_ptr", [](const Tensor& t) { return reinterpret_cast<std::uintptr_t>(t.data); })
        .def_static("from_ptr", [](std::uintptr_t ptr, std::vector<i64> shape, DType dt, u32 device) {
            return b200::tensor_from_ptr(reinterpret_cast<void*>(ptr), std::move(shape), dt, device);
        }, py::arg("ptr"), py::arg("shape"), py::arg("dtype"), py::arg("device") = 0,
           "A tensor over device memory the caller owns (for example another framework's buffer).");

    py::class_<StreamHandle>(m, "Stream")
        .def("sync", [](StreamHandle& s) { s.s->sync(); })
        .def_property_readonly("cuda_stream", [](StreamHandle& s) { return reinterpret_cast<std::uintptr_t>(b200::native_stream(*s.s)); });

    py::class_<Bound>(m, "BoundExecutable")
        .def("launch", [](Bound& b, std::vector<Tensor*> inputs, std::vector<Tensor*> outputs, StreamHandle& s) {
            b.exe->launch(inputs, outputs, *s.s);
            return b200::last_launch_status();
        }, "Enqueues every kernel of the plan on the stream; returns the cg_b200 status (0 = ok).")
        .def("set_output_gather", [](Bound& b, std::vector<std::uintptr_t> peers, int world, int rank) {
            std::vector<void*> p;
            for (auto x : peers) p.push_back(reinterpret_cast<void*>(x));
            return b200::set_output_gather(*b.exe, p.data(), world, rank);
        });

    m.def("add_cuda_device", [](Runtime& rt, u32 index) {
        auto d = b200::make_cuda_device(index);
        if (!d) return false;
        rt.add_device(std::move(d));
        return true;
    }, py::arg("runtime"), py::arg("index") = 0, "Registers CUDA device `index` with the runtime; False if it is not a usable sm_100 device.");

    m.def("bind", [](Runtime& rt, const Executable& exe, u32 index) -> std::unique_ptr<Bound> {
        auto bound = rt.bind(std::make_shared<Executable>(exe), DeviceId::cuda(index));
        if (!bound) return nullptr;   // None, as Runtime::bind's nullptr
        auto b = std::make_unique<Bound>();
        b->exe = std::move(bound);
        b->device_index = index;
        return b;
    }, py::arg("runtime"), py::arg("executable"), py::arg("index") = 0, py::keep_alive<0, 1>());

    m.def("create_stream", [](Runtime& rt, u32 index) -> std::unique_ptr<StreamHandle> {
        Device* d = rt.get_device(DeviceId::cuda(index));
        if (!d) return nullptr;
        auto s = std::make_unique<StreamHandle>();
        s->s = d->create_stream();
        return s;
    }, py::arg("runtime"), py::arg("index") = 0, py::keep_alive<0, 1>());
    m.def("wrap_stream", [](std::uintptr_t cuda_stream, u32 index) {
        auto s = std::make_unique<StreamHandle>();
        s->s = b200::wrap_stream(reinterpret_cast<void*>(cuda_stream), index);
        return s;
    }, py::arg("cuda_stream"), py::arg("index") = 0, "A Stream over an existing cudaStream_t (not owned).");

    m.def("alloc", [](Runtime& rt, std::vector<i64> shape, DType dt, u32 index) {
        Device* d = rt.get_device(DeviceId::cuda(index));
        if (!d) throw std::runtime_error("no such CUDA device registered");
        Tensor t = b200::make_tensor(*d, std::move(shape), dt);
        if (!t.data) throw std::runtime_error("device allocation failed");
        return t;
    }, py::arg("runtime"), py::arg("shape"), py::arg("dtype"), py::arg("index") = 0);
    m.def("free", [](Runtime& rt, Tensor& t, u32 index) {
        if (Device* d = rt.get_device(DeviceId::cuda(index))) b200::release_tensor(*d, t);
    }, py::arg("runtime"), py::arg("tensor"), py::arg("index") = 0);
    m.def("copy_to_device", [](Tensor& dst, py::buffer src, StreamHandle& s) {
        py::buffer_info info = src.request();
        return b200::copy_to_device(dst, info.ptr, static_cast<u64>(info.size * info.itemsize), *s.s);
    });
    m.def("copy_to_host", [](py::buffer dst, const Tensor& src, StreamHandle& s) {
        py::buffer_info info = dst.request(true);
        const int st = b200::copy_to_host(info.ptr, src, static_cast<u64>(info.size * info.itemsize), *s.s);
        s.s->sync();
        return st;
    });

    m.def("last_lowering_status", &b200::last_lowering_status);
    m.def("last_lowering_message", &b200::last_lowering_message);
    m.def("last_launch_status", &b200::last_launch_status);
    m.def("status_string", [](int st) { return std::string(cg_b200_status_string(st)); });

    m.def("plan_summary", [](const Executable& exe) {
        py::list out;
        auto plan = b200::LaunchPlan::deserialize(exe.machine_code);
        if (!plan) return out;
        static const char* names[] = {"?", "eltwise", "gemm", "softmax", "layernorm", "softmax_layernorm", "attention", "reduce"};
        for (const auto& r : plan->records) out.append(std::string(names[r.kind <= 7 ? r.kind : 0]));
        return out;
    }, "Kernel names of the launch plan an Executable carries (empty for text-only executables).");

    m.def("gemm_tuning_from_schedule", [](const Schedule& s) -> py::object {
        auto t = b200::gemm_tuning_from_schedule(s);
        if (!t) return py::none();
        return py::make_tuple(t->tile_n, t->cta_pair, t->tail_split);
    });
    m.def("make_gemm_benchmark", [](Runtime& rt, const Module& mod, u32 index, int iters, int warmup) -> BenchmarkFn {
        Device* d = rt.get_device(DeviceId::cuda(index));
        auto desc = b200::first_gemm_desc(mod);
        if (!d || !desc) throw std::runtime_error("needs a registered CUDA device and a module with a matmul");
        return b200::make_gemm_benchmark(*desc, *d, iters, warmup);
    }, py::arg("runtime"), py::arg("module"), py::arg("index") = 0, py::arg("iters") = 20, py::arg("warmup") = 3,
       "A benchmark function (Schedule -> seconds) that times the real kernel; pass it to bayesian_autotune.");
    m.def("autotune_and_cache", [](Runtime& rt, u64 key, const Module& mod, const ScheduleSpace& space, const BenchmarkFn& fn) {
        NvidiaBackend nv("sm_100a");
        auto r = b200::autotune_and_cache(rt, key, mod, space, fn, nv);
        py::dict d;
        d["executable"] = r.executable ? py::cast(*r.executable) : py::none();
        d["best_runtime"] = r.best_runtime;
        d["total_benchmarks"] = r.total_benchmarks;
        d["cache_hit"] = r.cache_hit;
        return d;
    });
    m.def("hardware_model", [](const std::string& peaks_json) {
        return peaks_json.empty() ? b200::hardware_model() : b200::hardware_model(b200::load_calibration(peaks_json));
    }, py::arg("peaks_json") = "", "HardwareModel of a B200; peaks from the given measurement file when there is one.");
}
