"""The C++ host layer from Python: the pybind11 module `cg_b200_host` built by build.py.

`host()` returns the module. Its classes carry the names the reference's `cantors_gift` module uses
(Module, Builder, TensorToCodegenLowering, NvidiaBackend, Executable, Runtime, KernelCache, Schedule,
ScheduleSpace ...), and add what the reference has no Python surface for: `Runtime.add_cuda_device`,
`Tensor.from_ptr`, `Runtime.bind` and `BoundExecutable.launch`. `tensor_of(t)` wraps a torch tensor.
"""
import importlib.util
import os
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
_mod = None


def module_path():
    return os.path.join(_HERE, "lib", "cg_b200_host" + sysconfig.get_config_var("EXT_SUFFIX"))


def host():
    global _mod
    if _mod is None:
        path = module_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `python __graft_entry__.py` (or cantors-gift_b200/build.py) first")
        spec = importlib.util.spec_from_file_location("cg_b200_host", path)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


_DTYPE_NAMES = {"torch.float32": "F32", "torch.bfloat16": "BF16", "torch.float16": "F16"}


def tensor_of(t):
    """A host-layer Tensor over a contiguous CUDA torch tensor's memory (the torch tensor keeps ownership)."""
    h = host()
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("tensor_of wants a contiguous CUDA tensor")
    return h.Tensor.from_ptr(t.data_ptr(), list(t.shape), getattr(h.DType, _DTYPE_NAMES[str(t.dtype)]),
                             h.DeviceId.cuda(t.device.index or 0))
