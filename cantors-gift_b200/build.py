"""Builds libcg_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python build.py [--force]. Objects are rebuilt when a source or header is newer.
nvcc cross-compiles without a GPU, so this runs on a CPU-only machine too.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libcg_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    t = os.path.getmtime(os.path.join(ROOT, "include", "cg_b200.h"))
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h")):
            t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def _compile(src, force, hdr_t, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_t):
        return obj, False
    cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj, True


def build_library(force=False, verbose=False):
    """Compiles every .cu under csrc/ and links lib/libcg_b200.so. Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_t = _headers_mtime()
    with ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(lambda s: _compile(s, force, hdr_t, verbose), _sources()))
    objs = [o for o, _ in results]
    if force or any(c for _, c in results) or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-Xlinker", "--no-undefined", "-ldl", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


HOST = os.path.join(HERE, "host")
HOST_LIB = os.path.join(LIB_DIR, "libcg_b200_host.so")
HOST_TESTS = os.path.join(LIB_DIR, "host_tests")


def build_host(force=False):
    """Builds the C++ host layer (libcg_b200_host.so) and its test executable (lib/host_tests,
    which also links the CPU oracle as its checker). Needs libcg_b200.so and oracle/libcg_oracle.so."""
    cxx = os.environ.get("CG_B200_CXX", "g++")   # the system compiler: its libstdc++ is the shared one torch also loads
    srcs = sorted(os.path.join(HOST, "src", f) for f in os.listdir(os.path.join(HOST, "src")) if f.endswith(".cpp"))
    hdr = os.path.join(HOST, "include", "cg", "b200_host.hpp")
    newest = max([os.path.getmtime(p) for p in srcs + [hdr, os.path.join(ROOT, "include", "cg_b200.h")]])
    common = ["-std=c++20", "-O2", "-Wall", "-Wextra", "-I" + os.path.join(HOST, "include"), "-I" + os.path.join(ROOT, "include")]
    if force or not os.path.exists(HOST_LIB) or os.path.getmtime(HOST_LIB) < newest:
        cmd = [cxx] + common + ["-fPIC", "-shared", "-o", HOST_LIB] + srcs + ["-L" + LIB_DIR, "-lcg_b200", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host library build failed:\n{r.stdout}\n{r.stderr}")
    test_src = os.path.join(HOST, "tests", "host_tests.cpp")
    oracle_dir = os.path.join(ROOT, "oracle")
    if os.path.exists(os.path.join(oracle_dir, "libcg_oracle.so")) and (
            force or not os.path.exists(HOST_TESTS) or os.path.getmtime(HOST_TESTS) < max(newest, os.path.getmtime(test_src))
            or os.path.getmtime(HOST_TESTS) < os.path.getmtime(HOST_LIB)):
        cmd = [cxx] + common + ["-ffp-contract=off", "-o", HOST_TESTS, test_src, "-L" + LIB_DIR, "-lcg_b200_host", "-lcg_b200",
                                "-L" + oracle_dir, "-lcg_oracle", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../oracle"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host tests build failed:\n{r.stdout}\n{r.stderr}")
    build_host_python(force, newest)
    return HOST_LIB


def host_python_module_path():
    import sysconfig
    return os.path.join(LIB_DIR, "cg_b200_host" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_host_python(force=False, newest=0.0):
    """The pybind11 module over libcg_b200_host.so (skipped, with a note, where pybind11 is absent)."""
    try:
        import pybind11
    except ImportError:
        print("pybind11 not importable: the Python module of the host layer is not built")
        return None
    import sysconfig
    cxx = os.environ.get("CG_B200_CXX", "g++")   # the system compiler: its libstdc++ is the shared one torch also loads
    src = os.path.join(HOST, "python", "bindings.cpp")
    out = host_python_module_path()
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(newest, os.path.getmtime(src), os.path.getmtime(HOST_LIB)):
        return out
    cmd = [cxx, "-std=c++20", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(HOST, "include"), "-I" + os.path.join(ROOT, "include"),
           "-o", out, src, "-L" + LIB_DIR, "-lcg_b200_host", "-lcg_b200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host python module build failed:\n{r.stdout}\n{r.stderr}")
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_host(force="--force" in sys.argv))
