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
OVERLAY = os.path.join(HOST, "_overlay")


def overlay_paths():
    """Where the host layer's build products are: the reference library with the B200 layer in place, the
    test executables, the command-line tool and the two Python modules."""
    return {"lib": os.path.join(OVERLAY, "lib", "libcantors_gift.so"), "bin": os.path.join(OVERLAY, "bin"),
            "python": os.path.join(OVERLAY, "python", "cantors_gift")}


def build_host(reference_dir, jobs=8):
    """Builds the C++ host layer. It implements four translation units of the reference project against
    the reference's own headers, so it needs the reference's source tree (`reference_dir`); every other
    reference source is compiled from there too (host/Makefile). Without the tree nothing is built and
    products of an earlier build are used as they are. Needs libcg_b200.so and oracle/libcg_oracle.so."""
    if not reference_dir:
        have = os.path.exists(overlay_paths()["lib"])
        print("reference tree not found: host layer " + ("kept as built earlier" if have else "not built"))
        return None
    r = subprocess.run(["make", "-C", HOST, f"REF={reference_dir}", f"-j{jobs}", "all"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("host layer build failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return overlay_paths()["lib"]


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    ref = os.environ.get("CG_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    print(build_host(ref if os.path.isdir(os.path.join(ref, "src", "backend")) else None))
