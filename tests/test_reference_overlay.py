"""The drop-in, shown against the reference's own interfaces: cantors-gift_b200/host implements four of
the reference's translation units (NvidiaBackend, TensorToCodegenLowering, Runtime + KernelCache,
VendorDispatcher) against the reference's own headers, and host/Makefile links them with every other
reference source compiled from where it lies. Checked here:
  - the reference's own 25 test executables pass against that library (backend_tests, finishing_tests,
    correctness_tests, tectonic_tests ... string-match the old PTX text and the dispatcher's choices);
  - the reference's own python/bindings.cpp, compiled unmodified against it, passes the reference's
    tests/python/test_bindings.py (run when the reference tree is on this machine);
  - this layer's own tests (planner, plan and cache formats; on a GPU: graphs through Runtime::bind and
    launch against the CPU oracle);
  - on a GPU: graphs built with the reference's Python module run through cg_b200_ext, and the
    command-line tool's `--backend nvidia --jit-run` executes.
The library and executables are built by __graft_entry__.build() where the reference tree is present; on
a machine without it the products of that build are used as they are."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OVERLAY = os.path.join(ROOT, "cantors-gift_b200", "host", "_overlay")
BIN = os.path.join(OVERLAY, "bin")
PYDIR = os.path.join(OVERLAY, "python", "cantors_gift")

REFERENCE_TESTS = ["autotuner_tests", "backend_tests", "correctness_tests", "cost_tests", "egraph_rules_tests",
                   "egraph_superoptimizer_tests", "egraph_tests", "exploitation_tests", "finishing_tests",
                   "fusion_profitability_tests", "gta_tests", "integration_tests", "ir_tests", "layout_tests",
                   "matmul_pipeline_tests", "memory_ir_tests", "migrated_passes_tests", "optimization_tests", "passes_tests",
                   "schedule_tests", "shape_tests", "tectonic_tests", "unified_analyzer_tests", "unified_opts_tests",
                   "view_algebra_tests"]


def _reference_dir():
    cand = os.environ.get("CG_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "backend")) else None


def _need(path):
    if not os.path.exists(path):
        pytest.fail(f"{path} missing: run `python __graft_entry__.py` where the reference tree is present")


def _run(cmd, env=None, timeout=900, cwd=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=cwd)
    assert r.returncode == 0, f"{' '.join(cmd)}\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return r.stdout + r.stderr


@pytest.mark.parametrize("name", REFERENCE_TESTS)
def test_reference_test_executable_passes_against_the_overlay(name, tmp_path):
    exe = os.path.join(BIN, name)
    _need(exe)
    out = _run([exe], cwd=str(tmp_path))   # some of them write a .cantors_cache directory
    assert "0 failed" in out


def test_reference_python_bindings_tests_pass_against_the_overlay(tmp_path):
    ref = _reference_dir()
    if ref is None:
        pytest.skip("the reference tree (its tests/python/test_bindings.py) is not on this machine")
    _need(os.path.join(PYDIR, "cg_b200_ext" + __import__("sysconfig").get_config_var("EXT_SUFFIX")))
    out = _run([sys.executable, "-m", "pytest", os.path.join(ref, "tests", "python", "test_bindings.py"), "-q",
                "-p", "no:cacheprovider"], env={"PYTHONPATH": PYDIR}, cwd=str(tmp_path))
    assert " passed" in out and "failed" not in out


def test_layer_tests_host_side(tmp_path):
    exe = os.path.join(BIN, "b200_overlay_tests")
    _need(exe)
    out = _run([exe], env={"CG_B200_TEST_GPU": "0"}, cwd=str(tmp_path))
    assert "0 failed" in out


def test_python_modules_compile_a_graph_without_a_device(tmp_path):
    code = (
        "import cantors_gift as cg, cg_b200_ext as ext\n"
        "m = cg.Module(); ty = cg.tensor_type([64, 64], cg.DType.F32)\n"
        "f = m.create_function('mm', [ty, ty], [ty]); b = cg.Builder(f)\n"
        "b.output_tensor(b.relu(b.matmul(f.args()[0], f.args()[1])))\n"
        "cgm = cg.TensorToCodegenLowering().lower(m); assert ext.last_lowering_status() == 0\n"
        "nv = cg.NvidiaBackend(); assert nv.target_info().name == 'nvidia_sm_80'\n"
        "exe = nv.compile(cgm)\n"
        "assert 'fma.rn' in exe.ptx_text and 'bar.sync' in exe.ptx_text and ext.plan_summary(exe) == ['gemm']\n"
        "rt = cg.Runtime(); assert rt.num_devices() == 0 and ext.bind(rt, exe, 0) is None\n"
        "res = rt.compile_and_cache(cg.KernelCache.compute_key('mm', '64', 'f32', 'b200'), cgm, nv)\n"
        "assert not res.cache_hit and rt.kernel_cache().size() == 1\n"
        "assert ext.hardware_model().num_cores == 148\n"
        "print('ok')\n")
    out = _run([sys.executable, "-c", code], env={"PYTHONPATH": PYDIR}, cwd=str(tmp_path))
    assert "ok" in out


@pytest.mark.gpu
def test_layer_tests_on_the_gpu(tmp_path):
    exe = os.path.join(BIN, "b200_overlay_tests")
    _need(exe)
    out = _run([exe], env={"CG_B200_TEST_GPU": "1"}, cwd=str(tmp_path))
    assert "0 failed" in out


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["chain", "block", "block_full"])
def test_graphs_run_through_the_reference_python_module(case, tmp_path):
    _need(PYDIR)
    out = _run([sys.executable, os.path.join(ROOT, "tests", "overlay_driver.py"), case], cwd=str(tmp_path), timeout=1200)
    assert " ok" in out


@pytest.mark.gpu
def test_cgc_nvidia_jit_run_executes(tmp_path):
    exe = os.path.join(BIN, "cgc")
    _need(exe)
    out = _run([exe, "--backend", "nvidia", "--jit-run", "--sm-target", "sm_100a", "--matmul", "1024,1024,1024", "-o",
                str(tmp_path / "out.ptx")], cwd=str(tmp_path))
    assert "kernel(s) on cuda:0" in out and "(ok)" in out
    text = (tmp_path / "out.ptx").read_text()
    assert ".entry" in text and "cg_b200_gemm" in text
