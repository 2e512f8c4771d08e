"""The complete reference-side binding (tests/binding/sm100_entry.cpp), compiled
against the reference's OWN headers: every public function of the hot path is DEFINED there with
the reference's declaration in scope, so a signature or record that drifted fails to compile."""
import os
import shutil
import subprocess

import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_binding_translation_unit_compiles_against_the_reference_headers(tmp_path):
    reference = O.reference_root()
    if not os.path.isdir(os.path.join(reference, "include", "fuse")):
        pytest.skip("the reference tree is not mounted here")
    compiler = shutil.which("g++", path="/usr/bin") or shutil.which("g++")
    if compiler is None:
        pytest.skip("no host C++ compiler")
    cutlass = subprocess.run(["python3", "-c", "import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), "
                              "'data', 'cutlass', 'include'))"], capture_output=True, text=True).stdout.strip()
    if not os.path.isdir(cutlass) or not os.path.isdir("/usr/local/cuda/include"):
        pytest.skip("no CUTLASS / CUDA headers for the reference's types")
    obj = tmp_path / "sm100_entry.o"
    cmd = [compiler, "-std=c++17", "-c", "-Wall", "-Werror", "-DFUSE_ARCH_SM103=1", f"-I{reference}/include",
           f"-I{ROOT}/include", "-I/usr/local/cuda/include", f"-I{cutlass}",
           os.path.join(ROOT, "tests", "binding", "sm100_entry.cpp"), "-o", str(obj)]
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-4000:]
    # every undefined fuse_* symbol of the object is exported by the library
    symbols = subprocess.run(["nm", "-u", str(obj)], capture_output=True, text=True).stdout.split()
    wanted = sorted({s for s in symbols if s.startswith("fuse_")})
    assert len(wanted) >= 40, wanted
    from fuse_b200 import _native as N
    lib = N.lib()
    missing = [s for s in wanted if not hasattr(lib, s)]
    assert not missing, missing


def test_a_caller_of_the_reference_interface_runs_over_the_binding(tmp_path):
    """tests/binding/probe_main.cpp uses only the reference's C++ interface; linked with the binding
    and the library it must see the reference's own validation answers (no device is touched)."""
    reference = O.reference_root()
    if not os.path.isdir(os.path.join(reference, "include", "fuse")):
        pytest.skip("the reference tree is not mounted here")
    compiler = shutil.which("g++", path="/usr/bin") or shutil.which("g++")
    cutlass = subprocess.run(["python3", "-c", "import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), "
                              "'data', 'cutlass', 'include'))"], capture_output=True, text=True).stdout.strip()
    if compiler is None or not os.path.isdir(cutlass) or not os.path.isdir("/usr/local/cuda/lib64"):
        pytest.skip("no host toolchain for the probe")
    from fuse_b200 import _native as N
    N.lib()  # builds the library when it is stale
    exe = tmp_path / "probe"
    lib_dir = os.path.join(ROOT, "fuse_b200")
    cmd = [compiler, "-std=c++17", "-Wall", "-DFUSE_ARCH_SM103=1", f"-I{reference}/include", f"-I{ROOT}/include",
           "-I/usr/local/cuda/include", f"-I{cutlass}", os.path.join(ROOT, "tests", "binding", "sm100_entry.cpp"),
           os.path.join(ROOT, "tests", "binding", "probe_main.cpp"), "-o", str(exe), f"-L{lib_dir}", "-lfuse_b200",
           f"-Wl,-rpath,{lib_dir}", "-L/usr/local/cuda/lib64", "-lcudart"]
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-4000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    # cudaErrorInvalidValue (1) for epoch 0, for a negative budget and for a plan without experts;
    # the output projection's tile geometry: 128 rows, 256 threads
    assert run.returncode == 0 and run.stdout.split() == ["1", "1", "1", "128", "256"], (run.stdout, run.stderr)
