"""The C++23 shim (include/q4k_b200_shim.hpp) compiles against the C ABI, links the library, and the
rejections that need no GPU behave like the reference's: typed error, nothing submitted."""
import shutil
import subprocess
from pathlib import Path

import pytest

from qw38_b200 import build

ROOT = Path(__file__).resolve().parents[1]


def test_shim_compiles_links_and_rejects(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    lib = build.build()
    exe = tmp_path / "shim_check"
    cmd = [gxx, "-std=c++23", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "shim" / "shim_check.cpp"),
           "-o", str(exe), f"-L{lib.parent}", "-lq4k_b200", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "shim check ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_shim_runs_the_path_on_the_device(tmp_path):
    """pack_q8 -> q4k_q8_project and launch_decode_mmv through the C++ shim, on weights that are all ones."""
    gxx = shutil.which("g++")
    cuda = Path("/usr/local/cuda")
    if gxx is None or not (cuda / "include" / "cuda_runtime.h").exists():
        pytest.skip("no g++ or CUDA headers")
    lib = build.build()
    exe = tmp_path / "shim_gpu"
    cmd = [gxx, "-std=c++23", "-Wall", "-Wextra", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}",
           str(ROOT / "tests" / "shim" / "shim_gpu.cpp"), "-o", str(exe), f"-L{lib.parent}", "-lq4k_b200",
           f"-L{cuda / 'lib64'}", "-lcudart", f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "shim gpu check ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_reference_operator_case_through_the_shim(tmp_path):
    """The reference's own test case for this path (tests/q4k_q8_test.cpp:36-142), restated in C++ against the shim:
    ten token counts, one PASS line each."""
    gxx = shutil.which("g++")
    cuda = Path("/usr/local/cuda")
    if gxx is None or not (cuda / "include" / "cuda_runtime.h").exists():
        pytest.skip("no g++ or CUDA headers")
    lib = build.build()
    exe = tmp_path / "q4k_q8_case"
    cmd = [gxx, "-std=c++23", "-O1", "-Wall", "-Wextra", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}",
           str(ROOT / "tests" / "shim" / "q4k_q8_case.cpp"), "-o", str(exe), f"-L{lib.parent}", "-lq4k_b200",
           f"-L{cuda / 'lib64'}", "-lcudart", f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.count(" PASS") == 10, r.stdout + r.stderr
