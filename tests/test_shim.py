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
