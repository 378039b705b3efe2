"""include/b200q.hpp (the C++ host shim with the reference's operator shapes) compiles against the
C ABI and rejects invalid problems on the host with std::invalid_argument, without a GPU."""
import os
import shutil
import subprocess

import pytest

from mlx_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_shim_compiles_and_validates(tmp_path):
    _lib.load()
    exe = str(tmp_path / "shim_check")
    libdir = os.path.dirname(_lib.LIB_PATH)
    cuda_inc = "/usr/local/cuda/include"
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "shim_check.cpp"),
           "-o", exe, "-L", libdir, "-lb200q", f"-Wl,-rpath,{libdir}"]
    if os.path.isdir(cuda_inc):
        cmd[3:3] = ["-I", cuda_inc]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "SHIM-OK" in res.stdout, res.stdout + res.stderr
