"""The Kokkos-free C++ call surface (include/lapis_b200.hpp): compiles everywhere, runs on a GPU box."""
import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
SRC = os.path.join(ROOT, "tests", "cpp", "driver.cpp")


def _env():
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    return env


def _compile(out, link):
    gxx = shutil.which("g++")
    if gxx is None or not os.path.isdir(os.path.join(CUDA, "include")):
        pytest.skip("needs g++ and the CUDA headers")
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), SRC]
    if link:
        lib = os.path.join(ROOT, "lapis_b200")
        cmd += ["-o", out, "-L", lib, "-llapis_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
                f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    else:
        cmd += ["-c", "-o", out]
    subprocess.run(cmd, check=True, env=_env())


def test_header_compiles(tmp_path):
    _compile(str(tmp_path / "driver.o"), link=False)


@pytest.mark.gpu
def test_cpp_driver_runs(tmp_path):
    assert torch.cuda.is_available(), "needs a CUDA device"
    exe = str(tmp_path / "driver")
    _compile(exe, link=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "driver ok" in r.stdout, r.stdout + r.stderr
