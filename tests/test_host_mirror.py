"""The C++ host mirror of the reference's Go API (go-nngpu_b200/host/gonngpu.hpp):
compiled with g++ against the C-ABI library, host-only checks on CPU, full run
on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "go-nngpu_b200")


def _compile(tmp_path, built_lib):
    exe = str(tmp_path / "host_mirror_test")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-o", exe,
                    os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"),
                    "-L" + PKG, "-lgonngpu_cuda", "-Wl,-rpath," + PKG], check=True)
    return exe


def test_host_mirror_compiles_and_host_logic_passes(tmp_path, built_lib):
    exe = _compile(tmp_path, built_lib)
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host mirror ok" in res.stdout


@pytest.mark.gpu
def test_host_mirror_on_gpu(tmp_path, gpu):
    exe = _compile(tmp_path, gpu)
    res = subprocess.run([exe, "gpu"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host mirror ok" in res.stdout
