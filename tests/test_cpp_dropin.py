"""The drop-in C++ headers (include/superkmeans/*.h) compile against the C ABI and keep the reference's
exception classes; with a GPU the same program also trains flat and hierarchical models."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "superkmeans_b200")


def _build(tmp_path):
    exe = str(tmp_path / "dropin_check")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "dropin_check.cpp"), "-o", exe,
           "-L", LIBDIR, "-lskm_b200", f"-Wl,-rpath,{LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_dropin_headers_compile_and_validate(tmp_path):
    import torch

    exe = _build(tmp_path)
    if torch.cuda.is_available():
        pytest.skip("covered by the GPU variant")
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "OK (cpu)" in res.stdout


@pytest.mark.gpu
def test_dropin_headers_train_on_gpu(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([exe, "gpu"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "OK (gpu)" in res.stdout
