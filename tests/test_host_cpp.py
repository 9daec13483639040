"""The C++ host layer (candy_b200/host/candy_cuda.hpp): builds with g++ against libcandyq.so; without
a GPU it must fail with an exception; on a GPU a QLinear forward must match the CPU oracle."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "candy_b200"


def build(tmp_path) -> Path:
    exe = tmp_path / "test_host"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", str(ROOT / "include"), "-I", str(PKG / "host"),
           str(ROOT / "tests" / "host" / "test_host.cpp"), "-o", str(exe), "-L", str(PKG), "-lcandyq", f"-Wl,-rpath,{PKG}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_host_layer_compiles_and_refuses_to_run_without_a_gpu(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([str(exe), "nogpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("OK") or r.stdout.startswith("SKIP")


@pytest.mark.gpu
def test_host_layer_qlinear_matches_oracle(tmp_path):
    from oracle import oracle_c as oc
    from helpers import rel_err
    exe = build(tmp_path)
    out = tmp_path / "host_out.bin"
    r = subprocess.run([str(exe), "gpu", str(out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    n, k, rows = 48, 256, 6
    raw = out.read_bytes()
    nb = n * (k // 32) * 18
    blocks = np.frombuffer(raw[:nb], dtype=np.uint8)
    x = np.frombuffer(raw[nb:nb + 4 * rows * k], dtype=np.float32).reshape(rows, k)
    y = np.frombuffer(raw[nb + 4 * rows * k:], dtype=np.float32).reshape(rows, n)
    assert rel_err(y, oc.qmatmul(oc.Q4_0, 0, x, blocks, n)) < 1e-4
