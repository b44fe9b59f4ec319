"""The C++ host-side mirror of the reference's backend trait (include/larql_backend.hpp): it compiles
and links against the C-ABI library, refuses to run without a device (no CPU fallback), and on a GPU
gives the oracle's results through the trait-shaped methods."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

import larql_b200
import oracle
from conftest import rel_l2, seeded_weights, seeded_x

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    out = tmp_path_factory.mktemp("cpp") / "mirror_check"
    lib_dir = Path(larql_b200.LIB_PATH).parent
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "tests/cpp/mirror_check.cpp"),
           "-L", str(lib_dir), "-llarql_b200", f"-Wl,-rpath,{lib_dir}", "-o", str(out)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return out


def test_mirror_compiles_links_and_has_no_cpu_fallback(exe):
    import torch
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    if torch.cuda.is_available():
        assert r.returncode == 0 and r.stdout.startswith("cuda-b200")
    else:
        assert r.returncode == 3 and "BackendError" in r.stderr   # no device: the mirror throws, it does not fall back


@pytest.mark.gpu
def test_mirror_matches_oracle(exe, tmp_path):
    rows, cols, k, batch = 300, 1024, 37, 3
    mats = [oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(0xC99 + j, rows, cols)) for j in range(3)]
    x = oracle.rms_norm(seeded_x(0xC9A, batch, cols))
    blob = np.array([rows, cols, k, batch], np.int32).tobytes() + b"".join(m.data.tobytes() for m in mats) + x.tobytes()
    (tmp_path / "in.bin").write_bytes(blob)
    r = subprocess.run([str(exe), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = (tmp_path / "out.bin").read_bytes()
    mv = np.frombuffer(raw, np.float32, rows)
    out = np.frombuffer(raw, np.float32, batch * cols, rows * 4).reshape(batch, cols)
    cnt = np.frombuffer(raw, np.int32, batch, (rows + batch * cols) * 4)
    hits = np.frombuffer(raw, np.uint32, int(cnt.sum()), (rows + batch * cols + batch) * 4)
    assert rel_l2(mv, mats[0].gemv(x[0])) < 1e-4
    off = 0
    for t in range(batch):
        want, idx, _ = oracle.walk_token(*mats, x[t], k)
        assert sorted(hits[off:off + cnt[t]].tolist()) == sorted(idx.tolist())
        assert rel_l2(out[t], want) < 1e-3
        off += int(cnt[t])
