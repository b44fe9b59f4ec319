"""Build liblarql_b200.so (sm_100a) in-tree with nvcc.

    python -m larql_b200.build [--force] [--verbose-ptxas]

Each .cu under csrc/ is compiled to an object with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and the objects are linked
into ``larql_b200/liblarql_b200.so``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_obj"
LIB = HERE / "liblarql_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _newer(a: Path, deps) -> bool:
    if not a.exists():
        return False
    t = a.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def build(force: bool = False, ptxas_verbose: bool = False) -> Path:
    extra = os.environ.get("LARQL_B200_NVCC_FLAGS", "").split()  # e.g. -DFW_CFG_THREADS=512 for tuning builds
    force = force or bool(extra)
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted((HERE.parent / "include").glob("*.h"))
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or ptxas_verbose or not _newer(o, [s] + hdrs):
            cmd = [NVCC] + FLAGS + extra + (["-Xptxas", "-v"] if ptxas_verbose else []) + ["-c", str(s), "-o", str(o)]
            jobs.append((s, cmd))

    def run(job):
        s, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for s, r in ex.map(run, jobs):
            if ptxas_verbose or r.returncode != 0:
                sys.stderr.write(f"--- {s.name}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {s.name}")
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if force or jobs or not _newer(LIB, objs):
        cmd = [NVCC, "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, ptxas_verbose="--verbose-ptxas" in sys.argv)
    print(p)
