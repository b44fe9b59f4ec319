"""Real multi-rank check of the feature-sharded walk: one process per GPU, the exchanges issued by the
library itself (lq_comm_init / lq_stack_create_sharded), both ways it has of making them: three NCCL
collectives per layer, and the persistent kernel that exchanges through peer memory.  Every rank's
output is compared with the unsharded CPU oracle and the union of the ranks' selections with the
oracle's top-K set.  The multi-rank cases skip on a box with fewer GPUs than ranks."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent('''
    import os, sys, pickle, numpy as np, torch
    sys.path.insert(0, os.environ["LQ_ROOT"]); sys.path.insert(0, os.path.join(os.environ["LQ_ROOT"], "tests"))
    import torch.distributed as dist
    import larql_b200, oracle
    from larql_b200 import sharded
    from conftest import seeded_weights, seeded_x, rel_l2
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    H, N, K, L, cap = [int(v) for v in os.environ["LQ_SHAPE"].split(",")]
    want_path = int(os.environ["LQ_WANT_PATH"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")          # plumbing only: hands the NCCL id round and collects the results
    be = larql_b200.CudaBackend(rank)
    ids = [larql_b200.CudaBackend.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    assert be.comm_init(rank, world, ids[0])
    lo, hi = sharded.shard_rows(N, world, rank)
    layers, full = [], []
    dev = torch.device("cuda", rank)
    # one seeded matrix; the nine matrices of the stack are its rows in other orders (rows quantise independently)
    base = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(900, N, H))
    row = base.row_bytes()
    def rolled(shift):
        d = np.roll(np.asarray(base.data).reshape(N, row), shift, axis=0).reshape(-1).copy()
        return oracle.Matrix(base.fmt, N, H, d)
    for l in range(L):
        mats = [rolled(1013 * (3 * l + j) + 7) for j in range(3)]
        full.append(mats)
        dm = []
        for m in mats:
            t = torch.from_numpy(np.asarray(m.data)[lo * row:hi * row].copy()).to(dev)
            dm.append(larql_b200.DeviceMatrix(larql_b200.FMT_Q4_K, hi - lo, H, t.data_ptr(), t.numel(), keepalive=t))
        layers.append(dm)
    st = be.stack_create_sharded([m[0] for m in layers], [m[1] for m in layers], [m[2] for m in layers], 1, K, N, lo, cap,
                                 larql_b200.WALK_FORCE_SPARSE)
    assert st is not None, be.last_refusal
    path = be.stack_path(st)
    ok = path == want_path
    print(f"rank {rank}: stack path {path} (expected {want_path})", flush=True)
    for q in range(3):
        h = seeded_x(77 + q, H)
        want = h.copy()
        for l in range(L):
            want, idx = oracle.run_ffn_token(*full[l], want, K)
        got = np.empty(H, np.float32)
        dist.barrier()
        assert be.stack_run_host(st, h.ctypes.data, got.ctypes.data), be.last_refusal
        mine = be.last_shard_hits(lo)                         # the last layer's selection of this rank, global rows
        allhits = [None] * world
        dist.all_gather_object(allhits, mine)
        union = sorted(x for part in allhits for x in part)
        outs = [None] * world
        dist.all_gather_object(outs, got.tobytes())
        same = all(o == outs[0] for o in outs)                # every rank holds the same residual, bit for bit
        ok = ok and rel_l2(got, want) < 1e-3 and union == sorted(idx.tolist()) and same
        print(f"rank {rank} query {q}: rel_l2 {rel_l2(got, want):.2e} union_ok {union == sorted(idx.tolist())} "
              f"ranks_identical {same}", flush=True)
    dist.barrier()
    be.stack_destroy(st); be.comm_destroy(); be.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 3)
''')

# hidden, features, top_k, layers, band capacity
SMALL = "2048,6144,700,3,2048"      # too few rows per rank for the persistent kernel: NCCL exchanges
LARGE = "4096,12288,1500,3,4096"    # persistent kernel on every rank, exchange through peer memory
LARGE8 = "4096,20480,2500,3,4096"   # the same with enough rows for eight ranks (a rank needs a tile per CTA)
PATH_SHARDED_NCCL, PATH_SHARDED_FUSED = 2, 3


def run_ranks(world, shape, want_path, tmp_path, extra_env=None):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, LQ_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29600 + world),
               WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0", LQ_SHAPE=shape, LQ_WANT_PATH=str(want_path))
    env.update(extra_env or {})
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_stack_over_nccl_matches_the_unsharded_oracle(world, tmp_path):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(world, SMALL, PATH_SHARDED_NCCL, tmp_path)
    run_ranks(world, LARGE, PATH_SHARDED_NCCL, tmp_path, {"LARQL_B200_SHARDED_NCCL": "1"})


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sharded_stack_on_the_persistent_kernel_matches_the_unsharded_oracle(world, tmp_path):
    '''Every rank walks all layers in one launch; histogram, band rows and partial outputs travel through
    peer memory.  world = 1 runs the same kernel and barriers on one GPU.'''
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(world, LARGE8 if world > 4 else LARGE, PATH_SHARDED_FUSED, tmp_path)
