"""Real multi-rank check of the feature-sharded walk: one process per GPU, NCCL between them, the
exchanges issued by the library itself (lq_comm_init / lq_stack_create_sharded).  Every rank's output
is compared with the unsharded CPU oracle and the union of the ranks' selections with the oracle's
top-K set.  Skips on a box with fewer than two GPUs."""
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
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")          # plumbing only: hands the NCCL id round and collects the results
    H, N, K, L, cap = 2048, 6144, 700, 3, 2048
    be = larql_b200.CudaBackend(rank)
    ids = [larql_b200.CudaBackend.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    assert be.comm_init(rank, world, ids[0])
    lo, hi = sharded.shard_rows(N, world, rank)
    layers, full = [], []
    dev = torch.device("cuda", rank)
    for l in range(L):
        mats = [oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(900 + 8 * l + j, N, H)) for j in range(3)]
        full.append(mats)
        row = mats[0].row_bytes()
        dm = []
        for m in mats:
            t = torch.from_numpy(np.asarray(m.data)[lo * row:hi * row].copy()).to(dev)
            dm.append(larql_b200.DeviceMatrix(larql_b200.FMT_Q4_K, hi - lo, H, t.data_ptr(), t.numel(), keepalive=t))
        layers.append(dm)
    st = be.stack_create_sharded([m[0] for m in layers], [m[1] for m in layers], [m[2] for m in layers], 1, K, N, lo, cap,
                                 larql_b200.WALK_FORCE_SPARSE)
    assert st is not None, be.last_refusal
    ok = True
    for q in range(2):
        h = seeded_x(77 + q, H)
        want = h.copy()
        for l in range(L):
            want, idx = oracle.run_ffn_token(*full[l], want, K)
        got = np.empty(H, np.float32)
        assert be.stack_run_host(st, h.ctypes.data, got.ctypes.data), be.last_refusal
        mine = be.last_shard_hits(lo)                         # the last layer's selection of this rank, global rows
        allhits = [None] * world
        dist.all_gather_object(allhits, mine)
        union = sorted(x for part in allhits for x in part)
        ok = ok and rel_l2(got, want) < 1e-3 and union == sorted(idx.tolist())
        print(f"rank {rank} query {q}: rel_l2 {rel_l2(got, want):.2e} union_ok {union == sorted(idx.tolist())}", flush=True)
    dist.barrier()
    be.stack_destroy(st); be.comm_destroy(); be.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 3)
''')


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_stack_over_nccl_matches_the_unsharded_oracle(world, tmp_path):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, LQ_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29600 + world),
               WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
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
        assert p.returncode == 0, f"rank {r} failed:\\n{out[-3000:]}"
