"""Feature-sharded walk on one GPU: the ranks are emulated one after another (one backend
context per rank, no kernel ever waits on another), the collectives are plain tensor sums and
concatenations.  Checks the C-ABI shard steps against the unsharded oracle walk."""
import numpy as np
import pytest

import oracle
from conftest import rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,h,n,k,fmt", [(2, 1024, 3072, 512, oracle.FMT_Q4_K), (4, 2560, 2048, 300, oracle.FMT_Q4_K),
                                             (8, 8192, 4096, 600, oracle.FMT_Q4_K), (2, 1024, 3072, 512, oracle.FMT_NVFP4),
                                             (4, 2048, 2048, 300, oracle.FMT_MXFP4), (3, 1024, 1000, 128, oracle.FMT_Q8_0)])
def test_emulated_ranks_match_unsharded_oracle(world, h, n, k, fmt):
    import torch

    import larql_b200
    from larql_b200 import sharded

    dev = torch.device("cuda", 0)
    mats = [oracle.quantize_matrix(fmt, seeded_weights(31 * world + j, n, h)) for j in range(3)]
    hin = seeded_x(5 + world, h)
    want, want_idx = oracle.run_ffn_token(*mats, hin, k)
    row = mats[0].row_bytes()
    srow = {oracle.FMT_MXFP4: h // 32, oracle.FMT_NVFP4: h // 16}.get(fmt, 0)   # scale bytes per row
    cap = 1024
    stride = 2 + 2 * cap
    flags = larql_b200.WALK_RMSNORM | larql_b200.WALK_FORCE_SPARSE
    bes, shards, spans = [], [], []
    for r in range(world):
        lo, hi = sharded.shard_rows(n, world, r)
        spans.append((lo, hi))
        bes.append(larql_b200.CudaBackend(0))
        dm = []
        for m in mats:
            t = torch.from_numpy(m.data[lo * row:hi * row].copy()).to(dev)
            sc = torch.from_numpy(m.scales[lo * srow:hi * srow].copy()).to(dev) if srow else None
            dm.append(larql_b200.DeviceMatrix(fmt, hi - lo, h, t.data_ptr(), t.numel(), sc.data_ptr() if srow else 0,
                                              sc.numel() if srow else 0, float(m.tensor_scale), keepalive=(t, sc)))
        shards.append(dm)
    x_d = torch.from_numpy(hin).to(dev)
    hists = [torch.zeros(sharded.HIST_WORDS, dtype=torch.int32, device=dev) for _ in range(world)]
    packs = torch.zeros(world, stride, dtype=torch.int32, device=dev)
    outs = [torch.zeros(h, dtype=torch.float32, device=dev) for _ in range(world)]
    torch.cuda.synchronize()
    try:
        for r in range(world):
            assert bes[r].dev_shard_scan(shards[r][0], x_d.data_ptr(), flags, r, world, hists[r].data_ptr())
            bes[r].synchronize()
        total = torch.stack(hists).sum(0).to(torch.int32)          # "all-reduce"
        for r in range(world):
            hists[r].copy_(total)
            torch.cuda.synchronize()
            assert bes[r].dev_shard_classify(shards[r][0], hists[r].data_ptr(), world, k, spans[r][0],
                                             packs[r].data_ptr(), cap)
            bes[r].synchronize()
            assert int(hists[r][:sharded.HIST_BINS].abs().sum()) == 0   # cleared for the next layer
        flat = packs.reshape(-1).contiguous()                       # "all-gather"
        for r in range(world):
            assert bes[r].dev_shard_gather(shards[r][1], shards[r][2], flat.data_ptr(), world, r, cap, k,
                                           spans[r][0], outs[r].data_ptr())
            bes[r].synchronize()
        out = torch.stack(outs).sum(0).cpu().numpy() + hin           # "all-reduce" + residual
        assert rel_l2(out - hin, want - hin) < 1e-3
        n_in = packs[:, 0].sum().item()
        assert 0 < n_in <= k
        # the union of the ranks' selections is the unsharded reference's top-K set
        got_idx = []
        for r in range(world):
            st = bes[r].last_shard_hits(spans[r][0])
            got_idx += st
        assert sorted(got_idx) == sorted(want_idx.tolist())
    finally:
        for b in bes:
            b.close()
