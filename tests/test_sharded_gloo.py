"""World-size-2 test of the feature-sharded walk protocol over gloo (CPU only).

The per-rank device steps are replaced by a numpy stand-in with the same contract (scores and
exact re-scores from the oracle), so this exercises the host-side protocol in
larql_b200/sharded.py — row partition, the three collectives, pack layout, the identical final
pick on every rank — and checks the result against the unsharded oracle walk."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from conftest import rel_l2, seeded_weights, seeded_x
from larql_b200 import sharded

H, N, K, LAYERS, CAP = 256, 192, 40, 2, 64


def _layers():
    return [[oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(100 * l + j, N, H)) for j in range(3)]
            for l in range(LAYERS)]


class NumpyShardCompute:
    """CPU stand-in for the three device steps (same inputs, outputs and pack layout)."""

    def __init__(self, layers, rank, world, lo, hi, top_k, cap):
        self.rank, self.world, self.lo, self.hi, self.top_k, self.cap = rank, world, lo, hi, top_k, cap
        row = H // 256 * 144
        self.sh = [[oracle.Matrix(oracle.FMT_Q4_K, hi - lo, H, m.data[lo * row:hi * row]) for m in ms] for ms in layers]
        self.hits = []

    def scan(self, l, h, hist):
        self.x = oracle.rms_norm(h.numpy())
        self.scores = self.sh[l][0].gemv(self.x) if self.hi > self.lo else np.zeros(0, np.float32)
        hv = hist.numpy()
        hv[sharded.HIST_BINS:] = 0
        keys = np.abs(self.scores).view(np.uint32) >> sharded.HIST_SHIFT
        np.add.at(hv, keys.astype(np.int64), 1)
        hv[sharded.HIST_BINS + self.rank] = np.float32(1e-6 * (self.rank + 1)).view(np.int32)

    def classify(self, l, hist, pack):
        hv = hist.numpy()
        B = hv[sharded.HIST_BINS:sharded.HIST_BINS + self.world].view(np.float32).max()
        suffix = np.cumsum(hv[:sharded.HIST_BINS][::-1])[::-1]
        bstar = int(np.max(np.nonzero(suffix >= self.top_k)[0]))
        t_lo = np.uint32(bstar << sharded.HIST_SHIFT).view(np.float32)
        t_hi = np.uint32(min((bstar + 1) << sharded.HIST_SHIFT, 0x7F800000)).view(np.float32)
        a = np.abs(self.scores)
        self.is_in = a > t_hi + 2 * B
        band = (~self.is_in) & (a >= t_lo - 2 * B)
        rows = np.nonzero(band)[0]
        assert len(rows) <= self.cap
        pv = pack.numpy()
        pv[:] = 0
        pv[0], pv[1] = int(self.is_in.sum()), len(rows)
        pv[2:2 + len(rows)] = rows + self.lo
        pv[2 + self.cap:2 + self.cap + len(rows)] = self.scores[rows].view(np.int32)
        hv[:sharded.HIST_BINS] = 0

    def gather(self, l, packs, out):
        stride = 2 + 2 * self.cap
        pv = packs.numpy().reshape(self.world, stride)
        need = self.top_k - int(pv[:, 0].sum())
        ent = []
        for r in range(self.world):
            nb = int(pv[r, 1])
            for j in range(nb):
                v = pv[r, 2 + self.cap + j:3 + self.cap + j].view(np.float32)[0]
                ent.append((-abs(float(v)), int(pv[r, 2 + j]), float(v)))
        ent.sort()
        winners = {row: v for _, row, v in ent[:max(need, 0)]}
        sel = [(int(i), float(self.scores[i])) for i in np.nonzero(self.is_in)[0]]
        sel += [(row - self.lo, v) for row, v in winners.items() if self.lo <= row < self.hi]
        o = np.zeros(H, np.float32)
        gate, up, down = self.sh[l]
        rb = up.row_bytes()
        for i, g in sel:
            u = oracle.q4k_row_dot(up.data[i * rb:(i + 1) * rb], self.x)
            act = np.float32(np.float32(g * oracle.sigmoid(g)) * u)
            if abs(act) > 1e-10:
                oracle.q4k_row_scaled_add(down.data[i * rb:(i + 1) * rb], float(act), o)
        self.hits.append(sorted(i + self.lo for i, _ in sel))
        out.copy_(torch.from_numpy(o))


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layers = _layers()
        lo, hi = sharded.shard_rows(N, world, rank)
        comp = NumpyShardCompute(layers, rank, world, lo, hi, K, CAP)
        sw = sharded.ShardedWalk(comp, rank, world, H, CAP, torch.device("cpu"))
        h = torch.from_numpy(seeded_x(7, H))
        out = sw.token(h, LAYERS)
        ret[rank] = (out.numpy().copy(), comp.hits, (lo, hi))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_walk_matches_unsharded_oracle():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    layers = _layers()
    h = seeded_x(7, H)
    want_hits = []
    for l in range(LAYERS):
        h, idx = oracle.run_ffn_token(*layers[l], h, K)
        want_hits.append(sorted(idx.tolist()))
    (o0, hits0, r0), (o1, hits1, r1) = ret[0], ret[1]
    assert r0 == (0, 96) and r1 == (96, 192)
    assert np.array_equal(o0, o1)                      # every rank ends with the same residual
    assert rel_l2(o0, h) < 1e-5
    for l in range(LAYERS):
        assert sorted(hits0[l] + hits1[l]) == want_hits[l]   # union of the ranks' picks == reference top-K


def test_shard_rows_partition():
    for n, w in [(28672, 8), (28672, 4), (3072, 2), (100, 8), (31, 4)]:
        spans = [sharded.shard_rows(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
