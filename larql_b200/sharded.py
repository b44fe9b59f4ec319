"""Feature-sharded walk across the GPUs of one box (one process per GPU, torch.distributed).

Each rank owns a contiguous range of feature rows of every layer's gate / up / down.  Per layer
and token the protocol is three device steps separated by three collectives::

    scan      local scores + local coarse |score| histogram + local error bound
      all-reduce(sum)   histogram [16384] and one bound slot per rank          (64 KB)
    classify  global band thresholds -> certain rows, band rows re-scored exactly, packed
      all-gather        {n_in, n_band, band rows, exact scores} of every rank  (<= 8*cap B/rank)
    gather    identical final pick on every rank; up/act/down of the rows this rank owns
      all-reduce(sum)   partial out[hidden]                                    (4*hidden B)
    h <- h + out

The union of the ranks' selections equals the unsharded reference top-K set exactly (the
histogram and the bound are global, the band is resolved with exact reference-order scores and
ties go to the lower GLOBAL row).  The reference itself has no feature sharding; it shards
layers or experts over HTTP (docs/ffn/distributed.md:14-40).

``ShardedWalk`` is the protocol for a host that brings its own collectives (torch.distributed
here); the per-rank arithmetic is a *compute* object with ``scan``, ``classify`` and ``gather``
methods.  ``CudaShardCompute`` runs them through the C ABI; the CPU test-suite plugs in a numpy
stand-in to exercise the protocol over the gloo backend.  The library runs the same protocol by
itself (``CudaBackend.comm_init`` / ``stack_create_sharded``: the exchanges are made from C++, on
the persistent kernel through peer memory where it applies); that is the path the benchmark times.

Ordering: the C-ABI steps are enqueued on the backend's own non-blocking stream.  When the compute
object exposes that stream (``stream()``), ``ShardedWalk.layer`` issues the collectives and the
residual add on the same stream, after making it wait for the caller's current stream, and makes
the caller's stream wait for it before returning: steps and collectives are ordered whatever
stream the caller is on.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

HIST_BINS = 16384
HIST_WORDS = HIST_BINS + 64
HIST_SHIFT = 17


def shard_rows(n_features: int, world: int, rank: int, multiple: int = 32):
    """Contiguous row range of `rank`: ranges are multiples of `multiple` rows except the last."""
    per = (n_features + world - 1) // world
    per = (per + multiple - 1) // multiple * multiple
    lo = min(n_features, rank * per)
    hi = min(n_features, lo + per)
    return lo, hi


class ShardedWalk:
    def __init__(self, compute, rank: int, world: int, hidden: int, cap: int, device, group=None):
        self.compute, self.rank, self.world, self.hidden, self.cap = compute, rank, world, hidden, cap
        self.group = group
        self.stride = 2 + 2 * cap
        self.hist = torch.zeros(HIST_WORDS, dtype=torch.int32, device=device)
        self.pack = torch.zeros(self.stride, dtype=torch.int32, device=device)
        self.packs = torch.zeros(world * self.stride, dtype=torch.int32, device=device)
        self.out = torch.zeros(hidden, dtype=torch.float32, device=device)
        handle = compute.stream() if hasattr(compute, "stream") else None
        self._stream = torch.cuda.ExternalStream(handle, device=device) if handle else None

    def layer(self, l: int, h: torch.Tensor) -> torch.Tensor:
        """h: [hidden] residual on the compute device. Returns h + walk_l(rmsnorm(h))."""
        if self._stream is None:
            return self._layer(l, h)
        caller = torch.cuda.current_stream(self._stream.device)
        self._stream.wait_stream(caller)          # h is ready before the first step reads it
        with torch.cuda.stream(self._stream):
            out = self._layer(l, h)
        caller.wait_stream(self._stream)          # the result is ready for whatever the caller enqueues next
        return out

    def _layer(self, l: int, h: torch.Tensor) -> torch.Tensor:
        c = self.compute
        c.scan(l, h, self.hist)
        if self.world > 1:
            dist.all_reduce(self.hist, group=self.group)
        c.classify(l, self.hist, self.pack)
        if self.world > 1:
            dist.all_gather(list(self.packs.view(self.world, self.stride).unbind(0)), self.pack, group=self.group)
        else:
            self.packs.copy_(self.pack)
        c.gather(l, self.packs, self.out)
        if self.world > 1:
            dist.all_reduce(self.out, group=self.group)
        return h + self.out

    def token(self, h: torch.Tensor, n_layers: int) -> torch.Tensor:
        for l in range(n_layers):
            h = self.layer(l, h)
        return h


class CudaShardCompute:
    """The three device steps through the C ABI (Q4_K shards resident in this rank's HBM)."""

    def __init__(self, backend, layers, rank: int, world: int, row_offset: int, top_k: int, cap: int, flags: int):
        # layers: list of (gate, up, down_fm) DeviceMatrix shards (rows = this rank's range)
        self.be, self.layers, self.rank, self.world = backend, layers, rank, world
        self.row_offset, self.top_k, self.cap, self.flags = row_offset, top_k, cap, flags

    def stream(self) -> int:
        """The CUDA stream the steps are enqueued on (a cudaStream_t as an integer)."""
        return self.be.stream()

    def scan(self, l, h, hist):
        ok = self.be.dev_shard_scan(self.layers[l][0], h.data_ptr(), self.flags, self.rank, self.world, hist.data_ptr())
        if not ok:
            raise RuntimeError("shard_scan refused: " + self.be.last_refusal)

    def classify(self, l, hist, pack):
        ok = self.be.dev_shard_classify(self.layers[l][0], hist.data_ptr(), self.world, self.top_k, self.row_offset,
                                        pack.data_ptr(), self.cap)
        if not ok:
            raise RuntimeError("shard_classify refused: " + self.be.last_refusal)

    def gather(self, l, packs, out):
        ok = self.be.dev_shard_gather(self.layers[l][1], self.layers[l][2], packs.data_ptr(), self.world, self.rank,
                                      self.cap, self.top_k, self.row_offset, out.data_ptr())
        if not ok:
            raise RuntimeError("shard_gather refused: " + self.be.last_refusal)
