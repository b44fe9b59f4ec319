#!/usr/bin/env python3
"""Benchmark of the vindex FFN walk on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME] [--batch B]

A step is one token batch through every layer of the workload (h <- h + walk_l(rmsnorm(h))).
Default workload: the Llama-3-70B-shaped Q4_K walk (hidden 8192, 28672 features, 80 layers,
top-K 4096, batch 1), which fits one GPU and is the configuration the multi-GPU metric is
quoted on.  Weights are seeded N(0, 0.02), generated on the device and quantised there (Q4_K, by
the library's own encoder, byte-identical to the CPU encoder) or on the host by the oracle's
encoders (the other formats); inputs are seeded N(0, 1) residuals.

Workloads (one per benchmark configuration):
    qwen06b_q4k        config 1: one Qwen3-0.6B-shaped layer, K = 512
    dense_sweep        config 2: dense matvec (K = all), Q4_K and Q8_0, three shapes, batch 1 / 8 / 32
    gemma12b_q4k       config 3: 48 Gemma-3-12B-shaped layers, K = 1024
    gptoss_mxfp4_moe   config 4: gpt-oss-20B-shaped MXFP4 MoE FFN, 32 experts, top-4, K = 768 per expert
    llama70b_q4k       config 5 (default): 80 Llama-3-70B-shaped Q4_K layers, K = 4096; --gpus N shards the features
    llama70b_nvfp4     config 5, NVFP4 variant

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (CUDA events on the launching
stream); `e2e` goes through the host-pointer C-ABI call with the host<->device copies inside the timed
region; `roofline` is the dominant kernel's algorithmic bytes per launch over its launch time against
the measured HBM copy bandwidth; `cpu_baseline` is the CPU oracle (a restatement of the reference CPU
backend, `kind: "port"` — the Rust reference cannot be built on this machine) timed on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FMT_Q4_K, FMT_Q8_0, FMT_MXFP4, FMT_NVFP4 = 0, 1, 2, 3
WORKLOADS = {
    # name: hidden, features, top_k, layers, fmt
    "llama70b_q4k": dict(hidden=8192, features=28672, top_k=4096, layers=80, fmt=FMT_Q4_K),
    "llama70b_nvfp4": dict(hidden=8192, features=28672, top_k=4096, layers=80, fmt=FMT_NVFP4),
    "gemma12b_q4k": dict(hidden=3840, features=15360, top_k=1024, layers=48, fmt=FMT_Q4_K),
    "qwen06b_q4k": dict(hidden=1024, features=3072, top_k=512, layers=1, fmt=FMT_Q4_K),
    "gptoss_mxfp4_moe": dict(hidden=2880, features=2880, top_k=768, layers=1, fmt=FMT_MXFP4, experts=32, top_e=4),
    "dense_sweep": dict(hidden=3840, features=15360, top_k=15360, layers=1, fmt=FMT_Q4_K),
}
FMT_NAME = {FMT_Q4_K: "Q4_K", FMT_Q8_0: "Q8_0", FMT_MXFP4: "MXFP4", FMT_NVFP4: "NVFP4"}


def row_bytes(fmt: int, hidden: int) -> int:
    """Bytes of one quantised row, scale streams included."""
    return {FMT_Q4_K: hidden // 256 * 144, FMT_Q8_0: hidden // 32 * 34, FMT_MXFP4: hidden // 32 * 17,
            FMT_NVFP4: hidden // 16 * 9}[fmt]


def algorithmic_bytes_per_token_layer(hidden: int, features: int, top_k: int, fmt: int = FMT_Q4_K) -> int:
    """gate rows once + the K selected up rows and down rows + activation in and out."""
    row = row_bytes(fmt, hidden)
    return int(features * row + 2 * top_k * row + 8 * hidden)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# phases of the persistent walk kernel between its clock stamps (CTA 0, last layer but one); in a sharded walk
# barrier_a also covers the barrier over this GPU's CTAs and the copy of its histogram to the other ranks
PHASE_NAMES = ["prepare", "scan", "barrier_a", "select", "rescore", "barrier_b", "pick", "gather", "merge",
               "barrier_c", "finish", "barrier_d"]


def config_of(args, wl):
    moe = f", {wl['experts']} experts top-{wl['top_e']}" if "experts" in wl else ""
    return {"workload": f"{args.workload}: hidden {wl['hidden']}, features {wl['features']}{moe}, top_k {wl['top_k']}, "
                        f"{wl['layers']} layer(s), {FMT_NAME[wl['fmt']]} gate/up/down N(0,0.02), batch {args.batch}",
            "batch": args.batch, "layers": wl["layers"],
            "l2": "inputs larger than L2: every step streams more distinct weight bytes than the 126 MB L2 holds "
                  "(small workloads rotate over copies)",
            "parallelism": f"features sharded over {args.gpus} GPU(s), three NCCL exchanges per layer issued by the "
                           f"library" if args.gpus > 1 else "single GPU"}


# ------------------------------------------------------------------ host-side weights (oracle encoders)
def host_matrix(wl, seed: int, fmt=None):
    import oracle
    rng = np.random.Generator(np.random.PCG64(seed))
    w = rng.standard_normal((wl["features"], wl["hidden"]), dtype=np.float32)
    w *= np.float32(0.02)
    return oracle.quantize_matrix(wl["fmt"] if fmt is None else fmt, w)


def host_layer(wl, layer: int):
    """One layer's gate/up/down quantised on the host with the oracle's encoder."""
    return [host_matrix(wl, 0x1A2B0000 + 8 * layer + j) for j in range(3)]


def oracle_inputs(wl, n=4):
    import oracle
    return [oracle.rms_norm(np.random.Generator(np.random.PCG64(0x5EED0000 + q)).standard_normal(
        wl["hidden"], dtype=np.float32)) for q in range(n)]


# ------------------------------------------------------------------ reference arm
def cpu_walk_sample(layers, wl, batch: int, budget_s: float, threads: int):
    """Times the oracle's threaded walk: calls of (one layer x `batch` tokens), rotating over `layers`
    (distinct weights) until `budget_s` has passed.  Returns (seconds per layer-call, calls, seconds)."""
    import oracle
    xs = oracle_inputs(wl)
    oracle.walk_token_mt(*layers[0], xs[0], wl["top_k"], threads)  # warm
    n, t0 = 0, time.perf_counter()
    while True:
        mats = layers[n % len(layers)]
        for b in range(batch):
            oracle.walk_token_mt(*mats, xs[(n + b) % 4], wl["top_k"], threads)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s:
            return dt / n, n, dt


def run_reference(args, wl):
    """The reference's CPU implementation of the path, as the oracle restates it (`kind: port`), on all host
    cores.  A step is a bounded sample of the workload: `sample_layers` distinct layers (of the workload's
    `layers`) for `batch` tokens; `ms_per_step` is what that sample took, `value` scales it to all layers."""
    import oracle
    threads = oracle.host_threads()
    if wl.get("experts") or args.workload == "dense_sweep":
        raise SystemExit("the reference arm covers the walk workloads")
    sample_layers = min(3, wl["layers"])
    layers = [host_layer(wl, l) for l in range(sample_layers)]
    xs = oracle_inputs(wl)

    def step(i):
        for mats in layers:
            for b in range(args.batch):
                oracle.walk_token_mt(*mats, xs[(i + b) % 4], wl["top_k"], threads)

    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(i)
    dt = time.perf_counter() - t0
    ms_step = dt / args.steps * 1e3
    tok_s = args.batch / (ms_step * 1e-3 / sample_layers * wl["layers"])
    sample = (f"each step = {sample_layers} distinct layers of {wl['layers']} x {args.batch} token(s), oracle "
              f"walk_token_mt on {threads} threads; tokens/s = batch / (step time / {sample_layers} x {wl['layers']})")
    line = {
        "impl": "reference", "metric": "walk_ffn_tokens_per_s", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(args, wl),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ device-side weights
def device_layers(be, wl, n_layers: int, dev, lo: int = 0, hi=None, first_layer: int = 0):
    """Seeded layers resident on the device.  Q4_K: generated and quantised on the device (rows [lo, hi) of the
    same global matrix on every rank).  Other formats: three matrices quantised on the host by the oracle's
    encoder; every layer gets its own device copy with the rows rotated (rows encode independently, so a rotation
    is another valid seeded layer)."""
    import torch

    import larql_b200
    H, N, fmt = wl["hidden"], wl["features"], wl["fmt"]
    hi = N if hi is None else hi
    n_loc = hi - lo
    layers = []
    if fmt == FMT_Q4_K:
        row = H // 256 * 144
        gen = torch.Generator(device=dev)
        tmp = torch.empty(N * H, dtype=torch.float32, device=dev)
        for l in range(first_layer, first_layer + n_layers):
            mats = []
            for j in range(3):
                gen.manual_seed(0x1A2B0000 + 8 * l + j)
                tmp.normal_(0.0, 0.02, generator=gen)
                q = torch.empty(n_loc * row, dtype=torch.uint8, device=dev)
                torch.cuda.synchronize()
                be.dev_quantize_q4k(tmp.data_ptr() + lo * H * 4, n_loc * H, q.data_ptr())
                be.synchronize()
                mats.append(larql_b200.DeviceMatrix(FMT_Q4_K, n_loc, H, q.data_ptr(), q.numel(), keepalive=q))
            layers.append(mats)
        del tmp
        torch.cuda.empty_cache()
        return layers
    base = host_layer(wl, first_layer)
    rb = int(len(base[0].data) // N)
    sb = int(len(base[0].scales) // N) if base[0].scales is not None and len(base[0].scales) else 0
    for l in range(n_layers):
        mats = []
        for j, m in enumerate(base):
            shift = (l * 977 + j * 131) % N
            d = np.roll(np.asarray(m.data).reshape(N, rb), shift, axis=0)[lo:hi].reshape(-1)
            t = torch.from_numpy(np.ascontiguousarray(d)).to(dev)
            if sb:
                s = np.roll(np.asarray(m.scales).reshape(N, sb), shift, axis=0)[lo:hi].reshape(-1)
                ts = torch.from_numpy(np.ascontiguousarray(s)).to(dev)
                mats.append(larql_b200.DeviceMatrix(fmt, n_loc, H, t.data_ptr(), t.numel(), ts.data_ptr(), ts.numel(),
                                                    float(m.tensor_scale), keepalive=(t, ts)))
            else:
                mats.append(larql_b200.DeviceMatrix(fmt, n_loc, H, t.data_ptr(), t.numel(), keepalive=t))
        layers.append(mats)
    return layers, base


def time_steps(fn, steps, warmup, ext, sync):
    import torch
    for i in range(warmup):
        fn(i)
    sync()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(ext)
    for i in range(steps):
        fn(i)
    ev1.record(ext)
    sync()
    return ev0.elapsed_time(ev1) / steps


# ------------------------------------------------------------------------ sharded arm (N > 1)
def run_sharded(args, wl, be, ext, dev, rank, world, local):
    """The intermediate (feature) dimension of every layer is split across the GPUs; the library issues the three
    NCCL exchanges per layer on its own stream (lq_comm_init / lq_stack_create_sharded).  Strong scaling: the same
    workload at every N.  Before timing, rank 0 checks a sharded run of the first layers against the one-GPU walk
    of the same layers on the same input and prints the result as `parity`."""
    import torch
    import torch.distributed as dist

    import larql_b200
    from larql_b200 import sharded

    H, N, K, L, B = wl["hidden"], wl["features"], wl["top_k"], wl["layers"], args.batch
    if wl["fmt"] != FMT_Q4_K or wl.get("experts") or args.workload == "dense_sweep":
        raise SystemExit("the sharded benchmark runs the Q4_K walk workloads")
    lo, hi = sharded.shard_rows(N, world, rank)
    ids = [larql_b200.CudaBackend.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    if not be.comm_init(rank, world, ids[0]):
        raise SystemExit("lq_comm_init refused: " + be.last_refusal)
    layers = device_layers(be, wl, L, dev, lo, hi)
    cap = 4096
    flags = larql_b200.WALK_FORCE_SPARSE

    def make_stack(ls, batch):
        st = be.stack_create_sharded([m[0] for m in ls], [m[1] for m in ls], [m[2] for m in ls], batch, K, N, lo, cap, flags)
        if st is None:
            raise SystemExit("lq_stack_create_sharded refused: " + be.last_refusal)
        return st

    # ---- parity: the first layers sharded vs the same layers on one GPU (rank 0), same input
    n_par = min(2, L)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0x5EED0000)
    h_in = torch.randn(8, B, H, dtype=torch.float32, device=dev, generator=gen)
    h_out = torch.empty(B, H, dtype=torch.float32, device=dev)
    st_par, st_one = make_stack(layers[:n_par], 1), make_stack(layers[:1], 1)
    out_sh = torch.empty(H, dtype=torch.float32, device=dev)
    be.stack_run(st_par, h_in[0, 0].data_ptr(), out_sh.data_ptr())
    be.synchronize()
    be.stack_run(st_one, h_in[0, 0].data_ptr(), h_out[0].data_ptr())
    be.synchronize()
    mine = be.last_shard_hits(lo)
    allhits = [None] * world
    dist.all_gather_object(allhits, mine)
    parity = None
    if rank == 0:
        full = device_layers(be, wl, n_par, dev)
        ref = be.stack_create([m[0] for m in full], [m[1] for m in full], [m[2] for m in full], 1, K, flags)
        out_ref = torch.empty(H, dtype=torch.float32, device=dev)
        be.stack_run(ref, h_in[0, 0].data_ptr(), out_ref.data_ptr())
        be.synchronize()
        idx = torch.zeros(K, dtype=torch.int32, device=dev)
        tmp_out = torch.empty(H, dtype=torch.float32, device=dev)
        be.dev_walk_ffn(full[0][0], full[0][1], full[0][2], h_in[0, 0].data_ptr(), 1, K,
                        flags | larql_b200.WALK_RMSNORM | larql_b200.WALK_RESIDUAL, tmp_out.data_ptr(), idx.data_ptr())
        be.synchronize()
        rel = float((out_sh - out_ref).double().norm() / out_ref.double().norm())
        union = sorted(x for part in allhits for x in part)
        parity = {"layers": n_par, "rel_l2_vs_one_gpu": rel, "ok": bool(rel < 1e-3),
                  "hit_set_equal_layer0": union == sorted(int(i) for i in idx.cpu().tolist())}
        be.stack_destroy(ref)
        del full
        torch.cuda.empty_cache()
    be.stack_destroy(st_par)
    be.stack_destroy(st_one)

    # ---- timing
    stack = make_stack(layers, B)
    launches0 = be.launch_count()
    be.stack_run(stack, h_in[0].data_ptr(), h_out.data_ptr())
    be.synchronize()
    launches_per_step = be.launch_count() - launches0

    def step(i):
        be.stack_run(stack, h_in[i % 8].data_ptr(), h_out.data_ptr())

    dist.barrier()
    with ClockSampler(physical_gpu_index(local)) as clk:
        ms_local = time_steps(step, args.steps, args.warmup, ext, lambda: (be.synchronize(), torch.cuda.synchronize()))
    dist.barrier()
    t = torch.tensor([ms_local], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item())
    tok_s = B / (ms_step * 1e-3)

    # end to end: pinned host residual in, host result out, every step
    hp_in = torch.randn(8, B, H, dtype=torch.float32).pin_memory()
    hp_out = torch.empty(B, H, dtype=torch.float32).pin_memory()
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step(i):
        if not be.stack_run_host(stack, hp_in[i % 8].data_ptr(), hp_out.data_ptr()):
            raise RuntimeError("lq_stack_run_host refused: " + be.last_refusal)

    e2e_step(0)
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i + 1)
    e2e_local = (time.perf_counter() - t0) / e2e_steps * 1e3
    t = torch.tensor([e2e_local], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())

    alg_bytes = algorithmic_bytes_per_token_layer(H, N, K) * L * B
    peak, peak_kind = measured_peaks()
    achieved = alg_bytes / world / (ms_step * 1e-3) / 1e9   # per GPU
    fused = be.stack_path(stack) == 3
    if fused:
        kernel = "walk_fused_q4k_sharded_kernel (one persistent launch per token and rank)"
        how = ("features sharded over %d GPU(s); every rank walks all layers in one persistent kernel and the ranks "
               "exchange histogram, band rows and partial outputs through peer memory (three all-rank barriers per layer)"
               % world)
        note = ("per GPU: algorithmic bytes / n_gpus / step time; at batch 1 a layer is bound by its five barriers and "
                "the serial selection steps between them, not by HBM")
        us = be.fused_phase_us()
        phases = dict(zip(PHASE_NAMES, [float(v) for v in us])) if us is not None else None
    else:
        kernel = "scan_q4k_kernel + gather_q4k_kernel per rank"
        how = "features sharded over %d GPU(s), three NCCL exchanges per layer issued by the library" % world
        note = ("per GPU: algorithmic bytes / n_gpus / step time; batch-1 sharding is bound by the latency "
                "of three exchanges and a dozen small launches per layer, not by HBM")
        phases = None
    cfg = config_of(args, wl)
    cfg["parallelism"] = how
    line = {
        "metric": "walk_ffn_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "walk_gbs": alg_bytes / (ms_step * 1e-3) / 1e9, "algorithmic_bytes_per_step": alg_bytes,
        "exchanges_per_layer": 3, "parity": parity, "phase_us_cta0": phases,
        "roofline": {"kernel": kernel, "bound": "hbm", "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "note": note},
        "cpu_baseline": None,
        "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "path": "lq_stack_run_host on every rank: pinned host residual -> sharded walk over all layers -> host"},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clk.summary(),
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    be.stack_destroy(stack)
    be.comm_destroy()
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    # Leave without running destructors: NCCL's own teardown otherwise races the CUDA context at interpreter exit.
    os._exit(0)


# ------------------------------------------------------------------------ MoE workload (config 4)
def run_moe(args, wl, be, ext, dev, local):
    import larql_b200
    import oracle
    E, H, N, K, T, top_e = wl["experts"], wl["hidden"], wl["features"], wl["top_k"], args.batch, wl["top_e"]
    experts = [[host_matrix(wl, 0x1A2B0000 + 4 * 4096 + 64 * e + j) for j in range(3)] for e in range(E)]
    hm = [[larql_b200.HostMatrix(m.fmt, m.rows, m.cols, m.data, m.scales, float(m.tensor_scale)) for m in ex] for ex in experts]
    gates, ups, downs = [e[0] for e in hm], [e[1] for e in hm], [e[2] for e in hm]
    rng = np.random.Generator(np.random.PCG64(0x5EED0000 + 4000))
    logits = [rng.standard_normal((T, E), dtype=np.float32) for _ in range(4)]
    xs = [oracle.rms_norm(rng.standard_normal((T, H), dtype=np.float32)) for _ in range(4)]
    launches0 = be.launch_count()
    be.moe_walk_ffn(gates, ups, downs, logits[0], xs[0], top_e, K, True, larql_b200.WALK_FORCE_SPARSE)  # uploads the experts
    launches_per_step = be.launch_count() - launches0

    def step(i):
        be.moe_walk_ffn(gates, ups, downs, logits[i % 4], xs[i % 4], top_e, K, True, larql_b200.WALK_FORCE_SPARSE)

    for i in range(args.warmup):
        step(i)
    with ClockSampler(physical_gpu_index(local)) as clk:
        t0 = time.perf_counter()
        for i in range(args.steps):
            step(i)
        ms_step = (time.perf_counter() - t0) / args.steps * 1e3
    tok_s = T / (ms_step * 1e-3)
    # per token: the four routed experts' gate matrices + K up and K down rows each (+ activations)
    alg = T * top_e * algorithmic_bytes_per_token_layer(H, N, K, FMT_MXFP4)
    peak, peak_kind = measured_peaks()
    achieved = alg / (ms_step * 1e-3) / 1e9
    threads = oracle.host_threads()
    cpu = None
    if args.cpu_budget > 0:
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < args.cpu_budget:
            wi, _ = oracle.moe_route(logits[0][n % T], top_e, True)
            for e in wi:
                oracle.walk_token_mt(*experts[int(e)], xs[0][n % T], K, threads)
            n += 1
        cpu = {"value": n / (time.perf_counter() - t0), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{n} tokens x {top_e} experts, oracle walk_token_mt"}
    line = {
        "metric": "moe_walk_ffn_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(args, wl),
        "roofline": {"kernel": "scan_exact_staged_kernel (MXFP4) + gather_fmt_kernel per routed expert", "bound": "hbm",
                     "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "algorithmic_bytes_per_launch": alg,
                     "note": "host-pointer call: routing read-back and one walk per (token, expert) inside the step"},
        "cpu_baseline": cpu,
        "e2e": {"value": tok_s, "unit": "tokens/s", "ms_per_step": ms_step, "h2d_bytes_per_step": T * (H + E) * 4,
                "d2h_bytes_per_step": T * H * 4, "path": "lq_moe_walk_ffn (host logits and activations in, host out)"},
        "gpu_launches": int(launches_per_step * args.steps), "clocks": clk.summary(),
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------ dense sweep (config 2)
def run_dense_sweep(args, wl, be, ext, dev, local):
    """Dense quantised matvec (the walk with K = all): Q4_K and Q8_0 at [1024x3072], [2560x10240], [3840x15360]
    (hidden x features), batch 1 / 8 / 32, through the host-pointer calls.  The line's headline is the largest
    Q4_K shape at --batch; `sweep` holds every combination."""
    import larql_b200
    import oracle
    shapes = [(1024, 3072), (2560, 10240), (3840, 15360)]
    peak, peak_kind = measured_peaks()
    sweep, headline = [], None
    with ClockSampler(physical_gpu_index(local)) as clk:
        for fmt in (FMT_Q4_K, FMT_Q8_0):
            for H, N in shapes:
                w = dict(hidden=H, features=N, fmt=fmt)
                copies = min(64, max(3, int(np.ceil(3 * 126e6 / (N * row_bytes(fmt, H))))))   # rotate past the L2
                base = host_matrix(w, 0x1A2B0000 + 2 * 4096 + H)
                rb = len(base.data) // N
                mats = []
                for c in range(copies):
                    d = np.roll(np.asarray(base.data).reshape(N, rb), c * 37, axis=0).reshape(-1)
                    mats.append(larql_b200.HostMatrix(fmt, N, H, np.ascontiguousarray(d), None, 1.0))
                for B in (1, 8, 32):
                    xs = oracle.rms_norm(np.random.Generator(np.random.PCG64(0x5EED0000 + 2000 + B)).standard_normal(
                        (B, H), dtype=np.float32))

                    def call(i):
                        m = mats[i % copies]
                        if fmt == FMT_Q4_K and B > 1:
                            return be.q4k_matmul(m.data, xs, N, H, B)
                        return [be.gemv(m, xs[t]) for t in range(B)]

                    for i in range(copies):
                        call(i)              # uploads every copy once
                    n_it = max(3, args.steps)
                    t0 = time.perf_counter()
                    for i in range(n_it):
                        call(i)
                    us_host = (time.perf_counter() - t0) / n_it * 1e6
                    alg = N * row_bytes(fmt, H) + B * 4 * (H + N)
                    rec = {"fmt": FMT_NAME[fmt], "hidden": H, "features": N, "batch": B, "us_per_call_host": us_host,
                           "gbs_host": alg / us_host * 1e-3, "algorithmic_bytes": alg}
                    if fmt == FMT_Q4_K and B == 1:
                        # the same matvec with everything resident: device pointers, CUDA events on the library's stream
                        import torch
                        dmats = [torch.from_numpy(np.asarray(m.data)).to(dev) for m in mats]
                        dx = torch.from_numpy(xs[0]).to(dev)
                        dout = torch.empty(N, dtype=torch.float32, device=dev)
                        torch.cuda.synchronize()

                        def dcall(i):
                            t = dmats[i % copies]
                            be.dev_q4k_matvec(t.data_ptr(), t.numel(), dx.data_ptr(), N, H, dout.data_ptr())

                        ms_dev = time_steps(dcall, max(20, args.steps), max(3, args.warmup), ext,
                                            lambda: (be.synchronize(), torch.cuda.synchronize()))
                        rec["us_per_call_dev"] = ms_dev * 1e3
                        rec["gbs_dev"] = alg / (ms_dev * 1e3) * 1e-3
                        del dmats
                    sweep.append(rec)
                    if fmt == FMT_Q4_K and (H, N) == shapes[-1] and B == args.batch:
                        headline = rec
                be.drop_weight_regions()
    headline = headline or sweep[0]
    line = {
        "metric": "dense_matvec_gbs", "value": headline["gbs_host"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": headline["us_per_call_host"] * 1e-3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(args, wl),
        "sweep": sweep,
        "roofline": {"kernel": "scan_q4k_kernel / scan_q4k_mma_kernel / scan_fmt_kernel", "bound": "hbm",
                     "achieved": headline.get("gbs_dev", headline["gbs_host"]), "peak": peak, "peak_kind": peak_kind,
                     "unit": "GB/s", "frac": headline.get("gbs_dev", headline["gbs_host"]) / peak, "traffic": None,
                     "note": "resident call (device pointers, CUDA events) where the record has `gbs_dev`, else the "
                             "host-pointer call, whose fixed cost (copies, launch, wait) dominates at these sizes"},
        "cpu_baseline": None,
        "e2e": {"value": headline["gbs_host"], "unit": "GB/s", "h2d_bytes_per_step": headline["batch"] * headline["hidden"] * 4,
                "d2h_bytes_per_step": headline["batch"] * headline["features"] * 4, "path": "lq_gemv / lq_q4k_matmul"},
        "gpu_launches": int(be.launch_count()), "clocks": clk.summary(),
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------ our arm
def run_ours(args, wl):
    import torch
    import torch.distributed as dist

    import larql_b200

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a short timeout: a rank that dies must fail the others' next collective, not park them
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=180))
    dev = torch.device("cuda", local)
    be = larql_b200.CudaBackend(local)
    ext = torch.cuda.ExternalStream(be.stream(), device=dev)

    if world > 1:
        return run_sharded(args, wl, be, ext, dev, rank, world, local)
    if wl.get("experts"):
        return run_moe(args, wl, be, ext, dev, local)
    if args.workload == "dense_sweep":
        return run_dense_sweep(args, wl, be, ext, dev, local)

    H, N, K, L, B, fmt = wl["hidden"], wl["features"], wl["top_k"], wl["layers"], args.batch, wl["fmt"]
    row = row_bytes(fmt, H)
    # Small workloads rotate over enough distinct weight copies to exceed L2 between reuses.
    copies = 1
    per_layer = 3 * N * row
    if per_layer * L < 3 * 126e6:
        copies = int(np.ceil(3 * 126e6 / (per_layer * L)))
    host_base = None
    if fmt == FMT_Q4_K:
        layers = device_layers(be, wl, L * copies, dev)
    else:
        layers, host_base = device_layers(be, wl, L * copies, dev)

    launches0 = be.launch_count()
    stacks = []
    for c in range(copies):
        ls = layers[c * L:(c + 1) * L]
        st = be.stack_create([m[0] for m in ls], [m[1] for m in ls], [m[2] for m in ls], B, K,
                             larql_b200.WALK_FORCE_SPARSE)
        if st is None:
            raise SystemExit("lq_stack_create refused: " + be.last_refusal)
        stacks.append(st)
    launches_per_step = max(1, (be.launch_count() - launches0) // copies)  # the eager warm-up pass of stack_create

    n_in = 8
    gen = torch.Generator(device=dev)
    gen.manual_seed(0x5EED0000)
    h_in = torch.randn(n_in, B, H, dtype=torch.float32, device=dev, generator=gen)
    h_out = torch.empty(B, H, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()

    def step(i):
        be.stack_run(stacks[i % copies], h_in[i % n_in].data_ptr(), h_out.data_ptr())

    with ClockSampler(physical_gpu_index(local)) as clk:
        ms_step = time_steps(step, args.steps, args.warmup, ext, lambda: (be.synchronize(), torch.cuda.synchronize()))
    tok_s = B / (ms_step * 1e-3)
    alg_bytes = algorithmic_bytes_per_token_layer(H, N, K, fmt) * L  # per token (gate read once per token at batch 1)
    # per step: at batch >= 2 the Q4_K gate matrix is read once per chunk of up to 64 tokens, the 2K up/down rows per token
    if B == 1 or fmt != FMT_Q4_K:
        step_bytes = alg_bytes * B
    else:
        step_bytes = L * (((B + 63) // 64) * N * row + B * (2 * K * row + 8 * H))
    walk_gbs = step_bytes / (ms_step * 1e-3) / 1e9

    fused = fmt == FMT_Q4_K and B == 1
    phase_us = be.fused_phase_us() if fused else None
    phase = dict(zip(PHASE_NAMES, [float(v) for v in phase_us])) if phase_us else {}
    phase_all = None
    if fused and args.phase_sweep:
        # The kernel records the clock stamps of ONE CTA (of the last but one layer); which one is read from the
        # environment at every stamped launch.
        import torch as _t
        rows = []
        for cta in range(_t.cuda.get_device_properties(local).multi_processor_count):
            os.environ["LARQL_B200_FUSED_STAMP_CTA"] = str(cta)
            step(0)
            be.synchronize()
            rows.append([float(v) for v in be.fused_phase_us()][:len(PHASE_NAMES)])
        os.environ.pop("LARQL_B200_FUSED_STAMP_CTA", None)
        arr = np.array(rows)
        phase_all = {n: {"min": float(arr[:, j].min()), "median": float(np.median(arr[:, j])), "max": float(arr[:, j].max())}
                     for j, n in enumerate(PHASE_NAMES)}
    peak, peak_kind = measured_peaks()
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # End to end through the host-pointer C-ABI call of the whole stack (lq_stack_run_host): per
    # step the H2D copy of the token's residual from pinned host memory, every layer on the
    # device, and the D2H read of the final residual, all inside the timed region.
    e2e_steps = max(1, min(args.steps, 10))
    hp_in = torch.randn(n_in, B, H, dtype=torch.float32).pin_memory()
    hp_a = torch.empty(B, H, dtype=torch.float32).pin_memory()

    def e2e_step(i):
        if not be.stack_run_host(stacks[i % copies], hp_in[i % n_in].data_ptr(), hp_a.data_ptr()):
            raise RuntimeError("lq_stack_run_host refused: " + be.last_refusal)

    e2e_step(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i + 1)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    e2e_tok_s = B / (e2e_ms * 1e-3)

    # CPU baseline: the oracle's threaded walk rotating over distinct layers' weights.
    import oracle
    threads = oracle.host_threads()
    cpu = None
    if args.cpu_budget > 0:
        if fmt == FMT_Q4_K:
            n_cpu = min(3, L * copies)
            host_layers = [[oracle.Matrix(FMT_Q4_K, N, H, m.keepalive.cpu().numpy()) for m in layers[l]] for l in range(n_cpu)]
        else:
            host_layers = [host_base]
        s_call, n_calls, dt = cpu_walk_sample(host_layers, wl, B, args.cpu_budget, threads)
        cpu = {"value": B / (s_call * L), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{n_calls} calls of (one layer x {B} token(s)) rotating over {len(host_layers)} distinct layer(s) "
                         f"in {dt:.1f}s, scaled to {L} layer(s)"}

    if fused:
        kernel = "walk_fused_q4k_kernel"
    elif fmt == FMT_Q4_K:
        kernel = "scan_q4k_mma_kernel + gather_q4k_kernel (batched path)"
    else:
        kernel = "scan_exact_staged_kernel + gather_fmt_kernel"
    traffic_ratio = 1.035   # DRAM read + write over algorithmic bytes, ncu capture of the 2-layer case of this workload
    line = {
        "metric": "walk_ffn_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(args, wl),
        "walk_gbs": walk_gbs, "walk_frac_of_measured_hbm": walk_gbs / peak,
        "algorithmic_bytes_per_token": alg_bytes,
        "phase_us_cta0": phase, "phase_us_all_ctas": phase_all,
        "roofline": {"kernel": kernel, "bound": "hbm", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (step_bytes * traffic_ratio) if (args.workload == "llama70b_q4k" and B == 1) else None,
                     "traffic_note": "DRAM read + write per launch = 1.035 x algorithmic, measured by ncu on the 2-layer "
                                     "case of this workload and scaled by layers (traffic grows with the layers)",
                     "algorithmic_bytes_per_launch": step_bytes if fused else None,
                     "avg_launch_ms": ms_step if fused else None, "launches_per_step": int(launches_per_step)},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "path": "lq_stack_run_host: pinned host residual in, all layers on the device, host residual out; "
                        "resident weights"},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clk.summary(),
    }
    if rank == 0:
        print(json.dumps(line))
    for s in stacks:
        be.stack_destroy(s)
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama70b_q4k", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU baseline work (0: skip)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small profiling cases)")
    ap.add_argument("--phase-sweep", action="store_true",
                    help="fused walk only: after the timed steps, stamp every CTA in turn (one more token per CTA) and "
                         "print min / median / max of every phase over the CTAs as `phase_us_all_ctas`")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.layers > 0:
        wl["layers"] = args.layers
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) == 0:
            run_reference(args, wl)
        return
    run_ours(args, wl)


if __name__ == "__main__":
    main()
