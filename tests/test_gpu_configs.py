"""GPU parity tests at the full sizes of the benchmark configurations, through the C ABI, against
the CPU oracle: the Qwen3-0.6B-shaped layer over 1000 queries, one Gemma-3-12B-shaped layer at
batch 1 / 16 / 64, the gpt-oss-shaped MXFP4 MoE with all 32 experts at 1 / 16 / 256 tokens and one
Llama-3-70B-shaped NVFP4 layer; plus the device Q4_K encoder against the CPU encoder and the
host-side refusals that keep misaligned weights away from the kernels.

Bar: selected feature sets and encoder bytes exact; outputs within 1e-3 relative L2 (f32)."""
import numpy as np
import pytest

import oracle
from conftest import rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3


@pytest.fixture(scope="module")
def be():
    import larql_b200
    b = larql_b200.CudaBackend(0)
    yield b
    b.close()


@pytest.fixture(autouse=True)
def _fresh_weight_cache(be):
    yield
    be.drop_weight_regions()


def host(m: oracle.Matrix):
    import larql_b200
    return larql_b200.HostMatrix(m.fmt, m.rows, m.cols, m.data, m.scales, float(m.tensor_scale))


def layer(seed, n, h, fmt=oracle.FMT_Q4_K):
    return [oracle.quantize_matrix(fmt, seeded_weights(seed + i, n, h)) for i in range(3)]


def check_tokens(be, gate, up, down, xs, k, tokens=None):
    import larql_b200
    res = be.walk_ffn(host(gate), host(up), host(down), xs, k, larql_b200.WALK_FORCE_SPARSE)
    assert res is not None, be.last_refusal
    out, hits = res
    xs2, out2 = xs.reshape(-1, gate.cols), out.reshape(-1, gate.cols)
    for t in (range(xs2.shape[0]) if tokens is None else tokens):
        want, idx, _ = oracle.walk_token(gate, up, down, xs2[t], k)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist()), f"token {t}: selected set differs"
        assert rel_l2(out2[t], want) < OUT_TOL, f"token {t}"
    return out


def test_device_q4k_encoder_is_byte_identical_to_the_cpu_encoder(be):
    """lq_dev_quantize_q4k against quantize_q4_k (q4_common/quantize.rs:89-189), byte for byte."""
    import torch
    rows, cols = 67, 2048
    w = seeded_weights(0xE0C, rows, cols)
    w[3, :256] = 0.0                       # an all-zero super-block
    w[5, :] *= np.float32(1e-4)            # tiny scales (f16-subnormal d / dmin)
    w[7, 100] = 3.0                        # an outlier that dominates its sub-block
    w[9, 256:512] = np.float32(0.25)       # a constant super-block (zero range in every sub-block)
    w[11, :] = np.abs(w[11, :])            # all positive: min clamps to zero
    w[13, :] = -np.abs(w[13, :])           # all negative: max clamps to zero
    w[15, ::2] *= np.float32(50.0)         # mixed magnitudes inside every sub-block
    want = oracle.quantize_matrix(oracle.FMT_Q4_K, w).data
    src = torch.from_numpy(w.reshape(-1)).cuda()
    dst = torch.zeros(rows * cols // 256 * 144, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert be.dev_quantize_q4k(src.data_ptr(), rows * cols, dst.data_ptr())
    be.synchronize()
    got = dst.cpu().numpy()
    assert got.tobytes() == np.asarray(want, dtype=np.uint8).tobytes()
    # a larger seeded matrix of the benchmark's distribution
    w2 = seeded_weights(0x1A2B0000, 512, 8192)
    want2 = oracle.quantize_matrix(oracle.FMT_Q4_K, w2).data
    src2 = torch.from_numpy(w2.reshape(-1)).cuda()
    dst2 = torch.zeros(512 * 8192 // 256 * 144, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert be.dev_quantize_q4k(src2.data_ptr(), w2.size, dst2.data_ptr())
    be.synchronize()
    assert dst2.cpu().numpy().tobytes() == np.asarray(want2, dtype=np.uint8).tobytes()


def test_config1_qwen_shaped_layer_1000_queries(be):
    """Hidden 1024, intermediate 3072, K = 512, 1000 seeded queries, one at a time and as batches."""
    import larql_b200
    gate, up, down = layer(0x1A2B0000 + 4096, 3072, 1024)
    xs = oracle.rms_norm(seeded_x(0x5EED0000 + 1000, 1000, 1024))
    out_b = check_tokens(be, gate, up, down, xs, 512)          # batched path, every token against the oracle
    # the batch-1 path (fused persistent walk) on a slice of the same queries, against the same oracle
    for q in range(0, 1000, 37):
        out1 = check_tokens(be, gate, up, down, xs[q], 512)
        assert rel_l2(out1.reshape(-1), out_b[q]) < OUT_TOL


@pytest.mark.parametrize("batch", [1, 16, 64])
def test_config3_gemma_shaped_layer_full_size(be, batch):
    """Hidden 3840, intermediate 15360, K = 1024 at batch 1, 16 and 64."""
    gate, up, down = layer(0x1A2B0000 + 3 * 4096, 15360, 3840)
    xs = oracle.rms_norm(seeded_x(0x5EED0000 + 3000 + batch, batch, 3840))
    check_tokens(be, gate, up, down, xs, 1024)


@pytest.fixture(scope="module")
def gpt_oss_experts():
    return [layer(0x1A2B0000 + 4 * 4096 + 64 * e, 2880, 2880, oracle.FMT_MXFP4) for e in range(32)]


@pytest.mark.parametrize("tokens", [1, 16, 256])
def test_config4_moe_32_experts(be, gpt_oss_experts, tokens):
    """gpt-oss-20B shape: hidden 2880, 32 experts of intermediate 2880 (MXFP4), top-4 routing by softmax over
    seeded N(0,1) logits, per-expert K = 768."""
    import larql_b200
    E, H, N, K = 32, 2880, 2880, 768
    experts = gpt_oss_experts
    logits = seeded_x(0x5EED0000 + 4000 + tokens, tokens, E)
    xs = oracle.rms_norm(seeded_x(0x5EED0000 + 4500 + tokens, tokens, H))
    got, idx, w = be.moe_walk_ffn([host(e[0]) for e in experts], [host(e[1]) for e in experts],
                                  [host(e[2]) for e in experts], logits, xs, 4, K, True,
                                  larql_b200.WALK_FORCE_SPARSE)
    for t in range(tokens):
        wi, ww = oracle.moe_route(logits[t], 4, True)
        assert idx[t].tolist() == wi.tolist()
        assert np.allclose(w[t], ww, rtol=0, atol=1e-6)
        want = np.zeros(H, np.float32)
        for e, we in zip(wi, ww):
            o, _, _ = oracle.walk_token(*experts[int(e)], xs[t], K)
            want += np.float32(we) * o
        assert rel_l2(got[t], want) < OUT_TOL, f"token {t}"


def test_config5_llama70b_shaped_nvfp4_layer(be):
    """Hidden 8192, intermediate 28672, K = 4096, NVFP4 (e2m1 values, e4m3 scale per 16, f32 tensor scale)."""
    n, h, k = 28672, 8192, 4096
    gate = oracle.quantize_matrix(oracle.FMT_NVFP4, seeded_weights(0x1A2B0000 + 5 * 4096, n, h))
    # up and down: the gate's rows in another order (rows quantise independently; this keeps the host-side
    # set-up of three 235 M-weight matrices within the test budget)
    def rolled(m, shift):
        d = np.roll(np.asarray(m.data).reshape(n, -1), shift, axis=0).reshape(-1).copy()
        s = np.roll(np.asarray(m.scales).reshape(n, -1), shift, axis=0).reshape(-1).copy()
        return oracle.Matrix(m.fmt, n, h, d, s, m.tensor_scale)
    up, down = rolled(gate, 7919), rolled(gate, 12345)
    for q in range(2):
        x = oracle.rms_norm(seeded_x(0x5EED0000 + 5000 + q, h))
        check_tokens(be, gate, up, down, x, k)


def test_misaligned_device_weights_are_refused_before_any_launch(be):
    """Only the host-side refusal is exercised: no kernel ever sees a misaligned pointer."""
    import torch

    import larql_b200
    n, h, k = 64, 256, 8
    row = h // 256 * 144
    buf = torch.zeros(n * row + 64, dtype=torch.uint8, device="cuda")
    x = torch.zeros(h, dtype=torch.float32, device="cuda")
    out = torch.zeros(h, dtype=torch.float32, device="cuda")
    ok = larql_b200.DeviceMatrix(larql_b200.FMT_Q4_K, n, h, buf.data_ptr(), n * row, keepalive=buf)
    bad = larql_b200.DeviceMatrix(larql_b200.FMT_Q4_K, n, h, buf.data_ptr() + 8, n * row, keepalive=buf)
    for trio in ((bad, ok, ok), (ok, bad, ok), (ok, ok, bad)):
        with pytest.raises(larql_b200.BackendError):
            be.dev_walk_ffn(*trio, x.data_ptr(), 1, k, larql_b200.WALK_FORCE_SPARSE, out.data_ptr())
    # a host matrix at an odd offset inside a registered region gets an aligned private copy and works
    gate, up, down = layer(0xA11, n, h)
    blob = np.zeros(gate.data.size + 8 + 16, np.uint8)
    off = (-blob.ctypes.data) % 16 + 8          # 8 mod 16
    blob[off:off + gate.data.size] = gate.data
    be.register_weight_region(blob)
    g2 = oracle.Matrix(gate.fmt, n, h, blob[off:off + gate.data.size])
    xq = oracle.rms_norm(seeded_x(0xA12, h))
    out_h, hits = be.walk_ffn(host(g2), host(up), host(down), xq, k, larql_b200.WALK_FORCE_SPARSE)
    want, idx, _ = oracle.walk_token(gate, up, down, xq, k)
    assert sorted(hits[0].tolist()) == sorted(idx.tolist()) and rel_l2(out_h, want) < OUT_TOL


def test_contexts_on_two_devices_in_one_process():
    """A host with several GPUs holds one context per device in one process (what a backend registry
    does); every call runs on its context's device whatever device is current."""
    import torch

    import larql_b200
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    b0, b1 = larql_b200.CudaBackend(0), larql_b200.CudaBackend(1)
    try:
        gate, up, down = layer(0xD0, 3072, 1024)
        x = oracle.rms_norm(seeded_x(0xD1, 1024))
        want, idx, _ = oracle.walk_token(gate, up, down, x, 512)
        torch.cuda.set_device(0)   # the "wrong" device for b1
        for b in (b1, b0, b1):
            out, hits = b.walk_ffn(host(gate), host(up), host(down), x, 512, larql_b200.WALK_FORCE_SPARSE)
            assert sorted(hits[0].tolist()) == sorted(idx.tolist()) and rel_l2(out, want) < OUT_TOL
        assert torch.cuda.current_device() == 0
    finally:
        b0.close()
        b1.close()
