"""Oracle checks for selection, router and the composed walk (CPU only)."""
import numpy as np
import pytest

import oracle
from conftest import rel_l2, seeded_weights, seeded_x


# ---- gate_knn/mod.rs:231-287 top_k_by_abs cases
def test_top_k_by_abs_reference_cases():
    idx, val = oracle.top_k_by_abs([0.1, -0.9, 0.5, 0.3], 2)
    assert idx.tolist() == [1, 2] and abs(val[0] + 0.9) < 1e-6
    assert oracle.top_k_by_abs([1.0, -2.0, 0.5], 1)[0].tolist() == [1]
    assert len(oracle.top_k_by_abs([1.0, 2.0], 10)[0]) == 2
    assert len(oracle.top_k_by_abs([1.0, 2.0, 3.0], 0)[0]) == 0
    assert len(oracle.top_k_by_abs([], 5)[0]) == 0
    _, v = oracle.top_k_by_abs([0.3, 0.1, 0.9, 0.5, 0.7], 3)
    assert np.all(np.abs(v[:-1]) >= np.abs(v[1:]))
    with pytest.raises(ValueError):
        oracle.top_k_by_abs([1.0, float("nan")], 1)


def test_top_k_total_order_equals_literal_heap():
    rng = np.random.Generator(np.random.PCG64(11))
    for n, k in [(1, 1), (7, 3), (64, 64), (1000, 17), (3072, 512), (5000, 4999)]:
        s = rng.standard_normal(n, dtype=np.float32)
        a = oracle.top_k_by_abs(s, k)
        b = oracle.top_k_by_abs(s, k, heap=True)
        assert a[0].tolist() == b[0].tolist()
    # ties (including across the K boundary): lower index wins in both
    s = np.array([1.0, -2.0, 2.0, 0.5, 2.0, -1.0, 1.0], np.float32)
    for k in range(1, 8):
        a = oracle.top_k_by_abs(s, k)
        b = oracle.top_k_by_abs(s, k, heap=True)
        assert a[0].tolist() == b[0].tolist()
    assert oracle.top_k_by_abs(s, 2)[0].tolist() == [1, 2]
    assert oracle.top_k_by_abs(np.zeros(5, np.float32), 2)[0].tolist() == [0, 1]


# ---- moe/math.rs:229-259 router top_k cases
def test_moe_top_k_reference_cases():
    idx, val = oracle.moe_top_k([0.1, 0.5, 0.3, 0.9, 0.2], 3)
    assert idx.tolist() == [3, 1, 2] and np.allclose(val, [0.9, 0.5, 0.3])
    assert oracle.moe_top_k([0.1, 0.5, 0.3], 99)[0].tolist() == [1, 2, 0]
    idx, val = oracle.moe_top_k([1.0, 2.0, 2.0, 0.5], 3)
    assert idx.tolist() == [1, 2, 0] and val.tolist() == [2.0, 2.0, 1.0]
    assert oracle.moe_top_k([0.5, 2.0, 2.0], 1)[0].tolist() == [1]
    assert oracle.moe_top_k([3.0, 3.0, 3.0, 3.0], 2)[0].tolist() == [0, 1]


def test_moe_route_softmax_top4_renormalised():
    logits = seeded_x(5, 32)
    idx, w = oracle.moe_route(logits, 4, True)
    p = np.exp(logits - logits.max())
    p /= p.sum()
    want = np.argsort(-p, kind="stable")[:4]
    assert idx.tolist() == want.tolist()
    assert abs(w.sum() - 1.0) < 1e-6 and np.allclose(w, p[want] / p[want].sum(), rtol=1e-5)


def test_rms_norm_matches_formula():
    x = seeded_x(3, 2, 1024)
    got = oracle.rms_norm(x)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6).astype(np.float32)
    assert np.array_equal(got, want.astype(np.float32))


@pytest.mark.parametrize("fmt", [oracle.FMT_Q4_K, oracle.FMT_Q8_0, oracle.FMT_MXFP4, oracle.FMT_NVFP4])
def test_walk_token_matches_dequantised_formula(fmt):
    h, n, k = 256, 96, 24
    gate = oracle.quantize_matrix(fmt, seeded_weights(100 + fmt, n, h))
    up = oracle.quantize_matrix(fmt, seeded_weights(200 + fmt, n, h))
    down = oracle.quantize_matrix(fmt, seeded_weights(300 + fmt, n, h))
    x = oracle.rms_norm(seeded_x(400 + fmt, h))
    out, idx, gs = oracle.walk_token(gate, up, down, x, k)
    g, u, d = gate.dequantize(), up.dequantize(), down.dequantize()
    scores = g.astype(np.float64) @ x
    want_idx = np.argsort(-np.abs(scores), kind="stable")[:k]
    assert sorted(idx.tolist()) == sorted(want_idx.tolist())
    act = scores[idx] / (1 + np.exp(-scores[idx])) * (u[idx].astype(np.float64) @ x)
    want = act @ d[idx].astype(np.float64)
    assert rel_l2(out, want) < 1e-5
    assert np.allclose(gs, scores[idx], rtol=1e-4, atol=1e-6)
    # threaded baseline: same hit set, output equal up to summation order
    out_mt, idx_mt = oracle.walk_token_mt(gate, up, down, x, k, 3)
    assert idx_mt.tolist() == idx.tolist() and rel_l2(out_mt, out) < 1e-5
    assert np.array_equal(oracle.gemv_mt(gate, x, 3), gate.gemv(x))
    # K >= N is every feature; the dense rewrite gives the same up to order
    out_all, idx_all, _ = oracle.walk_token(gate, up, down, x, n + 5)
    assert len(idx_all) == n
    assert rel_l2(oracle.walk_token_dense(gate, up, down, x), out_all) < 1e-5


def test_run_ffn_adds_residual():
    h, n = 256, 64
    m = [oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(s, n, h)) for s in (1, 2, 3)]
    hin = seeded_x(9, h)
    out, idx = oracle.run_ffn_token(*m, hin, 16)
    w, idx2, _ = oracle.walk_token(*m, oracle.rms_norm(hin), 16)
    assert idx.tolist() == idx2.tolist()
    assert np.array_equal(out, hin + w)
