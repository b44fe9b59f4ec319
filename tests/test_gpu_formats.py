"""GPU parity tests for the Q8_0 / MXFP4 / NVFP4 paths and the MoE router, through the C ABI,
against the CPU oracle.

Bar: exact-order gemv bit-identical to the CPU backend's arithmetic, top-K index sets exact,
walk outputs within 1e-3 relative L2 (f32), router selections exact and weights within 1e-6."""
import numpy as np
import pytest

import oracle
from conftest import bits, rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3
FMTS = [oracle.FMT_Q8_0, oracle.FMT_MXFP4, oracle.FMT_NVFP4]
NAMES = {oracle.FMT_Q8_0: "q8_0", oracle.FMT_MXFP4: "mxfp4", oracle.FMT_NVFP4: "nvfp4"}


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


def layer(seed, n, h, fmt):
    return [oracle.quantize_matrix(fmt, seeded_weights(seed + i, n, h)) for i in range(3)]


def test_supports_all_four_formats(be):
    for f in (oracle.FMT_Q4_K, *FMTS):
        assert be.supports_quant(f)


@pytest.mark.parametrize("fmt", FMTS, ids=NAMES.get)
@pytest.mark.parametrize("rows,cols", [(1, 32), (37, 512), (300, 2880), (1024, 1024), (96, 8192)])
def test_exact_gemv_is_bit_identical_to_cpu_backend(be, fmt, rows, cols):
    m = oracle.quantize_matrix(fmt, seeded_weights(rows * 7 + cols + fmt, rows, cols))
    x = seeded_x(cols + rows, cols)
    got = be.gemv(host(m), x, exact=True)
    assert bits(got).tolist() == bits(m.gemv(x)).tolist()


@pytest.mark.parametrize("fmt", FMTS, ids=NAMES.get)
@pytest.mark.parametrize("rows,cols", [(37, 512), (3072, 1024), (300, 2880), (10240, 2560)])
def test_fast_gemv_within_tolerance_and_deterministic(be, fmt, rows, cols):
    m = oracle.quantize_matrix(fmt, seeded_weights(rows + cols + fmt, rows, cols))
    x = seeded_x(cols, cols)
    got = be.gemv(host(m), x)
    want = m.gemv(x)
    scale = np.abs(m.dequantize()).astype(np.float64) @ np.abs(x).astype(np.float64)
    assert np.max(np.abs(got.astype(np.float64) - want) / scale) < 2e-4   # fixed-point planes: ~2^-15 of sum|w||x|
    assert rel_l2(got, want) < OUT_TOL
    assert np.array_equal(bits(got), bits(be.gemv(host(m), x)))


def test_trait_shaped_gemv_entry_points_and_refusals(be):
    x = seeded_x(5, 512)
    q8 = oracle.quantize_matrix(oracle.FMT_Q8_0, seeded_weights(1, 40, 512))
    mx = oracle.quantize_matrix(oracle.FMT_MXFP4, seeded_weights(2, 40, 512))
    nv = oracle.quantize_matrix(oracle.FMT_NVFP4, seeded_weights(3, 40, 512))
    assert rel_l2(be.q8_0_gemv(q8.data, x, 40, 512), q8.gemv(x)) < OUT_TOL
    assert rel_l2(be.quant_matvec(oracle.FMT_Q8_0, q8.data, x, 40, 512), q8.gemv(x)) < OUT_TOL
    assert rel_l2(be.mxfp4_gemv(mx.data, mx.scales, x, 40, 512), mx.gemv(x)) < OUT_TOL
    assert rel_l2(be.nvfp4_gemv(nv.data, nv.scales, float(nv.tensor_scale), x, 40, 512), nv.gemv(x)) < OUT_TOL
    # exact-length rules of q8_0_gemv / nvfp4_gemv: any mismatch is a refusal (None), as on the CPU backend
    assert be.q8_0_gemv(q8.data[:-1], x, 40, 512) is None
    assert be.q8_0_gemv(q8.data, x[:-1], 40, 512) is None
    assert be.q8_0_gemv(q8.data, x, 39, 512) is None
    assert be.nvfp4_gemv(nv.data, nv.scales[:-1], float(nv.tensor_scale), x, 40, 512) is None
    assert be.nvfp4_gemv(nv.data, nv.scales, float(nv.tensor_scale), x, 40, 500) is None
    # n == 0: empty result
    assert be.q8_0_gemv(np.zeros(0, np.uint8), x, 0, 512).size == 0


def _check_walk(be, gate, up, down, x, k, flags=4):
    out, hits = be.walk_ffn(host(gate), host(up), host(down), x, k, flags)
    x2, out2 = x.reshape(-1, gate.cols), out.reshape(-1, gate.cols)
    for t in range(x2.shape[0]):
        want, idx, _ = oracle.walk_token(gate, up, down, x2[t], k)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist()), f"token {t}: top-K index set differs"
        assert rel_l2(out2[t], want) < OUT_TOL, f"token {t}"
    return out, hits


@pytest.mark.parametrize("fmt", FMTS, ids=NAMES.get)
@pytest.mark.parametrize("h,n,k", [(256, 64, 8), (512, 300, 37), (1024, 3072, 512), (2880, 2880, 768),
                                   (3840, 2048, 256), (8192, 1024, 128)])
def test_walk_index_sets_exact_and_outputs_within_tolerance(be, fmt, h, n, k):
    gate, up, down = layer(h + n + fmt, n, h, fmt)
    for q in range(2):
        x = oracle.rms_norm(seeded_x(0x5EED0000 + q, h))
        _check_walk(be, gate, up, down, x, k)
    st = be.last_walk_stats()
    assert st.n_hits == min(k, n) and st.n_certain + st.need == k and st.n_band >= st.need


@pytest.mark.parametrize("fmt", FMTS, ids=NAMES.get)
def test_walk_edge_cases(be, fmt):
    import larql_b200
    gate, up, down = layer(77 + fmt, 96, 256, fmt)
    x = oracle.rms_norm(seeded_x(78, 256))
    F = larql_b200.WALK_FORCE_SPARSE
    out, hits = be.walk_ffn(host(gate), host(up), host(down), x, 1000, F)
    assert sorted(hits[0].tolist()) == list(range(96))
    assert rel_l2(out, oracle.walk_token(gate, up, down, x, 1000)[0]) < OUT_TOL
    out_d, hits_d = be.walk_ffn(host(gate), host(up), host(down), x, 80, 0)      # 80 % rule: dense
    assert len(hits_d[0]) == 96 and rel_l2(out_d, oracle.walk_token_dense(gate, up, down, x)) < OUT_TOL
    out0, hits0 = be.walk_ffn(host(gate), host(up), host(down), x, 0, F)
    assert len(hits0[0]) == 0 and not out0.any()
    outz, hitsz = be.walk_ffn(host(gate), host(up), host(down), np.zeros(256, np.float32), 10, F)
    assert sorted(hitsz[0].tolist()) == list(range(10)) and not outz.any()
    # duplicated gate rows: exact ties across the boundary resolve to the lower index
    rb = gate.row_bytes()
    sc = None if gate.scales is None else np.tile(gate.scales[:gate.scales.size // 96], 96)
    g2 = oracle.Matrix(gate.fmt, 96, 256, np.tile(gate.data[:rb], 96), sc, gate.tensor_scale)
    _, hits_t = be.walk_ffn(host(g2), host(up), host(down), x, 7, F)
    assert sorted(hits_t[0].tolist()) == list(range(7))
    xn = x.copy()
    xn[5] = np.nan
    with pytest.raises(larql_b200.BackendError):
        be.walk_ffn(host(gate), host(up), host(down), xn, 8, F)
    q4 = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(1, 96, 256))
    assert be.walk_ffn(host(gate), host(q4), host(down), x, 8) is None              # mixed formats refused


@pytest.mark.parametrize("fmt", FMTS, ids=NAMES.get)
def test_run_ffn_norm_residual_and_batch(be, fmt):
    import larql_b200
    gate, up, down = layer(91 + fmt, 512, 1024, fmt)
    hin = seeded_x(92, 3, 1024)
    flags = larql_b200.WALK_RMSNORM | larql_b200.WALK_RESIDUAL | larql_b200.WALK_FORCE_SPARSE
    out, hits = be.walk_ffn(host(gate), host(up), host(down), hin, 64, flags)
    for t in range(3):
        want, idx = oracle.run_ffn_token(gate, up, down, hin[t], 64)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist())
        assert rel_l2(out[t] - hin[t], want - hin[t]) < OUT_TOL


# ------------------------------------------------------------------------- MoE
def test_moe_route_matches_reference(be):
    rng = np.random.Generator(np.random.PCG64(11))
    logits = rng.standard_normal((64, 32)).astype(np.float32)
    for renorm in (True, False):
        idx, w = be.moe_route(logits, 4, renorm)
        for t in range(64):
            wi, ww = oracle.moe_route(logits[t], 4, renorm)
            assert idx[t].tolist() == wi.tolist()
            assert np.allclose(w[t], ww, rtol=0, atol=1e-6)
    # ties: equal logits resolve to the lower expert index, in index order
    tie = np.zeros((1, 8), np.float32)
    tie[0, 5] = 1.0
    idx, w = be.moe_route(tie, 3, True)
    assert idx[0].tolist() == [5, 0, 1]
    wi, ww = oracle.moe_route(tie[0], 3, True)
    assert wi.tolist() == [5, 0, 1] and np.allclose(w[0], ww, atol=1e-6)
    # top_k >= experts returns all, sorted by probability then index
    idx, w = be.moe_route(logits[:2, :6], 10, True)
    assert idx.shape == (2, 6) and np.allclose(w.sum(axis=1), 1.0, atol=1e-5)
    for t in range(2):
        assert idx[t].tolist() == oracle.moe_route(logits[t, :6], 10, True)[0].tolist()


def test_moe_expert_walk_gpt_oss_shape(be):
    # 8 experts of the gpt-oss expert shape (hidden 2880, intermediate 2880, MXFP4), top-4 routing,
    # per-expert K = 768, a few tokens
    import larql_b200
    E, H, N, K, T = 8, 2880, 2880, 768, 3
    experts = [layer(0x600 + 10 * e, N, H, oracle.FMT_MXFP4) for e in range(E)]
    rng = np.random.Generator(np.random.PCG64(5))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    xs = oracle.rms_norm(seeded_x(0x77, T, H))
    got, idx, w = be.moe_walk_ffn([host(e[0]) for e in experts], [host(e[1]) for e in experts],
                                  [host(e[2]) for e in experts], logits, xs, 4, K, True,
                                  larql_b200.WALK_FORCE_SPARSE)
    for t in range(T):
        wi, ww = oracle.moe_route(logits[t], 4, True)
        assert idx[t].tolist() == wi.tolist()
        want = np.zeros(H, np.float32)
        for e, we in zip(wi, ww):
            o, _, _ = oracle.walk_token(*experts[int(e)], xs[t], K)
            want += np.float32(we) * o
        assert rel_l2(got[t], want) < OUT_TOL


@pytest.mark.parametrize("fmt", [oracle.FMT_Q4_K, oracle.FMT_NVFP4, oracle.FMT_Q8_0],
                         ids=["q4k_pair_by_pair", "nvfp4_grouped", "q8_0_grouped"])
def test_moe_expert_walk_both_routes(be, fmt):
    """Block-format experts of one shape take the grouped route (all pairs in the same launches, experts through a
    device table); Q4_K experts are walked pair by pair.  Same contract, same tolerance; one token routes to
    every expert (top_e == experts), so every table entry is read."""
    import larql_b200
    E, H, N, K, T = 4, 512, 768, 96, 5
    experts = [layer(0x900 + 10 * e, N, H, fmt) for e in range(E)]
    rng = np.random.Generator(np.random.PCG64(23))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    xs = oracle.rms_norm(seeded_x(0x91, T, H))
    for top_e in (2, E):
        got, idx, w = be.moe_walk_ffn([host(e[0]) for e in experts], [host(e[1]) for e in experts],
                                      [host(e[2]) for e in experts], logits, xs, top_e, K, True,
                                      larql_b200.WALK_FORCE_SPARSE)
        for t in range(T):
            wi, ww = oracle.moe_route(logits[t], top_e, True)
            assert idx[t].tolist() == wi.tolist()
            assert np.allclose(w[t], ww, rtol=0, atol=1e-6)
            want = np.zeros(H, np.float32)
            for e, we in zip(wi, ww):
                o, _, _ = oracle.walk_token(*experts[int(e)], xs[t], K)
                want += np.float32(we) * o
            assert rel_l2(got[t], want) < OUT_TOL


# ---------------------------------------------------- device seam: multi gemv, f16 / bf16, top-k by value
def test_gemv_multi_matches_single_gemvs(be):
    """mxfp4_gemv_multi / nvfp4_gemv_multi (backend/matmul.rs:242-286): the results of the single gemvs."""
    k = 2880
    x = oracle.rms_norm(seeded_x(0x301, k))
    alive = []  # weights are cached on the device by host address: keep every matrix of this test alive
    for fmt in (oracle.FMT_MXFP4, oracle.FMT_NVFP4, oracle.FMT_Q8_0, oracle.FMT_Q4_K):
        kk = k if fmt != oracle.FMT_Q4_K else 2816
        xx = np.ascontiguousarray(x[:kk])
        mats = [oracle.quantize_matrix(fmt, seeded_weights(0x310 + i, n, kk)) for i, n in enumerate((96, 257, 33))]
        alive.append(mats)
        for exact in (True, False):
            outs = be.gemv_multi([host(m) for m in mats], xx, exact=exact)
            assert outs is not None and len(outs) == 3
            for m, o in zip(mats, outs):
                single = be.gemv(host(m), xx, exact=exact)
                assert np.array_equal(bits(o), bits(single))
                if exact:
                    assert np.array_equal(bits(o), bits(m.gemv(xx)))
    # a matrix whose k differs from the input's length: refusal, not a wrong answer
    bad = oracle.quantize_matrix(oracle.FMT_MXFP4, seeded_weights(1, 8, 64))
    assert be.gemv_multi([host(bad)], x) is None


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_f16_bf16_gemv_exact_order_and_fast(be, kind):
    """f16_gemv / bf16_gemv (backend/matmul.rs:124-147) against the reference test device's loop."""
    rng = np.random.Generator(np.random.PCG64(0x16))
    for n, k in ((37, 64), (300, 1000), (129, 4097)):
        w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05))
        if kind == "f16":
            wb = w.astype(np.float16).view(np.uint16)
        else:
            wb = (w.view(np.uint32) >> 16).astype(np.uint16)
        x = rng.standard_normal(k, dtype=np.float32)
        want = oracle.gemv16(wb, x, n, k, 0 if kind == "f16" else 1)
        got = be.gemv16(wb, x, n, k, kind, exact=True)
        assert np.array_equal(bits(got), bits(want))
        fast = be.gemv16(wb, x, n, k, kind, exact=False)
        assert rel_l2(fast, want) < 1e-5
        outs = be.gemv16_multi([(wb, n, k), (wb[: n // 2], n // 2, k)], x, kind, exact=True)
        assert np.array_equal(bits(outs[0]), bits(want)) and np.array_equal(bits(outs[1]), bits(want[: n // 2]))
    # shape refusals: short weights, wrong input length
    assert be.gemv16(np.zeros(10, np.uint16), np.zeros(4, np.float32), 3, 4, kind) is None
    assert be.gemv16(np.zeros(12, np.uint16), np.zeros(5, np.float32), 3, 4, kind) is None


def test_q4k_matvec_topk_by_value(be):
    """q4k_matvec_topk (backend/quant_matvec.rs:268-277): the rows a full q4k_matvec + CPU reduce picks."""
    n, h = 5000, 1024
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(0x7061, n, h))
    x = oracle.rms_norm(seeded_x(0x7062, h))
    scores = oracle.q4k_matvec(m.data, x, n, h)
    for k in (1, 8, 100, 5000, 9000):
        got = be.q4k_matvec_topk(m.data, x, n, h, k)
        idx, val = oracle.top_k_by_value(scores, k)
        assert [r for r, _ in got] == idx.tolist()
        assert np.array_equal(bits(np.array([v for _, v in got], np.float32)), bits(val))
    # ties resolve to the lower row: duplicate one row many times
    d = np.asarray(m.data).reshape(n, -1).copy()
    best = int(oracle.top_k_by_value(scores, 1)[0][0])
    d[100:140] = d[best]
    s2 = oracle.q4k_matvec(d.reshape(-1), x, n, h)
    got = be.q4k_matvec_topk(d.reshape(-1), x, n, h, 7)
    assert [r for r, _ in got] == oracle.top_k_by_value(s2, 7)[0].tolist()
    # f16 LM-head form
    rng = np.random.Generator(np.random.PCG64(0x7063))
    wf = (rng.standard_normal((3000, 512), dtype=np.float32) * np.float32(0.05)).astype(np.float16).view(np.uint16)
    xs = rng.standard_normal(512, dtype=np.float32)
    sf = oracle.gemv16(wf, xs, 3000, 512, 0)
    gotf = be.f16_gemv_topk(wf, xs, 3000, 512, 16)
    assert [r for r, _ in gotf] == oracle.top_k_by_value(sf, 16)[0].tolist()


def test_fp4_fast_scan_with_band_keeps_the_exact_selection():
    """The switchable fast scan + band route of the FP4 walks (bound c1 * sum |w x| per row) selects the same rows
    as the exact-order scan.  The switch is read once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    child = textwrap.dedent('''
        import sys
        sys.path.insert(0, %r); sys.path.insert(0, %r)
        import numpy as np, larql_b200, oracle
        from conftest import seeded_weights, seeded_x, rel_l2
        be = larql_b200.CudaBackend(0)
        ok = True
        for fmt in (oracle.FMT_MXFP4, oracle.FMT_NVFP4):
            n, h, k = 3072, 2048, 400
            g, u, d = (oracle.quantize_matrix(fmt, seeded_weights(0xF4 + i + fmt, n, h)) for i in range(3))
            hm = lambda m: larql_b200.HostMatrix(m.fmt, m.rows, m.cols, m.data, m.scales, float(m.tensor_scale))
            for q in range(3):
                x = oracle.rms_norm(seeded_x(0xF5 + q, h))
                want, idx, _ = oracle.walk_token(g, u, d, x, k)
                out, hits = be.walk_ffn(hm(g), hm(u), hm(d), x, k, larql_b200.WALK_FORCE_SPARSE)
                ok = ok and sorted(hits[0].tolist()) == sorted(idx.tolist()) and rel_l2(out.reshape(-1), want) < 1e-3
        sys.exit(0 if ok else 3)
    ''') % (root, os.path.join(root, "tests"))
    env = dict(os.environ, LARQL_B200_FMT_FAST_SCAN="1")
    r = subprocess.run([sys.executable, "-c", child], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
