"""GPU parity tests for the Q4_K path, through the C ABI, against the CPU oracle.

Bar: dequantised weights, exact-order scores and top-K index sets bit-exact; walk
outputs within 1e-3 relative L2 (f32)."""
import numpy as np
import pytest

import oracle
from conftest import bits, rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3  # relative L2 on f32 outputs, the tolerance the path is specified to


@pytest.fixture(scope="module")
def be():
    import larql_b200
    b = larql_b200.CudaBackend(0)
    yield b
    b.close()


@pytest.fixture(autouse=True)
def _fresh_weight_cache(be):
    # Weights are cached on the device by host (address, length), which is only sound for
    # long-lived immutable memory (the reference's mmap slices).  Test arrays are freed and
    # their addresses reused, so the cache is emptied between tests.
    yield
    be.drop_weight_regions()


def host(m: oracle.Matrix):
    import larql_b200
    return larql_b200.HostMatrix(m.fmt, m.rows, m.cols, m.data, m.scales, float(m.tensor_scale))


def layer(seed, n, h, fmt=oracle.FMT_Q4_K):
    return [oracle.quantize_matrix(fmt, seeded_weights(seed + i, n, h)) for i in range(3)]


@pytest.mark.parametrize("fmt", [oracle.FMT_Q4_K, oracle.FMT_Q8_0, oracle.FMT_MXFP4, oracle.FMT_NVFP4])
def test_dequantised_weights_bit_exact(be, fmt):
    rng = np.random.Generator(np.random.PCG64(3))
    w = seeded_weights(17 + fmt, 37, 512)
    w[3, :64] = 0.0          # an all-zero group / block
    w[5, :] *= 1e-4          # tiny scales (f16-subnormal d for Q4_K/Q8_0)
    w[7, 100] = 3.0          # an outlier
    m = oracle.quantize_matrix(fmt, w)
    got = be.dequantize(host(m))
    assert bits(got).tolist() == bits(m.dequantize()).tolist()
    # every code / scale byte pattern, not just what the encoder emits
    if fmt in (oracle.FMT_MXFP4, oracle.FMT_NVFP4):
        gsz = 32 if fmt == oracle.FMT_MXFP4 else 16
        rows, cols = 16, 256
        packed = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
        scales = np.arange(rows * cols // gsz, dtype=np.uint32).astype(np.uint8)
        m2 = oracle.Matrix(fmt, rows, cols, packed, scales, 0.37)
        a, b = bits(be.dequantize(host(m2))), bits(m2.dequantize())
        nan = np.isnan(m2.dequantize().reshape(-1))
        assert np.array_equal(a.reshape(-1)[~nan], b.reshape(-1)[~nan])
        assert np.all(np.isnan(be.dequantize(host(m2)).reshape(-1)[nan]))


@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (33, 1024), (70, 2560), (64, 3840), (48, 8192)])
def test_exact_matvec_is_bit_identical_to_cpu_backend(be, rows, cols):
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(rows * 7 + cols, rows, cols))
    x = oracle.rms_norm(seeded_x(cols + 1, cols))
    got = be.q4k_matvec(m.data, x, rows, cols, exact=True)
    assert bits(got).tolist() == bits(oracle.q4k_matvec(m.data, x, rows, cols)).tolist()


@pytest.mark.parametrize("rows,cols", [(1, 256), (7, 512), (3072, 1024), (1000, 2560), (777, 3840), (512, 8192)])
def test_fast_matvec_within_tolerance_and_deterministic(be, rows, cols):
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(rows + cols, rows, cols))
    x = seeded_x(cols + 2, cols)
    want = oracle.q4k_matvec(m.data, x, rows, cols)
    got = be.q4k_matvec(m.data, x, rows, cols)
    # error measured against the magnitude of the terms, sum |w||x| (a single dot can cancel)
    scale = np.abs(m.dequantize()).astype(np.float64) @ np.abs(x).astype(np.float64)
    assert np.max(np.abs(got.astype(np.float64) - want) / scale) < 2e-5
    if rows >= 100:
        assert rel_l2(got, want) < 1e-4
    assert np.array_equal(bits(got), bits(be.q4k_matvec(m.data, x, rows, cols)))


def test_matvec_refusals_and_empty(be):
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(1, 4, 256))
    x = seeded_x(2, 256)
    assert be.q4k_matvec(m.data[:-1], x, 4, 256) is None          # short weights
    assert be.q4k_matvec(m.data, x[:-1], 4, 256) is None          # x_len != hidden
    assert be.q4k_matvec(m.data, seeded_x(2, 200), 4, 200) is None  # hidden % 256
    assert be.q4k_matvec(m.data, x, 0, 256).size == 0              # zero rows: the empty product
    assert be.quant_matvec(99, m.data, x, 4, 256) is None


def test_matmul_matches_matvec_rows(be):
    rows, cols, seq = 300, 1024, 3
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(5, rows, cols))
    x = seeded_x(6, seq, cols)
    got = be.q4k_matmul(m.data, x, rows, cols, seq)
    want = oracle.q4k_matmul(m.data, x, rows, cols, seq)
    assert got.shape == (seq, rows) and rel_l2(got, want) < 1e-4


def test_top_k_by_abs_matches_reference_order(be):
    rng = np.random.Generator(np.random.PCG64(5))
    for n, k in [(4, 2), (3, 1), (2, 10), (3, 0), (1000, 17), (3072, 512), (28672, 4096), (50000, 100), (4097, 4096)]:
        s = rng.standard_normal(n, dtype=np.float32)
        gi, gv = be.top_k_by_abs(s, k)
        wi, wv = oracle.top_k_by_abs(s, k)
        assert gi.tolist() == wi.tolist() and bits(gv).tolist() == bits(wv).tolist(), (n, k)
    # ties, including across the K boundary, zeros and signed zeros: lower index wins
    s = np.array([1.0, -2.0, 2.0, 0.5, 2.0, -1.0, 1.0, 0.0, -0.0, 2.0], np.float32)
    for k in range(0, 12):
        assert be.top_k_by_abs(s, k)[0].tolist() == oracle.top_k_by_abs(s, k)[0].tolist()
    z = np.zeros(777, np.float32)
    assert be.top_k_by_abs(z, 40)[0].tolist() == list(range(40))
    many = np.repeat(np.array([3.0, -3.0, 1.0], np.float32), 500)
    assert be.top_k_by_abs(many, 700)[0].tolist() == oracle.top_k_by_abs(many, 700)[0].tolist()
    import larql_b200
    with pytest.raises(larql_b200.BackendError):
        be.top_k_by_abs(np.array([1.0, np.nan, 2.0], np.float32), 2)


def test_rms_norm(be):
    x = seeded_x(8, 3, 1024)
    got = be.rms_norm(x)
    want = oracle.rms_norm(x)
    # the f64 tree sum can differ from the sequential one in the last f64 bit only
    assert np.max(np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))) <= 1
    assert np.mean(bits(got) == bits(want)) > 0.999


def _check_walk(be, gate, up, down, x, k, flags=0):
    import larql_b200
    res = be.walk_ffn(host(gate), host(up), host(down), x, k, flags | larql_b200.WALK_FORCE_SPARSE)
    assert res is not None, be.last_refusal
    out, hits = res
    x2 = x.reshape(-1, gate.cols)
    out2 = out.reshape(-1, gate.cols)
    for t in range(x2.shape[0]):
        want, idx, _ = oracle.walk_token(gate, up, down, x2[t], k)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist()), f"token {t}: top-K index set differs"
        assert rel_l2(out2[t], want) < OUT_TOL, f"token {t}"
    return out, hits


@pytest.mark.parametrize("h,n,k", [(256, 64, 8), (512, 300, 37), (1024, 3072, 512), (2560, 1024, 100),
                                   (3840, 2048, 256), (8192, 1024, 128)])
def test_walk_index_sets_exact_and_outputs_within_tolerance(be, h, n, k):
    gate, up, down = layer(h + n, n, h)
    for q in range(3):
        x = oracle.rms_norm(seeded_x(0x5EED0000 + q, h))
        _check_walk(be, gate, up, down, x, k)
    st = be.last_walk_stats()
    assert st.n_hits == min(k, n) and st.n_certain + st.need == k and st.n_band >= st.need


def test_walk_config1_qwen_shape_many_queries(be):
    # hidden 1024, intermediate 3072, K=512, seeded N(0,0.02) Q4_K, RMS-normed N(0,1) residuals
    gate, up, down = layer(0x1A2B0000, 3072, 1024)
    xs = oracle.rms_norm(seeded_x(0x5EED0000, 24, 1024))
    out, hits = _check_walk(be, gate, up, down, xs, 512)
    out2, hits2 = be.walk_ffn(host(gate), host(up), host(down), xs, 512, 4)
    assert np.array_equal(bits(out), bits(out2))  # run-to-run identical
    assert all(sorted(a.tolist()) == sorted(b.tolist()) for a, b in zip(hits, hits2))


def test_walk_edge_cases(be):
    import larql_b200
    gate, up, down = layer(77, 96, 256)
    x = oracle.rms_norm(seeded_x(78, 256))
    # K >= N forced sparse: every feature
    out, hits = be.walk_ffn(host(gate), host(up), host(down), x, 1000, larql_b200.WALK_FORCE_SPARSE)
    assert sorted(hits[0].tolist()) == list(range(96))
    assert rel_l2(out, oracle.walk_token(gate, up, down, x, 1000)[0]) < OUT_TOL
    # K >= 80% of N without the force flag: the dense rewrite (all features)
    out_d, hits_d = be.walk_ffn(host(gate), host(up), host(down), x, 80, 0)
    assert len(hits_d[0]) == 96 and rel_l2(out_d, oracle.walk_token_dense(gate, up, down, x)) < OUT_TOL
    # K = 0: empty selection, zero output
    out0, hits0 = be.walk_ffn(host(gate), host(up), host(down), x, 0, larql_b200.WALK_FORCE_SPARSE)
    assert len(hits0[0]) == 0 and not out0.any()
    # all-zero activation: every score ties at 0 -> the K lowest indices
    outz, hitsz = be.walk_ffn(host(gate), host(up), host(down), np.zeros(256, np.float32), 10,
                              larql_b200.WALK_FORCE_SPARSE)
    assert sorted(hitsz[0].tolist()) == list(range(10)) and not outz.any()
    # duplicated gate rows: exact ties across the boundary resolve to the lower index
    g2 = oracle.Matrix(gate.fmt, 96, 256, np.tile(gate.data[:144], 96))
    _, hits_t = be.walk_ffn(host(g2), host(up), host(down), x, 7, larql_b200.WALK_FORCE_SPARSE)
    assert sorted(hits_t[0].tolist()) == list(range(7))
    # NaN activation: the reference panics in top_k_by_abs
    xn = x.copy()
    xn[5] = np.nan
    with pytest.raises(larql_b200.BackendError):
        be.walk_ffn(host(gate), host(up), host(down), xn, 8, larql_b200.WALK_FORCE_SPARSE)
    # shape refusals
    bad = oracle.Matrix(gate.fmt, 96, 256, gate.data[:-1])
    assert be.walk_ffn(host(bad), host(up), host(down), x, 8) is None
    up2 = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(1, 95, 256))
    assert be.walk_ffn(host(gate), host(up2), host(down), x, 8) is None


def test_run_ffn_norm_and_residual(be):
    import larql_b200
    gate, up, down = layer(91, 512, 1024)
    hin = seeded_x(92, 2, 1024)
    flags = larql_b200.WALK_RMSNORM | larql_b200.WALK_RESIDUAL | larql_b200.WALK_FORCE_SPARSE
    out, hits = be.walk_ffn(host(gate), host(up), host(down), hin, 64, flags)
    for t in range(2):
        want, idx = oracle.run_ffn_token(gate, up, down, hin[t], 64)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist())
        assert rel_l2(out[t] - hin[t], want - hin[t]) < OUT_TOL


def test_weight_residency_cache(be):
    gate, up, down = layer(55, 128, 512)
    be.drop_weight_regions()
    blob = np.concatenate([gate.data, up.data, down.data])
    be.register_weight_region(blob)
    assert be.device_ptr(blob) is not None
    n = gate.data.size
    x = oracle.rms_norm(seeded_x(56, 512))
    got = be.q4k_matvec(blob[n:2 * n], x, 128, 512, exact=True)   # a slice inside the registered region
    assert bits(got).tolist() == bits(oracle.q4k_matvec(up.data, x, 128, 512)).tolist()
    be.drop_weight_regions()
    assert be.device_ptr(blob) is None


def test_full_size_llama70b_layer_properties(be):
    """One layer at the headline shape (hidden 8192, 28672 features, K=4096): index set
    and output against the oracle, plus size-independent properties."""
    import larql_b200
    h, n, k = 8192, 28672, 4096
    gate, up, down = layer(0x1A2B5000, n, h)
    x = oracle.rms_norm(seeded_x(0x5EED5000, h))
    out, hits = _check_walk(be, gate, up, down, x, k)
    st = be.last_walk_stats()
    assert st.n_hits == k and 0 < st.n_band < n // 8, (st.n_certain, st.n_band)
    # linearity in the down matrix: a walk whose hits are known is additive over a split of the hit set
    idx = np.sort(hits[0])
    assert len(np.unique(idx)) == k
    # idempotence / determinism
    out2, hits2 = be.walk_ffn(host(gate), host(up), host(down), x, k, larql_b200.WALK_FORCE_SPARSE)
    assert np.array_equal(bits(out), bits(out2)) and sorted(hits2[0].tolist()) == sorted(hits[0].tolist())
    # scaling the activation by 2 keeps the index set (scores scale exactly by a power of two)
    _, hits3 = be.walk_ffn(host(gate), host(up), host(down), 2.0 * x, k, larql_b200.WALK_FORCE_SPARSE)
    assert sorted(hits3[0].tolist()) == sorted(hits[0].tolist())


@pytest.mark.parametrize("h,n,k,batch", [(512, 300, 37, 70), (1024, 3072, 512, 33), (2560, 1024, 100, 16),
                                         (8192, 1024, 128, 5), (256, 64, 8, 2)])
def test_batched_walk_tensor_core_scan(be, h, n, k, batch):
    # batches take one integer-MMA scan for all tokens and one launch of each selection / gather
    # kernel; every token must still select the reference's exact top-K set
    gate, up, down = layer(3 * h + n + batch, n, h)
    xs = oracle.rms_norm(seeded_x(0xBA7C4 + batch, batch, h))
    out, hits = _check_walk(be, gate, up, down, xs, k)
    out2, hits2 = be.walk_ffn(host(gate), host(up), host(down), xs, k, 4)
    assert np.array_equal(bits(out), bits(out2))  # run-to-run identical
    # norm + residual through the batched path
    import larql_b200
    hin = seeded_x(0xBA7C5 + batch, min(batch, 4), h)
    flags = larql_b200.WALK_RMSNORM | larql_b200.WALK_RESIDUAL | larql_b200.WALK_FORCE_SPARSE
    o3, h3 = be.walk_ffn(host(gate), host(up), host(down), hin, k, flags)
    for t in range(hin.shape[0]):
        want, idx = oracle.run_ffn_token(gate, up, down, hin[t], k)
        assert sorted(h3[t].tolist()) == sorted(idx.tolist())
        assert rel_l2(o3[t] - hin[t], want - hin[t]) < OUT_TOL


@pytest.mark.parametrize("rows,cols,seq", [(300, 1024, 8), (3072, 1024, 32), (1000, 2560, 70)])
def test_matmul_on_tensor_cores_matches_reference(be, rows, cols, seq):
    # seq >= 2 runs the integer-MMA scan; the reference is q4k_matmul_into (decode, then 8 strided accumulators)
    m = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(rows + seq, rows, cols))
    x = seeded_x(cols + seq, seq, cols)
    got = be.q4k_matmul(m.data, x, rows, cols, seq)
    want = oracle.q4k_matmul(m.data, x, rows, cols, seq)
    assert got.shape == (seq, rows) and rel_l2(got, want) < 1e-4
    scale = np.abs(x).astype(np.float64) @ np.abs(m.dequantize()).astype(np.float64).T
    assert np.max(np.abs(got.astype(np.float64) - want) / scale) < 2e-4
    assert np.array_equal(bits(got), bits(be.q4k_matmul(m.data, x, rows, cols, seq)))


def test_stack_run_host_matches_layer_by_layer_oracle(be):
    import larql_b200
    h, n, k, L = 1024, 3072, 512, 3
    ls = [layer(0x57AC + 10 * l, n, h) for l in range(L)]
    st = be.stack_create([host(m[0]) for m in ls], [host(m[1]) for m in ls], [host(m[2]) for m in ls], 1, k,
                         larql_b200.WALK_FORCE_SPARSE)
    hin = seeded_x(0x57AD, 1, h)
    out = np.empty_like(hin)
    assert be.stack_run_host(st, hin.ctypes.data, out.ctypes.data)
    want = hin[0].copy()
    for l in range(L):
        want, _ = oracle.run_ffn_token(*ls[l], want, k)
    assert rel_l2(out[0] - hin[0], want - hin[0]) < OUT_TOL
    be.stack_destroy(st)


@pytest.mark.parametrize("n,k", [(4096, 100), (10000, 37)])
def test_massive_ties_resolve_to_lowest_rows(be, n, k):
    # every gate row identical: all |scores| tie, the band is the whole layer (beyond what the final pick
    # can rank by counting, and for n = 10000 beyond what it can stage in shared memory)
    import larql_b200
    h = 256
    base = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(0x71E5, 1, h))
    gate = oracle.Matrix(oracle.FMT_Q4_K, n, h, np.tile(base.data[:144], n))
    up = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(0x71E6, n, h))
    down = oracle.quantize_matrix(oracle.FMT_Q4_K, seeded_weights(0x71E7, n, h))
    x = oracle.rms_norm(seeded_x(0x71E8, h))
    out, hits = be.walk_ffn(host(gate), host(up), host(down), x, k, larql_b200.WALK_FORCE_SPARSE)
    assert sorted(hits[0].tolist()) == list(range(k))
    want, idx, _ = oracle.walk_token(gate, up, down, x, k)
    assert sorted(idx.tolist()) == list(range(k)) and rel_l2(out, want) < OUT_TOL
