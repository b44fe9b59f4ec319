"""GPU parity tests for Q6_K rows, the walk with gate / up / down each Q4_K or Q6_K (real Q4_K vindexes keep
down as Q6_K), and the fused gate+up Q4_K matvec, through the C ABI against the CPU oracle.

Bar: decode, q6k_matvec and q4k_dual_matvec bit-identical to the CPU backend's arithmetic; selected feature
sets exact; walk outputs within 1e-3 relative L2 (f32)."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from conftest import bits, rel_l2, seeded_weights, seeded_x

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3
GOLDEN = Path(__file__).resolve().parent / "golden"
Q4, Q6 = oracle.FMT_Q4_K, oracle.FMT_Q6_K


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


def test_q6k_decode_of_the_ggml_golden_block(be):
    g = json.loads((GOLDEN / "ggml_kquant_golden.json").read_text())
    case = next(c for c in g["cases"] if c["encoding"] == "q6_K")
    raw = np.frombuffer(bytes.fromhex(case["quantised_hex"]), np.uint8)
    got = be.dequantize_q6k(raw, case["elements"])
    assert bits(got).tolist() == case["dequantised_bits"]
    assert be.dequantize_q6k(raw[:-1], case["elements"]) is None      # short buffer: refused
    assert be.dequantize_q6k(raw, 100) is None                        # not a multiple of 256


@pytest.mark.parametrize("rows,cols", [(1, 256), (37, 512), (300, 2816), (1024, 1024), (96, 8192)])
def test_q6k_matvec_is_bit_identical_to_the_cpu_backend(be, rows, cols):
    m = oracle.quantize_matrix(Q6, seeded_weights(rows * 5 + cols, rows, cols))
    x = seeded_x(cols + rows, cols)
    got = be.q6k_matvec(m.data, x, rows, cols)
    assert bits(got).tolist() == bits(oracle.q6k_matvec(m.data, x, rows, cols)).tolist()
    assert bits(be.gemv(host(m), x, exact=True)).tolist() == bits(got).tolist()
    deq = be.dequantize_q6k(m.data, rows * cols)
    assert bits(deq).tolist() == bits(oracle.dequantize_q6_k(m.data, rows * cols)).tolist()
    assert be.q6k_matvec(m.data, x[:-1], rows, cols) is None          # x_len != hidden


@pytest.mark.parametrize("rows,cols", [(1, 256), (40, 768), (515, 2560), (64, 8192)])
def test_q4k_dual_matvec_is_bit_identical_to_the_cpu_backend(be, rows, cols):
    wa = oracle.quantize_matrix(Q4, seeded_weights(rows + cols, rows, cols))
    wb = oracle.quantize_matrix(Q4, seeded_weights(rows + cols + 1, rows, cols))
    x = seeded_x(cols, cols)
    ga, gb = be.q4k_dual_matvec(wa.data, wb.data, x, rows, cols)
    wa_, wb_ = oracle.q4k_dual_matvec(wa.data, wb.data, x, rows, cols)
    assert bits(ga).tolist() == bits(wa_).tolist() and bits(gb).tolist() == bits(wb_).tolist()
    assert be.q4k_dual_matvec(wa.data, wb.data[:-1], x, rows, cols) is None


MIXES = [(Q4, Q4, Q6), (Q6, Q6, Q6), (Q6, Q4, Q4), (Q4, Q6, Q4)]


@pytest.mark.parametrize("mix", MIXES, ids=lambda m: "-".join(oracle.FMT_NAMES[f] for f in m))
@pytest.mark.parametrize("n,h,k", [(3072, 1024, 512), (700, 2560, 64), (2048, 4096, 2048)])
def test_walk_with_mixed_kquant_matrices(be, mix, n, h, k):
    import larql_b200
    ws = [seeded_weights(0x6A00 + 16 * i + n, n, h) for i in range(3)]
    gate, up, down = (oracle.quantize_matrix(f, w) for f, w in zip(mix, ws))
    for q in range(2):
        x = oracle.rms_norm(seeded_x(0x6B00 + q + h, h))
        want, idx, _ = oracle.walk_token(gate, up, down, x, k)
        res = be.walk_ffn(host(gate), host(up), host(down), x, k, larql_b200.WALK_FORCE_SPARSE)
        assert res is not None, be.last_refusal
        out, hits = res
        assert sorted(hits[0].tolist()) == sorted(idx.tolist())
        assert rel_l2(out.reshape(-1), want) < OUT_TOL


def test_walk_q6k_down_batch_and_dense(be):
    """A batch (token by token on this path) and K = all features."""
    import larql_b200
    n, h = 1024, 2048
    gate = oracle.quantize_matrix(Q4, seeded_weights(0x6C01, n, h))
    up = oracle.quantize_matrix(Q4, seeded_weights(0x6C02, n, h))
    down = oracle.quantize_matrix(Q6, seeded_weights(0x6C03, n, h))
    xs = oracle.rms_norm(seeded_x(0x6C04, 5, h))
    out, hits = be.walk_ffn(host(gate), host(up), host(down), xs, 100, larql_b200.WALK_FORCE_SPARSE)
    for t in range(5):
        want, idx, _ = oracle.walk_token(gate, up, down, xs[t], 100)
        assert sorted(hits[t].tolist()) == sorted(idx.tolist()) and rel_l2(out[t], want) < OUT_TOL
    dense = be.walk_ffn(host(gate), host(up), host(down), xs[0], n)[0]
    assert rel_l2(dense.reshape(-1), oracle.walk_token_dense(gate, up, down, xs[0])) < OUT_TOL


def test_walk_over_weights_read_from_a_vindex_directory(be, tmp_path):
    """Files laid out as the reference's writer does (gate / up Q4_K, feature-major down Q6_K, hidden 2880 padded
    to 3072), mapped by the reader and walked as they are: the activation is zero-padded to the padded width."""
    import larql_b200
    from test_vindex_files import write_vindex
    hidden, feats, k = 2880, 512, 64
    write_vindex(tmp_path, 2, hidden, feats)
    v = larql_b200.VindexFiles(tmp_path)
    for l in range(2):
        gate, up, _, down_fm = v.layer(l)
        og, ou, od = (oracle.Matrix(m.fmt, m.rows, m.cols, m.data) for m in (gate, up, down_fm))
        x = np.zeros(gate.cols, np.float32)
        x[:hidden] = oracle.rms_norm(seeded_x(0x7100 + l, hidden))
        want, idx, _ = oracle.walk_token(og, ou, od, x, k)
        out, hits = be.walk_ffn(gate, up, down_fm, x, k, larql_b200.WALK_FORCE_SPARSE)
        assert sorted(hits[0].tolist()) == sorted(idx.tolist())
        assert rel_l2(out.reshape(-1), want) < OUT_TOL
        assert np.all(out.reshape(-1)[hidden:] == 0.0)      # the padded tail of every down row decodes to zero
    v.close()
