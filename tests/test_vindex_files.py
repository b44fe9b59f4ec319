"""The on-disk K-quant FFN weights of a vindex directory, written here exactly as the reference's writer lays them
out (write_kquant/ffn.rs, feature_major_down.rs) and read back through the C ABI.  Host code only: no GPU."""
import json

import numpy as np
import pytest

import oracle
from conftest import seeded_weights

Q4, Q6 = oracle.FMT_Q4_K, oracle.FMT_Q6_K
TAG = {Q4: "Q4_K", Q6: "Q6_K"}


def pad_rows(w: np.ndarray) -> np.ndarray:
    """pad_rows_to_block: zero-pad every row to a whole number of 256-element super-blocks."""
    rows, cols = w.shape
    pc = (cols + 255) // 256 * 256
    out = np.zeros((rows, pc), np.float32)
    out[:, :cols] = w
    return out


def write_vindex(tmp, layers, hidden, feats, down_fmt=Q6, sidecar=True, names=("interleaved_kquant", "down_features_kquant")):
    """Returns the per-layer (gate, up, down, down_fm) quantised bytes it wrote."""
    ffn, ffn_man, fm, fm_man, written = bytearray(), [], bytearray(), [], []
    for l in range(layers):
        gate = pad_rows(seeded_weights(100 + 3 * l, feats, hidden))
        up = pad_rows(seeded_weights(101 + 3 * l, feats, hidden))
        down = pad_rows(seeded_weights(102 + 3 * l, hidden, feats))        # [hidden, padded intermediate]
        mats = []
        for key, w, fmt in ((f"layers.{l}.ffn_gate", gate, Q4), (f"layers.{l}.ffn_up", up, Q4),
                            (f"layers.{l}.ffn_down", down, down_fmt)):
            q = oracle.quantize_matrix(fmt, w).data
            ffn_man.append({"key": key, "shape": list(w.shape), "format": TAG[fmt], "offset": len(ffn), "length": int(q.size)})
            ffn += q.tobytes()
            mats.append(q)
        # feature-major down: transpose to [padded intermediate, hidden], re-pad rows, same precision
        dfm = pad_rows(np.ascontiguousarray(down.T))
        q = oracle.quantize_matrix(down_fmt, dfm).data
        fm_man.append({"key": f"layers.{l}.ffn_down", "shape": list(dfm.shape), "format": TAG[down_fmt],
                       "offset": len(fm), "length": int(q.size)})
        fm += q.tobytes()
        mats.append(q)
        written.append(mats)
    (tmp / f"{names[0]}.bin").write_bytes(bytes(ffn))
    (tmp / f"{names[0]}_manifest.json").write_text(json.dumps(ffn_man, indent=2))
    if sidecar:
        (tmp / f"{names[1]}.bin").write_bytes(bytes(fm))
        (tmp / f"{names[1]}_manifest.json").write_text(json.dumps(fm_man, indent=2))
    return written


def test_padded_cols_formula():
    import larql_b200
    for cols, want in ((0, 0), (1, 256), (256, 256), (257, 512), (2880, 3072), (1152, 1280), (8192, 8192)):
        assert larql_b200.k_quant_padded_cols(cols) == want


@pytest.mark.parametrize("down_fmt", [Q6, Q4])
def test_reads_back_what_the_writer_lays_out(tmp_path, down_fmt):
    import larql_b200
    hidden, feats, layers = 2880, 300, 3          # the GPT-OSS width: 2880 -> 3072, and 300 -> 512 features
    written = write_vindex(tmp_path, layers, hidden, feats, down_fmt)
    v = larql_b200.VindexFiles(tmp_path)
    assert v.num_layers == layers
    for l in range(layers):
        gate, up, down, down_fm = v.layer(l)
        assert (gate.fmt, gate.rows, gate.cols) == (Q4, feats, 3072) and (up.fmt, up.rows, up.cols) == (Q4, feats, 3072)
        assert (down.fmt, down.rows, down.cols) == (down_fmt, hidden, 512)
        assert (down_fm.fmt, down_fm.rows, down_fm.cols) == (down_fmt, 512, 3072)
        for got, want in zip((gate, up, down, down_fm), written[l]):
            assert got.data.tobytes() == want.tobytes()
    with pytest.raises(IndexError):
        v.layer(layers)
    # the padded tail of a row decodes to zeros, the logical part to the writer's values
    gate0 = v.layer(0)[0]
    deq = oracle.dequantize_q4_k(gate0.data, gate0.rows * gate0.cols).reshape(gate0.rows, gate0.cols)
    assert np.all(deq[:, hidden:] == 0.0)
    v.close()


def test_directory_without_the_feature_major_sidecar_and_with_legacy_names(tmp_path):
    import larql_b200
    write_vindex(tmp_path, 2, 512, 256, sidecar=False, names=("interleaved_q4k", "down_features_q4k"))
    v = larql_b200.VindexFiles(tmp_path)
    assert v.num_layers == 2 and v.layer(1)[3] is None
    v.close()


def test_refusals(tmp_path):
    import larql_b200
    with pytest.raises(larql_b200.BackendError, match="not found"):
        larql_b200.VindexFiles(tmp_path)
    write_vindex(tmp_path, 2, 512, 256)
    man = tmp_path / "interleaved_kquant_manifest.json"
    good = json.loads(man.read_text())
    for mutate, what in (
        (lambda m: m[1].update(format="Q5_K"), "unknown format"),
        (lambda m: m[2].update(length=m[2]["length"] - 1), "length does not match"),
        (lambda m: m[5].update(offset=m[5]["offset"] + 4096), "past the end"),
        (lambda m: m[0].update(shape=[256, 500]), "padded to 256"),
        (lambda m: m.pop(), "three entries"),
        (lambda m: m[0].update(dtype="x"), "unknown field"),
    ):
        m = json.loads(json.dumps(good))
        mutate(m)
        man.write_text(json.dumps(m))
        with pytest.raises(larql_b200.BackendError, match=what):
            larql_b200.VindexFiles(tmp_path)
    man.write_text(json.dumps(good))
    (tmp_path / "down_features_kquant_manifest.json").unlink()
    with pytest.raises(larql_b200.BackendError, match="manifest .* missing"):
        larql_b200.VindexFiles(tmp_path)


def test_nvfp4_pack_split_matches_the_stored_layout():
    import larql_b200
    rows, k = 24, 160
    m = oracle.quantize_matrix(oracle.FMT_NVFP4, seeded_weights(9, rows, k))
    payload = np.concatenate([m.data, m.scales, np.array([m.tensor_scale], np.float32).view(np.uint8)])
    hm = larql_b200.nvfp4_pack_split(payload, rows, k)
    assert hm.data.tobytes() == m.data.tobytes() and hm.scales.tobytes() == m.scales.tobytes()
    assert np.float32(hm.tensor_scale) == np.float32(m.tensor_scale)
    assert larql_b200.nvfp4_pack_split(payload[:-1], rows, k) is None          # wrong length
    assert larql_b200.nvfp4_pack_split(payload, rows, k + 8) is None           # k not a whole number of groups
