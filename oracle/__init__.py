"""CPU oracle for the vindex FFN walk — TEST INFRASTRUCTURE, not product code.

A ctypes wrapper over ``larql_oracle.c`` (a C restatement of the reference's
CPU arithmetic, each function citing the reference file:line it follows).
Only the test-suite, the smoke check and the benchmark's CPU-baseline arm may
import this package; the CUDA library never does.

``build()`` compiles the C file with contraction disabled (``-ffp-contract=off``)
because the reference never fuses a multiply with an add.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "larql_oracle.c"
_SO = _HERE / "_build" / "liblarql_oracle.so"

FMT_Q4_K, FMT_Q8_0, FMT_MXFP4, FMT_NVFP4, FMT_Q6_K = 0, 1, 2, 3, 4
FMT_NAMES = {FMT_Q4_K: "q4_k", FMT_Q8_0: "q8_0", FMT_MXFP4: "mxfp4", FMT_NVFP4: "nvfp4", FMT_Q6_K: "q6_k"}


def build(force: bool = False) -> Path:
    """Compile the oracle shared library (gcc; seconds)."""
    if not force and _SO.exists() and _SO.stat().st_mtime >= _SRC.stat().st_mtime:
        return _SO
    _SO.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-pthread",
           "-fvisibility=hidden", "-o", str(_SO), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return _SO


class _Matrix(C.Structure):
    _fields_ = [("fmt", C.c_int32), ("data", C.c_void_p), ("scales", C.c_void_p),
                ("tensor_scale", C.c_float), ("rows", C.c_size_t), ("cols", C.c_size_t)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        f = _lib
        f.orc_f16_to_f32.restype = C.c_float
        f.orc_f16_to_f32.argtypes = [C.c_uint16]
        f.orc_f32_to_f16_trunc.restype = C.c_uint16
        f.orc_f32_to_f16_trunc.argtypes = [C.c_float]
        f.orc_f32_to_f16_nearest.restype = C.c_uint16
        f.orc_f32_to_f16_nearest.argtypes = [C.c_float]
        f.orc_e4m3_to_f32.restype = C.c_float
        f.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        f.orc_f32_to_e4m3.restype = C.c_uint8
        f.orc_f32_to_e4m3.argtypes = [C.c_float]
        f.orc_e2m1_to_f32.restype = C.c_float
        f.orc_e2m1_to_f32.argtypes = [C.c_uint8]
        f.orc_f32_to_e2m1.restype = C.c_uint8
        f.orc_f32_to_e2m1.argtypes = [C.c_float]
        f.orc_e8m0_to_f32.restype = C.c_float
        f.orc_e8m0_to_f32.argtypes = [C.c_uint8]
        f.orc_nearest_mxfp4_code.restype = C.c_uint8
        f.orc_nearest_mxfp4_code.argtypes = [C.c_float]
        f.orc_q4k_row_dot.restype = C.c_float
        f.orc_q6k_row_dot.restype = C.c_float
        f.orc_nvfp4_tensor_scale_for.restype = C.c_float
        f.orc_sigmoid.restype = C.c_float
        f.orc_sigmoid.argtypes = [C.c_float]
        f.orc_silu.restype = C.c_float
        f.orc_silu.argtypes = [C.c_float]
        for name in ("orc_top_k_by_abs", "orc_top_k_by_abs_heap", "orc_walk_token", "orc_run_ffn_token",
                     "orc_walk_token_mt"):
            getattr(f, name).restype = C.c_int64
        f.orc_moe_top_k.restype = C.c_size_t
        f.orc_moe_route.restype = C.c_size_t
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _sz(v):
    return C.c_size_t(int(v))


# ---------------------------------------------------------------- scalars
def f16_to_f32(bits: int) -> float:
    return lib().orc_f16_to_f32(bits)


def f32_to_f16_trunc(v: float) -> int:
    return lib().orc_f32_to_f16_trunc(C.c_float(v))


def f32_to_f16_nearest(v: float) -> int:
    return lib().orc_f32_to_f16_nearest(C.c_float(v))


def e4m3_to_f32(b: int) -> float:
    return lib().orc_e4m3_to_f32(b)


def f32_to_e4m3(v: float) -> int:
    return lib().orc_f32_to_e4m3(C.c_float(v))


def e2m1_to_f32(c: int) -> float:
    return lib().orc_e2m1_to_f32(c)


def f32_to_e2m1(v: float) -> int:
    return lib().orc_f32_to_e2m1(C.c_float(v))


def e8m0_to_f32(b: int) -> float:
    return lib().orc_e8m0_to_f32(b)


def nearest_mxfp4_code(v: float) -> int:
    return lib().orc_nearest_mxfp4_code(C.c_float(v))


def sigmoid(v: float) -> float:
    return lib().orc_sigmoid(C.c_float(v))


# ------------------------------------------------------------- quantisers
def quantize_q4_k(data) -> np.ndarray:
    d = _f32(data).reshape(-1)
    assert d.size % 256 == 0, "data length must be a multiple of 256"
    out = np.empty(d.size // 256 * 144, np.uint8)
    lib().orc_quantize_q4_k(_p(d), _sz(d.size), _p(out))
    return out


def dequantize_q4_k(data, n: int) -> np.ndarray:
    b = _u8(data)
    assert n % 256 == 0 and b.size >= n // 256 * 144
    out = np.empty(n, np.float32)
    lib().orc_dequantize_q4_k(_p(b), _sz(n), _p(out))
    return out


def quantize_q6_k(data) -> np.ndarray:
    d = _f32(data).reshape(-1)
    assert d.size % 256 == 0, "data length must be a multiple of 256"
    out = np.empty(d.size // 256 * 210, np.uint8)
    lib().orc_quantize_q6_k(_p(d), _sz(d.size), _p(out))
    return out


def dequantize_q6_k(data, n: int) -> np.ndarray:
    b = _u8(data)
    assert n % 256 == 0 and b.size >= n // 256 * 210
    out = np.empty(n, np.float32)
    lib().orc_dequantize_q6_k(_p(b), _sz(n), _p(out))
    return out


def quantize_q8_0(data) -> np.ndarray:
    d = _f32(data).reshape(-1)
    assert d.size % 32 == 0
    out = np.empty(d.size // 32 * 34, np.uint8)
    lib().orc_quantize_q8_0(_p(d), _sz(d.size), _p(out))
    return out


def dequantize_q8_0(data, n: int) -> np.ndarray:
    b = _u8(data)
    assert n % 32 == 0 and b.size >= n // 32 * 34
    out = np.empty(n, np.float32)
    lib().orc_dequantize_q8_0(_p(b), _sz(n), _p(out))
    return out


def nvfp4_tensor_scale_for(values) -> float:
    v = _f32(values).reshape(-1)
    return float(lib().orc_nvfp4_tensor_scale_for(_p(v), _sz(v.size)))


def quantize_nvfp4(values, rows: int, k: int, tensor_scale: float | None = None):
    """Returns (packed[rows*k/2], scales[rows*k/16], tensor_scale) or None on bad geometry."""
    v = _f32(values).reshape(-1)
    if k % 16 != 0 or v.size != rows * k:
        return None
    ts = nvfp4_tensor_scale_for(v) if tensor_scale is None else float(tensor_scale)
    packed = np.empty(rows * k // 2, np.uint8)
    scales = np.empty(rows * k // 16, np.uint8)
    rc = lib().orc_quantize_nvfp4(_p(v), _sz(rows), _sz(k), C.c_float(ts), _p(packed), _p(scales))
    assert rc == 0
    return packed, scales, np.float32(ts)


def dequantize_nvfp4(packed, scales, tensor_scale, rows: int, k: int) -> np.ndarray:
    out = np.empty(rows * k, np.float32)
    rc = lib().orc_dequantize_nvfp4(_p(_u8(packed)), _p(_u8(scales)), C.c_float(tensor_scale), _sz(rows), _sz(k),
                                    _p(out))
    assert rc == 0
    return out


def quantize_mxfp4(values, rows: int, k: int):
    v = _f32(values).reshape(-1)
    if k % 32 != 0 or v.size != rows * k:
        return None
    packed = np.empty(rows * k // 2, np.uint8)
    scales = np.empty(rows * k // 32, np.uint8)
    rc = lib().orc_quantize_mxfp4(_p(v), _sz(rows), _sz(k), _p(packed), _p(scales))
    assert rc == 0
    return packed, scales


def dequantize_mxfp4(packed, scales, rows: int, groups: int) -> np.ndarray:
    out = np.empty(rows * groups * 32, np.float32)
    lib().orc_dequantize_mxfp4(_p(_u8(packed)), _p(_u8(scales)), _sz(rows), _sz(groups), _p(out))
    return out


# ------------------------------------------------------------------ dots
def q4k_matvec(w, x, rows: int, cols: int):
    """Association A (backend q4k_matvec). None on a shape refusal."""
    w = _u8(w)
    x = _f32(x)
    out = np.empty(rows, np.float32)
    rc = lib().orc_q4k_matvec(_p(w), _sz(w.size), _p(x), _sz(x.size), _sz(rows), _sz(cols), _p(out), _sz(rows))
    return None if rc else out


def q6k_matvec(w, x, rows: int, cols: int):
    """Backend q6k_matvec (per sub-block sum, then acc += sc * sub). None on a shape refusal."""
    w = _u8(w)
    x = _f32(x)
    out = np.empty(rows, np.float32)
    rc = lib().orc_q6k_matvec(_p(w), _sz(w.size), _p(x), _sz(x.size), _sz(rows), _sz(cols), _p(out))
    return None if rc else out


def q6k_row_dot(row, x) -> np.float32:
    row = _u8(row)
    x = _f32(x)
    return np.float32(lib().orc_q6k_row_dot(_p(row), _p(x), _sz(x.size)))


def q6k_row_scaled_add(row, alpha: float, out: np.ndarray) -> None:
    row = _u8(row)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    lib().orc_q6k_row_scaled_add(_p(row), C.c_float(alpha), _p(out), _sz(out.size))


def q4k_dual_matvec(w_a, w_b, x, rows: int, cols: int):
    """Gate and up against one activation (q4k_dual_matvec_into): one running sum per row. None on a refusal."""
    w_a, w_b, x = _u8(w_a), _u8(w_b), _f32(x)
    out_a, out_b = np.empty(rows, np.float32), np.empty(rows, np.float32)
    rc = lib().orc_q4k_dual_matvec(_p(w_a), _sz(w_a.size), _p(w_b), _sz(w_b.size), _p(x), _sz(x.size), _sz(rows),
                                   _sz(cols), _p(out_a), _p(out_b))
    return None if rc else (out_a, out_b)


def q4k_row_dot(row, x) -> np.float32:
    row = _u8(row)
    x = _f32(x)
    return np.float32(lib().orc_q4k_row_dot(_p(row), _p(x), _sz(x.size)))


def q4k_row_scaled_add(row, alpha: float, out: np.ndarray) -> None:
    row = _u8(row)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    lib().orc_q4k_row_scaled_add(_p(row), C.c_float(alpha), _p(out), _sz(out.size))


def q4k_matmul(w, x, rows: int, hidden: int, seq: int) -> np.ndarray:
    w = _u8(w)
    x = _f32(x)
    out = np.empty(seq * rows, np.float32)
    lib().orc_q4k_matmul(_p(w), _sz(w.size), _p(x), _sz(rows), _sz(hidden), _sz(seq), _p(out))
    return out.reshape(seq, rows)


def q8_0_gemv(blocks, x, n: int, k: int):
    b = _u8(blocks)
    x = _f32(x)
    out = np.empty(n, np.float32)
    rc = lib().orc_q8_0_gemv(_p(b), _sz(b.size), _p(x), _sz(x.size), _sz(n), _sz(k), _p(out))
    return None if rc else out


def nvfp4_gemv(packed, scales, tensor_scale, x, n: int, k: int):
    p, s, x = _u8(packed), _u8(scales), _f32(x)
    out = np.empty(n, np.float32)
    rc = lib().orc_nvfp4_gemv(_p(p), _sz(p.size), _p(s), _sz(s.size), C.c_float(tensor_scale), _p(x), _sz(x.size),
                              _sz(n), _sz(k), _p(out))
    return None if rc else out


def mxfp4_gemv(packed, scales, x, n: int, k: int):
    p, s, x = _u8(packed), _u8(scales), _f32(x)
    out = np.empty(n, np.float32)
    rc = lib().orc_mxfp4_gemv(_p(p), _sz(p.size), _p(s), _sz(s.size), _p(x), _sz(x.size), _sz(n), _sz(k), _p(out))
    return None if rc else out


def gemv16(w_bits, x, n: int, k: int, kind: int):
    """f16 (kind 0) / bf16 (kind 1) gemv in the reference test device's order; None on a shape mismatch."""
    w = np.ascontiguousarray(w_bits).view(np.uint8).reshape(-1)
    x = _f32(x)
    out = np.empty(n, np.float32)
    rc = lib().orc_gemv16(_p(w), _sz(w.size), _p(x), _sz(x.size), _sz(n), _sz(k), C.c_int(kind), _p(out))
    return None if rc else out


def top_k_by_value(scores, top_k: int):
    """(idx, val) of the top_k largest values, descending, ties to the lower index. Raises on NaN."""
    s = _f32(scores).reshape(-1)
    k = min(int(top_k), s.size)
    idx = np.empty(max(k, 1), np.uint32)
    val = np.empty(max(k, 1), np.float32)
    lib().orc_top_k_by_value.restype = C.c_long
    got = lib().orc_top_k_by_value(_p(s), _sz(s.size), _sz(top_k), _p(idx), _p(val))
    if got < 0:
        raise ValueError("NaN score")
    return idx[:got].copy(), val[:got].copy()


# ---------------------------------------------------------------- top-K
def top_k_by_abs(scores, top_k: int, heap: bool = False):
    """Returns (idx uint32[k'], val float32[k']) sorted (|v| desc, idx asc). Raises on NaN."""
    s = _f32(scores).reshape(-1)
    k = min(int(top_k), s.size)
    idx = np.empty(max(k, 1), np.uint32)
    val = np.empty(max(k, 1), np.float32)
    fn = lib().orc_top_k_by_abs_heap if heap else lib().orc_top_k_by_abs
    got = fn(_p(s), _sz(s.size), _sz(top_k), _p(idx), _p(val))
    if got < 0:
        raise ValueError("NaN score in top_k_by_abs (the reference panics)")
    return idx[:got].copy(), val[:got].copy()


def rms_norm(x, eps: float = 1e-6) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    lib().orc_rms_norm(_p(x2), _sz(x2.shape[0]), _sz(x2.shape[1]), C.c_double(eps), _p(out))
    return out.reshape(x.shape)


def softmax(v) -> np.ndarray:
    a = _f32(v).copy()
    lib().orc_softmax(_p(a), _sz(a.size))
    return a


def moe_top_k(v, k: int):
    a = _f32(v)
    kk = min(k, a.size)
    idx = np.empty(max(kk, 1), np.uint32)
    val = np.empty(max(kk, 1), np.float32)
    got = lib().orc_moe_top_k(_p(a), _sz(a.size), _sz(k), _p(idx), _p(val))
    return idx[:got].copy(), val[:got].copy()


def moe_route(logits, top_k: int, renormalise: bool = True):
    a = _f32(logits)
    kk = min(top_k, a.size)
    idx = np.empty(max(kk, 1), np.uint32)
    w = np.empty(max(kk, 1), np.float32)
    got = lib().orc_moe_route(_p(a), _sz(a.size), _sz(top_k), C.c_int(1 if renormalise else 0), _p(idx), _p(w))
    return idx[:got].copy(), w[:got].copy()


# ----------------------------------------------------------------- walk
class Matrix:
    """A quantised [rows, cols] matrix in one of the block formats (host memory)."""

    def __init__(self, fmt: int, rows: int, cols: int, data, scales=None, tensor_scale: float = 1.0):
        self.fmt, self.rows, self.cols = fmt, rows, cols
        self.data = _u8(data)
        self.scales = _u8(scales) if scales is not None else None
        self.tensor_scale = np.float32(tensor_scale)

    def c(self) -> _Matrix:
        return _Matrix(self.fmt, self.data.ctypes.data, self.scales.ctypes.data if self.scales is not None else None,
                       float(self.tensor_scale), self.rows, self.cols)

    @property
    def nbytes(self) -> int:
        return self.data.nbytes + (self.scales.nbytes if self.scales is not None else 0)

    def row_bytes(self) -> int:
        return {FMT_Q4_K: self.cols // 256 * 144, FMT_Q8_0: self.cols // 32 * 34, FMT_MXFP4: self.cols // 32 * 16,
                FMT_NVFP4: self.cols // 16 * 8, FMT_Q6_K: self.cols // 256 * 210}[self.fmt]

    def gemv(self, x):
        if self.fmt == FMT_Q4_K:
            return q4k_matvec(self.data, x, self.rows, self.cols)
        if self.fmt == FMT_Q8_0:
            return q8_0_gemv(self.data, x, self.rows, self.cols)
        if self.fmt == FMT_Q6_K:
            return q6k_matvec(self.data, x, self.rows, self.cols)
        if self.fmt == FMT_MXFP4:
            return mxfp4_gemv(self.data, self.scales, x, self.rows, self.cols)
        return nvfp4_gemv(self.data, self.scales, self.tensor_scale, x, self.rows, self.cols)

    def dequantize(self) -> np.ndarray:
        n = self.rows * self.cols
        if self.fmt == FMT_Q4_K:
            return dequantize_q4_k(self.data, n).reshape(self.rows, self.cols)
        if self.fmt == FMT_Q8_0:
            return dequantize_q8_0(self.data, n).reshape(self.rows, self.cols)
        if self.fmt == FMT_Q6_K:
            return dequantize_q6_k(self.data, n).reshape(self.rows, self.cols)
        if self.fmt == FMT_MXFP4:
            return dequantize_mxfp4(self.data, self.scales, self.rows, self.cols // 32).reshape(self.rows, self.cols)
        return dequantize_nvfp4(self.data, self.scales, self.tensor_scale, self.rows, self.cols).reshape(
            self.rows, self.cols)


def quantize_matrix(fmt: int, w) -> Matrix:
    """Quantise an f32 [rows, cols] matrix with the reference's encoder for ``fmt``."""
    w = _f32(w)
    rows, cols = w.shape
    if fmt == FMT_Q4_K:
        return Matrix(fmt, rows, cols, quantize_q4_k(w))
    if fmt == FMT_Q8_0:
        return Matrix(fmt, rows, cols, quantize_q8_0(w))
    if fmt == FMT_Q6_K:
        return Matrix(fmt, rows, cols, quantize_q6_k(w))
    if fmt == FMT_MXFP4:
        p, s = quantize_mxfp4(w, rows, cols)
        return Matrix(fmt, rows, cols, p, s)
    p, s, ts = quantize_nvfp4(w, rows, cols)
    return Matrix(fmt, rows, cols, p, s, ts)


def walk_token(gate: Matrix, up: Matrix, down_fm: Matrix, x, top_k: int):
    """One token of the sparse walk. Returns (out[H], idx[k'], gate_score[k']) with hits in |score| order."""
    x = _f32(x)
    h, n = gate.cols, gate.rows
    out = np.empty(h, np.float32)
    kk = max(min(top_k, n), 1)
    idx = np.empty(kk, np.uint32)
    val = np.empty(kk, np.float32)
    g, u, d = gate.c(), up.c(), down_fm.c()
    got = lib().orc_walk_token(C.byref(g), C.byref(u), C.byref(d), _p(x), _sz(top_k), _p(out), _p(idx), _p(val))
    if got < 0:
        raise ValueError("NaN gate score")
    return out, idx[:got].copy(), val[:got].copy()


def walk_token_dense(gate: Matrix, up: Matrix, down_fm: Matrix, x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(gate.cols, np.float32)
    g, u, d = gate.c(), up.c(), down_fm.c()
    lib().orc_walk_token_dense(C.byref(g), C.byref(u), C.byref(d), _p(x), _p(out))
    return out


def run_ffn_token(gate: Matrix, up: Matrix, down_fm: Matrix, h_in, top_k: int, eps: float = 1e-6):
    h_in = _f32(h_in)
    out = np.empty(gate.cols, np.float32)
    kk = max(min(top_k, gate.rows), 1)
    idx = np.empty(kk, np.uint32)
    g, u, d = gate.c(), up.c(), down_fm.c()
    got = lib().orc_run_ffn_token(C.byref(g), C.byref(u), C.byref(d), _p(h_in), _sz(top_k), C.c_double(eps), _p(out),
                                  _p(idx))
    if got < 0:
        raise ValueError("NaN gate score")
    return out, idx[:got].copy()


def gemv_mt(m: Matrix, x, threads: int) -> np.ndarray:
    x = _f32(x)
    out = np.empty(m.rows, np.float32)
    mc = m.c()
    lib().orc_gemv_mt(C.byref(mc), _p(x), _p(out), C.c_int(threads))
    return out


def walk_token_mt(gate: Matrix, up: Matrix, down_fm: Matrix, x, top_k: int, threads: int):
    x = _f32(x)
    out = np.empty(gate.cols, np.float32)
    kk = max(min(top_k, gate.rows), 1)
    idx = np.empty(kk, np.uint32)
    g, u, d = gate.c(), up.c(), down_fm.c()
    got = lib().orc_walk_token_mt(C.byref(g), C.byref(u), C.byref(d), _p(x), _sz(top_k), _p(out), _p(idx),
                                  C.c_int(threads))
    if got < 0:
        raise ValueError("NaN gate score")
    return out, idx[:got].copy()


def host_threads() -> int:
    return os.cpu_count() or 1
