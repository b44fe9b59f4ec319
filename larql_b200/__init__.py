"""larql_b200 — B200 (sm_100a) backend for LARQL's vindex FFN walk.

The product is ``liblarql_b200.so`` (hand-written CUDA behind the C ABI in
``include/larql_cuda.h``).  This package is the thin host-side binding used by the
tests and the benchmark: :class:`CudaBackend` mirrors the method names, argument
meaning and refusal behaviour of the reference's ``ComputeBackend`` /
``QuantMatVec`` / ``MatMul`` traits for the walk path (``None`` = "cannot compute
this", never a wrong answer).

There is no CPU fallback: importing works anywhere, but constructing a backend
without the built library or without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

import numpy as np

_HERE = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("LARQL_B200_LIB") or (_HERE / "liblarql_b200.so"))  # override: a tuning build

FMT_Q4_K, FMT_Q8_0, FMT_MXFP4, FMT_NVFP4, FMT_Q6_K = 0, 1, 2, 3, 4
MAT_DEVICE = 0x100  # OR-ed into a matrix format: data/scales are device pointers
WALK_RMSNORM, WALK_RESIDUAL, WALK_FORCE_SPARSE = 1, 2, 4

LQ_OK = 0
LQ_REFUSED_SHAPE, LQ_REFUSED_UNSUPPORTED, LQ_ERR_NAN_SCORE = 1, 2, 3
LQ_ERR_CUDA, LQ_ERR_TIMEOUT, LQ_ERR_ARGUMENT = -1, -2, -3

# Every symbol include/larql_cuda.h declares (checked by the CPU test-suite).
EXPORTS = [
    "lq_create", "lq_destroy", "lq_last_error", "lq_device_info", "lq_supports_quant", "lq_synchronize",
    "lq_stream", "lq_launch_count", "lq_register_weight_region", "lq_seal_weight_regions",
    "lq_drop_weight_regions", "lq_device_ptr", "lq_q4k_matvec", "lq_q4k_matmul", "lq_q4k_matvec_exact",
    "lq_topk_abs", "lq_rms_norm", "lq_dequantize", "lq_walk_ffn", "lq_dev_q4k_matvec", "lq_dev_walk_ffn",
    "lq_stack_create", "lq_stack_run", "lq_stack_destroy", "lq_last_walk_stats", "lq_dev_quantize_q4k",
    "lq_profile_walk", "lq_fused_phase_us", "lq_q4k_matvec_static", "lq_dev_shard_scan", "lq_dev_shard_classify",
    "lq_dev_shard_gather", "lq_gemv", "lq_q8_0_gemv", "lq_mxfp4_gemv", "lq_nvfp4_gemv", "lq_moe_route",
    "lq_moe_walk_ffn", "lq_stack_run_host", "lq_dev_shard_hits", "lq_gemv_multi", "lq_mxfp4_gemv_multi",
    "lq_nvfp4_gemv_multi", "lq_gemv16", "lq_gemv16_multi", "lq_f16_gemv", "lq_bf16_gemv", "lq_q4k_matvec_topk",
    "lq_gemv16_topk", "lq_f16_gemv_topk", "lq_comm_unique_id", "lq_comm_init", "lq_comm_destroy",
    "lq_stack_create_sharded", "lq_stack_path", "lq_q6k_matvec", "lq_dequantize_q6k", "lq_q4k_dual_matvec",
    "lq_k_quant_padded_cols", "lq_vindex_open", "lq_vindex_num_layers", "lq_vindex_layer", "lq_vindex_close",
    "lq_nvfp4_pack_split",
]


class BackendError(RuntimeError):
    """A device/runtime failure (negative status) or the reference's panic cases."""


class LqMatrix(C.Structure):
    _fields_ = [("fmt", C.c_int32), ("data", C.c_void_p), ("data_len", C.c_size_t), ("scales", C.c_void_p),
                ("scales_len", C.c_size_t), ("tensor_scale", C.c_float), ("rows", C.c_int64), ("cols", C.c_int64)]


class WalkStats(C.Structure):
    _fields_ = [("n_certain", C.c_int32), ("n_band", C.c_int32), ("n_hits", C.c_int32), ("need", C.c_int32),
                ("tau", C.c_float), ("bound", C.c_float)]


_lib = None


def load_library() -> C.CDLL:
    """dlopen the built CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise BackendError(f"{LIB_PATH} is missing: run `python -m larql_b200.build` (no CPU fallback exists)")
    lib = C.CDLL(str(LIB_PATH))
    vp, sz, u32p, f32p = C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p
    mp = C.POINTER(LqMatrix)
    sig = {
        "lq_create": (C.c_int, [C.c_int, C.POINTER(vp)]),
        "lq_destroy": (None, [vp]),
        "lq_last_error": (C.c_char_p, [vp]),
        "lq_device_info": (C.c_int, [vp, C.c_char_p, sz]),
        "lq_supports_quant": (C.c_int, [vp, C.c_int]),
        "lq_synchronize": (C.c_int, [vp]),
        "lq_stream": (vp, [vp]),
        "lq_launch_count": (C.c_uint64, [vp]),
        "lq_register_weight_region": (C.c_int, [vp, vp, sz]),
        "lq_seal_weight_regions": (C.c_int, [vp]),
        "lq_drop_weight_regions": (C.c_int, [vp]),
        "lq_device_ptr": (vp, [vp, vp, sz]),
        "lq_q4k_matvec": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p, sz]),
        "lq_q4k_matvec_exact": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p, sz]),
        "lq_q4k_matmul": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, sz, f32p, sz]),
        "lq_topk_abs": (C.c_int, [vp, f32p, sz, sz, u32p, f32p, C.POINTER(sz)]),
        "lq_rms_norm": (C.c_int, [vp, f32p, sz, sz, C.c_double, f32p]),
        "lq_dequantize": (C.c_int, [vp, mp, f32p, sz]),
        "lq_walk_ffn": (C.c_int, [vp, mp, mp, mp, f32p, sz, sz, C.c_uint32, f32p, u32p, u32p]),
        "lq_dev_q4k_matvec": (C.c_int, [vp, vp, sz, f32p, sz, sz, f32p]),
        "lq_dev_walk_ffn": (C.c_int, [vp, mp, mp, mp, f32p, sz, sz, C.c_uint32, f32p, u32p, u32p]),
        "lq_stack_create": (C.c_int, [vp, mp, mp, mp, sz, sz, sz, C.c_uint32, C.POINTER(vp)]),
        "lq_stack_run": (C.c_int, [vp, vp, f32p, f32p]),
        "lq_stack_run_host": (C.c_int, [vp, vp, f32p, f32p]),
        "lq_dev_shard_hits": (C.c_int, [vp, u32p, sz, C.POINTER(sz)]),
        "lq_stack_destroy": (None, [vp, vp]),
        "lq_stack_path": (C.c_int, [vp]),
        "lq_k_quant_padded_cols": (sz, [sz]),
        "lq_vindex_open": (C.c_int, [C.c_char_p, C.POINTER(vp), C.c_char_p, sz]),
        "lq_vindex_num_layers": (sz, [vp]),
        "lq_vindex_layer": (C.c_int, [vp, sz, mp, mp, mp, mp]),
        "lq_vindex_close": (None, [vp]),
        "lq_nvfp4_pack_split": (C.c_int, [vp, sz, sz, sz, mp]),
        "lq_q6k_matvec": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p]),
        "lq_dequantize_q6k": (C.c_int, [vp, vp, sz, sz, f32p]),
        "lq_q4k_dual_matvec": (C.c_int, [vp, vp, sz, vp, sz, f32p, sz, sz, sz, f32p, f32p]),
        "lq_last_walk_stats": (C.c_int, [vp, C.POINTER(WalkStats)]),
        "lq_dev_quantize_q4k": (C.c_int, [vp, f32p, sz, vp]),
        "lq_profile_walk": (C.c_int, [vp, mp, mp, mp, f32p, sz, C.c_uint32, f32p, f32p]),
        "lq_fused_phase_us": (C.c_int, [vp, f32p, sz]),
        "lq_dev_shard_scan": (C.c_int, [vp, mp, f32p, C.c_uint32, C.c_int, C.c_int, vp]),
        "lq_dev_shard_classify": (C.c_int, [vp, mp, vp, C.c_int, sz, sz, vp, sz]),
        "lq_dev_shard_gather": (C.c_int, [vp, mp, mp, vp, C.c_int, C.c_int, sz, sz, sz, f32p]),
        "lq_gemv": (C.c_int, [vp, mp, f32p, sz, f32p, sz, C.c_int]),
        "lq_q8_0_gemv": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p]),
        "lq_mxfp4_gemv": (C.c_int, [vp, vp, sz, vp, sz, f32p, sz, sz, sz, f32p]),
        "lq_nvfp4_gemv": (C.c_int, [vp, vp, sz, vp, sz, C.c_float, f32p, sz, sz, sz, f32p]),
        "lq_moe_route": (C.c_int, [vp, f32p, sz, sz, sz, C.c_int, u32p, f32p]),
        "lq_moe_walk_ffn": (C.c_int, [vp, mp, mp, mp, sz, f32p, f32p, sz, sz, C.c_int, sz, C.c_uint32, f32p, u32p,
                                      f32p]),
        "lq_q4k_matvec_static": (C.c_int, [vp, sz, f32p, sz, sz, f32p, vp, C.c_char_p, sz]),
        "lq_comm_unique_id": (C.c_int, [vp, sz]),
        "lq_comm_init": (C.c_int, [vp, C.c_int, C.c_int, vp, sz]),
        "lq_comm_destroy": (C.c_int, [vp]),
        "lq_stack_create_sharded": (C.c_int, [vp, mp, mp, mp, sz, sz, sz, sz, sz, C.c_uint32, sz, C.POINTER(vp)]),
        "lq_gemv_multi": (C.c_int, [vp, vp, sz, f32p, sz, vp, C.c_int]),
        "lq_mxfp4_gemv_multi": (C.c_int, [vp, vp, sz, f32p, sz, vp]),
        "lq_nvfp4_gemv_multi": (C.c_int, [vp, vp, sz, f32p, sz, vp]),
        "lq_gemv16": (C.c_int, [vp, C.c_int, vp, sz, f32p, sz, sz, sz, f32p, C.c_int]),
        "lq_gemv16_multi": (C.c_int, [vp, C.c_int, sz, vp, vp, vp, sz, f32p, sz, vp, C.c_int]),
        "lq_f16_gemv": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p]),
        "lq_bf16_gemv": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, f32p]),
        "lq_q4k_matvec_topk": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, sz, u32p, f32p, C.POINTER(sz)]),
        "lq_gemv16_topk": (C.c_int, [vp, C.c_int, vp, sz, f32p, sz, sz, sz, sz, u32p, f32p, C.POINTER(sz)]),
        "lq_f16_gemv_topk": (C.c_int, [vp, vp, sz, f32p, sz, sz, sz, sz, u32p, f32p, C.POINTER(sz)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _ptr(a):
    return a.ctypes.data if a is not None and a.size else None


class HostMatrix:
    """A quantised [rows, cols] matrix held in host memory (numpy), as the reference's mmap slices are."""

    def __init__(self, fmt: int, rows: int, cols: int, data, scales=None, tensor_scale: float = 1.0):
        self.fmt, self.rows, self.cols = int(fmt), int(rows), int(cols)
        self.data = _u8(data)
        self.scales = _u8(scales) if scales is not None else None
        self.tensor_scale = float(tensor_scale)

    def c(self) -> LqMatrix:
        return LqMatrix(self.fmt, _ptr(self.data), self.data.size, _ptr(self.scales) if self.scales is not None else None,
                        self.scales.size if self.scales is not None else 0, self.tensor_scale, self.rows, self.cols)


def k_quant_padded_cols(cols: int) -> int:
    """Row width of a K-quant matrix on disk: the next multiple of 256 (k_quant_padded_cols)."""
    return int(load_library().lq_k_quant_padded_cols(int(cols)))


def _host_matrix_of(m: "LqMatrix", keepalive=None) -> "HostMatrix":
    def view(ptr, n):
        if not ptr or not n:
            return None
        a = np.ctypeslib.as_array((C.c_ubyte * n).from_address(ptr))
        a.flags.writeable = False
        return a
    hm = HostMatrix.__new__(HostMatrix)
    hm.fmt, hm.rows, hm.cols = int(m.fmt), int(m.rows), int(m.cols)
    hm.data, hm.scales = view(m.data, m.data_len), view(m.scales, m.scales_len)
    hm.tensor_scale = float(m.tensor_scale)
    hm.keepalive = keepalive
    return hm


class VindexFiles:
    """The K-quant FFN weights of a vindex directory, mapped read-only (interleaved_kquant.bin and, when present,
    the feature-major down sidecar).  ``layer(l)`` returns (gate, up, down, down_fm) as HostMatrix views into the
    mappings; down_fm is None without the sidecar.  Raises BackendError with the reader's reason on a refusal."""

    def __init__(self, directory):
        self._lib = load_library()
        self._h = C.c_void_p()
        err = C.create_string_buffer(512)
        rc = self._lib.lq_vindex_open(str(directory).encode(), C.byref(self._h), err, len(err))
        if rc != LQ_OK:
            raise BackendError(err.value.decode() or f"lq_vindex_open: status {rc}")

    @property
    def num_layers(self) -> int:
        return int(self._lib.lq_vindex_num_layers(self._h))

    def layer(self, l: int):
        g, u, d, f = LqMatrix(), LqMatrix(), LqMatrix(), LqMatrix()
        if self._lib.lq_vindex_layer(self._h, int(l), C.byref(g), C.byref(u), C.byref(d), C.byref(f)) != LQ_OK:
            raise IndexError(f"layer {l} out of range")
        return (_host_matrix_of(g, self), _host_matrix_of(u, self), _host_matrix_of(d, self),
                _host_matrix_of(f, self) if f.fmt >= 0 else None)

    def close(self):
        if self._h:
            self._lib.lq_vindex_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nvfp4_pack_split(payload, rows: int, k: int):
    """The stored form of an NVFP4 tensor {codes | scales | f32 tensor scale} as a HostMatrix view; None on a
    shape refusal (k not a multiple of 16, or a length that does not match [rows, k])."""
    b = _u8(payload)
    m = LqMatrix()
    rc = load_library().lq_nvfp4_pack_split(_ptr(b), b.size, int(rows), int(k), C.byref(m))
    return _host_matrix_of(m, b) if rc == LQ_OK else None


class DeviceMatrix:
    """A quantised matrix resident in device memory (raw device pointers, e.g. from torch tensors)."""

    def __init__(self, fmt: int, rows: int, cols: int, data_ptr: int, data_len: int, scales_ptr: int = 0,
                 scales_len: int = 0, tensor_scale: float = 1.0, keepalive=None):
        self.fmt, self.rows, self.cols = int(fmt), int(rows), int(cols)
        self.data_ptr, self.data_len, self.scales_ptr, self.scales_len = data_ptr, data_len, scales_ptr, scales_len
        self.tensor_scale = float(tensor_scale)
        self.keepalive = keepalive

    def c(self) -> LqMatrix:
        return LqMatrix(self.fmt | MAT_DEVICE, self.data_ptr, self.data_len, self.scales_ptr or None,
                        self.scales_len, self.tensor_scale, self.rows, self.cols)


def q4k_matvec_static(w_ptr: int, w_len: int, x_ptr: int, num_rows: int, hidden: int, out_ptr: int, stream: int = 0):
    """The allocation-free Q4_K matvec (device pointers; no context, no cudaMalloc inside).

    For hosts that cannot allocate device memory while running; scratch is a fixed 128 KiB array
    in the library image, so hidden <= 16384.  Returns (status, message)."""
    lib = load_library()
    buf = C.create_string_buffer(256)
    rc = lib.lq_q4k_matvec_static(w_ptr, w_len, x_ptr, num_rows, hidden, out_ptr, stream or None, buf, 256)
    return rc, buf.value.decode()


class CudaBackend:
    """Host-side mirror of the reference's backend trait for the walk path.

    Method names and argument meaning follow ``QuantMatVec`` / ``MatMul``
    (crates/larql-compute/src/backend/quant_matvec.rs, matmul.rs).  Methods return
    ``None`` on a refusal (bad geometry, unsupported format) and raise
    :class:`BackendError` on device errors and on the reference's panic cases.
    """

    def __init__(self, device: int = 0):
        self._lib = load_library()
        h = C.c_void_p()
        rc = self._lib.lq_create(device, C.byref(h))
        if rc != 0 or not h.value:
            raise BackendError(f"lq_create(device={device}) failed with status {rc}: no usable CUDA device "
                               f"(there is no CPU fallback)")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._lib.lq_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- plumbing ------------------------------------------------------------
    def _status(self, rc: int):
        """0 -> True, refusal -> None... returns True when ok, False when refused, raises otherwise."""
        if rc == LQ_OK:
            return True
        msg = self._lib.lq_last_error(self._h).decode()
        if rc in (LQ_REFUSED_SHAPE, LQ_REFUSED_UNSUPPORTED):
            self.last_refusal = msg
            return False
        raise BackendError(f"status {rc}: {msg}")

    def name(self) -> str:
        return "cuda-b200"

    def device_info(self) -> str:
        buf = C.create_string_buffer(512)
        self._lib.lq_device_info(self._h, buf, 512)
        return buf.value.decode()

    def supports_quant(self, fmt: int) -> bool:
        return bool(self._lib.lq_supports_quant(self._h, fmt))

    def synchronize(self):
        self._status(self._lib.lq_synchronize(self._h))

    def stream(self) -> int:
        return self._lib.lq_stream(self._h)

    def launch_count(self) -> int:
        return int(self._lib.lq_launch_count(self._h))

    def register_weight_region(self, arr: np.ndarray):
        self._status(self._lib.lq_register_weight_region(self._h, arr.ctypes.data, arr.nbytes))

    def seal_weight_regions(self):
        self._status(self._lib.lq_seal_weight_regions(self._h))

    def drop_weight_regions(self):
        self._status(self._lib.lq_drop_weight_regions(self._h))

    def device_ptr(self, arr: np.ndarray):
        return self._lib.lq_device_ptr(self._h, arr.ctypes.data, arr.nbytes)

    # -- QuantMatVec ----------------------------------------------------------
    def q4k_matvec(self, q4k_data, x, num_rows: int, hidden: int, exact: bool = False):
        w, x = _u8(q4k_data), _f32(x)
        out = np.empty(num_rows, np.float32)
        fn = self._lib.lq_q4k_matvec_exact if exact else self._lib.lq_q4k_matvec
        ok = self._status(fn(self._h, _ptr(w), w.size, _ptr(x), x.size, num_rows, hidden, _ptr(out), out.size))
        return out if ok else None

    def q4k_matmul(self, q4k_data, x, num_rows: int, hidden: int, seq_len: int):
        w, x = _u8(q4k_data), _f32(x)
        out = np.empty(seq_len * num_rows, np.float32)
        ok = self._status(self._lib.lq_q4k_matmul(self._h, _ptr(w), w.size, _ptr(x), x.size, num_rows, hidden,
                                                  seq_len, _ptr(out), out.size))
        return out.reshape(seq_len, num_rows) if ok else None

    def quant_matvec(self, fmt: int, weights, x, num_rows: int, hidden: int):
        """Format-dispatched matvec (quant_matvec.rs:50-98): formats that are one byte slice."""
        if fmt == FMT_Q4_K:
            return self.q4k_matvec(weights, x, num_rows, hidden)
        if fmt == FMT_Q8_0:
            return self.q8_0_gemv(weights, x, num_rows, hidden)
        return None

    def gemv(self, m: "HostMatrix", x, exact: bool = False):
        """out[rows] = m . x for any of the four formats; exact=True is the CPU backend's f32 order."""
        x = _f32(x).reshape(-1)
        out = np.empty(m.rows, np.float32)
        mc = m.c()
        ok = self._status(self._lib.lq_gemv(self._h, C.byref(mc), _ptr(x), x.size, _ptr(out), out.size, int(exact)))
        return out if ok else None

    def q8_0_gemv(self, blocks, x, n: int, k: int):
        """QuantMatVec::q8_0_gemv: None on any geometry mismatch."""
        w, x = _u8(blocks), _f32(x)
        out = np.empty(n, np.float32)
        ok = self._status(self._lib.lq_q8_0_gemv(self._h, _ptr(w), w.size, _ptr(x), x.size, n, k, _ptr(out)))
        return out if ok else None

    def mxfp4_gemv(self, packed, scales, x, n: int, k: int):
        """MatMul::mxfp4_gemv."""
        w, sc, x = _u8(packed), _u8(scales), _f32(x)
        out = np.empty(n, np.float32)
        ok = self._status(self._lib.lq_mxfp4_gemv(self._h, _ptr(w), w.size, _ptr(sc), sc.size, _ptr(x), x.size, n, k,
                                                  _ptr(out)))
        return out if ok else None

    def nvfp4_gemv(self, packed, scales, tensor_scale: float, x, n: int, k: int):
        """QuantMatVec::nvfp4_gemv: None on any geometry mismatch."""
        w, sc, x = _u8(packed), _u8(scales), _f32(x)
        out = np.empty(n, np.float32)
        ok = self._status(self._lib.lq_nvfp4_gemv(self._h, _ptr(w), w.size, _ptr(sc), sc.size, float(tensor_scale),
                                                  _ptr(x), x.size, n, k, _ptr(out)))
        return out if ok else None

    def gemv_multi(self, mats, x, exact: bool = False):
        """MatMul::mxfp4_gemv_multi / nvfp4_gemv_multi (any block format): several matrices, one input, one
        submission.  Returns a list of outputs, or None on refusal."""
        x = _f32(x).reshape(-1)
        n = len(mats)
        arr = (LqMatrix * max(n, 1))(*[m.c() for m in mats])
        outs = [np.empty(m.rows, np.float32) for m in mats]
        ptrs = (C.c_void_p * max(n, 1))(*[o.ctypes.data for o in outs])
        ok = self._status(self._lib.lq_gemv_multi(self._h, arr, n, _ptr(x), x.size, ptrs, int(exact)))
        return outs if ok else None

    def gemv16(self, w_bits, x, n: int, k: int, kind: str = "f16", exact: bool = False):
        """MatMul::f16_gemv / bf16_gemv: w_bits holds n*k little-endian 16-bit words."""
        w = np.ascontiguousarray(w_bits).view(np.uint8).reshape(-1)
        x = _f32(x).reshape(-1)
        out = np.empty(n, np.float32)
        ok = self._status(self._lib.lq_gemv16(self._h, 0 if kind == "f16" else 1, _ptr(w), w.size, _ptr(x), x.size, n, k,
                                              _ptr(out), int(exact)))
        return out if ok else None

    def gemv16_multi(self, weights, x, kind: str = "f16", exact: bool = False):
        """MatMul::f16_gemv_multi / bf16_gemv_multi: weights = [(w_bits, n, k), ...], every k == len(x)."""
        x = _f32(x).reshape(-1)
        ws = [np.ascontiguousarray(w).view(np.uint8).reshape(-1) for w, _, _ in weights]
        ns = [int(n) for _, n, _ in weights]
        if any(int(k) != x.size for _, _, k in weights):
            return None
        m = len(weights)
        outs = [np.empty(n, np.float32) for n in ns]
        wp = (C.c_void_p * max(m, 1))(*[w.ctypes.data for w in ws])
        wl = (C.c_size_t * max(m, 1))(*[w.size for w in ws])
        nn = (C.c_size_t * max(m, 1))(*ns)
        op = (C.c_void_p * max(m, 1))(*[o.ctypes.data for o in outs])
        ok = self._status(self._lib.lq_gemv16_multi(self._h, 0 if kind == "f16" else 1, m, wp, wl, nn, x.size, _ptr(x),
                                                    x.size, op, int(exact)))
        return outs if ok else None

    def q6k_matvec(self, q6k_data, x, num_rows: int, hidden: int):
        """QuantMatVec::q6k_matvec; None on a shape refusal."""
        w, x = _u8(q6k_data), _f32(x).reshape(-1)
        out = np.empty(num_rows, np.float32)
        ok = self._status(self._lib.lq_q6k_matvec(self._h, _ptr(w), w.size, _ptr(x), x.size, num_rows, hidden, _ptr(out)))
        return out if ok else None

    def dequantize_q6k(self, data, n_elems: int):
        d = _u8(data)
        out = np.empty(n_elems, np.float32)
        ok = self._status(self._lib.lq_dequantize_q6k(self._h, _ptr(d), d.size, n_elems, _ptr(out)))
        return out if ok else None

    def q4k_dual_matvec(self, q4k_a, q4k_b, x, num_rows: int, hidden: int):
        """QuantMatVec::q4k_dual_matvec: (out_a, out_b); None on a shape refusal."""
        a, b, x = _u8(q4k_a), _u8(q4k_b), _f32(x).reshape(-1)
        oa, ob = np.empty(num_rows, np.float32), np.empty(num_rows, np.float32)
        ok = self._status(self._lib.lq_q4k_dual_matvec(self._h, _ptr(a), a.size, _ptr(b), b.size, _ptr(x), x.size,
                                                       num_rows, hidden, _ptr(oa), _ptr(ob)))
        return (oa, ob) if ok else None

    def q4k_matvec_topk(self, q4k_data, x, num_rows: int, hidden: int, top_k: int):
        """QuantMatVec::q4k_matvec_topk: [(row, score)] sorted by score descending, ties to the lower row."""
        w, x = _u8(q4k_data), _f32(x).reshape(-1)
        k = max(1, min(int(top_k), num_rows))
        idx, val, cnt = np.empty(k, np.uint32), np.empty(k, np.float32), C.c_size_t(0)
        ok = self._status(self._lib.lq_q4k_matvec_topk(self._h, _ptr(w), w.size, _ptr(x), x.size, num_rows, hidden,
                                                       int(top_k), idx.ctypes.data, val.ctypes.data, C.byref(cnt)))
        return list(zip(idx[:cnt.value].tolist(), val[:cnt.value].tolist())) if ok else None

    def f16_gemv_topk(self, w_bits, x, n: int, k: int, top_k: int, kind: str = "f16"):
        """MatMul::f16_gemv_topk (and its bf16 sibling)."""
        w = np.ascontiguousarray(w_bits).view(np.uint8).reshape(-1)
        x = _f32(x).reshape(-1)
        kk = max(1, min(int(top_k), n))
        idx, val, cnt = np.empty(kk, np.uint32), np.empty(kk, np.float32), C.c_size_t(0)
        ok = self._status(self._lib.lq_gemv16_topk(self._h, 0 if kind == "f16" else 1, _ptr(w), w.size, _ptr(x), x.size,
                                                   n, k, int(top_k), idx.ctypes.data, val.ctypes.data, C.byref(cnt)))
        return list(zip(idx[:cnt.value].tolist(), val[:cnt.value].tolist())) if ok else None

    # -- MoE --------------------------------------------------------------------
    def moe_route(self, logits, top_k: int, renormalise: bool = True):
        """softmax -> top-k experts (value desc, index asc) -> weights; logits [tokens, experts]."""
        lg = _f32(logits)
        lg = lg.reshape(-1, lg.shape[-1])
        t, e = lg.shape
        k = min(int(top_k), e)
        idx = np.zeros((t, max(k, 1)), np.uint32)
        w = np.zeros((t, max(k, 1)), np.float32)
        ok = self._status(self._lib.lq_moe_route(self._h, _ptr(lg), t, e, int(top_k), int(renormalise), idx.ctypes.data,
                                                 w.ctypes.data))
        return (idx[:, :k], w[:, :k]) if ok else None

    def moe_walk_ffn(self, gates, ups, downs, logits, x, top_e: int, top_k: int, renormalise: bool = True,
                     flags: int = 0):
        """out[t] = sum over the token's top_e experts of w * walk(expert, x[t]); returns (out, idx, w)."""
        x = _f32(x)
        x2 = x.reshape(-1, x.shape[-1])
        lg = _f32(logits).reshape(x2.shape[0], -1)
        ne = len(gates)
        arr = lambda ms: (LqMatrix * ne)(*[m.c() for m in ms])
        ga, ua, da = arr(gates), arr(ups), arr(downs)
        ke = min(int(top_e), ne)
        out = np.empty_like(x2)
        idx = np.zeros((x2.shape[0], max(ke, 1)), np.uint32)
        w = np.zeros((x2.shape[0], max(ke, 1)), np.float32)
        ok = self._status(self._lib.lq_moe_walk_ffn(self._h, ga, ua, da, ne, _ptr(lg), _ptr(x2), x2.shape[0], int(top_e),
                                                    int(renormalise), int(top_k), int(flags), _ptr(out),
                                                    idx.ctypes.data, w.ctypes.data))
        return (out.reshape(x.shape), idx[:, :ke], w[:, :ke]) if ok else None

    # -- selection, norm, decode ----------------------------------------------
    def top_k_by_abs(self, scores, top_k: int):
        s = _f32(scores).reshape(-1)
        k = min(int(top_k), s.size)
        idx = np.empty(max(k, 1), np.uint32)
        val = np.empty(max(k, 1), np.float32)
        cnt = C.c_size_t(0)
        self._status(self._lib.lq_topk_abs(self._h, _ptr(s), s.size, int(top_k), idx.ctypes.data, val.ctypes.data,
                                           C.byref(cnt)))
        return idx[:cnt.value].copy(), val[:cnt.value].copy()

    def rms_norm(self, x, eps: float = 1e-6):
        x = _f32(x)
        x2 = x.reshape(-1, x.shape[-1])
        out = np.empty_like(x2)
        ok = self._status(self._lib.lq_rms_norm(self._h, _ptr(x2), x2.shape[0], x2.shape[1], eps, _ptr(out)))
        return out.reshape(x.shape) if ok else None

    def dequantize(self, m: HostMatrix):
        out = np.empty(m.rows * m.cols, np.float32)
        mc = m.c()
        ok = self._status(self._lib.lq_dequantize(self._h, C.byref(mc), _ptr(out), out.size))
        return out.reshape(m.rows, m.cols) if ok else None

    # -- the walk -------------------------------------------------------------
    def walk_ffn(self, gate: HostMatrix, up: HostMatrix, down_fm: HostMatrix, x, top_k: int, flags: int = 0,
                 want_idx: bool = True):
        """One layer for x [batch, hidden] (host). Returns (out, idx_list) or None on refusal."""
        x = _f32(x)
        x2 = x.reshape(-1, gate.cols) if gate.cols else x.reshape(x.shape[0] if x.ndim > 1 else 1, 0)
        batch = x2.shape[0]
        n = gate.rows
        k_eff = n if (not (flags & WALK_FORCE_SPARSE) and top_k >= (n * 4) // 5) else min(top_k, n)
        out = np.empty_like(x2)
        idx = np.zeros((batch, max(k_eff, 1)), np.uint32)
        cnt = np.zeros(batch, np.uint32)
        g, u, d = gate.c(), up.c(), down_fm.c()
        ok = self._status(self._lib.lq_walk_ffn(self._h, C.byref(g), C.byref(u), C.byref(d), _ptr(x2), batch,
                                                int(top_k), flags, _ptr(out), idx.ctypes.data if want_idx else None,
                                                cnt.ctypes.data if want_idx else None))
        if not ok:
            return None
        hits = [idx[t, :cnt[t]].copy() for t in range(batch)] if want_idx else None
        return out.reshape(x.shape), hits

    def fused_phase_us(self):
        us = (C.c_float * 13)()
        ok = self._status(self._lib.lq_fused_phase_us(self._h, us, 13))
        return list(us) if ok else None

    def last_walk_stats(self) -> WalkStats:
        s = WalkStats()
        self._lib.lq_last_walk_stats(self._h, C.byref(s))
        return s

    # -- device-pointer API (torch tensors or raw pointers) --------------------
    def dev_q4k_matvec(self, w_ptr: int, w_len: int, x_ptr: int, num_rows: int, hidden: int, out_ptr: int):
        return self._status(self._lib.lq_dev_q4k_matvec(self._h, w_ptr, w_len, x_ptr, num_rows, hidden, out_ptr))

    def dev_walk_ffn(self, gate: DeviceMatrix, up: DeviceMatrix, down_fm: DeviceMatrix, x_ptr: int, batch: int,
                     top_k: int, flags: int, out_ptr: int, idx_ptr: int = 0, count_ptr: int = 0):
        g, u, d = gate.c(), up.c(), down_fm.c()
        return self._status(self._lib.lq_dev_walk_ffn(self._h, C.byref(g), C.byref(u), C.byref(d), x_ptr, batch,
                                                      int(top_k), flags, out_ptr, idx_ptr or None, count_ptr or None))

    def dev_quantize_q4k(self, src_ptr: int, n_elems: int, dst_ptr: int):
        return self._status(self._lib.lq_dev_quantize_q4k(self._h, src_ptr, n_elems, dst_ptr))

    def profile_walk(self, gate, up, down_fm, x_ptr: int, top_k: int, flags: int, out_ptr: int):
        """Per-phase device milliseconds of one token: prepare, scan, select, re-score, gather, finish."""
        ms = (C.c_float * 6)()
        g, u, d = gate.c(), up.c(), down_fm.c()
        ok = self._status(self._lib.lq_profile_walk(self._h, C.byref(g), C.byref(u), C.byref(d), x_ptr, int(top_k),
                                                    flags, out_ptr, ms))
        return list(ms) if ok else None

    # -- feature-sharded walk: the steps between the collectives --------------------
    def dev_shard_scan(self, gate, x_ptr: int, flags: int, rank: int, world: int, hist_ptr: int):
        g = gate.c()
        return self._status(self._lib.lq_dev_shard_scan(self._h, C.byref(g), x_ptr, flags, rank, world, hist_ptr))

    def last_shard_hits(self, row_offset: int = 0):
        """Global rows this rank selected in its last shard gather (unordered)."""
        cnt = C.c_size_t(0)
        self._status(self._lib.lq_dev_shard_hits(self._h, None, 0, C.byref(cnt)))
        idx = np.zeros(max(cnt.value, 1), np.uint32)
        self._status(self._lib.lq_dev_shard_hits(self._h, idx.ctypes.data, cnt.value, C.byref(cnt)))
        return [int(i) + int(row_offset) for i in idx[:cnt.value]]

    def dev_shard_classify(self, gate, hist_ptr: int, world: int, top_k: int, row_offset: int, pack_ptr: int, cap: int):
        g = gate.c()
        return self._status(self._lib.lq_dev_shard_classify(self._h, C.byref(g), hist_ptr, world, int(top_k),
                                                            int(row_offset), pack_ptr, int(cap)))

    def dev_shard_gather(self, up, down, packs_ptr: int, world: int, rank: int, cap: int, top_k: int,
                         row_offset: int, out_ptr: int):
        u, d = up.c(), down.c()
        return self._status(self._lib.lq_dev_shard_gather(self._h, C.byref(u), C.byref(d), packs_ptr, world, rank,
                                                          int(cap), int(top_k), int(row_offset), out_ptr))

    # -- multi-GPU: one NCCL communicator per context, feature-sharded stacks ---------------
    @staticmethod
    def comm_unique_id() -> bytes:
        """The 128-byte NCCL id rank 0 makes and hands to the other ranks (any channel)."""
        buf = C.create_string_buffer(128)
        rc = load_library().lq_comm_unique_id(buf, 128)
        if rc != 0:
            raise BackendError(f"lq_comm_unique_id failed ({rc}): libnccl.so.2 not loadable?")
        return buf.raw

    def comm_init(self, rank: int, world: int, unique_id: bytes):
        buf = C.create_string_buffer(unique_id, len(unique_id))
        return self._status(self._lib.lq_comm_init(self._h, rank, world, buf, len(unique_id)))

    def comm_destroy(self):
        return self._status(self._lib.lq_comm_destroy(self._h))

    def stack_create_sharded(self, gates, ups, downs, batch: int, top_k: int, n_features_global: int, row_offset: int,
                             cap: int, flags: int = 0):
        """This rank's row range of every layer; run with stack_run / stack_run_host on every rank alike."""
        n = len(gates)
        arr = (LqMatrix * n)
        ga, ua, da = arr(*[m.c() for m in gates]), arr(*[m.c() for m in ups]), arr(*[m.c() for m in downs])
        h = C.c_void_p()
        ok = self._status(self._lib.lq_stack_create_sharded(self._h, ga, ua, da, n, batch, int(top_k),
                                                            int(n_features_global), int(row_offset), flags, int(cap),
                                                            C.byref(h)))
        return h if ok else None

    def stack_path(self, stack) -> int:
        """STACK_PATH_*: which implementation the stack runs on."""
        return int(self._lib.lq_stack_path(stack))

    def stack_create(self, gates, ups, downs, batch: int, top_k: int, flags: int = 0):
        n = len(gates)
        arr = (LqMatrix * n)
        ga, ua, da = arr(*[m.c() for m in gates]), arr(*[m.c() for m in ups]), arr(*[m.c() for m in downs])
        h = C.c_void_p()
        ok = self._status(self._lib.lq_stack_create(self._h, ga, ua, da, n, batch, int(top_k), flags, C.byref(h)))
        return h if ok else None

    def stack_run(self, stack, h_in_ptr: int, h_out_ptr: int):
        return self._status(self._lib.lq_stack_run(self._h, stack, h_in_ptr, h_out_ptr))

    def stack_run_host(self, stack, h_in_ptr: int, h_out_ptr: int):
        """All layers of a stack on HOST residuals (pointers to batch*hidden floats): upload, walk, download."""
        return self._status(self._lib.lq_stack_run_host(self._h, stack, h_in_ptr, h_out_ptr))

    def stack_destroy(self, stack):
        self._lib.lq_stack_destroy(self._h, stack)
