//! `larql-compute-cuda`: the B200 backend behind `dyn larql_compute::ComputeBackend`.
//!
//! Every accelerated method is a pure delegation to one `extern "C"` entry point of
//! `include/larql_cuda.h`; the status convention of that header maps onto the traits' contract:
//!
//! * `0`             → `Some(..)`
//! * positive status → `None` ("cannot compute this": the caller falls back or fails loudly, never a wrong
//!                     or zero-filled answer — crates/larql-compute/src/backend/quant_matvec.rs:378-427,
//!                     cpu/ops/kernel_shape.rs:1-17)
//! * `3` (NaN score) → panic, as `top_k_by_abs` does on the CPU
//!                     (crates/larql-vindex/src/index/compute/gate_knn/mod.rs:47-49)
//! * negative status → device error: logged, then `None`.
//!
//! The two REQUIRED methods of `MatMul` — dense f32 `matmul` / `matmul_transb`
//! (crates/larql-compute/src/backend/matmul.rs:46-49) — are off the quantised walk path; this crate
//! satisfies them by holding a `CpuBackend` and forwarding to it, the same way the Metal backend sends
//! small products to the CPU.  Everything else not listed here keeps the trait's refusing default.
//!
//! Device calls are serialised behind a mutex, as `DevicePlanBackend` does for any device backend
//! (crates/larql-vindex/src/format/vindex3/opplan/exec/device.rs:39-42).

use std::any::Any;
use std::ffi::{c_char, c_int, c_void, CStr};
use std::sync::Mutex;

use larql_compute::backend::{Capability, ComputeBackend, DecodeBackend, MatMul, QuantMatVec};
use larql_compute::cpu::CpuBackend;
use larql_compute::QuantFormat;
use ndarray::{Array2, ArrayView2};

/// Mirrors `lq_matrix` (include/larql_cuda.h).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct LqMatrix {
    pub fmt: i32,
    pub data: *const c_void,
    pub data_len: usize,
    pub scales: *const c_void,
    pub scales_len: usize,
    pub tensor_scale: f32,
    pub rows: i64,
    pub cols: i64,
}

pub const LQ_FMT_Q4_K: i32 = 0;
pub const LQ_FMT_Q8_0: i32 = 1;
pub const LQ_FMT_MXFP4: i32 = 2;
pub const LQ_FMT_NVFP4: i32 = 3;
pub const LQ_WALK_RMSNORM: u32 = 1;
pub const LQ_WALK_RESIDUAL: u32 = 2;
pub const LQ_WALK_FORCE_SPARSE: u32 = 4;
const LQ_ERR_NAN_SCORE: c_int = 3;

#[repr(C)]
pub struct LqCtx {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct LqStack {
    _opaque: [u8; 0],
}

extern "C" {
    fn lq_create(device: c_int, out: *mut *mut LqCtx) -> c_int;
    fn lq_destroy(ctx: *mut LqCtx);
    fn lq_last_error(ctx: *mut LqCtx) -> *const c_char;
    fn lq_device_info(ctx: *mut LqCtx, buf: *mut c_char, cap: usize) -> c_int;
    fn lq_supports_quant(ctx: *mut LqCtx, fmt: c_int) -> c_int;
    fn lq_register_weight_region(ctx: *mut LqCtx, host: *const c_void, len: usize) -> c_int;
    fn lq_seal_weight_regions(ctx: *mut LqCtx) -> c_int;
    fn lq_q4k_matvec(ctx: *mut LqCtx, w: *const u8, w_len: usize, x: *const f32, x_len: usize, num_rows: usize,
                     hidden: usize, out: *mut f32, out_len: usize) -> c_int;
    fn lq_q4k_matmul(ctx: *mut LqCtx, w: *const u8, w_len: usize, x: *const f32, x_len: usize, num_rows: usize,
                     hidden: usize, seq_len: usize, out: *mut f32, out_len: usize) -> c_int;
    fn lq_q4k_matvec_topk(ctx: *mut LqCtx, w: *const u8, w_len: usize, x: *const f32, x_len: usize, num_rows: usize,
                          hidden: usize, top_k: usize, idx: *mut u32, val: *mut f32, count: *mut usize) -> c_int;
    fn lq_q6k_matvec(ctx: *mut LqCtx, w: *const u8, w_len: usize, x: *const f32, x_len: usize, num_rows: usize,
                     hidden: usize, out: *mut f32) -> c_int;
    fn lq_q4k_dual_matvec(ctx: *mut LqCtx, w_a: *const u8, wa_len: usize, w_b: *const u8, wb_len: usize, x: *const f32,
                          x_len: usize, num_rows: usize, hidden: usize, out_a: *mut f32, out_b: *mut f32) -> c_int;
    fn lq_q8_0_gemv(ctx: *mut LqCtx, blocks: *const u8, blocks_len: usize, x: *const f32, x_len: usize, n: usize,
                    k: usize, out: *mut f32) -> c_int;
    fn lq_mxfp4_gemv(ctx: *mut LqCtx, packed: *const u8, packed_len: usize, scales: *const u8, scales_len: usize,
                     x: *const f32, x_len: usize, n: usize, k: usize, out: *mut f32) -> c_int;
    fn lq_nvfp4_gemv(ctx: *mut LqCtx, packed: *const u8, packed_len: usize, scales: *const u8, scales_len: usize,
                     tensor_scale: f32, x: *const f32, x_len: usize, n: usize, k: usize, out: *mut f32) -> c_int;
    fn lq_gemv_multi(ctx: *mut LqCtx, mats: *const LqMatrix, n_mats: usize, x: *const f32, x_len: usize,
                     outs: *const *mut f32, exact: c_int) -> c_int;
    fn lq_gemv16(ctx: *mut LqCtx, kind: c_int, w: *const u8, w_len: usize, x: *const f32, x_len: usize, n: usize,
                 k: usize, out: *mut f32, exact: c_int) -> c_int;
    fn lq_gemv16_multi(ctx: *mut LqCtx, kind: c_int, n_mats: usize, ws: *const *const u8, w_lens: *const usize,
                       ns: *const usize, k: usize, x: *const f32, x_len: usize, outs: *const *mut f32,
                       exact: c_int) -> c_int;
    fn lq_gemv16_topk(ctx: *mut LqCtx, kind: c_int, w: *const u8, w_len: usize, x: *const f32, x_len: usize, n: usize,
                      k: usize, top_k: usize, idx: *mut u32, val: *mut f32, count: *mut usize) -> c_int;
    fn lq_walk_ffn(ctx: *mut LqCtx, gate: *const LqMatrix, up: *const LqMatrix, down_fm: *const LqMatrix,
                   x: *const f32, batch: usize, top_k: usize, flags: u32, out: *mut f32, idx_out: *mut u32,
                   count_out: *mut u32) -> c_int;
    fn lq_stack_create(ctx: *mut LqCtx, gates: *const LqMatrix, ups: *const LqMatrix, downs_fm: *const LqMatrix,
                       n_layers: usize, batch: usize, top_k: usize, flags: u32, out: *mut *mut LqStack) -> c_int;
    fn lq_stack_run_host(ctx: *mut LqCtx, stack: *mut LqStack, h_in: *const f32, h_out: *mut f32) -> c_int;
    fn lq_stack_destroy(ctx: *mut LqCtx, stack: *mut LqStack);
}

struct Ctx(*mut LqCtx);
// The context is only ever touched under the mutex below.
unsafe impl Send for Ctx {}

pub struct CudaBackend {
    ctx: Mutex<Ctx>,
    cpu: CpuBackend,
    info: String,
}

impl CudaBackend {
    /// `None` when no usable B200 is present (the registry then reports the backend as unavailable).
    pub fn new(device: i32) -> Option<Self> {
        let mut raw: *mut LqCtx = std::ptr::null_mut();
        if unsafe { lq_create(device, &mut raw) } != 0 || raw.is_null() {
            return None;
        }
        let mut buf = vec![0 as c_char; 256];
        let info = if unsafe { lq_device_info(raw, buf.as_mut_ptr(), buf.len()) } == 0 {
            unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
        } else {
            "cuda".to_string()
        };
        Some(Self { ctx: Mutex::new(Ctx(raw)), cpu: CpuBackend, info })
    }

    /// Runs `f` with the context locked and maps the status onto the traits' contract.
    fn call<T>(&self, f: impl FnOnce(*mut LqCtx) -> (c_int, T)) -> Option<T> {
        let guard = self.ctx.lock().unwrap_or_else(|e| e.into_inner());
        let (rc, value) = f(guard.0);
        if rc == 0 {
            return Some(value);
        }
        let msg = unsafe { CStr::from_ptr(lq_last_error(guard.0)) }.to_string_lossy().into_owned();
        if rc == LQ_ERR_NAN_SCORE {
            panic!("NaN gate score (top_k_by_abs): {msg}");
        }
        if rc < 0 {
            eprintln!("larql-compute-cuda: device error {rc}: {msg}");
        }
        None
    }

    /// The vindex FFN walk of one layer (walk_ffn_sparse,
    /// crates/larql-inference/src/vindex/walk_ffn/sparse.rs:60-306): `x` is `[batch, hidden]`; returns the
    /// output `[batch, hidden]` and, per token, the selected feature ids (the set is the CPU path's).
    /// There is no trait method for the fused walk: `WalkFfn` reaches this through `as_any()`.
    pub fn walk_ffn(&self, gate: &LqMatrix, up: &LqMatrix, down_fm: &LqMatrix, x: &[f32], batch: usize,
                    top_k: usize, flags: u32) -> Option<(Vec<f32>, Vec<Vec<u32>>)> {
        let hidden = gate.cols as usize;
        let n = gate.rows as usize;
        if x.len() != batch * hidden {
            return None;
        }
        let dense = flags & LQ_WALK_FORCE_SPARSE == 0 && top_k >= (n * 4) / 5;
        let stride = if dense { n } else { top_k.min(n) };
        let mut out = vec![0f32; batch * hidden];
        let mut idx = vec![0u32; (batch * stride).max(1)];
        let mut cnt = vec![0u32; batch.max(1)];
        self.call(|c| {
            let rc = unsafe {
                lq_walk_ffn(c, gate, up, down_fm, x.as_ptr(), batch, top_k, flags, out.as_mut_ptr(), idx.as_mut_ptr(),
                            cnt.as_mut_ptr())
            };
            (rc, ())
        })?;
        let hits = (0..batch).map(|t| idx[t * stride..t * stride + cnt[t] as usize].to_vec()).collect();
        Some((out, hits))
    }

    /// A stack of walk layers kept on the device: `h <- h + walk_l(rmsnorm(h))` for every layer with one
    /// upload and one download per token (run_ffn per layer, crates/larql-compute/src/forward/layer.rs:61-127).
    pub fn stack(&self, gates: &[LqMatrix], ups: &[LqMatrix], downs_fm: &[LqMatrix], batch: usize, top_k: usize,
                 flags: u32) -> Option<WalkStack<'_>> {
        if gates.len() != ups.len() || gates.len() != downs_fm.len() || gates.is_empty() {
            return None;
        }
        let mut raw: *mut LqStack = std::ptr::null_mut();
        self.call(|c| {
            let rc = unsafe {
                lq_stack_create(c, gates.as_ptr(), ups.as_ptr(), downs_fm.as_ptr(), gates.len(), batch, top_k, flags,
                                &mut raw)
            };
            (rc, ())
        })?;
        Some(WalkStack { backend: self, raw, len: batch * gates[0].cols as usize })
    }
}

impl Drop for CudaBackend {
    fn drop(&mut self) {
        let guard = self.ctx.lock().unwrap_or_else(|e| e.into_inner());
        unsafe { lq_destroy(guard.0) };
    }
}

pub struct WalkStack<'a> {
    backend: &'a CudaBackend,
    raw: *mut LqStack,
    len: usize,
}

impl WalkStack<'_> {
    pub fn run(&self, h_in: &[f32]) -> Option<Vec<f32>> {
        if h_in.len() != self.len {
            return None;
        }
        let mut out = vec![0f32; self.len];
        self.backend
            .call(|c| (unsafe { lq_stack_run_host(c, self.raw, h_in.as_ptr(), out.as_mut_ptr()) }, ()))
            .map(|_| out)
    }
}

impl Drop for WalkStack<'_> {
    fn drop(&mut self) {
        let guard = self.backend.ctx.lock().unwrap_or_else(|e| e.into_inner());
        unsafe { lq_stack_destroy(guard.0, self.raw) };
    }
}

impl MatMul for CudaBackend {
    // Required, dense f32, off the quantised walk path: forwarded to the CPU backend (see the module docs).
    fn matmul(&self, a: ArrayView2<f32>, b: ArrayView2<f32>) -> Array2<f32> {
        self.cpu.matmul(a, b)
    }
    fn matmul_transb(&self, a: ArrayView2<f32>, b: ArrayView2<f32>) -> Array2<f32> {
        self.cpu.matmul_transb(a, b)
    }

    fn f16_gemv(&self, w_f16: &[u8], x: &[f32], n: usize, k: usize) -> Option<Vec<f32>> {
        self.gemv16(0, w_f16, x, n, k)
    }
    fn bf16_gemv(&self, w_bf16: &[u8], x: &[f32], n: usize, k: usize) -> Option<Vec<f32>> {
        self.gemv16(1, w_bf16, x, n, k)
    }
    fn f16_gemv_multi(&self, weights: &[(&[u8], usize, usize)], x: &[f32]) -> Option<Vec<Vec<f32>>> {
        self.gemv16_multi(0, weights, x)
    }
    fn bf16_gemv_multi(&self, weights: &[(&[u8], usize, usize)], x: &[f32]) -> Option<Vec<Vec<f32>>> {
        self.gemv16_multi(1, weights, x)
    }
    fn f16_gemv_topk(&self, w_f16: &[u8], x: &[f32], n: usize, k: usize, top_k: usize) -> Option<Vec<(u32, f32)>> {
        let kk = top_k.min(n);
        let (mut idx, mut val, mut count) = (vec![0u32; kk.max(1)], vec![0f32; kk.max(1)], 0usize);
        self.call(|c| {
            let rc = unsafe {
                lq_gemv16_topk(c, 0, w_f16.as_ptr(), w_f16.len(), x.as_ptr(), x.len(), n, k, top_k, idx.as_mut_ptr(),
                               val.as_mut_ptr(), &mut count)
            };
            (rc, ())
        })?;
        Some(idx.into_iter().zip(val).take(count).collect())
    }

    fn mxfp4_gemv(&self, packed: &[u8], scales: &[u8], x: &[f32], n: usize, k: usize) -> Option<Vec<f32>> {
        let mut out = vec![0f32; n];
        self.call(|c| {
            let rc = unsafe {
                lq_mxfp4_gemv(c, packed.as_ptr(), packed.len(), scales.as_ptr(), scales.len(), x.as_ptr(), x.len(), n, k,
                              out.as_mut_ptr())
            };
            (rc, ())
        })
        .map(|_| out)
    }
    fn mxfp4_gemv_multi(&self, weights: &[(&[u8], &[u8], usize, usize)], x: &[f32]) -> Option<Vec<Vec<f32>>> {
        let mats: Vec<LqMatrix> = weights
            .iter()
            .map(|&(p, s, n, k)| block_matrix(LQ_FMT_MXFP4, p, s, 1.0, n, k))
            .collect();
        self.gemv_multi(&mats, x)
    }
    fn nvfp4_gemv(&self, packed: &[u8], scales: &[u8], tensor_scale: f32, x: &[f32], n: usize, k: usize)
                  -> Option<Vec<f32>> {
        let mut out = vec![0f32; n];
        self.call(|c| {
            let rc = unsafe {
                lq_nvfp4_gemv(c, packed.as_ptr(), packed.len(), scales.as_ptr(), scales.len(), tensor_scale, x.as_ptr(),
                              x.len(), n, k, out.as_mut_ptr())
            };
            (rc, ())
        })
        .map(|_| out)
    }
    fn nvfp4_gemv_multi(&self, weights: &[larql_compute::backend::matmul::Nvfp4Operand<'_>], x: &[f32])
                        -> Option<Vec<Vec<f32>>> {
        let mats: Vec<LqMatrix> = weights
            .iter()
            .map(|&(p, s, ts, n, k)| block_matrix(LQ_FMT_NVFP4, p, s, ts, n, k))
            .collect();
        self.gemv_multi(&mats, x)
    }
    fn wire_resident(&self, buffers: &[&[u8]]) {
        for b in buffers {
            self.register_weight_region(b);
        }
    }
}

fn block_matrix(fmt: i32, packed: &[u8], scales: &[u8], tensor_scale: f32, n: usize, k: usize) -> LqMatrix {
    LqMatrix {
        fmt,
        data: packed.as_ptr() as *const c_void,
        data_len: packed.len(),
        scales: scales.as_ptr() as *const c_void,
        scales_len: scales.len(),
        tensor_scale,
        rows: n as i64,
        cols: k as i64,
    }
}

impl CudaBackend {
    fn gemv16(&self, kind: c_int, w: &[u8], x: &[f32], n: usize, k: usize) -> Option<Vec<f32>> {
        let mut out = vec![0f32; n];
        self.call(|c| {
            (unsafe { lq_gemv16(c, kind, w.as_ptr(), w.len(), x.as_ptr(), x.len(), n, k, out.as_mut_ptr(), 0) }, ())
        })
        .map(|_| out)
    }
    fn gemv16_multi(&self, kind: c_int, weights: &[(&[u8], usize, usize)], x: &[f32]) -> Option<Vec<Vec<f32>>> {
        if weights.iter().any(|&(_, _, k)| k != x.len()) {
            return None;
        }
        let ws: Vec<*const u8> = weights.iter().map(|w| w.0.as_ptr()).collect();
        let lens: Vec<usize> = weights.iter().map(|w| w.0.len()).collect();
        let ns: Vec<usize> = weights.iter().map(|w| w.1).collect();
        let mut outs: Vec<Vec<f32>> = ns.iter().map(|&n| vec![0f32; n]).collect();
        let ptrs: Vec<*mut f32> = outs.iter_mut().map(|o| o.as_mut_ptr()).collect();
        self.call(|c| {
            let rc = unsafe {
                lq_gemv16_multi(c, kind, ws.len(), ws.as_ptr(), lens.as_ptr(), ns.as_ptr(), x.len(), x.as_ptr(), x.len(),
                                ptrs.as_ptr(), 0)
            };
            (rc, ())
        })
        .map(|_| outs)
    }
    fn gemv_multi(&self, mats: &[LqMatrix], x: &[f32]) -> Option<Vec<Vec<f32>>> {
        let mut outs: Vec<Vec<f32>> = mats.iter().map(|m| vec![0f32; m.rows as usize]).collect();
        let ptrs: Vec<*mut f32> = outs.iter_mut().map(|o| o.as_mut_ptr()).collect();
        self.call(|c| {
            (unsafe { lq_gemv_multi(c, mats.as_ptr(), mats.len(), x.as_ptr(), x.len(), ptrs.as_ptr(), 0) }, ())
        })
        .map(|_| outs)
    }
    /// ggml Q8_0 gemv with f32 activations.  The reference calls `kquant_gemv::q8_0_gemv` directly
    /// (crates/larql-vindex/src/format/vindex3/represent/kquant.rs:293); no trait method carries it.
    pub fn q8_0_gemv(&self, blocks: &[u8], x: &[f32], n: usize, k: usize) -> Option<Vec<f32>> {
        let mut out = vec![0f32; n];
        self.call(|c| {
            let rc = unsafe { lq_q8_0_gemv(c, blocks.as_ptr(), blocks.len(), x.as_ptr(), x.len(), n, k, out.as_mut_ptr()) };
            (rc, ())
        })
        .map(|_| out)
    }
}

impl QuantMatVec for CudaBackend {
    fn q4k_matvec(&self, q4k_data: &[u8], x: &[f32], num_rows: usize, hidden: usize) -> Option<Vec<f32>> {
        let mut out = vec![0f32; num_rows];
        self.call(|c| {
            let rc = unsafe {
                lq_q4k_matvec(c, q4k_data.as_ptr(), q4k_data.len(), x.as_ptr(), x.len(), num_rows, hidden,
                              out.as_mut_ptr(), out.len())
            };
            (rc, ())
        })
        .map(|_| out)
    }
    fn q6k_matvec(&self, q6k_data: &[u8], x: &[f32], num_rows: usize, hidden: usize) -> Option<Vec<f32>> {
        let mut out = vec![0f32; num_rows];
        self.call(|c| {
            let rc = unsafe {
                lq_q6k_matvec(c, q6k_data.as_ptr(), q6k_data.len(), x.as_ptr(), x.len(), num_rows, hidden,
                              out.as_mut_ptr())
            };
            (rc, ())
        })
        .map(|_| out)
    }
    fn q4k_dual_matvec(&self, q4k_a: &[u8], q4k_b: &[u8], x: &[f32], num_rows: usize, hidden: usize)
                       -> Option<(Vec<f32>, Vec<f32>)> {
        let (mut a, mut b) = (vec![0f32; num_rows], vec![0f32; num_rows]);
        self.call(|c| {
            let rc = unsafe {
                lq_q4k_dual_matvec(c, q4k_a.as_ptr(), q4k_a.len(), q4k_b.as_ptr(), q4k_b.len(), x.as_ptr(), x.len(),
                                   num_rows, hidden, a.as_mut_ptr(), b.as_mut_ptr())
            };
            (rc, ())
        })
        .map(|_| (a, b))
    }
    fn q4k_matvec_topk(&self, q4k_data: &[u8], x: &[f32], num_rows: usize, hidden: usize, top_k: usize)
                       -> Option<Vec<(u32, f32)>> {
        let kk = top_k.min(num_rows);
        let (mut idx, mut val, mut count) = (vec![0u32; kk.max(1)], vec![0f32; kk.max(1)], 0usize);
        self.call(|c| {
            let rc = unsafe {
                lq_q4k_matvec_topk(c, q4k_data.as_ptr(), q4k_data.len(), x.as_ptr(), x.len(), num_rows, hidden, top_k,
                                   idx.as_mut_ptr(), val.as_mut_ptr(), &mut count)
            };
            (rc, ())
        })?;
        Some(idx.into_iter().zip(val).take(count).collect())
    }
    fn q4k_matmul(&self, q4k_data: &[u8], x: &[f32], num_rows: usize, hidden: usize, seq_len: usize)
                  -> Option<Vec<f32>> {
        let mut out = vec![0f32; num_rows * seq_len];
        self.call(|c| {
            let rc = unsafe {
                lq_q4k_matmul(c, q4k_data.as_ptr(), q4k_data.len(), x.as_ptr(), x.len(), num_rows, hidden, seq_len,
                              out.as_mut_ptr(), out.len())
            };
            (rc, ())
        })
        .map(|_| out)
    }
    fn supports_quant(&self, format: QuantFormat) -> bool {
        // what the trait's `quant_matvec` dispatch can reach on this backend: Q4_K (and its Q4_KF twin)
        matches!(format, QuantFormat::Q4_K | QuantFormat::Q4_KF)
            && self.call(|c| (0, unsafe { lq_supports_quant(c, LQ_FMT_Q4_K) } != 0)).unwrap_or(false)
    }
}

// Every method of DecodeBackend has a refusing default (crates/larql-compute/src/backend/decode.rs:219-...):
// attention and the full decode pipeline stay with the caller's other backends.
impl DecodeBackend for CudaBackend {}

impl ComputeBackend for CudaBackend {
    fn name(&self) -> &str {
        "cuda-b200"
    }
    fn device_info(&self) -> String {
        self.info.clone()
    }
    fn supports(&self, _cap: Capability) -> bool {
        false // the capability menu (capability.rs:22-102) lists decode-pipeline features; none is claimed
    }
    fn register_weight_region(&self, region: &[u8]) {
        let _ = self.call(|c| {
            (unsafe { lq_register_weight_region(c, region.as_ptr() as *const c_void, region.len()) }, ())
        });
    }
    fn seal_weight_regions(&self) {
        let _ = self.call(|c| (unsafe { lq_seal_weight_regions(c) }, ()));
    }
    fn as_any(&self) -> &dyn Any {
        self
    }
}

/// `BackendCtor` for `BackendKind::Cuda` (crates/larql-compute/src/backend/factory.rs:127-130); the binary
/// registers it next to the Metal one (crates/larql-cli/src/backend_select.rs:26-36).
pub fn cuda_backend() -> Option<Box<dyn ComputeBackend>> {
    CudaBackend::new(0).map(|b| Box::new(b) as Box<dyn ComputeBackend>)
}
