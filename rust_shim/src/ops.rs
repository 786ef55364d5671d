//! Bodies of the `kaio-ops` hot-path functions over `libkaio_b200.so`.
//!
//! NOT COMPILED IN THIS REPOSITORY: no Rust toolchain is available where it was written.
//!
//! Each function keeps the reference's signature and its `validate_dims_*` call; only the
//! tail that built a PTX module, loaded it and launched it is replaced by one FFI call.  Like
//! the reference, every call enqueues on `device.stream()` and returns without synchronising
//! (kaio-ops/src/matmul_int8_kernel.rs:1497-1511); a kernel fault surfaces at the caller's
//! next synchronisation.
//!
//! cudarc accessors used (cudarc 0.19, to be checked against the pinned 0.19.4):
//!   `CudaSlice::<T>::device_ptr(&self, &CudaStream) -> (CUdeviceptr, SyncOnDrop)`
//!   `CudaSlice::<T>::device_ptr_mut(&mut self, &CudaStream) -> (CUdeviceptr, SyncOnDrop)`
//!   `CudaStream::cu_stream(&self) -> CUstream`
//!   `CudaStream::context(&self) -> &Arc<CudaContext>`, `CudaContext::bind_to_thread(&self)`
//! The guards returned beside the pointers record the stream's use of the buffers; they must
//! live until the FFI call has returned, which the `let` bindings below ensure.

use std::ffi::c_void;

use cudarc::driver::{DevicePtr, DevicePtrMut};
use half::f16;
use kaio_runtime::{GpuBuffer, KaioDevice, KaioError, Result};

use crate::ffi;
use crate::status::check;

/// The library launches on the calling thread's current device; the reference binds the
/// context when the `KaioDevice` is created (kaio-runtime/src/device.rs:77-82) and cudarc
/// re-binds it on use, so it is bound again here before every call.
fn bind(device: &KaioDevice) -> Result<u32> {
    device.stream().context().bind_to_thread()?;
    let (major, minor) = device.info()?.compute_capability;
    Ok(major * 10 + minor)
}

fn raw_stream(device: &KaioDevice) -> *mut c_void {
    device.stream().cu_stream() as *mut c_void
}

/// kaio-ops/src/matmul_int8_kernel.rs:1468-1512.
#[allow(clippy::too_many_arguments)]
pub fn matmul_int8(
    device: &KaioDevice,
    a: &GpuBuffer<i8>,
    b: &GpuBuffer<i8>,
    c: &mut GpuBuffer<f32>,
    scale: f32,
    m: u32,
    n: u32,
    k: u32,
) -> Result<()> {
    validate_dims_int8(a, b, c, m, n, k)?; // unchanged: matmul_int8_kernel.rs:108-150
    let sm = bind(device)?;
    let stream = device.stream();
    let (a_len, b_len, c_len) = (a.len(), b.len(), c.len());
    let (ap, _ga) = a.inner().device_ptr(stream);
    let (bp, _gb) = b.inner().device_ptr(stream);
    let (cp, _gc) = c.inner_mut().device_ptr_mut(stream);
    // SAFETY: the pointers are live device allocations of at least `*_len` elements on the
    // bound device; the library reads a, b and writes c[0 .. m*n) only.
    let code = unsafe {
        ffi::kaio_b200_matmul_int8(
            ap as *const i8, a_len, bp as *const i8, b_len, cp as *mut f32, c_len, scale, m, n, k,
            raw_stream(device),
        )
    };
    check(code, sm)
}

/// kaio-ops/src/matmul_int4_kernel.rs:2126-2171.
#[allow(clippy::too_many_arguments)]
pub fn matmul_int4(
    device: &KaioDevice,
    a: &GpuBuffer<f16>,
    b_packed: &GpuBuffer<u32>,
    scales: &GpuBuffer<f16>,
    c: &mut GpuBuffer<f32>,
    m: u32,
    n: u32,
    k: u32,
    group_size: u32,
) -> Result<()> {
    validate_dims_int4(a, b_packed, scales, c, m, n, k, group_size)?; // :112-174
    let sm = bind(device)?;
    let stream = device.stream();
    let (a_len, b_len, s_len, c_len) = (a.len(), b_packed.len(), scales.len(), c.len());
    let (ap, _ga) = a.inner().device_ptr(stream);
    let (bp, _gb) = b_packed.inner().device_ptr(stream);
    let (sp, _gs) = scales.inner().device_ptr(stream);
    let (cp, _gc) = c.inner_mut().device_ptr_mut(stream);
    // SAFETY: as in matmul_int8; b_packed is the flat word buffer `pack_s4_weights` produces
    // (kaio-ops/tests/matmul_int4_e2e.rs:37-54), indexed (k/8) + col * (K/8) by the library.
    let code = unsafe {
        ffi::kaio_b200_matmul_int4(
            ap as *const u16, a_len, bp as *const u32, b_len, sp as *const u16, s_len,
            cp as *mut f32, c_len, m, n, k, group_size, raw_stream(device),
        )
    };
    check(code, sm)
}

/// kaio-ops/src/matmul_tc_kernel.rs:1583-1626.
pub fn matmul_tc(
    device: &KaioDevice,
    a: &GpuBuffer<f16>,
    b: &GpuBuffer<f16>,
    c: &mut GpuBuffer<f32>,
    m: u32,
    n: u32,
    k: u32,
) -> Result<()> {
    validate_dims_tc(a, b, c, m, n, k)?; // matmul_tc_kernel.rs:123-164
    let sm = bind(device)?;
    let stream = device.stream();
    let (a_len, b_len, c_len) = (a.len(), b.len(), c.len());
    let (ap, _ga) = a.inner().device_ptr(stream);
    let (bp, _gb) = b.inner().device_ptr(stream);
    let (cp, _gc) = c.inner_mut().device_ptr_mut(stream);
    // SAFETY: as in matmul_int8.
    let code = unsafe {
        ffi::kaio_b200_matmul_tc(
            ap as *const u16, a_len, bp as *const u16, b_len, cp as *mut f32, c_len, m, n, k,
            raw_stream(device),
        )
    };
    check(code, sm)
}

/// kaio-ops/src/matmul_tc_async_kernel.rs:960-1003 (same contract as `matmul_tc`; the two
/// differ in the reference only in how they stage shared memory).
pub fn matmul_tc_async(
    device: &KaioDevice,
    a: &GpuBuffer<f16>,
    b: &GpuBuffer<f16>,
    c: &mut GpuBuffer<f32>,
    m: u32,
    n: u32,
    k: u32,
) -> Result<()> {
    validate_dims_tc(a, b, c, m, n, k)?;
    let sm = bind(device)?;
    let stream = device.stream();
    let (a_len, b_len, c_len) = (a.len(), b.len(), c.len());
    let (ap, _ga) = a.inner().device_ptr(stream);
    let (bp, _gb) = b.inner().device_ptr(stream);
    let (cp, _gc) = c.inner_mut().device_ptr_mut(stream);
    // SAFETY: as in matmul_int8.
    let code = unsafe {
        ffi::kaio_b200_matmul_tc_async(
            ap as *const u16, a_len, bp as *const u16, b_len, cp as *mut f32, c_len, m, n, k,
            raw_stream(device),
        )
    };
    check(code, sm)
}

/// The reference documents that the three outputs must be distinct allocations
/// (kaio-ops/src/qkv_project_int8_kernel.rs:1881-1892) and defers the device-pointer check;
/// with the raw pointers in hand it costs nothing, so it is made here (the library checks
/// again).
fn distinct(op: &str, q: u64, k: u64, v: u64) -> Result<()> {
    if q == k || q == v || k == v {
        return Err(KaioError::InvalidConfig(format!(
            "{op}: the three output buffers must be distinct allocations"
        )));
    }
    Ok(())
}

/// kaio-ops/src/qkv_project_int8_kernel.rs:2008-2064 (W8A16, scalar scale per projection).
#[allow(clippy::too_many_arguments)]
pub fn qkv_project_int8(
    device: &KaioDevice,
    x: &GpuBuffer<f16>,
    w_q: &GpuBuffer<i8>,
    w_k: &GpuBuffer<i8>,
    w_v: &GpuBuffer<i8>,
    scale_q: f32,
    scale_k: f32,
    scale_v: f32,
    q_out: &mut GpuBuffer<f16>,
    k_out: &mut GpuBuffer<f16>,
    v_out: &mut GpuBuffer<f16>,
    m: u32,
    n: u32,
    k: u32,
) -> Result<()> {
    validate_dims_qkv_int8(x, w_q, w_k, w_v, q_out, k_out, v_out, m, n, k)?; // :1894-1953
    let sm = bind(device)?;
    let stream = device.stream();
    let (x_len, wq_len, wk_len, wv_len) = (x.len(), w_q.len(), w_k.len(), w_v.len());
    let (q_len, k_len, v_len) = (q_out.len(), k_out.len(), v_out.len());
    let (xp, _gx) = x.inner().device_ptr(stream);
    let (wqp, _g1) = w_q.inner().device_ptr(stream);
    let (wkp, _g2) = w_k.inner().device_ptr(stream);
    let (wvp, _g3) = w_v.inner().device_ptr(stream);
    let (qp, _g4) = q_out.inner_mut().device_ptr_mut(stream);
    let (kp, _g5) = k_out.inner_mut().device_ptr_mut(stream);
    let (vp, _g6) = v_out.inner_mut().device_ptr_mut(stream);
    distinct("qkv_project_int8", qp as u64, kp as u64, vp as u64)?;
    // SAFETY: as in matmul_int8; the three outputs do not alias (checked above).
    let code = unsafe {
        ffi::kaio_b200_qkv_project_int8(
            xp as *const u16, x_len, wqp as *const i8, wq_len, wkp as *const i8, wk_len,
            wvp as *const i8, wv_len, scale_q, scale_k, scale_v, qp as *mut u16, q_len,
            kp as *mut u16, k_len, vp as *mut u16, v_len, m, n, k, raw_stream(device),
        )
    };
    check(code, sm)
}

/// kaio-ops/src/qkv_project_int4_kernel.rs:1495-1555 (W4A16, group-128 f16 scales).
#[allow(clippy::too_many_arguments)]
pub fn qkv_project_int4(
    device: &KaioDevice,
    x: &GpuBuffer<f16>,
    w_q_packed: &GpuBuffer<u32>,
    w_k_packed: &GpuBuffer<u32>,
    w_v_packed: &GpuBuffer<u32>,
    scales_q: &GpuBuffer<f16>,
    scales_k: &GpuBuffer<f16>,
    scales_v: &GpuBuffer<f16>,
    q_out: &mut GpuBuffer<f16>,
    k_out: &mut GpuBuffer<f16>,
    v_out: &mut GpuBuffer<f16>,
    m: u32,
    n: u32,
    k: u32,
    group_size: u32,
) -> Result<()> {
    validate_dims_qkv_int4(
        x, w_q_packed, w_k_packed, w_v_packed, scales_q, scales_k, scales_v, q_out, k_out, v_out,
        m, n, k, group_size,
    )?; // :1344-1433
    let sm = bind(device)?;
    let stream = device.stream();
    let x_len = x.len();
    let (wq_len, wk_len, wv_len) = (w_q_packed.len(), w_k_packed.len(), w_v_packed.len());
    let (sq_len, sk_len, sv_len) = (scales_q.len(), scales_k.len(), scales_v.len());
    let (q_len, k_len, v_len) = (q_out.len(), k_out.len(), v_out.len());
    let (xp, _gx) = x.inner().device_ptr(stream);
    let (wqp, _g1) = w_q_packed.inner().device_ptr(stream);
    let (wkp, _g2) = w_k_packed.inner().device_ptr(stream);
    let (wvp, _g3) = w_v_packed.inner().device_ptr(stream);
    let (sqp, _g4) = scales_q.inner().device_ptr(stream);
    let (skp, _g5) = scales_k.inner().device_ptr(stream);
    let (svp, _g6) = scales_v.inner().device_ptr(stream);
    let (qp, _g7) = q_out.inner_mut().device_ptr_mut(stream);
    let (kp, _g8) = k_out.inner_mut().device_ptr_mut(stream);
    let (vp, _g9) = v_out.inner_mut().device_ptr_mut(stream);
    distinct("qkv_project_int4", qp as u64, kp as u64, vp as u64)?;
    // SAFETY: as in qkv_project_int8.
    let code = unsafe {
        ffi::kaio_b200_qkv_project_int4(
            xp as *const u16, x_len, wqp as *const u32, wq_len, wkp as *const u32, wk_len,
            wvp as *const u32, wv_len, sqp as *const u16, sq_len, skp as *const u16, sk_len,
            svp as *const u16, sv_len, qp as *mut u16, q_len, kp as *mut u16, k_len,
            vp as *mut u16, v_len, m, n, k, group_size, raw_stream(device),
        )
    };
    check(code, sm)
}

/// `attention_tc_dispatch` (kaio-ops/src/attention_tc_kernel.rs:2273-2333) with the launch
/// tail replaced; `attention_tc` (:2240-2252) and `attention_tc_causal` (:2261-2273) call it
/// with `causal = false / true` exactly as before.
#[allow(clippy::too_many_arguments)]
fn attention_tc_dispatch(
    device: &KaioDevice,
    q: &GpuBuffer<f16>,
    k: &GpuBuffer<f16>,
    v: &GpuBuffer<f16>,
    out: &mut GpuBuffer<f32>,
    seq_q: u32,
    seq_k: u32,
    d_k: u32,
    d_v: u32,
    causal: bool,
) -> Result<()> {
    validate_attention_tc_dims(q, k, v, out, seq_q, seq_k, d_k, d_v)?; // :139-223
    let sm = bind(device)?;
    let stream = device.stream();
    let (q_len, k_len, v_len, o_len) = (q.len(), k.len(), v.len(), out.len());
    let (qp, _g1) = q.inner().device_ptr(stream);
    let (kp, _g2) = k.inner().device_ptr(stream);
    let (vp, _g3) = v.inner().device_ptr(stream);
    let (op, _g4) = out.inner_mut().device_ptr_mut(stream);
    // SAFETY: as in matmul_int8.
    let code = unsafe {
        ffi::kaio_b200_attention_tc(
            qp as *const u16, q_len, kp as *const u16, k_len, vp as *const u16, v_len,
            op as *mut f32, o_len, seq_q, seq_k, d_k, d_v, i32::from(causal), raw_stream(device),
        )
    };
    check(code, sm)
}

/// kaio-ops/src/attention_tc_kernel.rs:2240-2252.
#[allow(clippy::too_many_arguments)]
pub fn attention_tc(
    device: &KaioDevice,
    q: &GpuBuffer<f16>,
    k: &GpuBuffer<f16>,
    v: &GpuBuffer<f16>,
    out: &mut GpuBuffer<f32>,
    seq_q: u32,
    seq_k: u32,
    d_k: u32,
    d_v: u32,
) -> Result<()> {
    attention_tc_dispatch(device, q, k, v, out, seq_q, seq_k, d_k, d_v, false)
}

/// kaio-ops/src/attention_tc_kernel.rs:2261-2273.
#[allow(clippy::too_many_arguments)]
pub fn attention_tc_causal(
    device: &KaioDevice,
    q: &GpuBuffer<f16>,
    k: &GpuBuffer<f16>,
    v: &GpuBuffer<f16>,
    out: &mut GpuBuffer<f32>,
    seq_q: u32,
    seq_k: u32,
    d_k: u32,
    d_v: u32,
) -> Result<()> {
    attention_tc_dispatch(device, q, k, v, out, seq_q, seq_k, d_k, d_v, true)
}
