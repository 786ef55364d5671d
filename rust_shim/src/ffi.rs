//! `extern "C"` declarations of `libkaio_b200.so` (see `include/kaio_b200.h`).
//!
//! NOT COMPILED IN THIS REPOSITORY: no Rust toolchain is available where it was written.
//!
//! Conventions: device pointers, element counts of the caller's buffers (`GpuBuffer::len()`),
//! a `CUstream` as `*mut c_void`; `f16` crosses as its `u16` bit pattern (`half::f16` is
//! `#[repr(transparent)]` over `u16`).  Every function returns a status code
//! (`status::check` turns it into `Result<()>`).

use std::ffi::c_void;
use std::os::raw::c_char;

pub const KAIO_B200_OK: i32 = 0;
pub const KAIO_B200_ERR_INVALID_CONFIG: i32 = 1;
pub const KAIO_B200_ERR_CUDA: i32 = 2;
pub const KAIO_B200_ERR_UNSUPPORTED_ARCH: i32 = 3;
pub const KAIO_B200_ERR_TIMEOUT: i32 = 4;

#[link(name = "kaio_b200")]
extern "C" {
    /// Replaces the launch tail of `matmul_int8` (kaio-ops/src/matmul_int8_kernel.rs:1468-1512).
    pub fn kaio_b200_matmul_int8(
        a: *const i8, a_len: usize, b: *const i8, b_len: usize, c: *mut f32, c_len: usize,
        scale: f32, m: u32, n: u32, k: u32, stream: *mut c_void,
    ) -> i32;

    /// Replaces the launch tail of `matmul_int4` (kaio-ops/src/matmul_int4_kernel.rs:2126-2171).
    pub fn kaio_b200_matmul_int4(
        a: *const u16, a_len: usize, b_packed: *const u32, b_len: usize, scales: *const u16,
        scales_len: usize, c: *mut f32, c_len: usize, m: u32, n: u32, k: u32, group_size: u32,
        stream: *mut c_void,
    ) -> i32;

    /// Replaces `matmul_tc` (kaio-ops/src/matmul_tc_kernel.rs:1583-1626).
    pub fn kaio_b200_matmul_tc(
        a: *const u16, a_len: usize, b: *const u16, b_len: usize, c: *mut f32, c_len: usize,
        m: u32, n: u32, k: u32, stream: *mut c_void,
    ) -> i32;

    /// Replaces `matmul_tc_async` (kaio-ops/src/matmul_tc_async_kernel.rs:960-1003).
    pub fn kaio_b200_matmul_tc_async(
        a: *const u16, a_len: usize, b: *const u16, b_len: usize, c: *mut f32, c_len: usize,
        m: u32, n: u32, k: u32, stream: *mut c_void,
    ) -> i32;

    /// Replaces `qkv_project_int8` (kaio-ops/src/qkv_project_int8_kernel.rs:2008-2064).
    pub fn kaio_b200_qkv_project_int8(
        x: *const u16, x_len: usize, w_q: *const i8, w_q_len: usize, w_k: *const i8,
        w_k_len: usize, w_v: *const i8, w_v_len: usize, scale_q: f32, scale_k: f32, scale_v: f32,
        q_out: *mut u16, q_len: usize, k_out: *mut u16, k_len: usize, v_out: *mut u16,
        v_len: usize, m: u32, n: u32, k: u32, stream: *mut c_void,
    ) -> i32;

    /// Replaces `qkv_project_int4` (kaio-ops/src/qkv_project_int4_kernel.rs:1495-1555).
    pub fn kaio_b200_qkv_project_int4(
        x: *const u16, x_len: usize, w_q_packed: *const u32, w_q_len: usize,
        w_k_packed: *const u32, w_k_len: usize, w_v_packed: *const u32, w_v_len: usize,
        scales_q: *const u16, scales_q_len: usize, scales_k: *const u16, scales_k_len: usize,
        scales_v: *const u16, scales_v_len: usize, q_out: *mut u16, q_len: usize,
        k_out: *mut u16, k_len: usize, v_out: *mut u16, v_len: usize, m: u32, n: u32, k: u32,
        group_size: u32, stream: *mut c_void,
    ) -> i32;

    /// Replaces `attention_tc_dispatch` behind `attention_tc` / `attention_tc_causal`
    /// (kaio-ops/src/attention_tc_kernel.rs:2240-2333); `causal` is 0 or 1.
    pub fn kaio_b200_attention_tc(
        q: *const u16, q_len: usize, k: *const u16, k_len: usize, v: *const u16, v_len: usize,
        out: *mut f32, out_len: usize, seq_q: u32, seq_k: u32, d_k: u32, d_v: u32, causal: i32,
        stream: *mut c_void,
    ) -> i32;

    /// The calling thread's last error message (valid until its next call into the library).
    pub fn kaio_b200_last_error() -> *const c_char;

    /// Synchronises `stream` and reports a device-side wait that gave up (status 4), if any.
    pub fn kaio_b200_device_status(stream: *mut c_void, code: *mut u32) -> i32;
}
