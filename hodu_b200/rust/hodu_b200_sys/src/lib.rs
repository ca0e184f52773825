//! Raw declarations of the C ABI in `include/hodu_b200.h`, one per exported function, in the
//! header's order.  `usize` is `size_t` on every target Hodu supports, so the metadata
//! `Vec<usize>` built by `crates/hodu_core/src/op_metadatas.rs` is passed as it is
//! (`as_ptr()`, `len()`).  Not compiled in this repository's build image (no cargo).
#![allow(non_camel_case_types)]
use core::ffi::{c_char, c_int, c_void};

/// `DType` discriminants (`crates/hodu_core/src/types/dtype.rs:6-30`).
pub mod dtype {
    pub const BOOL: u8 = 0;
    pub const F8E4M3: u8 = 1;
    pub const F8E5M2: u8 = 2;
    pub const BF16: u8 = 3;
    pub const F16: u8 = 4;
    pub const F32: u8 = 5;
    pub const F64: u8 = 6;
    pub const U8: u8 = 7;
    pub const U16: u8 = 8;
    pub const U32: u8 = 9;
    pub const U64: u8 = 10;
    pub const I8: u8 = 11;
    pub const I16: u8 = 12;
    pub const I32: u8 = 13;
    pub const I64: u8 = 14;
}

/// Return codes; one per `CudaKernelError` variant plus the device-status code.
pub mod code {
    pub const OK: i32 = 0;
    pub const INVALID_KERNEL: i32 = -1;
    pub const INVALID_INPUT: i32 = -2;
    pub const LAUNCH: i32 = -3;
    pub const MEMORY: i32 = -4;
    pub const DEVICE_STATUS: i32 = -5;
    pub const NOT_INITIALISED: i32 = -6;
}

pub const SWIGLU_ROUND_EACH_OP: u32 = 0;
pub const SWIGLU_ROUND_ONCE: u32 = 1;
pub const LINEAR_ROUND_EACH_OP: u32 = 0;
pub const LINEAR_ROUND_ONCE: u32 = 1;
pub const STATIC_SCRATCH_BYTES: usize = 32 << 20;

extern "C" {
    pub fn hodu_b200_init(device: c_int) -> c_int;
    pub fn hodu_b200_shutdown(device: c_int);
    pub fn hodu_b200_matmul(device: c_int, stream: *mut c_void, dtype: u8, lhs: *const c_void,
        rhs: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_dot(device: c_int, stream: *mut c_void, dtype: u8, lhs: *const c_void,
        rhs: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_matmul_ex(device: c_int, stream: *mut c_void, in_dtype: u8, out_dtype: u8,
        lhs: *const c_void, rhs: *const c_void, out: *mut c_void, metadata: *const usize,
        metadata_len: usize, scale_lhs: f32, scale_rhs: f32, epilogue: u32) -> c_int;
    pub fn hodu_b200_dot_ex(device: c_int, stream: *mut c_void, in_dtype: u8, out_dtype: u8,
        lhs: *const c_void, rhs: *const c_void, out: *mut c_void, metadata: *const usize,
        metadata_len: usize, scale_lhs: f32, scale_rhs: f32, epilogue: u32) -> c_int;
    pub fn hodu_b200_cast(device: c_int, stream: *mut c_void, src_dtype: u8, dst_dtype: u8,
        input: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_contiguous(device: c_int, stream: *mut c_void, dtype: u8, input: *const c_void,
        out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_swiglu(device: c_int, stream: *mut c_void, dtype: u8, x: *const c_void,
        w_gate: *const c_void, w_up: *const c_void, out: *mut c_void, metadata: *const usize,
        metadata_len: usize, flags: u32) -> c_int;
    pub fn hodu_b200_linear(device: c_int, stream: *mut c_void, dtype: u8, x: *const c_void,
        w: *const c_void, bias: *const c_void, out: *mut c_void, metadata: *const usize,
        metadata_len: usize, flags: u32) -> c_int;
    pub fn hodu_b200_einsum(device: c_int, stream: *mut c_void, dtype: u8, inputs: *const *const c_void,
        num_inputs: usize, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_conv2d(device: c_int, stream: *mut c_void, dtype: u8, input: *const c_void,
        weight: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_matmul_host(device: c_int, in_dtype: u8, out_dtype: u8, lhs: *const c_void,
        rhs: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize,
        scale_lhs: f32, scale_rhs: f32) -> c_int;
    pub fn hodu_b200_dot_host(device: c_int, in_dtype: u8, out_dtype: u8, lhs: *const c_void,
        rhs: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize,
        scale_lhs: f32, scale_rhs: f32) -> c_int;
    pub fn hodu_b200_swiglu_mlp_host(device: c_int, dtype: u8, x_host: *const c_void, w_gate: *const c_void,
        w_up: *const c_void, w_down: *const c_void, y_host: *mut c_void, metadata: *const usize,
        metadata_len: usize, flags: u32) -> c_int;
    pub fn hodu_b200_dot_f32_static(device: c_int, stream: *mut c_void, lhs: *const c_void,
        rhs: *const c_void, out: *mut c_void, metadata: *const usize, metadata_len: usize) -> c_int;
    pub fn hodu_b200_dot_f32_static_status(device: c_int, word: *mut u32) -> c_int;
    pub fn hodu_b200_strerror(code: c_int) -> *const c_char;
    pub fn hodu_b200_last_error_message() -> *const c_char;
    pub fn hodu_b200_last_status(device: c_int, word: *mut u32) -> c_int;
    pub fn hodu_b200_force_path(path: c_int) -> c_int;
    pub fn hodu_b200_last_path() -> c_int;
    pub fn hodu_b200_debug_wait_timeout(device: c_int, stream: *mut c_void, limit_ms: u32) -> c_int;
    pub fn hodu_b200_launch_count() -> u64;
    pub fn hodu_b200_version() -> c_int;
}
