//! Replacement bodies for `call_ops_matmul` and `call_ops_dot` of
//! `crates/hodu_cuda_kernels/src/kernels/ops_matrix.rs` (:415-429 and :611-625; the helper
//! functions `call_ops_matmul_kernel` / `call_ops_dot_kernel` at :328-384 and :539-585 and the
//! PTX they load are then unused).  Signatures, error type and stream are the reference's, so
//! `hodu_core::be_cuda::storage::ops_matrix` (`:50`, `:126`) calls them unchanged.
//! Not compiled in this repository's build image (no cargo).
use std::{ffi::CStr, sync::Arc};

use cudarc::driver::{CudaContext, CudaSlice, DevicePtr, DevicePtrMut, DeviceRepr};

use crate::{
    error::{CudaKernelError, Result},
    kernel::Kernels,
    kernels::macros::Kernel,
};

/// "hodu_cuda_matmul_bf16" -> `DType::BF16 as u8`, by `DType`'s `Display` names
/// (`crates/hodu_core/src/types/dtype.rs:31-58`).
pub(crate) fn dtype_code(name: &str) -> Option<u8> {
    Some(match name {
        "bool" => 0, "f8e4m3" => 1, "f8e5m2" => 2, "bf16" => 3, "f16" => 4, "f32" => 5, "f64" => 6,
        "u8" => 7, "u16" => 8, "u32" => 9, "u64" => 10, "i8" => 11, "i16" => 12, "i32" => 13, "i64" => 14,
        _ => return None,
    })
}

pub(crate) fn dtype_of(kernel: &Kernel, prefix: &str) -> Result<u8> {
    kernel.0.strip_prefix(prefix).and_then(dtype_code)
        .ok_or_else(|| CudaKernelError::InvalidKernel(kernel.0.to_string()))
}

/// Maps a return code of the C ABI onto the reference's error variants
/// (`crates/hodu_cuda_kernels/src/error.rs:7-18`).
pub(crate) fn check(code: i32) -> Result<()> {
    if code == 0 {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(hodu_b200_sys::hodu_b200_last_error_message()) }.to_string_lossy().into_owned();
    Err(match code {
        -1 => CudaKernelError::InvalidKernel(msg),
        -2 => CudaKernelError::InvalidInput(msg),
        -3 => CudaKernelError::LaunchError(msg),
        -4 => CudaKernelError::MemoryError(msg),
        _ => CudaKernelError::Message(msg),
    })
}

pub fn call_ops_matmul<T: DeviceRepr>(
    kernel: Kernel,
    _kernels: &Kernels,
    context: &Arc<CudaContext>,
    lhs: &CudaSlice<T>,
    rhs: &CudaSlice<T>,
    output: &mut CudaSlice<T>,
    metadata: &[usize],
) -> Result<()> {
    let dtype = dtype_of(&kernel, "hodu_cuda_matmul_")?;
    let stream = context.default_stream();
    let (l, _gl) = lhs.device_ptr(&stream);
    let (r, _gr) = rhs.device_ptr(&stream);
    let (o, _go) = output.device_ptr_mut(&stream);
    check(unsafe {
        hodu_b200_sys::hodu_b200_matmul(context.ordinal() as i32, stream.cu_stream() as *mut _, dtype,
            l as *const _, r as *const _, o as *mut _, metadata.as_ptr(), metadata.len())
    })
}

pub fn call_ops_dot<T: DeviceRepr>(
    kernel: Kernel,
    _kernels: &Kernels,
    context: &Arc<CudaContext>,
    lhs: &CudaSlice<T>,
    rhs: &CudaSlice<T>,
    output: &mut CudaSlice<T>,
    metadata: &[usize],
) -> Result<()> {
    let dtype = dtype_of(&kernel, "hodu_cuda_dot_")?;
    let stream = context.default_stream();
    let (l, _gl) = lhs.device_ptr(&stream);
    let (r, _gr) = rhs.device_ptr(&stream);
    let (o, _go) = output.device_ptr_mut(&stream);
    check(unsafe {
        hodu_b200_sys::hodu_b200_dot(context.ordinal() as i32, stream.cu_stream() as *mut _, dtype,
            l as *const _, r as *const _, o as *mut _, metadata.as_ptr(), metadata.len())
    })
}
