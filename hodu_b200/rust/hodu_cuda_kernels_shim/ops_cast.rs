//! Replacement body for `call_ops_cast` of `crates/hodu_cuda_kernels/src/kernels/ops_cast.rs:27-64`
//! (call site `crates/hodu_core/src/be_cuda/storage.rs:619`).  The kernel name
//! "hodu_cuda_cast_{src}_to_{dst}" selects the dtype pair; pairs the library does not implement
//! come back as `InvalidKernel`, and the caller may keep the reference's own kernel for those.
//! Not compiled in this repository's build image (no cargo).
use std::sync::Arc;

use cudarc::driver::{CudaContext, CudaSlice, DevicePtr, DevicePtrMut, DeviceRepr};

use super::ops_matrix::{check, dtype_code};
use crate::{
    error::{CudaKernelError, Result},
    kernel::Kernels,
    kernels::macros::Kernel,
};

pub fn call_ops_cast<I: DeviceRepr, O: DeviceRepr>(
    kernel: Kernel,
    _kernels: &Kernels,
    context: &Arc<CudaContext>,
    input: &CudaSlice<I>,
    output: &mut CudaSlice<O>,
    metadata: &[usize],
) -> Result<()> {
    let bad = || CudaKernelError::InvalidKernel(kernel.0.to_string());
    let rest = kernel.0.strip_prefix("hodu_cuda_cast_").ok_or_else(bad)?;
    let (src, dst) = rest.split_once("_to_").ok_or_else(bad)?;
    let (src, dst) = (dtype_code(src).ok_or_else(bad)?, dtype_code(dst).ok_or_else(bad)?);
    let stream = context.default_stream();
    let (i, _gi) = input.device_ptr(&stream);
    let (o, _go) = output.device_ptr_mut(&stream);
    check(unsafe {
        hodu_b200_sys::hodu_b200_cast(context.ordinal() as i32, stream.cu_stream() as *mut _, src, dst,
            i as *const _, o as *mut _, metadata.as_ptr(), metadata.len())
    })
}
