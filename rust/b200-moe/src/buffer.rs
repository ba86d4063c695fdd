//! Caller-owned device memory and the library context.
use std::os::raw::c_void;

use b200_moe_sys as sys;

use crate::error::{guarded, Exception};

/// Element types the library understands (values of `B200_F32` / `B200_BF16` / `B200_F16`; u32 is used for
/// packed weights and indices and never passed as a dtype).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum DType {
    Float32,
    Bfloat16,
    Float16,
    Uint32,
}
impl DType {
    pub fn size(self) -> usize {
        match self {
            DType::Float32 | DType::Uint32 => 4,
            DType::Bfloat16 | DType::Float16 => 2,
        }
    }
    pub(crate) fn code(self) -> i32 {
        match self {
            DType::Float32 => sys::B200_F32,
            DType::Bfloat16 => sys::B200_BF16,
            DType::Float16 => sys::B200_F16,
            DType::Uint32 => -1,
        }
    }
}

/// Where output buffers come from.  The host program implements it over its own CUDA allocator; the
/// library itself only allocates its scratch arena (`Context::reserve`) and the expert-parallel buffers.
pub trait DeviceAllocator {
    fn alloc(&self, bytes: usize) -> *mut c_void;
    fn free(&self, ptr: *mut c_void);
}

/// A dense row-major tensor in device memory: pointer, dtype, shape.  Does not own the memory unless it
/// was produced by an op (then it frees it through the allocator it came from).
pub struct DeviceBuf<'a> {
    pub ptr: *mut c_void,
    pub dtype: DType,
    pub shape: Vec<i64>,
    owner: Option<&'a dyn DeviceAllocator>,
}
impl<'a> DeviceBuf<'a> {
    /// Wraps memory the caller owns.
    pub fn borrowed(ptr: *mut c_void, dtype: DType, shape: &[i64]) -> Self {
        Self { ptr, dtype, shape: shape.to_vec(), owner: None }
    }
    pub(crate) fn new_in(alloc: &'a dyn DeviceAllocator, dtype: DType, shape: &[i64]) -> Self {
        let n: i64 = shape.iter().product();
        Self { ptr: alloc.alloc(n as usize * dtype.size()), dtype, shape: shape.to_vec(), owner: Some(alloc) }
    }
    pub fn numel(&self) -> i64 {
        self.shape.iter().product()
    }
    pub fn dim(&self, i: isize) -> i64 {
        let n = self.shape.len() as isize;
        self.shape[((i + n) % n) as usize]
    }
}
impl Drop for DeviceBuf<'_> {
    fn drop(&mut self) {
        if let Some(a) = self.owner {
            a.free(self.ptr);
        }
    }
}

/// A CUDA stream handle (`cudaStream_t`), the counterpart of `mlx_rs::Stream`.
#[derive(Debug, Clone, Copy)]
pub struct Stream(pub *mut c_void);
impl Stream {
    pub fn default_stream() -> Self {
        Stream(std::ptr::null_mut())
    }
}

/// Owns the library's scratch memory on one device; one per thread and device, like the reference's
/// per-thread default streams.
pub struct Context {
    pub(crate) raw: *mut sys::b200_ctx,
}
impl Context {
    #[track_caller]
    pub fn new(device: i32) -> Result<Self, Exception> {
        let mut raw = std::ptr::null_mut();
        guarded(|| unsafe { sys::b200_ctx_create(&mut raw, device) })?;
        Ok(Self { raw })
    }
    /// Pre-sizes the scratch so that later calls do not allocate.
    #[track_caller]
    pub fn reserve(&self, cfg: &sys::b200_moe_config, max_tokens: i64) -> Result<(), Exception> {
        guarded(|| unsafe { sys::b200_ctx_reserve(self.raw, cfg, max_tokens) })
    }
    /// Synchronises `stream` and reports device-side findings (index out of range, expired wait).
    #[track_caller]
    pub fn check(&self, stream: Stream) -> Result<(), Exception> {
        guarded(|| unsafe { sys::b200_ctx_check(self.raw, stream.0) })
    }
}
impl Drop for Context {
    fn drop(&mut self) {
        unsafe { sys::b200_ctx_destroy(self.raw) };
    }
}
