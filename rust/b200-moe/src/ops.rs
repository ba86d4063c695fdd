//! Op wrappers with the names, argument order and defaults of the reference
//! (`mlx-rs/src/ops/quantization.rs:48-230`, `ops/sort.rs:57-83,186-226`, `ops/indexing/mod.rs:374-453`,
//! `ops/arithmetic.rs:1312-1327`, `fast.rs:178-205`).  Every function takes the context, an allocator for
//! its result and a stream where the reference takes a `Stream`; the `_device` suffix follows
//! `mlx-internal-macros/src/lib.rs:44-104`.
use b200_moe_sys as sys;

use crate::buffer::{Context, DType, DeviceAllocator, DeviceBuf, Stream};
use crate::error::guarded;
use crate::Result;

pub const DEFAULT_GROUP_SIZE: i32 = sys::B200_DEFAULT_GROUP_SIZE;
pub const DEFAULT_BITS: i32 = sys::B200_DEFAULT_BITS;

fn opt<'b>(b: Option<&'b DeviceBuf<'_>>) -> *const u32 {
    b.map_or(std::ptr::null(), |t| t.ptr as *const u32)
}

/// `quantize(w, group_size, bits) -> (w_q, scales, biases)` along the last axis.
#[track_caller]
pub fn quantize_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, w: &DeviceBuf<'_>, group_size: impl Into<Option<i32>>,
                           bits: impl Into<Option<i32>>, stream: Stream) -> Result<(DeviceBuf<'a>, DeviceBuf<'a>, DeviceBuf<'a>)> {
    let (gs, bits) = (group_size.into().unwrap_or(DEFAULT_GROUP_SIZE), bits.into().unwrap_or(DEFAULT_BITS));
    let k = w.dim(-1);
    let rows = w.numel() / k;
    let mut qs = w.shape.clone();
    *qs.last_mut().unwrap() = k * bits as i64 / 32;
    let mut ss = w.shape.clone();
    *ss.last_mut().unwrap() = k / gs as i64;
    let (wq, s, b) = (DeviceBuf::new_in(alloc, DType::Uint32, &qs), DeviceBuf::new_in(alloc, w.dtype, &ss), DeviceBuf::new_in(alloc, w.dtype, &ss));
    guarded(|| unsafe {
        sys::b200_quantize(ctx.raw, w.ptr, w.dtype.code(), rows, k, gs, bits, wq.ptr as *mut u32, s.ptr, b.ptr, stream.0)
    })?;
    Ok((wq, s, b))
}

/// `dequantize(w, scales, biases, group_size, bits)`.
#[track_caller]
pub fn dequantize_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, w: &DeviceBuf<'_>, scales: &DeviceBuf<'_>,
                             biases: &DeviceBuf<'_>, group_size: impl Into<Option<i32>>, bits: impl Into<Option<i32>>,
                             stream: Stream) -> Result<DeviceBuf<'a>> {
    let (gs, bits) = (group_size.into().unwrap_or(DEFAULT_GROUP_SIZE), bits.into().unwrap_or(DEFAULT_BITS));
    let k = w.dim(-1) * 32 / bits as i64;
    let rows = w.numel() / w.dim(-1);
    let mut shape = w.shape.clone();
    *shape.last_mut().unwrap() = k;
    let out = DeviceBuf::new_in(alloc, scales.dtype, &shape);
    guarded(|| unsafe {
        sys::b200_dequantize(ctx.raw, w.ptr as *const u32, scales.ptr, biases.ptr, scales.dtype.code(), rows, k, gs, bits, out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `quantized_matmul(x, w, scales, biases, transpose, group_size, bits)`; `transpose` defaults to false like
/// the reference's wrapper (`mlx-rs/src/ops/quantization.rs:101`), layers pass true.
#[track_caller]
pub fn quantized_matmul_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, x: &DeviceBuf<'_>, w: &DeviceBuf<'_>,
                                   scales: &DeviceBuf<'_>, biases: &DeviceBuf<'_>, transpose: impl Into<Option<bool>>,
                                   group_size: impl Into<Option<i32>>, bits: impl Into<Option<i32>>, stream: Stream) -> Result<DeviceBuf<'a>> {
    let transpose = transpose.into().unwrap_or(false);
    let (gs, bits) = (group_size.into().unwrap_or(DEFAULT_GROUP_SIZE), bits.into().unwrap_or(DEFAULT_BITS));
    let k = x.dim(-1);
    let m = x.numel() / k;
    let n = if transpose { w.dim(0) } else { w.dim(1) * 32 / bits as i64 };
    let mut shape = x.shape.clone();
    *shape.last_mut().unwrap() = n;
    let out = DeviceBuf::new_in(alloc, x.dtype, &shape);
    guarded(|| unsafe {
        sys::b200_quantized_matmul(ctx.raw, x.ptr, w.ptr as *const u32, scales.ptr, biases.ptr, transpose as i32, gs, bits,
                                   x.dtype.code(), m, k, n, out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, transpose, group_size, bits, sorted_indices)`;
/// defaults: transpose true, group 64, bits 4, sorted false.
#[allow(clippy::too_many_arguments)]
#[track_caller]
pub fn gather_qmm_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, x: &DeviceBuf<'_>, w: &DeviceBuf<'_>,
                             scales: &DeviceBuf<'_>, biases: &DeviceBuf<'_>, lhs_indices: Option<&DeviceBuf<'_>>,
                             rhs_indices: &DeviceBuf<'_>, transpose: impl Into<Option<bool>>, group_size: impl Into<Option<i32>>,
                             bits: impl Into<Option<i32>>, sorted_indices: impl Into<Option<bool>>, stream: Stream) -> Result<DeviceBuf<'a>> {
    let transpose = transpose.into().unwrap_or(true);
    let (gs, bits) = (group_size.into().unwrap_or(DEFAULT_GROUP_SIZE), bits.into().unwrap_or(DEFAULT_BITS));
    let sorted = sorted_indices.into().unwrap_or(false);
    let (m, k) = (x.dim(-2), x.dim(-1));
    let bx = x.numel() / (m * k);
    let n = if transpose { w.dim(-2) } else { w.dim(-1) * 32 / bits as i64 };
    let e = w.numel() / (w.dim(-2) * w.dim(-1));
    let n_idx = rhs_indices.numel();
    let mut shape = rhs_indices.shape.clone();
    shape.extend_from_slice(&[m, n]);
    let out = DeviceBuf::new_in(alloc, x.dtype, &shape);
    guarded(|| unsafe {
        sys::b200_gather_qmm(ctx.raw, x.ptr, w.ptr as *const u32, scales.ptr, biases.ptr, opt(lhs_indices),
                             rhs_indices.ptr as *const u32, transpose as i32, gs, bits, sorted as i32, x.dtype.code(), bx, m, k, e, n,
                             n_idx, out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `gather_mm(a, b, lhs_indices, rhs_indices)` (un-quantised).
#[track_caller]
pub fn gather_mm_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, a: &DeviceBuf<'_>, b: &DeviceBuf<'_>,
                            lhs_indices: Option<&DeviceBuf<'_>>, rhs_indices: Option<&DeviceBuf<'_>>, stream: Stream) -> Result<DeviceBuf<'a>> {
    let (m, k, n) = (a.dim(-2), a.dim(-1), b.dim(-1));
    let (ba, bb) = (a.numel() / (m * k), b.numel() / (k * n));
    let idx = lhs_indices.or(rhs_indices).expect("gather_mm: at least one index array");
    let mut shape = idx.shape.clone();
    shape.extend_from_slice(&[m, n]);
    let out = DeviceBuf::new_in(alloc, a.dtype, &shape);
    guarded(|| unsafe {
        sys::b200_gather_mm(ctx.raw, a.ptr, b.ptr, opt(lhs_indices), opt(rhs_indices), ba, bb, m, k, n, idx.numel(), out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `softmax_axis(a, -1, precise)`.
#[track_caller]
pub fn softmax_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, a: &DeviceBuf<'_>, precise: impl Into<Option<bool>>,
                               stream: Stream) -> Result<DeviceBuf<'a>> {
    let cols = a.dim(-1);
    let out = DeviceBuf::new_in(alloc, a.dtype, &a.shape);
    guarded(|| unsafe {
        sys::b200_softmax_axis(ctx.raw, a.ptr, a.numel() / cols, cols, precise.into().unwrap_or(false) as i32, out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `argpartition_axis(a, kth, -1)`.
#[track_caller]
pub fn argpartition_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, a: &DeviceBuf<'_>, kth: i32, stream: Stream) -> Result<DeviceBuf<'a>> {
    let cols = a.dim(-1);
    let out = DeviceBuf::new_in(alloc, DType::Uint32, &a.shape);
    guarded(|| unsafe { sys::b200_argpartition_axis(ctx.raw, a.ptr, a.numel() / cols, cols, kth, out.ptr as *mut u32, stream.0) })?;
    Ok(out)
}

/// `argsort_axis(keys, -1)` for small unsigned keys (stable).
#[track_caller]
pub fn argsort_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, keys: &DeviceBuf<'_>, key_bound: i32, stream: Stream) -> Result<DeviceBuf<'a>> {
    let cols = keys.dim(-1);
    let out = DeviceBuf::new_in(alloc, DType::Uint32, &keys.shape);
    guarded(|| unsafe {
        sys::b200_argsort_axis(ctx.raw, keys.ptr as *const u32, keys.numel() / cols.max(1), cols, key_bound, out.ptr as *mut u32, stream.0)
    })?;
    Ok(out)
}

/// `take_along_axis(a, indices, -1)`.
#[track_caller]
pub fn take_along_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, a: &DeviceBuf<'_>, indices: &DeviceBuf<'_>, stream: Stream) -> Result<DeviceBuf<'a>> {
    let (cols, icols) = (a.dim(-1), indices.dim(-1));
    let out = DeviceBuf::new_in(alloc, a.dtype, &indices.shape);
    guarded(|| unsafe {
        sys::b200_take_along_axis(ctx.raw, a.ptr, a.numel() / cols, cols, indices.ptr as *const u32, icols, out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `take_axis(x, indices, 0)`.
#[track_caller]
pub fn take_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, x: &DeviceBuf<'_>, indices: &DeviceBuf<'_>, stream: Stream) -> Result<DeviceBuf<'a>> {
    let out = DeviceBuf::new_in(alloc, x.dtype, &[indices.numel(), x.dim(1)]);
    guarded(|| unsafe {
        sys::b200_take_axis(ctx.raw, x.ptr, indices.ptr as *const u32, indices.numel(), x.dim(0), x.dim(1), out.ptr, stream.0)
    })?;
    Ok(out)
}

/// `topk_axis(a, k, -1)`.
#[track_caller]
pub fn topk_axis_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, a: &DeviceBuf<'_>, k: i32, stream: Stream) -> Result<DeviceBuf<'a>> {
    let cols = a.dim(-1);
    let mut shape = a.shape.clone();
    *shape.last_mut().unwrap() = k as i64;
    let out = DeviceBuf::new_in(alloc, a.dtype, &shape);
    guarded(|| unsafe { sys::b200_topk_axis(ctx.raw, a.ptr, a.numel() / cols, cols, k, out.ptr, stream.0) })?;
    Ok(out)
}

/// `fast::rms_norm(x, weight, eps)`.
#[track_caller]
pub fn rms_norm_device<'a>(ctx: &Context, alloc: &'a dyn DeviceAllocator, x: &DeviceBuf<'_>, weight: Option<&DeviceBuf<'_>>, eps: f32,
                           stream: Stream) -> Result<DeviceBuf<'a>> {
    let cols = x.dim(-1);
    let out = DeviceBuf::new_in(alloc, x.dtype, &x.shape);
    let w = weight.map_or(std::ptr::null(), |t| t.ptr as *const std::os::raw::c_void);
    guarded(|| unsafe { sys::b200_rms_norm(ctx.raw, x.ptr, w, eps, x.numel() / cols, cols, out.ptr, stream.0) })?;
    Ok(out)
}
