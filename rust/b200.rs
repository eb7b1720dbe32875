//! Glue between hanzo-quant's `QuantMethod` layers and libhanzoquant_b200, in the style of
//! hanzo-quant/src/gguf/fast_mmvq.rs and gguf/cuda.rs.  NOT COMPILED in this repository (no Rust toolchain in
//! the build image; `hanzo-ml` is not vendored): the types named here (`Tensor`, `CudaStorage`, `QTensor`,
//! `slice_ptr`) are the reference's (hanzo-quant/src/utils/mod.rs:43-72, gguf/cuda.rs:436-491).
//!
//! What changes for a maintainer: `GgufMatMul::forward_raw` / `gather_forward_raw` (hanzo-quant/src/gguf/mod.rs:156-230),
//! `BlockwiseFP8Linear::{forward_raw, gather_forward_raw}` (blockwise_fp8/mod.rs:72-198) and
//! `MXFP4Layer::{forward_raw, gather_forward_raw}` (mxfp4/mod.rs:89-174) call `linear` / `gather` below on CUDA
//! devices of compute capability 10.0 instead of their own launch wrappers; nothing above the trait changes.
use crate::b200::ffi::*; // rust/ffi.rs
use hanzo_ml::{cuda_backend::CudaStorage, DType, Result, Shape, Storage, Tensor};
use std::ffi::c_void;

fn dt_code(dt: DType) -> Result<i32> {
    Ok(match dt {
        DType::F32 => HQ_DT_F32,
        DType::F16 => HQ_DT_F16,
        DType::BF16 => HQ_DT_BF16,
        other => hanzo_ml::bail!("hanzoquant_b200: unsupported activation dtype {other:?}"),
    })
}

/// The library's format code of a GGML weight type, `None` for types it does not run: the list of
/// `fast_mmvq::supports` (hanzo-quant/src/gguf/fast_mmvq.rs:36-50), served for any row count.
pub fn gguf_format(dtype: hanzo_ml::quantized::GgmlDType) -> Option<i32> {
    use hanzo_ml::quantized::GgmlDType as G;
    Some(match dtype {
        G::Q8_0 => HQ_FMT_Q8_0,
        G::Q4_0 => HQ_FMT_Q4_0,
        G::Q4_1 => HQ_FMT_Q4_1,
        G::Q5_0 => HQ_FMT_Q5_0,
        G::Q5_1 => HQ_FMT_Q5_1,
        G::Q2K => HQ_FMT_Q2_K,
        G::Q3K => HQ_FMT_Q3_K,
        G::Q4K => HQ_FMT_Q4_K,
        G::Q5K => HQ_FMT_Q5_K,
        G::Q6K => HQ_FMT_Q6_K,
        _ => return None,
    })
}

fn check(rc: i32, what: &str) -> Result<()> {
    if rc == HQ_OK {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(hq_error_string(rc)) }.to_string_lossy();
    hanzo_ml::bail!("hanzoquant_b200: {what}: {msg} ({rc})")
}

/// A quantized matrix or expert bank that already lives on the device in the reference's own byte layout
/// (GGUF blocks: `QTensor::device_ptr()`; FP8: weight + `weight_scale_inv`; MXFP4: blocks + scales).
pub struct B200Weight {
    pub desc: hq_weight,
    /// keeps the device buffers alive for as long as `desc` points into them
    pub _owners: Vec<Tensor>,
}
unsafe impl Send for B200Weight {}
unsafe impl Sync for B200Weight {}

/// y = x . W^T (+ b) for any leading dims of `x` (QuantMethod::forward_raw).
pub fn linear(w: &B200Weight, x: &Tensor, out_dtype: DType) -> Result<Tensor> {
    let k = w.desc.k as usize;
    let dims = x.dims().to_vec();
    if *dims.last().unwrap() != k {
        hanzo_ml::bail!("shape mismatch: input has {} features, weight expects {k}", dims.last().unwrap());
    }
    let m: usize = dims[..dims.len() - 1].iter().product();
    let x = x.contiguous()?;
    let (x_storage, x_layout) = x.storage_and_layout();
    let Storage::Cuda(xs) = &*x_storage else { hanzo_ml::bail!("hanzoquant_b200 has no CPU path") };
    let dev = xs.device().clone();
    let stream = dev.cuda_stream();
    // raw pointer + guard that orders the access on the stream (hanzo-quant/src/utils/mod.rs:43-72)
    let (x_ptr, _x_guard) = crate::utils::slice_ptr_dyn(xs, x_layout.start_offset(), &stream)?;
    let n = w.desc.n as usize;
    let out = unsafe { dev.alloc_dyn(out_dtype, m * n)? };
    let (y_ptr, _y_guard) = crate::utils::slice_ptr_mut_dyn(&out, 0, &stream)?;
    check(
        unsafe {
            hq_linear_forward_ws(
                &w.desc, x_ptr as *const c_void, dt_code(x.dtype())?, k as i64, y_ptr as *mut c_void,
                dt_code(out_dtype)?, n as i64, m as i64, std::ptr::null_mut(), 0, std::ptr::null_mut(),
                stream.cu_stream() as *mut c_void,
            )
        },
        "hq_linear_forward_ws",
    )?;
    let mut out_dims = dims;
    *out_dims.last_mut().unwrap() = n;
    Ok(Tensor::from((Storage::Cuda(CudaStorage::wrap_dyn(out, dev)), Shape::from_dims(&out_dims))))
}

/// out[t, s, :] = W[ids[t, s]] . x_row (QuantMethod::gather_forward_raw): x is [T, K] / [T, 1, K] (one row per token)
/// or [T, k, K] (one row per slot), ids u32 [T, k]; returns [T, k, N].
pub fn gather(w: &B200Weight, x: &Tensor, ids: &Tensor, per_slot: bool, out_dtype: DType) -> Result<Tensor> {
    let (t, top_k) = ids.dims2()?;
    let e = w.desc.n_experts;
    let x = x.contiguous()?;
    let ids = ids.contiguous()?;
    let (x_storage, x_layout) = x.storage_and_layout();
    let (i_storage, i_layout) = ids.storage_and_layout();
    let (Storage::Cuda(xs), Storage::Cuda(is)) = (&*x_storage, &*i_storage) else {
        hanzo_ml::bail!("hanzoquant_b200 has no CPU path")
    };
    let dev = xs.device().clone();
    let stream = dev.cuda_stream();
    let raw = stream.cu_stream() as *mut c_void;
    let (x_ptr, _g0) = crate::utils::slice_ptr_dyn(xs, x_layout.start_offset(), &stream)?;
    let (i_ptr, _g1) = crate::utils::slice_ptr_dyn(is, i_layout.start_offset(), &stream)?;
    // dispatch tables + workspace: per-device scratch grown on demand, as the reference keeps its Q8_1 and
    // dispatch scratch (hanzo-quant/src/gguf/cuda.rs:21-132)
    let ws_bytes = unsafe { hq_moe_dispatch_workspace_bytes(t as i64, top_k as i32, e) };
    let mut scratch = crate::b200::scratch::ensure(&dev, (e as usize + 1 + 3 * t * top_k) * 4 + ws_bytes as usize)?;
    let (bounds, sorted_assign, sorted_token, inv_perm, ws) = scratch.carve(e as usize, t * top_k);
    check(
        unsafe {
            hq_moe_dispatch_build(i_ptr as *const u32, t as i64, top_k as i32, e, bounds, sorted_assign,
                                  sorted_token, inv_perm, ws, ws_bytes, raw)
        },
        "hq_moe_dispatch_build",
    )?;
    let n = w.desc.n as usize;
    let out = unsafe { dev.alloc_dyn(out_dtype, t * top_k * n)? };
    let (y_ptr, _g2) = crate::utils::slice_ptr_mut_dyn(&out, 0, &stream)?;
    check(
        unsafe {
            hq_moe_gather_forward(
                &w.desc, std::ptr::null(), std::ptr::null(), x_ptr as *const c_void, dt_code(x.dtype())?,
                if per_slot { HQ_ROWS_PER_SLOT } else { HQ_ROWS_PER_TOKEN }, t as i64, top_k as i32, bounds,
                sorted_assign, sorted_token, ws, y_ptr as *mut c_void, dt_code(out_dtype)?, HQ_ROWS_PER_SLOT,
                std::ptr::null_mut(), raw,
            )
        },
        "hq_moe_gather_forward",
    )?;
    Ok(Tensor::from((Storage::Cuda(CudaStorage::wrap_dyn(out, dev)), Shape::from_dims(&[t, top_k, n]))))
}
