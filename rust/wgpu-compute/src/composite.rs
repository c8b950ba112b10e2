//! Composites (original: `src/composite/*.rs`).  In the original each is a recipe of primitive
//! ops; here each is one call into the library, whose resolver sees the same recipe and fuses it
//! (rms-norm runs as one single-pass row kernel, rope as one kernel).
use crate::element_wise::CastTensor;
use crate::tensor::{DataType, Tensor};
use crate::Device;
use std::ptr;
use wgf_sys as sys;

// ---- arange (original: `src/composite/arange.rs:3-23`) -----------------------------------------
impl<D: DataType> Tensor<1, D> {
    pub fn arange(device: &Device, start: D, end: D) -> Self {
        Self::arange_step(device, start, end, D::one())
    }

    /// Values start, start + step, ... below (above, for a negative step) `end`, accumulated in the
    /// element type on the host like the original's loop, then uploaded.
    pub fn arange_step(device: &Device, start: D, end: D, step: D) -> Self {
        let mut values = Vec::new();
        let mut at = start;
        let upwards = step >= D::zero();
        while (upwards && at < end) || (!upwards && at > end) {
            values.push(at);
            at += step;
        }
        let n = values.len();
        Tensor::from_vec(device, values, [n])
    }
}

// ---- cat (original: `src/composite/cat.rs:3-40`) -------------------------------------------------
impl<const R: usize, D: DataType> Tensor<R, D> {
    pub fn cat(vectors: impl IntoIterator<Item = Self>, dim: usize) -> Self {
        let parts: Vec<Self> = vectors.into_iter().collect();
        assert!(!parts.is_empty(), "cat of nothing");
        let handles: Vec<*mut sys::wgf_tensor> = parts.iter().map(|p| p.raw).collect();
        let mut raw = ptr::null_mut();
        crate::error::expect(unsafe {
            sys::wgf_tensor_cat(handles.as_ptr(), handles.len() as u32, dim as u32, &mut raw)
        });
        Tensor::from_raw(raw, &parts[0].device)
    }

    // ---- narrow (original: `src/composite/narrow.rs:3-15`) ----------------------------------------
    pub fn narrow(&self, axis: usize, start: usize, length: usize) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_narrow(self.raw, axis as u32, start as i64, length as i64, out) })
    }

    // ---- silu (original: `src/composite/silu.rs:3-7`): x / (1 + exp(-x)) --------------------------
    pub fn silu(&self) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_silu(self.raw, out) })
    }
}

// ---- rms-norm (original: `src/composite/rms_norm.rs:3-15`, where it is called layer_norm) --------
impl<T> Tensor<2, T>
where
    T: DataType + CastTensor<f32>,
    f32: CastTensor<T>,
{
    /// x / sqrt(mean(x^2 over the last axis) + eps) * weight, computed in f32 and rounded once.
    pub fn layer_norm(self, weight: Tensor<1, T>, eps: f32) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_layer_norm(self.raw, weight.raw, eps, out) })
    }
}

// ---- softmax (original: `src/composite/softmax.rs:3-10`): rank 1, exp(x) / sum(exp(x)) ------------
impl<D: DataType> Tensor<1, D> {
    pub fn softmax(&self) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_softmax(self.raw, out) })
    }
}

// ---- rope (original: `src/composite/rope.rs:12-22`) -----------------------------------------------
impl<D: DataType> Tensor<3, D> {
    /// Rotary embedding of [heads, seq, embed] with cos / sin [>= seq, embed / 2] (rotate-half form).
    pub fn rope(self, cos: Tensor<2, D>, sin: Tensor<2, D>) -> Tensor<3, D> {
        self.build(|out| unsafe { sys::wgf_tensor_rope(self.raw, cos.raw, sin.raw, out) })
    }
}

// ---- unsqueeze (original: `src/composite/unsqueeze.rs:16-53`) -------------------------------------
pub trait Unsqueeze {
    type Output;

    fn unsqueeze(&self, axis: usize) -> Self::Output;
}

macro_rules! unsqueeze_for_rank {
    ($($rank:literal),*) => {$(
        impl<D: DataType> Unsqueeze for Tensor<$rank, D> {
            type Output = Tensor<{ $rank + 1 }, D>;

            fn unsqueeze(&self, axis: usize) -> Self::Output {
                self.build(|out| unsafe { sys::wgf_tensor_unsqueeze(self.raw, axis as u32, out) })
            }
        }
    )*};
}

// the library's largest rank is 8 (the original goes on to 20)
unsqueeze_for_rank!(1, 2, 3, 4, 5, 6, 7);
