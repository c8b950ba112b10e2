//! Views that never copy: `slice`, `transpose`, `broadcast` (original: `src/map_layout.rs:41-98`).
use crate::tensor::{DataType, Tensor};
use std::ops::Range;
use wgf_sys as sys;

pub(crate) fn dims<const N: usize>(values: [usize; N]) -> [i64; N] {
    values.map(|v| v as i64)
}

impl<const R: usize, T: DataType> Tensor<R, T> {
    pub fn slice(&self, slices: [Range<usize>; R]) -> Tensor<R, T> {
        let starts: [i64; R] = std::array::from_fn(|i| slices[i].start as i64);
        let ends: [i64; R] = std::array::from_fn(|i| slices[i].end as i64);
        self.build(|out| unsafe { sys::wgf_tensor_slice(self.raw, starts.as_ptr(), ends.as_ptr(), out) })
    }

    pub fn transpose(&self, first_axis: usize, second_axis: usize) -> Tensor<R, T> {
        self.build(|out| unsafe { sys::wgf_tensor_transpose(self.raw, first_axis as u32, second_axis as u32, out) })
    }

    /// Adds ONE stride-0 axis where the common prefix of the two shapes ends
    /// (original: `src/map_layout.rs:69-98`).  `broadcast_axis` names the position instead.
    pub fn broadcast<const R2: usize>(&self, out_shape: [usize; R2]) -> Tensor<R2, T> {
        let shape = dims(out_shape);
        self.build(|out| unsafe { sys::wgf_tensor_broadcast(self.raw, R2 as u32, shape.as_ptr(), out) })
    }

    /// `broadcast` with the new axis' position stated (no counterpart in the original).
    pub fn broadcast_axis<const R2: usize>(&self, axis: usize, size: usize) -> Tensor<R2, T> {
        assert_eq!(R2, R + 1, "broadcast_axis adds exactly one axis");
        self.build(|out| unsafe { sys::wgf_tensor_broadcast_axis(self.raw, axis as u32, size as i64, out) })
    }

    /// Stretches axes of extent 1 to `out_shape` with stride 0 (no counterpart in the original).
    pub fn expand(&self, out_shape: [usize; R]) -> Tensor<R, T> {
        let shape = dims(out_shape);
        self.build(|out| unsafe { sys::wgf_tensor_expand(self.raw, shape.as_ptr(), out) })
    }
}
