//! `slice_assign` (original: `src/slice_assign.rs:76-79`).  The original writes into the target's
//! buffer whoever else still holds it; the library copies first unless nothing can see the target.
use crate::tensor::{DataType, Tensor};
use std::ops::Range;

impl<const R: usize, T: DataType> Tensor<R, T> {
    pub fn slice_assign(&self, slices: [Range<usize>; R], value: &Self) -> Self {
        let starts: [i64; R] = std::array::from_fn(|i| slices[i].start as i64);
        let ends: [i64; R] = std::array::from_fn(|i| slices[i].end as i64);
        self.build(|out| unsafe {
            wgf_sys::wgf_tensor_slice_assign(self.raw, starts.as_ptr(), ends.as_ptr(), value.raw, out)
        })
    }
}
