//! `resize` (zero-filled growth or cut) and `reshape` (original: `src/resize.rs:121-144`).
use crate::map_layout::dims;
use crate::tensor::{DataType, Tensor};

impl<const R: usize, T: DataType> Tensor<R, T> {
    pub fn resize(&self, new_shape: [usize; R]) -> Tensor<R, T> {
        let shape = dims(new_shape);
        self.build(|out| unsafe { wgf_sys::wgf_tensor_resize(self.raw, shape.as_ptr(), out) })
    }

    pub fn reshape<const R2: usize>(&self, new_shape: [usize; R2]) -> Tensor<R2, T> {
        let shape = dims(new_shape);
        self.build(|out| unsafe { wgf_sys::wgf_tensor_reshape(self.raw, R2 as u32, shape.as_ptr(), out) })
    }
}
