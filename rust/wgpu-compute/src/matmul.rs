//! `mat_mul` (original: `src/matmul.rs:25-29`).  Rank 2, or rank 3 as a batch of matrices (an
//! addition).  16-bit operands run on the tensor cores with fp32 accumulation in tensor memory.
use crate::tensor::{DataType, Tensor};

impl<const R: usize, T: DataType> Tensor<R, T> {
    pub fn mat_mul(&self, other: &Self) -> Self {
        self.build(|out| unsafe { wgf_sys::wgf_tensor_matmul(self.raw, other.raw, out) })
    }
}
