//! Unary math, scalar operators and casts (original: `src/element_wise.rs:197-1471`).  Each call adds
//! one element-wise node; the resolver folds chains of them, and the pair-wise and reduce nodes they
//! feed, into one kernel.
use crate::tensor::{DataType, Tensor};
use std::ops::{Add, Div, Mul, Neg, Sub};
use wgf_sys as sys;

impl<const R: usize, D: DataType> Tensor<R, D> {
    pub(crate) fn unary(&self, opcode: u32) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_unary(self.raw, opcode, out) })
    }

    pub(crate) fn scalar(&self, opcode: u32, c: f32) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_scalar(self.raw, opcode, c, out) })
    }
}

// tensor (op) f32 and f32 (op) tensor; the scalar is always an f32, converted to the element type
// inside the kernel (original: `src/element_wise.rs:197-651`)
macro_rules! scalar_operator {
    ($trait:ident, $method:ident, $tensor_first:expr, $scalar_first:expr) => {
        impl<const R: usize, T: DataType> $trait<f32> for Tensor<R, T> {
            type Output = Tensor<R, T>;

            fn $method(self, rhs: f32) -> Self::Output {
                self.scalar($tensor_first, rhs)
            }
        }

        impl<const R: usize, T: DataType> $trait<Tensor<R, T>> for f32 {
            type Output = Tensor<R, T>;

            fn $method(self, rhs: Tensor<R, T>) -> Self::Output {
                rhs.scalar($scalar_first, self)
            }
        }
    };
}

scalar_operator!(Add, add, sys::WGF_OP_ADD_C, sys::WGF_OP_ADD_C);
scalar_operator!(Sub, sub, sys::WGF_OP_SUB_C, sys::WGF_OP_RSUB_C);
scalar_operator!(Mul, mul, sys::WGF_OP_MUL_C, sys::WGF_OP_MUL_C);
scalar_operator!(Div, div, sys::WGF_OP_DIV_C, sys::WGF_OP_RDIV_C);

// the 19 unary functions (original: `src/element_wise.rs:678-1342`)
macro_rules! unary_functions {
    ($($name:ident => $opcode:ident),* $(,)?) => {
        impl<const R: usize, D: DataType> Tensor<R, D> {
            $(
                pub fn $name(&self) -> Self {
                    self.unary(sys::$opcode)
                }
            )*
        }
    };
}

unary_functions!(
    exp => WGF_OP_EXP, exp2 => WGF_OP_EXP2, log => WGF_OP_LOG, log2 => WGF_OP_LOG2, sqr => WGF_OP_SQR,
    sqrt => WGF_OP_SQRT, sin => WGF_OP_SIN, cos => WGF_OP_COS, tan => WGF_OP_TAN, asin => WGF_OP_ASIN,
    acos => WGF_OP_ACOS, atan => WGF_OP_ATAN, sinh => WGF_OP_SINH, cosh => WGF_OP_COSH, tanh => WGF_OP_TANH,
    asinh => WGF_OP_ASINH, acosh => WGF_OP_ACOSH, atanh => WGF_OP_ATANH, abs => WGF_OP_ABS,
);

impl<const R: usize, D: DataType> Neg for Tensor<R, D> {
    type Output = Tensor<R, D>;

    fn neg(self) -> Self {
        self.unary(sys::WGF_OP_NEG)
    }
}

impl<const R: usize, T> Tensor<R, T> {
    /// `tensor.cast::<half::f16>()` (original: `src/element_wise.rs:1408-1415`).
    pub fn cast<T2>(self) -> Tensor<R, T2>
    where
        T: CastTensor<T2>,
    {
        T::cast(self)
    }
}

/// Element types a tensor of `Self` can be converted to (original: `src/element_wise.rs:1417-1471`):
/// the identity, f32 -> f16 (round to nearest even) and f16 -> f32 (exact); bf16 both ways as well.
pub trait CastTensor<T>: Sized {
    /// Casts the tensor to another type
    fn cast<const R: usize>(tensor: Tensor<R, Self>) -> Tensor<R, T>;
}

impl<T> CastTensor<T> for T {
    fn cast<const R: usize>(tensor: Tensor<R, Self>) -> Tensor<R, Self> {
        tensor
    }
}

macro_rules! cast_between {
    ($from:ty, $to:ty) => {
        impl CastTensor<$to> for $from {
            fn cast<const R: usize>(tensor: Tensor<R, Self>) -> Tensor<R, $to> {
                let code = <$to as DataType>::WGSL_TYPE.code();
                tensor.build(|out| unsafe { sys::wgf_tensor_cast(tensor.raw, code, out) })
            }
        }
    };
}

cast_between!(f32, half::f16);
cast_between!(half::f16, f32);
cast_between!(f32, half::bf16);
cast_between!(half::bf16, f32);
