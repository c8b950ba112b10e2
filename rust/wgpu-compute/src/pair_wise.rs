//! `+ - * /` and `pow` between tensors of one shape and type, owned or by reference (original:
//! `src/pair_wise.rs:205-528`).  The two operands' graphs are merged by the library on first contact.
use crate::tensor::{DataType, Tensor};
use std::ops::{Add, Div, Mul, Sub};
use wgf_sys as sys;

impl<const R: usize, T: DataType> Tensor<R, T> {
    pub(crate) fn binary(&self, other: &Self, opcode: u32) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_binary(self.raw, other.raw, opcode, out) })
    }

    pub fn pow(&self, other: &Self) -> Self {
        self.binary(other, sys::WGF_OP_POW)
    }
}

macro_rules! pair_operator {
    ($trait:ident, $method:ident, $opcode:ident) => {
        impl<const R: usize, T: DataType> $trait<Tensor<R, T>> for Tensor<R, T> {
            type Output = Tensor<R, T>;

            fn $method(self, rhs: Tensor<R, T>) -> Self::Output {
                self.binary(&rhs, sys::$opcode)
            }
        }

        impl<const R: usize, T: DataType> $trait<&Tensor<R, T>> for &Tensor<R, T> {
            type Output = Tensor<R, T>;

            fn $method(self, rhs: &Tensor<R, T>) -> Self::Output {
                self.binary(rhs, sys::$opcode)
            }
        }
    };
}

pair_operator!(Add, add, WGF_OP_ADD);
pair_operator!(Sub, sub, WGF_OP_SUB);
pair_operator!(Mul, mul, WGF_OP_MUL);
pair_operator!(Div, div, WGF_OP_DIV);
