//! `sum`, `max`, `min`, `product` over one axis, rank R -> R - 1 (original: `src/reduce.rs:433-815`).
//! Implemented for ranks 1..=8, the library's largest rank (the original goes to 20).
use crate::tensor::{DataType, Tensor};
use wgf_sys as sys;

/// The original exports this type with a private constructor (`src/reduce.rs:390-419`): user code can
/// name it but not build one.  Kept for that; it names one of the four reductions.
#[derive(Clone, Debug, PartialEq, Eq)]
pub struct ReduceFunction {
    name: Option<String>,
    builtin: &'static str,
    pub(crate) opcode: u32,
}

impl ReduceFunction {
    const fn builtin(builtin: &'static str, opcode: u32) -> Self {
        ReduceFunction { name: None, builtin, opcode }
    }

    /// The name given with `with_name`, else the reduction's own (the original answers "reduce" for
    /// an unnamed function, `src/reduce.rs:407-409`; here the four reductions are told apart).
    pub fn name(&self) -> &str {
        self.name.as_deref().unwrap_or(self.builtin)
    }

    /// A label for traces and timing records (`src/reduce.rs:411-414`); the arithmetic is unchanged.
    pub fn with_name(mut self, name: impl ToString) -> Self {
        self.name = Some(name.to_string());
        self
    }
}

pub(crate) const SUM: ReduceFunction = ReduceFunction::builtin("sum", sys::WGF_OP_SUM);
pub(crate) const MAX: ReduceFunction = ReduceFunction::builtin("max", sys::WGF_OP_MAX);
pub(crate) const MIN: ReduceFunction = ReduceFunction::builtin("min", sys::WGF_OP_MIN);
pub(crate) const PRODUCT: ReduceFunction = ReduceFunction::builtin("product", sys::WGF_OP_PRODUCT);

impl<const R: usize, D: DataType> Tensor<R, D> {
    pub(crate) fn reduce<const OUT: usize>(&self, function: &ReduceFunction, dim: usize) -> Tensor<OUT, D> {
        self.build(|out| unsafe { sys::wgf_tensor_reduce(self.raw, function.opcode, dim as u32, out) })
    }
}

pub trait Sum {
    type Output;

    fn sum(&self, dim: usize) -> Self::Output;
}

pub trait Max {
    type Output;

    fn max(&self, dim: usize) -> Self::Output;
}

pub trait Min {
    type Output;

    fn min(&self, dim: usize) -> Self::Output;
}

pub trait Product {
    type Output;

    fn product(&self, dim: usize) -> Self::Output;
}

macro_rules! reductions_for_rank {
    ($($rank:literal),*) => {$(
        impl<D: DataType> Sum for Tensor<$rank, D> {
            type Output = Tensor<{ $rank - 1 }, D>;

            fn sum(&self, dim: usize) -> Self::Output {
                self.reduce(&SUM, dim)
            }
        }

        impl<D: DataType> Max for Tensor<$rank, D> {
            type Output = Tensor<{ $rank - 1 }, D>;

            fn max(&self, dim: usize) -> Self::Output {
                self.reduce(&MAX, dim)
            }
        }

        impl<D: DataType> Min for Tensor<$rank, D> {
            type Output = Tensor<{ $rank - 1 }, D>;

            fn min(&self, dim: usize) -> Self::Output {
                self.reduce(&MIN, dim)
            }
        }

        impl<D: DataType> Product for Tensor<$rank, D> {
            type Output = Tensor<{ $rank - 1 }, D>;

            fn product(&self, dim: usize) -> Self::Output {
                self.reduce(&PRODUCT, dim)
            }
        }
    )*};
}

reductions_for_rank!(1, 2, 3, 4, 5, 6, 7, 8);
