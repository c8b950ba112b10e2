//! `Layout` (original: `src/layout.rs:33-94`): offset, shape and strides in elements.  On this
//! backend layouts live inside the library; this type describes a materialised tensor
//! (`Tensor::layout`) and keeps the original's constructors and accessors.
use std::ops::Range;

#[derive(Clone, Debug, PartialEq, Eq)]
pub struct Layout {
    offset: usize,
    shape: Box<[usize]>,
    strides: Box<[usize]>,
}

impl Layout {
    pub fn contiguous(shape: &[usize]) -> Self {
        let mut strides = vec![0usize; shape.len()];
        let mut run = 1usize;
        for axis in (0..shape.len()).rev() {
            strides[axis] = run;
            run *= shape[axis];
        }
        Layout { offset: 0, shape: shape.into(), strides: strides.into() }
    }

    pub fn from_parts(offset: usize, shape: Box<[usize]>, strides: Box<[usize]>) -> Self {
        Layout { offset, shape, strides }
    }

    /// Row-major with no gaps AND offset 0, as in the original (`src/layout.rs:58-60`).
    pub fn is_contiguous(&self) -> bool {
        self.offset == 0 && *self == Layout::contiguous(&self.shape)
    }

    pub fn slice(&self, slices: &[Range<usize>]) -> Self {
        let offset = self.offset + slices.iter().zip(self.strides.iter()).map(|(r, s)| r.start * s).sum::<usize>();
        let shape = slices.iter().map(|r| r.end - r.start).collect();
        Layout { offset, shape, strides: self.strides.clone() }
    }

    pub fn rank(&self) -> usize {
        self.shape.len()
    }

    pub fn shape(&self) -> &[usize] {
        &self.shape
    }

    pub fn strides(&self) -> &[usize] {
        &self.strides
    }

    pub fn offset(&self) -> usize {
        self.offset
    }
}
