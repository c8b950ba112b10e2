//! The `wgpu-compute` API over the B200 (sm_100a) backend.
//!
//! Module layout follows the original crate (`src/lib.rs:1-27` there): the same names are exported
//! from the same places, so `use wgpu_compute::*;` brings the same items into scope.  Each module
//! states which file of the original it stands in for.
//!
//! Written without a Rust toolchain at hand: see README.md.

pub use composite::*;
pub use device::*;
pub use element_wise::CastTensor;
pub use error::*;
pub use extras::*;
pub use layout::*;
pub use query::*;
pub use reduce::*;
pub use tensor::*;

mod composite;
mod device;
mod element_wise;
mod error;
mod extras;
mod layout;
mod map_layout;
mod matmul;
mod pair_wise;
mod query;
mod reduce;
mod resize;
mod slice_assign;
mod tensor;

/// Stand-in for the two `wgpu` names that user code of the original crate spells out: the argument
/// of the poll loop and the error type of `as_slice`.  Code that says `wgpu::PollType::Wait` after
/// `use wgpu_compute::*;` resolves to this module when it has no `wgpu` dependency of its own.
pub mod wgpu {
    /// `wgpu::PollType`: ignored, CUDA streams make progress on their own.
    #[derive(Clone, Copy, Debug, PartialEq, Eq)]
    pub enum PollType {
        Wait,
        Poll,
    }
    pub type BufferAsyncError = crate::Error;
    pub type RequestDeviceError = crate::Error;
}
