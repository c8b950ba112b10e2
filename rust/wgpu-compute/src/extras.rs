//! What the B200 backend offers beyond the original crate's API.  Nothing here is needed to run
//! existing user code; all of it maps one-to-one on entry points of `include/wgf.h`.
use crate::error::{check, expect, Error};
use crate::tensor::{DataType, Tensor};
use crate::Device;
use std::ptr;
use wgf_sys as sys;

impl<const R: usize, D: DataType> Tensor<R, D> {
    /// Max-subtracted softmax over the last axis, any rank: one single-pass row kernel.
    pub fn softmax_last_dim(&self) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_softmax_last_dim(self.raw, out) })
    }

    /// All-reduce of this tensor over the communicator's GPUs (`op` = the reduction that combines
    /// the ranks' values).  A whole-tensor reduction below it is exchanged over peer memory.
    pub fn all_reduce(&self, comm: &Comm, op: AllReduceOp) -> Self {
        self.build(|out| unsafe { sys::wgf_tensor_all_reduce(self.raw, comm.raw, op as u32, out) })
    }
}

/// How `all_reduce` combines the ranks.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
#[repr(u32)]
pub enum AllReduceOp {
    Sum = sys::WGF_OP_SUM,
    Max = sys::WGF_OP_MAX,
    Min = sys::WGF_OP_MIN,
    Product = sys::WGF_OP_PRODUCT,
}

/// Several tensors resolved as ONE request (`wgf_tensor_materialize_many`): a reduction of a whole
/// tensor to a scalar among them rides along in the row kernel of another one over the same index
/// space, so its input is read once.  Each argument is any `Tensor`; ranks and types may differ.
#[macro_export]
macro_rules! materialize_many {
    ($($tensor:expr),+ $(,)?) => {{
        let handles = [$($crate::raw_handle(&$tensor)),+];
        $crate::materialize_handles(&handles)
    }};
}

#[doc(hidden)]
pub fn raw_handle<const R: usize, D>(t: &Tensor<R, D>) -> *mut sys::wgf_tensor {
    t.raw
}

#[doc(hidden)]
pub fn materialize_handles(handles: &[*mut sys::wgf_tensor]) -> Result<(), Error> {
    check(unsafe { sys::wgf_tensor_materialize_many(handles.as_ptr(), handles.len() as u32) })
}

impl<D: DataType> Tensor<3, D> {
    /// softmax(scale * q k^T [+ mask]) v for [batch * heads, seq, head_dim] tensors.  16-bit elements,
    /// head_dim 128 and equal sequence lengths that are multiples of 128 run as one fused
    /// tensor-core kernel that keeps the scores in tensor memory; other shapes, and any explicit
    /// mask, run as mat_mul, softmax_last_dim, mat_mul.
    pub fn attention(&self, k: &Self, v: &Self, mask: Option<&Tensor<2, D>>, causal: bool, scale: f32) -> Self {
        let mask = mask.map_or(ptr::null_mut(), |m| m.raw);
        self.build(|out| unsafe {
            sys::wgf_tensor_attention(self.raw, k.raw, v.raw, mask, causal as i32, scale, out)
        })
    }

    /// Llama-style decoder block forward on [batch, seq, hidden]; see `wgf_tensor_llama_block`.
    /// `weights` = [Wq, Wk, Wv, Wo, Wg, Wu, Wd], each stored [out_features, in_features];
    /// `mask` = additive [seq, seq], or `None` for causal attention through the fused kernel.
    #[allow(clippy::too_many_arguments)]
    pub fn llama_block(
        &self,
        weights: &[Tensor<2, D>; 7],
        norm1: &Tensor<1, D>,
        norm2: &Tensor<1, D>,
        cos: &Tensor<2, D>,
        sin: &Tensor<2, D>,
        mask: Option<&Tensor<2, D>>,
        n_heads: usize,
        eps: f32,
    ) -> Self {
        let handles: [*mut sys::wgf_tensor; 7] = std::array::from_fn(|i| weights[i].raw);
        let mask = mask.map_or(ptr::null_mut(), |m| m.raw);
        self.build(|out| unsafe {
            sys::wgf_tensor_llama_block(
                self.raw,
                handles.as_ptr(),
                norm1.raw,
                norm2.raw,
                cos.raw,
                sin.raw,
                mask,
                n_heads as u32,
                eps,
                out,
            )
        })
    }
}

/// One rank of a multi-GPU job (one process or thread per GPU); wraps NCCL plus the peer-memory
/// mailboxes used for scalar all-reduces.
pub struct Comm {
    pub(crate) raw: *mut sys::wgf_comm,
}

impl Comm {
    /// Made on rank 0 and handed to the other ranks by the launcher.
    pub fn unique_id() -> Result<[u8; sys::WGF_COMM_ID_BYTES], Error> {
        let mut id = [0u8; sys::WGF_COMM_ID_BYTES];
        check(unsafe { sys::wgf_comm_unique_id(id.as_mut_ptr()) })?;
        Ok(id)
    }

    pub fn new(device: &Device, world: usize, rank: usize, id: &[u8; sys::WGF_COMM_ID_BYTES]) -> Result<Self, Error> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::wgf_comm_create(device.raw, world as i32, rank as i32, id.as_ptr(), &mut raw) })?;
        Ok(Comm { raw })
    }
}

impl Drop for Comm {
    fn drop(&mut self) {
        unsafe { sys::wgf_comm_release(self.raw) };
    }
}

/// Contiguous block partition of `n_units` over `world` ranks; the first `n_units % world` ranks
/// get one unit more.
pub fn shard_range(n_units: usize, world: usize, rank: usize) -> std::ops::Range<usize> {
    let (mut begin, mut end) = (0i64, 0i64);
    expect(unsafe { sys::wgf_shard_range(n_units as i64, world as i32, rank as i32, &mut begin, &mut end) });
    begin as usize..end as usize
}

/// The kernels of one or more materialisations, recorded once as a CUDA graph and replayed with one
/// call (`wgf_schedule_*`).  Inputs are tensors made before `record`; refill them between launches.
pub struct Schedule {
    raw: *mut sys::wgf_schedule,
}

impl Schedule {
    /// Records everything `body` materialises on `device`.
    pub fn record(device: &Device, body: impl FnOnce() -> Result<(), Error>) -> Result<Self, Error> {
        check(unsafe { sys::wgf_schedule_begin(device.raw) })?;
        let outcome = body();
        let mut raw = ptr::null_mut();
        let ended = check(unsafe { sys::wgf_schedule_end(device.raw, &mut raw) });
        outcome?;
        ended?;
        Ok(Schedule { raw })
    }

    /// Queues one replay on the device's stream; does not wait.
    pub fn launch(&self) -> Result<(), Error> {
        check(unsafe { sys::wgf_schedule_launch(self.raw) })
    }

    pub fn kernel_count(&self) -> u64 {
        let mut n = 0u64;
        unsafe { sys::wgf_schedule_kernel_count(self.raw, &mut n) };
        n
    }
}

impl Drop for Schedule {
    fn drop(&mut self) {
        if !self.raw.is_null() {
            unsafe { sys::wgf_schedule_destroy(self.raw) };
        }
    }
}

impl<const R: usize, D: DataType> Tensor<R, D> {
    /// New contents for a materialised, contiguous tensor, written into the buffer it already has:
    /// how the inputs of a recorded `Schedule` are fed.
    pub fn write(&self, data: &[D]) -> Result<(), Error> {
        let layout = self.layout()?;
        assert_eq!(
            layout.strides(),
            crate::Layout::contiguous(layout.shape()).strides(),
            "write needs a contiguous tensor"
        );
        assert_eq!(data.len(), self.shape().iter().product::<usize>(), "element count does not match the shape");
        let mut desc = std::mem::MaybeUninit::<sys::wgf_tensor_desc>::zeroed();
        check(unsafe { sys::wgf_tensor_desc_of(self.raw, desc.as_mut_ptr()) })?;
        let desc = unsafe { desc.assume_init() };
        let size = std::mem::size_of::<D>() as u64;
        let status = unsafe {
            sys::wgf_buffer_upload(
                desc.buf,
                desc.offset as u64 * size,
                data.as_ptr() as *const core::ffi::c_void,
                data.len() as u64 * size,
            )
        };
        unsafe { sys::wgf_buffer_release(desc.buf) };
        check(status)
    }
}
