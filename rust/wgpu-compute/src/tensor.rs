//! `Tensor<R, D>`, `DataType`, `IntoTensor`, `TensorSlice` (original: `src/tensor.rs`).
//!
//! A `Tensor` is a handle on a node of the library's lazy compute graph (`wgf_tensor`).  Building
//! ops only adds nodes; `as_slice().await` resolves the graph -- fusing it into as few kernels as
//! the resolver manages -- runs the kernels and downloads the result.
use crate::error::{check, expect, Error};
use crate::layout::Layout;
use crate::query::QueryResults;
use crate::Device;
use std::fmt::{self, Debug, Display};
use std::marker::PhantomData;
use std::ops::{Add, AddAssign, Div, DivAssign, Index, Mul, MulAssign, Sub, SubAssign};
use std::ptr;

/// Element types a tensor can hold (original: `src/tensor.rs:22-65`; `bf16` is an addition).
pub trait DataType:
    Add<Output = Self>
    + AddAssign
    + Sub<Output = Self>
    + SubAssign
    + Mul<Output = Self>
    + MulAssign
    + Div<Output = Self>
    + DivAssign
    + PartialOrd
    + bytemuck::NoUninit
    + bytemuck::AnyBitPattern
    + Debug
    + Display
{
    /// Name kept from the original, where it selects the WGSL scalar type; here it selects `WGF_F32` / `WGF_F16` / `WGF_BF16`.
    const WGSL_TYPE: DataTypeEnum;

    fn zero() -> Self;
    fn one() -> Self;
    /// Scalars of `arange` and of the scalar operators are f32 in the C ABI.
    fn to_f32(self) -> f32;
}

impl DataType for f32 {
    const WGSL_TYPE: DataTypeEnum = DataTypeEnum::F32;
    fn zero() -> Self {
        0.0
    }
    fn one() -> Self {
        1.0
    }
    fn to_f32(self) -> f32 {
        self
    }
}

impl DataType for half::f16 {
    const WGSL_TYPE: DataTypeEnum = DataTypeEnum::F16;
    fn zero() -> Self {
        half::f16::ZERO
    }
    fn one() -> Self {
        half::f16::ONE
    }
    fn to_f32(self) -> f32 {
        half::f16::to_f32(self)
    }
}

impl DataType for half::bf16 {
    const WGSL_TYPE: DataTypeEnum = DataTypeEnum::BF16;
    fn zero() -> Self {
        half::bf16::ZERO
    }
    fn one() -> Self {
        half::bf16::ONE
    }
    fn to_f32(self) -> f32 {
        half::bf16::to_f32(self)
    }
}

#[non_exhaustive]
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum DataTypeEnum {
    F32,
    F16,
    BF16,
}

impl DataTypeEnum {
    pub fn as_str(&self) -> &'static str {
        match self {
            DataTypeEnum::F32 => "f32",
            DataTypeEnum::F16 => "f16",
            DataTypeEnum::BF16 => "bf16",
        }
    }

    pub fn element_size(&self) -> usize {
        match self {
            DataTypeEnum::F32 => 4,
            DataTypeEnum::F16 | DataTypeEnum::BF16 => 2,
        }
    }

    pub(crate) fn code(&self) -> u32 {
        match self {
            DataTypeEnum::F32 => wgf_sys::WGF_F32,
            DataTypeEnum::F16 => wgf_sys::WGF_F16,
            DataTypeEnum::BF16 => wgf_sys::WGF_BF16,
        }
    }

    pub(crate) fn from_code(code: u32) -> Self {
        match code {
            wgf_sys::WGF_F16 => DataTypeEnum::F16,
            wgf_sys::WGF_BF16 => DataTypeEnum::BF16,
            _ => DataTypeEnum::F32,
        }
    }
}

impl Display for DataTypeEnum {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        f.write_str(self.as_str())
    }
}

/// Graphviz text of a compute graph (`Tensor::graphvis`).  The original returns a `tabbycat::Graph`;
/// its only use is to be printed, which this does too.
pub struct Graph(pub String);

impl Display for Graph {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        f.write_str(&self.0)
    }
}

/// A lazily evaluated tensor of rank `R` with elements of type `D` (original: `src/tensor.rs:418-421`).
pub struct Tensor<const R: usize, D> {
    pub(crate) raw: *mut wgf_sys::wgf_tensor,
    pub(crate) device: Device,
    shape: [usize; R],
    datatype: PhantomData<D>,
}

impl<const R: usize, D> Clone for Tensor<R, D> {
    /// A second handle on the same graph node (`src/tensor.rs:432-439`).
    fn clone(&self) -> Self {
        let mut raw = ptr::null_mut();
        expect(unsafe { wgf_sys::wgf_tensor_clone(self.raw, &mut raw) });
        Tensor { raw, device: self.device.clone(), shape: self.shape, datatype: PhantomData }
    }
}

impl<const R: usize, D> Drop for Tensor<R, D> {
    fn drop(&mut self) {
        unsafe { wgf_sys::wgf_tensor_release(self.raw) };
    }
}

impl<const R: usize, D> Tensor<R, D> {
    /// Wraps a handle the library just returned; reads its shape back and checks the rank.
    pub(crate) fn from_raw(raw: *mut wgf_sys::wgf_tensor, device: &Device) -> Self {
        let (mut dtype, mut rank) = (0u32, 0u32);
        let mut dims = [0i64; wgf_sys::WGF_MAX_RANK];
        expect(unsafe { wgf_sys::wgf_tensor_info(raw, &mut dtype, &mut rank, dims.as_mut_ptr()) });
        assert_eq!(rank as usize, R, "the library returned a tensor of rank {rank}, the type says {R}");
        let mut shape = [0usize; R];
        for (dst, src) in shape.iter_mut().zip(dims.iter()) {
            *dst = *src as usize;
        }
        Tensor { raw, device: device.clone(), shape, datatype: PhantomData }
    }

    /// Runs `f(out_handle)` and wraps what it stored.  Panics with the library's message on failure,
    /// where the original panics on shape and type misuse.
    pub(crate) fn build<const R2: usize, D2>(
        &self,
        f: impl FnOnce(*mut *mut wgf_sys::wgf_tensor) -> i32,
    ) -> Tensor<R2, D2> {
        let mut raw = ptr::null_mut();
        expect(f(&mut raw));
        Tensor::from_raw(raw, &self.device)
    }

    pub fn shape(&self) -> &[usize; R] {
        &self.shape
    }

    pub fn rank(&self) -> usize {
        R
    }

    pub fn device(&self) -> &Device {
        &self.device
    }
}

/// Nested iterators of `&D` up to three deep (original: `src/tensor.rs:441-515`).
pub trait IntoTensor<const R: usize, D> {
    fn into_tensor(self, device: &Device) -> Tensor<R, D>;
}

impl<'a, I, D: DataType> IntoTensor<1, D> for I
where
    I: IntoIterator<Item = &'a D>,
    I::IntoIter: ExactSizeIterator,
{
    fn into_tensor(self, device: &Device) -> Tensor<1, D> {
        let flat: Vec<D> = self.into_iter().copied().collect();
        let n = flat.len();
        Tensor::from_vec(device, flat, [n])
    }
}

impl<'a, I, I2, D: DataType> IntoTensor<2, D> for I
where
    I: IntoIterator<Item = I2>,
    I::IntoIter: ExactSizeIterator,
    I2: IntoIterator<Item = &'a D>,
    I2::IntoIter: ExactSizeIterator,
{
    fn into_tensor(self, device: &Device) -> Tensor<2, D> {
        let rows = self.into_iter();
        let n_rows = rows.len();
        let mut width = None;
        let mut flat = Vec::new();
        for row in rows {
            let row = row.into_iter();
            let len = row.len();
            let expected = *width.get_or_insert(len);
            if len != expected {
                panic!("expected a rectangular matrix. The first inner iterator size was {expected}, but another inner iterator size was {len}");
            }
            flat.extend(row.copied());
        }
        Tensor::from_vec(device, flat, [n_rows, width.unwrap_or(0)])
    }
}

impl<'a, I, I2, I3, D: DataType> IntoTensor<3, D> for I
where
    I: IntoIterator<Item = I2>,
    I::IntoIter: ExactSizeIterator,
    I2: IntoIterator<Item = I3>,
    I2::IntoIter: ExactSizeIterator,
    I3: IntoIterator<Item = &'a D>,
    I3::IntoIter: ExactSizeIterator,
{
    fn into_tensor(self, device: &Device) -> Tensor<3, D> {
        let planes = self.into_iter();
        let n_planes = planes.len();
        let (mut height, mut width) = (None, None);
        let mut flat = Vec::new();
        for plane in planes {
            let plane = plane.into_iter();
            let len = plane.len();
            let expected = *height.get_or_insert(len);
            if len != expected {
                panic!("expected a rectangular matrix. The first inner iterator size was {expected}, but another inner iterator size was {len}");
            }
            for row in plane {
                let row = row.into_iter();
                let len = row.len();
                let expected = *width.get_or_insert(len);
                if len != expected {
                    panic!("expected a rectangular matrix. The first inner inner iterator size was {expected}, but another inner inner iterator size was {len}");
                }
                flat.extend(row.copied());
            }
        }
        Tensor::from_vec(device, flat, [n_planes, height.unwrap_or(0), width.unwrap_or(0)])
    }
}

impl<D: DataType, const R: usize> Tensor<R, D> {
    /// `Tensor::new(&device, &[[1., 2.], [3., 4.]])` (original: `src/tensor.rs:518-520`).
    pub fn new(device: &Device, data: impl IntoTensor<R, D>) -> Self {
        data.into_tensor(device)
    }

    /// Row-major elements + shape: uploads at once, like the original's mapped-at-creation buffer.
    pub fn from_vec(device: &Device, flat: Vec<D>, shape: [usize; R]) -> Self {
        assert_eq!(flat.len(), shape.iter().product::<usize>(), "element count does not match the shape");
        let dims: Vec<i64> = shape.iter().map(|&s| s as i64).collect();
        let mut raw = ptr::null_mut();
        expect(unsafe {
            wgf_sys::wgf_tensor_from_host(
                device.raw,
                D::WGSL_TYPE.code(),
                R as u32,
                dims.as_ptr(),
                flat.as_ptr() as *const core::ffi::c_void,
                &mut raw,
            )
        });
        Tensor::from_raw(raw, device)
    }

    pub fn datatype(&self) -> DataTypeEnum {
        D::WGSL_TYPE
    }

    /// Queues the kernels of this tensor's graph without waiting (`LazyTensorData::materialize`,
    /// `src/tensor.rs:286-288`).
    pub fn materialize(&self) -> Result<(), Error> {
        check(unsafe { wgf_sys::wgf_tensor_materialize(self.raw) })
    }

    /// Resolves the graph, waits and downloads (original: `src/tensor.rs:551-554`).  `async` as in
    /// the original; the download itself blocks the calling thread on the CUDA stream.
    pub async fn as_slice(&self) -> Result<TensorSlice<R, D>, Error> {
        let count: usize = self.shape.iter().product();
        let mut data: Vec<D> = vec![D::zero(); count];
        check(unsafe {
            wgf_sys::wgf_tensor_download(
                self.raw,
                data.as_mut_ptr() as *mut core::ffi::c_void,
                (count * std::mem::size_of::<D>()) as u64,
            )
        })?;
        Ok(TensorSlice { data, layout: Layout::contiguous(&self.shape) })
    }

    /// Device time of every kernel launched so far while resolving this tensor's graph
    /// (original: `src/tensor.rs:556-558`).
    pub async fn all_timing_information(&self) -> Vec<QueryResults> {
        // the kernels have to have been queued before their times can be asked for
        expect(unsafe { wgf_sys::wgf_tensor_materialize(self.raw) });
        let mut count = 0u32;
        expect(unsafe { wgf_sys::wgf_tensor_timing(self.raw, ptr::null_mut(), 0, &mut count) });
        let mut nanos = vec![0u64; count as usize];
        expect(unsafe { wgf_sys::wgf_tensor_timing(self.raw, nanos.as_mut_ptr(), count, &mut count) });
        nanos.truncate(count as usize);
        nanos.into_iter().map(QueryResults::from_nanos).collect()
    }

    /// Graphviz text of the graph below this tensor (original: `src/tensor.rs:641-643`).
    pub fn graphvis(&self) -> Graph {
        let mut needed = 0u64;
        expect(unsafe { wgf_sys::wgf_tensor_graphviz(self.raw, ptr::null_mut(), 0, &mut needed) });
        let mut text = vec![0u8; needed as usize];
        expect(unsafe {
            wgf_sys::wgf_tensor_graphviz(self.raw, text.as_mut_ptr() as *mut core::ffi::c_char, needed, &mut needed)
        });
        while text.last() == Some(&0) {
            text.pop();
        }
        Graph(String::from_utf8_lossy(&text).into_owned())
    }

    /// Layout of the materialised result in device memory (may be a strided view).
    pub fn layout(&self) -> Result<Layout, Error> {
        let mut desc = std::mem::MaybeUninit::<wgf_sys::wgf_tensor_desc>::zeroed();
        check(unsafe { wgf_sys::wgf_tensor_desc_of(self.raw, desc.as_mut_ptr()) })?;
        let desc = unsafe { desc.assume_init() };
        unsafe { wgf_sys::wgf_buffer_release(desc.buf) };
        let rank = desc.rank as usize;
        Ok(Layout::from_parts(
            desc.offset as usize,
            desc.shape[..rank].iter().map(|&v| v as usize).collect(),
            desc.stride[..rank].iter().map(|&v| v as usize).collect(),
        ))
    }
}

/// Host copy of a materialised tensor (original: `src/tensor.rs:669-855`).  The original keeps the
/// whole downloaded allocation and indexes it through the view's layout; the library compacts on
/// the device, so this holds exactly the logical elements in row-major order.
pub struct TensorSlice<const R: usize, D> {
    data: Vec<D>,
    layout: Layout,
}

impl<D: DataType, const R: usize> TensorSlice<R, D> {
    /// The elements in row-major order.
    pub fn as_slice(&self) -> &[D] {
        &self.data
    }

    pub fn shape(&self) -> &[usize] {
        self.layout.shape()
    }

    /// `None` outside the shape (original: `src/tensor.rs:833-846`).
    pub fn get(&self, index: [usize; R]) -> Option<&D> {
        let mut at = 0usize;
        for ((&i, &stride), &extent) in index.iter().zip(self.layout.strides()).zip(self.layout.shape()) {
            if i >= extent {
                return None;
            }
            at += i * stride;
        }
        self.data.get(at)
    }
}

impl<D: DataType, const R: usize> Index<[usize; R]> for TensorSlice<R, D> {
    type Output = D;

    fn index(&self, index: [usize; R]) -> &D {
        self.get(index).expect("index outside the tensor")
    }
}

impl<const R: usize, D: DataType + PartialEq> PartialEq for TensorSlice<R, D> {
    fn eq(&self, other: &Self) -> bool {
        self.layout.shape() == other.layout.shape() && self.data == other.data
    }
}

impl<'a, D: DataType> PartialEq<&'a [D]> for TensorSlice<1, D> {
    fn eq(&self, other: &&'a [D]) -> bool {
        self.data.as_slice() == *other
    }
}

impl<const N: usize, D: DataType> PartialEq<[D; N]> for TensorSlice<1, D> {
    fn eq(&self, other: &[D; N]) -> bool {
        self.data.as_slice() == other.as_slice()
    }
}

impl<'a, D: DataType> PartialEq<TensorSlice<1, D>> for &'a [D] {
    fn eq(&self, other: &TensorSlice<1, D>) -> bool {
        *self == other.data.as_slice()
    }
}

impl<'a, const N: usize, D: DataType> PartialEq<TensorSlice<1, D>> for &'a [D; N] {
    fn eq(&self, other: &TensorSlice<1, D>) -> bool {
        self.as_slice() == other.data.as_slice()
    }
}

impl<D: DataType> Debug for TensorSlice<0, D> {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        self.get([]).fmt(f)
    }
}

impl<D: DataType> Debug for TensorSlice<1, D> {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        f.debug_list().entries(self.data.iter()).finish()
    }
}

impl<D: DataType> Debug for TensorSlice<2, D> {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        let width = self.layout.shape()[1].max(1);
        f.debug_list().entries(self.data.chunks(width)).finish()
    }
}

impl<D: DataType> Debug for TensorSlice<3, D> {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        let (height, width) = (self.layout.shape()[1].max(1), self.layout.shape()[2].max(1));
        let planes: Vec<Vec<&[D]>> = self.data.chunks(height * width).map(|p| p.chunks(width).collect()).collect();
        f.debug_list().entries(planes.iter()).finish()
    }
}
