//! Raw bindings of `include/wgf.h`, the C ABI of the B200 (sm_100a) backend: one `extern "C"`
//! declaration per function of the header, in the header's order, with the header's comments.
//!
//! This crate holds no logic.  `wgpu-compute` (the sibling crate) restates the public API of the
//! original `wgpu-compute` crate (`Tensor<R, D>`, `Device`, the operator impls and traits) on top of
//! these declarations.
//!
//! Linking: `build.rs` adds `libwgf.so` (built by `wgpu-kernal-fusion_b200/build.py`) from the
//! directory named by the environment variable `WGF_LIB_DIR`.
//!
//! NOTE: written on a machine without a Rust toolchain; it has not been compiled.  A test of the
//! repository (`tests/test_rust_bindings.py`) checks that every function of the header is declared
//! here with the same number of parameters and the same parameter types.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_void};

pub const WGF_MAX_RANK: usize = 8;
pub const WGF_COMM_ID_BYTES: usize = 128;

// status codes
pub const WGF_OK: i32 = 0;
pub const WGF_ERR_SHAPE: i32 = 1;
pub const WGF_ERR_DTYPE: i32 = 2;
pub const WGF_ERR_RANK: i32 = 3;
pub const WGF_ERR_OOM: i32 = 4;
pub const WGF_ERR_CUDA: i32 = 5;
pub const WGF_ERR_NCCL: i32 = 6;
pub const WGF_ERR_TIMEOUT: i32 = 7;
pub const WGF_ERR_INVALID_HANDLE: i32 = 8;
pub const WGF_ERR_INVALID_ARGUMENT: i32 = 9;
pub const WGF_ERR_COMPILE: i32 = 10;
pub const WGF_ERR_UNSUPPORTED: i32 = 11;

// element types (DataTypeEnum, src/tensor.rs:67-72; bf16 is an addition)
pub const WGF_F32: u32 = 0;
pub const WGF_F16: u32 = 1;
pub const WGF_BF16: u32 = 2;

// opcodes: unary functions (src/element_wise.rs:678-1380)
pub const WGF_OP_EXP: u32 = 0;
pub const WGF_OP_EXP2: u32 = 1;
pub const WGF_OP_LOG: u32 = 2;
pub const WGF_OP_LOG2: u32 = 3;
pub const WGF_OP_SQR: u32 = 4;
pub const WGF_OP_SQRT: u32 = 5;
pub const WGF_OP_SIN: u32 = 6;
pub const WGF_OP_COS: u32 = 7;
pub const WGF_OP_TAN: u32 = 8;
pub const WGF_OP_ASIN: u32 = 9;
pub const WGF_OP_ACOS: u32 = 10;
pub const WGF_OP_ATAN: u32 = 11;
pub const WGF_OP_SINH: u32 = 12;
pub const WGF_OP_COSH: u32 = 13;
pub const WGF_OP_TANH: u32 = 14;
pub const WGF_OP_ASINH: u32 = 15;
pub const WGF_OP_ACOSH: u32 = 16;
pub const WGF_OP_ATANH: u32 = 17;
pub const WGF_OP_ABS: u32 = 18;
pub const WGF_OP_NEG: u32 = 19;
// scalar forms (src/element_wise.rs:197-651)
pub const WGF_OP_ADD_C: u32 = 32;
pub const WGF_OP_SUB_C: u32 = 33;
pub const WGF_OP_RSUB_C: u32 = 34;
pub const WGF_OP_MUL_C: u32 = 35;
pub const WGF_OP_DIV_C: u32 = 36;
pub const WGF_OP_RDIV_C: u32 = 37;
pub const WGF_OP_CAST: u32 = 48;
// binary (src/pair_wise.rs:205-528)
pub const WGF_OP_ADD: u32 = 64;
pub const WGF_OP_SUB: u32 = 65;
pub const WGF_OP_MUL: u32 = 66;
pub const WGF_OP_DIV: u32 = 67;
pub const WGF_OP_POW: u32 = 68;
// reductions (src/reduce.rs:433-815)
pub const WGF_OP_SUM: u32 = 96;
pub const WGF_OP_MAX: u32 = 97;
pub const WGF_OP_MIN: u32 = 98;
pub const WGF_OP_PRODUCT: u32 = 99;

macro_rules! opaque {
    ($($name:ident),*) => {$(
        #[repr(C)]
        pub struct $name {
            _private: [u8; 0],
        }
    )*};
}
opaque!(wgf_device, wgf_buffer, wgf_tensor, wgf_comm, wgf_timing, wgf_schedule);

/// Layout {offset, shape, strides} + DataTypeEnum + buffer: src/layout.rs:33-38, src/tensor.rs:300-306.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct wgf_tensor_desc {
    pub buf: *mut wgf_buffer,
    pub dtype: u32,
    pub rank: u32,
    pub offset: i64,
    pub shape: [i64; WGF_MAX_RANK],
    pub stride: [i64; WGF_MAX_RANK],
}

/// ElementWiseFunction, src/element_wise.rs:167-172; `chain[0]` is applied first.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct wgf_ew_op {
    pub opcode: u16,
    /// only read for WGF_OP_CAST
    pub out_dtype: u16,
    /// only read for the scalar forms
    pub imm: f32,
}

extern "C" {
    pub fn wgf_last_error() -> *const c_char;
    /// Version of this ABI; bumped on any incompatible change.
    pub fn wgf_abi_version() -> i32;
    pub fn wgf_device_create(ordinal: i32, out: *mut *mut wgf_device) -> i32;
    pub fn wgf_device_retain(dev: *mut wgf_device) -> i32;
    pub fn wgf_device_release(dev: *mut wgf_device) -> i32;
    /// Blocks until all work queued on the device's stream has finished.
    pub fn wgf_device_sync(dev: *mut wgf_device) -> i32;
    /// No-op kept so callers that spawn the crate's `device.poll(Wait)` loop still link.
    pub fn wgf_device_poll(dev: *mut wgf_device) -> i32;
    /// Per-kernel CUDA-event timing on/off (default on, like the crate's timestamp queries).
    pub fn wgf_device_set_timing(dev: *mut wgf_device, enabled: i32) -> i32;
    /// Number of kernels this library has launched on the device since creation.
    pub fn wgf_device_launch_count(dev: *mut wgf_device, out: *mut u64) -> i32;
    /// Number of run-time kernel compilations so far (cache misses).
    pub fn wgf_device_compile_count(dev: *mut wgf_device, out: *mut u64) -> i32;
    /// Bytes held from the driver / bytes handed out to live buffers.
    pub fn wgf_device_memory(dev: *mut wgf_device, reserved: *mut u64, in_use: *mut u64) -> i32;
    /// Number of SMs and the raw cudaStream_t (as void*) for interop with the caller's runtime.
    pub fn wgf_device_info(dev: *mut wgf_device, sm_count: *mut i32, stream: *mut *mut c_void) -> i32;
    pub fn wgf_buffer_alloc(dev: *mut wgf_device, bytes: u64, zero: i32, out: *mut *mut wgf_buffer) -> i32;
    pub fn wgf_buffer_retain(buf: *mut wgf_buffer) -> i32;
    pub fn wgf_buffer_release(buf: *mut wgf_buffer) -> i32;
    /// Arc::strong_count analogue that gates in-place reuse, src/tensor.rs:413-415.
    pub fn wgf_buffer_use_count(buf: *mut wgf_buffer, out: *mut i64) -> i32;
    pub fn wgf_buffer_upload(buf: *mut wgf_buffer, offset_bytes: u64, src: *const c_void, bytes: u64) -> i32;
    pub fn wgf_buffer_download(buf: *mut wgf_buffer, offset_bytes: u64, dst: *mut c_void, bytes: u64) -> i32;
    /// Stream-ordered upload from PAGE-LOCKED host memory (wgf_host_alloc) that does not wait: the copy
    /// runs on the upload stream behind everything queued on the device stream so far; later kernels
    /// that read the buffer are ordered behind it.  `done` (may be NULL) receives a handle on the copy:
    /// wgf_timing_wait returns once `src` may be reused, wgf_timing_elapsed_ns gives the copy time.
    pub fn wgf_buffer_upload_async(
        buf: *mut wgf_buffer,
        offset_bytes: u64,
        src: *const c_void,
        bytes: u64,
        done: *mut *mut wgf_timing,
    ) -> i32;
    pub fn wgf_buffer_device_ptr(buf: *mut wgf_buffer, ptr: *mut *mut c_void, bytes: *mut u64) -> i32;
    /// Page-locked host memory, so that uploads and downloads run at full PCIe speed (the crate
    /// gets this from wgpu's mapped staging buffers, src/tensor.rs:345-381 and :533-549).
    pub fn wgf_host_alloc(bytes: u64, out: *mut *mut c_void) -> i32;
    pub fn wgf_host_free(ptr: *mut c_void) -> i32;
    /// Waits for the kernels the call queued and stores the sum of their device times.
    pub fn wgf_timing_elapsed_ns(t: *mut wgf_timing, out_ns: *mut u64) -> i32;
    /// Waits for them without reading the time.
    pub fn wgf_timing_wait(t: *mut wgf_timing) -> i32;
    /// Number of kernels (or copies) the call queued.
    pub fn wgf_timing_kernel_count(t: *mut wgf_timing, out: *mut u32) -> i32;
    pub fn wgf_timing_release(t: *mut wgf_timing) -> i32;
    /// UntypedElementWiseKernel::run_with_query, src/element_wise.rs:89-164.
    /// `inplace_ok` != 0 lets the result reuse `in`'s buffer when the dtype width is unchanged
    /// (the crate decides this from the buffer's reference count, src/element_wise.rs:98-99).
    /// `out->buf` is a new reference the caller must release.
    pub fn wgf_launch_elementwise(
        dev: *mut wgf_device,
        in_: *const wgf_tensor_desc,
        chain: *const wgf_ew_op,
        n_ops: u32,
        inplace_ok: i32,
        out: *mut wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// UntypedPairWiseKernel::run_with_query, src/pair_wise.rs:85-176: out = post(op(preA(a), preB(b))).
    pub fn wgf_launch_pairwise(
        dev: *mut wgf_device,
        a: *const wgf_tensor_desc,
        b: *const wgf_tensor_desc,
        pre_a: *const wgf_ew_op,
        n_pre_a: u32,
        pre_b: *const wgf_ew_op,
        n_pre_b: u32,
        opcode: u32,
        post: *const wgf_ew_op,
        n_post: u32,
        out: *mut wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// UntypedReduceKernel::run_with_query, src/reduce.rs:283-386: out = post(reduce_axis(pre(in))).
    pub fn wgf_launch_reduce(
        dev: *mut wgf_device,
        in_: *const wgf_tensor_desc,
        axis: u32,
        pre: *const wgf_ew_op,
        n_pre: u32,
        reduce_opcode: u32,
        post: *const wgf_ew_op,
        n_post: u32,
        out: *mut wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// UntypedMatMul::run_with_query, src/matmul.rs:157-214.  Rank 2, or rank 3 = batched.
    /// Strides and offsets are honoured.  `acc_dtype` names the accumulator type: WGF_F32 is the
    /// one this backend has for every element type (fp32 accumulators in tensor memory for 16-bit
    /// operands, FFMA for f32); anything else is WGF_ERR_UNSUPPORTED.  (The crate accumulates in
    /// the element type, src/matmul.rs:87-149.)
    pub fn wgf_launch_matmul(
        dev: *mut wgf_device,
        a: *const wgf_tensor_desc,
        b: *const wgf_tensor_desc,
        acc_dtype: u32,
        out: *mut wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// UntypedResizeKernel::run_with_query, src/resize.rs:90-118: copy `in` into the leading
    /// `fill_shape` box of a zero-filled tensor of `new_shape`.
    pub fn wgf_launch_resize(
        dev: *mut wgf_device,
        in_: *const wgf_tensor_desc,
        new_rank: u32,
        new_shape: *const i64,
        fill_shape: *const i64,
        out: *mut wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// UntypedSliceAssignKernel::run_with_query, src/slice_assign.rs:39-74: writes `value` into
    /// target[starts..ends) IN PLACE on the target's buffer.
    pub fn wgf_launch_slice_assign(
        dev: *mut wgf_device,
        target: *const wgf_tensor_desc,
        starts: *const i64,
        ends: *const i64,
        value: *const wgf_tensor_desc,
        timing: *mut *mut wgf_timing,
    ) -> i32;
    /// Tensor::new, src/tensor.rs:518-531 (row-major host data of `dtype`).
    pub fn wgf_tensor_from_host(
        dev: *mut wgf_device,
        dtype: u32,
        rank: u32,
        shape: *const i64,
        data: *const c_void,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Same, from PAGE-LOCKED host memory (wgf_host_alloc) without waiting: the copy runs on a
    /// separate upload stream and overlaps kernels and downloads already queued; every consumer is
    /// ordered behind it.  `data` must stay unchanged until a synchronising call (wgf_device_sync,
    /// a download of a dependent tensor) has returned.  Pageable memory is rejected.
    pub fn wgf_tensor_from_host_pinned(
        dev: *mut wgf_device,
        dtype: u32,
        rank: u32,
        shape: *const i64,
        data: *const c_void,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Wraps an existing buffer + layout as a graph leaf (TensorData::new_from_parts).
    pub fn wgf_tensor_from_desc(
        dev: *mut wgf_device,
        desc: *const wgf_tensor_desc,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Tensor::arange / arange_step, src/composite/arange.rs:4-23 (host loop + upload).
    pub fn wgf_tensor_arange(
        dev: *mut wgf_device,
        dtype: u32,
        start: f32,
        end: f32,
        step: f32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Clone, src/tensor.rs:432-439: a second handle on the same node.
    pub fn wgf_tensor_clone(t: *mut wgf_tensor, out: *mut *mut wgf_tensor) -> i32;
    pub fn wgf_tensor_release(t: *mut wgf_tensor) -> i32;
    /// shape() / rank() / datatype(), src/tensor.rs:629-639
    pub fn wgf_tensor_info(t: *mut wgf_tensor, dtype: *mut u32, rank: *mut u32, shape: *mut i64) -> i32;
    /// 19 unary functions + Neg, src/element_wise.rs:678-1380
    pub fn wgf_tensor_unary(t: *mut wgf_tensor, opcode: u32, out: *mut *mut wgf_tensor) -> i32;
    /// t+c, t-c, c-t, t*c, t/c, c/t, src/element_wise.rs:197-651
    pub fn wgf_tensor_scalar(t: *mut wgf_tensor, opcode: u32, c: f32, out: *mut *mut wgf_tensor) -> i32;
    /// CastTensor::cast, src/element_wise.rs:1408-1471
    pub fn wgf_tensor_cast(t: *mut wgf_tensor, dtype: u32, out: *mut *mut wgf_tensor) -> i32;
    /// + - * / pow on equal shapes and dtypes, src/pair_wise.rs:205-528
    pub fn wgf_tensor_binary(
        a: *mut wgf_tensor,
        b: *mut wgf_tensor,
        opcode: u32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// sum / max / min / product over one axis, src/reduce.rs:433-815
    pub fn wgf_tensor_reduce(t: *mut wgf_tensor, opcode: u32, axis: u32, out: *mut *mut wgf_tensor) -> i32;
    /// mat_mul, src/matmul.rs:25-29 (rank 2; rank 3 = batched, an addition)
    pub fn wgf_tensor_matmul(a: *mut wgf_tensor, b: *mut wgf_tensor, out: *mut *mut wgf_tensor) -> i32;
    /// slice / transpose / broadcast, src/map_layout.rs:41-98
    pub fn wgf_tensor_slice(
        t: *mut wgf_tensor,
        starts: *const i64,
        ends: *const i64,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    pub fn wgf_tensor_transpose(
        t: *mut wgf_tensor,
        axis_a: u32,
        axis_b: u32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Inserts ONE stride-0 axis; its position is the length of the common leading-dims prefix
    /// of the two shapes (src/map_layout.rs:73-77).
    pub fn wgf_tensor_broadcast(
        t: *mut wgf_tensor,
        out_rank: u32,
        out_shape: *const i64,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Same, with the position of the new axis stated (no counterpart in the crate).
    pub fn wgf_tensor_broadcast_axis(
        t: *mut wgf_tensor,
        axis: u32,
        size: i64,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Stride-0 expansion of size-1 axes to `out_shape` (no counterpart in the crate).
    pub fn wgf_tensor_expand(t: *mut wgf_tensor, out_shape: *const i64, out: *mut *mut wgf_tensor) -> i32;
    /// resize / reshape, src/resize.rs:121-144
    pub fn wgf_tensor_resize(t: *mut wgf_tensor, new_shape: *const i64, out: *mut *mut wgf_tensor) -> i32;
    pub fn wgf_tensor_reshape(
        t: *mut wgf_tensor,
        new_rank: u32,
        new_shape: *const i64,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// slice_assign, src/slice_assign.rs:76-79
    pub fn wgf_tensor_slice_assign(
        target: *mut wgf_tensor,
        starts: *const i64,
        ends: *const i64,
        value: *mut wgf_tensor,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Composites (graph recipes, no kernels of their own), src/composite/
    pub fn wgf_tensor_cat(
        parts: *const *mut wgf_tensor,
        n_parts: u32,
        dim: u32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// cat.rs:4-40
    pub fn wgf_tensor_narrow(
        t: *mut wgf_tensor,
        axis: u32,
        start: i64,
        length: i64,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// narrow.rs:4-15
    pub fn wgf_tensor_unsqueeze(t: *mut wgf_tensor, axis: u32, out: *mut *mut wgf_tensor) -> i32;
    /// unsqueeze.rs:16-53
    pub fn wgf_tensor_silu(t: *mut wgf_tensor, out: *mut *mut wgf_tensor) -> i32;
    /// silu.rs:4-7
    pub fn wgf_tensor_layer_norm(
        t: *mut wgf_tensor,
        weight: *mut wgf_tensor,
        eps: f32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// rms_norm.rs:8-15
    pub fn wgf_tensor_softmax(t: *mut wgf_tensor, out: *mut *mut wgf_tensor) -> i32;
    /// Max-subtracted softmax over the last axis of any rank (no counterpart in the crate).
    pub fn wgf_tensor_softmax_last_dim(t: *mut wgf_tensor, out: *mut *mut wgf_tensor) -> i32;
    pub fn wgf_tensor_rope(
        t: *mut wgf_tensor,
        cos: *mut wgf_tensor,
        sin: *mut wgf_tensor,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// softmax(scale * q k^T + mask) v for q [n, seq_q, d], k and v [n, seq_k, d] (n = batch * heads).
    /// `mask` is an additive [seq_q, seq_k] tensor or NULL.  With mask == NULL, `causal` != 0 masks the
    /// keys after each query; for 16-bit elements, d == 128 and seq_q == seq_k a multiple of 128 this
    /// runs as ONE fused tensor-core kernel that keeps the scores in tensor memory.  Other shapes
    /// (and any explicit mask) run as mat_mul, scale, add, softmax_last_dim, mat_mul; a causal
    /// request that cannot be fused fails with WGF_ERR_UNSUPPORTED and asks for a mask.  No
    /// counterpart in the crate.
    pub fn wgf_tensor_attention(
        q: *mut wgf_tensor,
        k: *mut wgf_tensor,
        v: *mut wgf_tensor,
        mask: *mut wgf_tensor,
        causal: i32,
        scale: f32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// Llama-style decoder block forward, composed from the primitives above (no counterpart in the
    /// crate; its README lists the ops such a block needs, README.md:24-38).
    /// h = x + Wo.attn(rope(Wq.n1), rope(Wk.n1), Wv.n1), n1 = rms_norm(x, norm1);
    /// out = h + Wd.(silu(Wg.n2) * (Wu.n2)),             n2 = rms_norm(h, norm2).
    /// x [batch, seq, hidden]; weights[7] = {Wq, Wk, Wv, Wo, Wg, Wu, Wd}, each stored
    /// [out_features, in_features]; norm1/norm2 [hidden]; cos/sin [>= seq, head_dim/2];
    /// mask [seq, seq] additive (0 where attended, -inf where not), or NULL for causal attention
    /// through wgf_tensor_attention's fused kernel.
    pub fn wgf_tensor_llama_block(
        x: *mut wgf_tensor,
        weights: *const *mut wgf_tensor,
        norm1: *mut wgf_tensor,
        norm2: *mut wgf_tensor,
        cos: *mut wgf_tensor,
        sin: *mut wgf_tensor,
        mask: *mut wgf_tensor,
        n_heads: u32,
        eps: f32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    /// LazyTensorData::materialize, src/tensor.rs:286-288: resolves the graph below `t`
    /// (src/compute_graph/resolve.rs:16-248) and queues its kernels; does not wait.
    pub fn wgf_tensor_materialize(t: *mut wgf_tensor) -> i32;
    /// Materialises `n` tensors as one request.  Same results as n calls of wgf_tensor_materialize;
    /// in addition, a reduction of a whole tensor to a scalar (e.g. t.sum(0).sum(0), also below
    /// wgf_tensor_all_reduce) that is requested together with a row-fused tensor over the same
    /// index space (layer_norm, softmax_last_dim, ...) is computed inside that tensor's kernel and
    /// reads nothing from memory a second time.  No counterpart in the crate, which resolves one
    /// tensor per call (src/tensor.rs:551-554) and names sibling-reduce fusion as future work
    /// (README.md:19-22).
    pub fn wgf_tensor_materialize_many(tensors: *const *mut wgf_tensor, n: u32) -> i32;
    /// The layout and buffer of the materialised result (TensorData, src/tensor.rs:300-306).
    /// `out->buf` is a new reference.
    pub fn wgf_tensor_desc_of(t: *mut wgf_tensor, out: *mut wgf_tensor_desc) -> i32;
    /// Tensor::as_slice, src/tensor.rs:551-554, compacted: materialises, waits, and copies the
    /// logical elements in row-major order to `dst` (`bytes` must equal numel * sizeof(dtype)).
    pub fn wgf_tensor_download(t: *mut wgf_tensor, dst: *mut c_void, bytes: u64) -> i32;
    /// Tensor::all_timing_information, src/tensor.rs:556-558: device time in ns of each kernel
    /// launched while resolving `t`'s graph.  Call with out_ns == NULL to get the count.
    pub fn wgf_tensor_timing(t: *mut wgf_tensor, out_ns: *mut u64, capacity: u32, count: *mut u32) -> i32;
    /// Kernel names matching wgf_tensor_timing, one per line (elementwise, rows, stream_reduce,
    /// col_reduce, copy, sgemm, matmul_tc, gemv_kn, ...).  Same size protocol as wgf_tensor_graphviz.
    pub fn wgf_tensor_timing_labels(
        t: *mut wgf_tensor,
        dst: *mut c_char,
        capacity: u64,
        needed: *mut u64,
    ) -> i32;
    /// Graphviz DOT text of the graph below `t` (Tensor::graphvis, src/tensor.rs:641-643).
    pub fn wgf_tensor_graphviz(t: *mut wgf_tensor, dst: *mut c_char, capacity: u64, needed: *mut u64) -> i32;
    /// Number of live graph nodes reachable from the graph `t` belongs to (debug aid).
    pub fn wgf_tensor_graph_size(t: *mut wgf_tensor, nodes: *mut u64) -> i32;
    /// Contiguous block partition of `n_units` over `world` ranks: the first n_units % world
    /// ranks get one extra unit.
    pub fn wgf_shard_range(n_units: i64, world: i32, rank: i32, begin: *mut i64, end: *mut i64) -> i32;
    pub fn wgf_comm_unique_id(id: *mut u8) -> i32;
    pub fn wgf_comm_create(
        dev: *mut wgf_device,
        world: i32,
        rank: i32,
        id: *const u8,
        out: *mut *mut wgf_comm,
    ) -> i32;
    pub fn wgf_comm_release(comm: *mut wgf_comm) -> i32;
    /// Lazy node: all-reduce (WGF_OP_SUM / MAX / MIN / PRODUCT) of `t` over the communicator,
    /// queued on the device stream directly behind the kernel that produces `t`.
    pub fn wgf_tensor_all_reduce(
        t: *mut wgf_tensor,
        comm: *mut wgf_comm,
        opcode: u32,
        out: *mut *mut wgf_tensor,
    ) -> i32;
    pub fn wgf_schedule_begin(dev: *mut wgf_device) -> i32;
    pub fn wgf_schedule_end(dev: *mut wgf_device, out: *mut *mut wgf_schedule) -> i32;
    pub fn wgf_schedule_launch(s: *mut wgf_schedule) -> i32;
    /// Kernels (and copies) one launch runs.
    pub fn wgf_schedule_kernel_count(s: *mut wgf_schedule, out: *mut u64) -> i32;
    /// Waits for replays in flight, then frees the graph and returns its memory to the pool.
    pub fn wgf_schedule_destroy(s: *mut wgf_schedule) -> i32;
    pub fn wgf_full_reduce_f32_noalloc(
        x: *const f32,
        n: u64,
        pre_opcode: u32,
        reduce_opcode: u32,
        out: *mut f32,
        cuda_stream: *mut c_void,
    ) -> i32;
}
