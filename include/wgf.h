/*
 * wgf.h -- C ABI of the B200 (sm_100a) backend for the lazy, kernel-fusing tensor runtime
 * whose behaviour is defined by the Rust crate `wgpu-compute`.
 *
 * The crate has no FFI layer of its own: its only contact with a GPU is five wgpu seams
 * (device creation, buffer allocation/upload, kernel dispatch, queue submit, download and
 * timestamp queries).  This header places one plain-C entry point at each of those seams
 * ("kernel-level" section) and, above them, restates the crate's public `Tensor` API as
 * opaque-handle calls ("graph-level" section) so that a host written in any language gets
 * the lazy graph and the fusion resolver as well.  Every declaration cites the crate item it
 * replaces as `path:line` relative to the crate root.
 *
 * Conventions
 *   - every function returns a status (WGF_OK == 0); on failure `wgf_last_error()` gives a
 *     thread-local message.  Nothing aborts, nothing throws across this boundary.
 *   - handles are reference counted; `*_release` drops one reference.
 *   - shapes, strides and offsets are in ELEMENTS and 64-bit (the crate passes u32 to its
 *     shaders, src/kernel.rs:326-333).
 *   - one CUDA stream per device handle; all work on a device is ordered on that stream.
 *   - there is no CPU fallback: a call that needs the GPU fails with WGF_ERR_CUDA without one.
 */
#ifndef WGF_H
#define WGF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WGF_MAX_RANK 8

/* ---- status codes ------------------------------------------------------------------ */
enum {
    WGF_OK = 0,
    WGF_ERR_SHAPE = 1,          /* the crate panics: src/pair_wise.rs:92, src/matmul.rs:194 */
    WGF_ERR_DTYPE = 2,
    WGF_ERR_RANK = 3,           /* src/visit_tiled.rs:71 */
    WGF_ERR_OOM = 4,
    WGF_ERR_CUDA = 5,           /* RequestDeviceError / BufferAsyncError: src/device.rs:14, src/tensor.rs:551 */
    WGF_ERR_NCCL = 6,
    WGF_ERR_TIMEOUT = 7,
    WGF_ERR_INVALID_HANDLE = 8,
    WGF_ERR_INVALID_ARGUMENT = 9,
    WGF_ERR_COMPILE = 10,       /* run-time kernel compilation failed (create_shader_module, src/kernel.rs:244-272) */
    WGF_ERR_UNSUPPORTED = 11
};

/* ---- element types: DataTypeEnum, src/tensor.rs:67-72 (bf16 is an addition) ---------- */
enum { WGF_F32 = 0, WGF_F16 = 1, WGF_BF16 = 2 };

/* ---- opcodes ------------------------------------------------------------------------
 * Unary functions: src/element_wise.rs:678-1380.  Scalar forms: src/element_wise.rs:197-651.
 * Binary: src/pair_wise.rs:205-528.  Reductions: src/reduce.rs:433-815. */
enum {
    WGF_OP_EXP = 0, WGF_OP_EXP2, WGF_OP_LOG, WGF_OP_LOG2, WGF_OP_SQR, WGF_OP_SQRT,
    WGF_OP_SIN, WGF_OP_COS, WGF_OP_TAN, WGF_OP_ASIN, WGF_OP_ACOS, WGF_OP_ATAN,
    WGF_OP_SINH, WGF_OP_COSH, WGF_OP_TANH, WGF_OP_ASINH, WGF_OP_ACOSH, WGF_OP_ATANH,
    WGF_OP_ABS, WGF_OP_NEG,
    WGF_OP_ADD_C = 32,  /* x + c */
    WGF_OP_SUB_C,       /* x - c */
    WGF_OP_RSUB_C,      /* c - x */
    WGF_OP_MUL_C,       /* x * c */
    WGF_OP_DIV_C,       /* x / c */
    WGF_OP_RDIV_C,      /* c / x */
    WGF_OP_CAST = 48,   /* to out_dtype: src/element_wise.rs:1408-1471 */
    WGF_OP_ADD = 64, WGF_OP_SUB, WGF_OP_MUL, WGF_OP_DIV, WGF_OP_POW,
    WGF_OP_SUM = 96, WGF_OP_MAX, WGF_OP_MIN, WGF_OP_PRODUCT
};

typedef struct wgf_device wgf_device;
typedef struct wgf_buffer wgf_buffer;
typedef struct wgf_tensor wgf_tensor;
typedef struct wgf_comm wgf_comm;
/* Device time of what ONE call queued (PerformanceQueries / QueryResults, src/query.rs:10-126):
 * created by the call, read later -- nothing waits until wgf_timing_elapsed_ns. */
typedef struct wgf_timing wgf_timing;

const char* wgf_last_error(void);
/* Version of this ABI; bumped on any incompatible change. */
int32_t wgf_abi_version(void);

/* ======================================================================================
 * Device  (replaces Device::new / Clone / wgpu_device().poll, src/device.rs:8-52)
 * ==================================================================================== */
int32_t wgf_device_create(int32_t ordinal, wgf_device** out);
int32_t wgf_device_retain(wgf_device* dev);
int32_t wgf_device_release(wgf_device* dev);
/* Blocks until all work queued on the device's stream has finished. */
int32_t wgf_device_sync(wgf_device* dev);
/* No-op kept so callers that spawn the crate's `device.poll(Wait)` loop still link. */
int32_t wgf_device_poll(wgf_device* dev);
/* Per-kernel CUDA-event timing on/off (default on, like the crate's timestamp queries). */
int32_t wgf_device_set_timing(wgf_device* dev, int32_t enabled);
/* Number of kernels this library has launched on the device since creation. */
int32_t wgf_device_launch_count(wgf_device* dev, uint64_t* out);
/* Number of run-time kernel compilations so far (cache misses). */
int32_t wgf_device_compile_count(wgf_device* dev, uint64_t* out);
/* Bytes held from the driver / bytes handed out to live buffers. */
int32_t wgf_device_memory(wgf_device* dev, uint64_t* reserved, uint64_t* in_use);
/* Number of SMs and the raw cudaStream_t (as void*) for interop with the caller's runtime. */
int32_t wgf_device_info(wgf_device* dev, int32_t* sm_count, void** stream);

/* ======================================================================================
 * Buffers  (replaces TensorData::new_for_shape/new_inner/owned, src/tensor.rs:331-415,
 *           and the download in src/tensor.rs:533-549)
 * ==================================================================================== */
int32_t wgf_buffer_alloc(wgf_device* dev, uint64_t bytes, int32_t zero, wgf_buffer** out);
int32_t wgf_buffer_retain(wgf_buffer* buf);
int32_t wgf_buffer_release(wgf_buffer* buf);
/* Arc::strong_count analogue that gates in-place reuse, src/tensor.rs:413-415. */
int32_t wgf_buffer_use_count(wgf_buffer* buf, int64_t* out);
int32_t wgf_buffer_upload(wgf_buffer* buf, uint64_t offset_bytes, const void* src, uint64_t bytes);
int32_t wgf_buffer_download(wgf_buffer* buf, uint64_t offset_bytes, void* dst, uint64_t bytes);
/* Stream-ordered upload from PAGE-LOCKED host memory (wgf_host_alloc) that does not wait: the copy
 * runs on the upload stream behind everything queued on the device stream so far; later kernels
 * that read the buffer are ordered behind it.  `done` (may be NULL) receives a handle on the copy:
 * wgf_timing_wait returns once `src` may be reused, wgf_timing_elapsed_ns gives the copy time. */
int32_t wgf_buffer_upload_async(wgf_buffer* buf, uint64_t offset_bytes, const void* src, uint64_t bytes,
                                wgf_timing** done);
int32_t wgf_buffer_device_ptr(wgf_buffer* buf, void** ptr, uint64_t* bytes);
/* Page-locked host memory, so that uploads and downloads run at full PCIe speed (the crate
 * gets this from wgpu's mapped staging buffers, src/tensor.rs:345-381 and :533-549). */
int32_t wgf_host_alloc(uint64_t bytes, void** out);
int32_t wgf_host_free(void* ptr);

/* ======================================================================================
 * Timing handles  (replace PerformanceQueries::wait_for_results / QueryResults::elapsed,
 *                  src/query.rs:35-41 and :78-112)
 * ==================================================================================== */
/* Waits for the kernels the call queued and stores the sum of their device times. */
int32_t wgf_timing_elapsed_ns(wgf_timing* t, uint64_t* out_ns);
/* Waits for them without reading the time. */
int32_t wgf_timing_wait(wgf_timing* t);
/* Number of kernels (or copies) the call queued. */
int32_t wgf_timing_kernel_count(wgf_timing* t, uint32_t* out);
int32_t wgf_timing_release(wgf_timing* t);

/* ======================================================================================
 * Kernel-level launches  (replace Untyped*Kernel::run_with_query)
 * Each takes an optional `timing` out-parameter, the analogue of the crate's
 * `Option<&PerformanceQueries>` argument: NULL = untimed; otherwise *timing receives a new
 * handle (release it with wgf_timing_release).  The launch itself never waits.
 * ==================================================================================== */
/* Layout {offset, shape, strides} + DataTypeEnum + buffer: src/layout.rs:33-38, src/tensor.rs:300-306 */
typedef struct wgf_tensor_desc {
    wgf_buffer* buf;
    uint32_t dtype;
    uint32_t rank;
    int64_t offset;
    int64_t shape[WGF_MAX_RANK];
    int64_t stride[WGF_MAX_RANK];
} wgf_tensor_desc;

/* ElementWiseFunction, src/element_wise.rs:167-172; `chain[0]` is applied first. */
typedef struct wgf_ew_op {
    uint16_t opcode;
    uint16_t out_dtype;   /* only read for WGF_OP_CAST */
    float imm;            /* only read for the scalar forms */
} wgf_ew_op;

/* UntypedElementWiseKernel::run_with_query, src/element_wise.rs:89-164.
 * `inplace_ok` != 0 lets the result reuse `in`'s buffer when the dtype width is unchanged
 * (the crate decides this from the buffer's reference count, src/element_wise.rs:98-99).
 * `out->buf` is a new reference the caller must release. */
int32_t wgf_launch_elementwise(wgf_device* dev, const wgf_tensor_desc* in, const wgf_ew_op* chain,
                               uint32_t n_ops, int32_t inplace_ok, wgf_tensor_desc* out,
                               wgf_timing** timing);
/* UntypedPairWiseKernel::run_with_query, src/pair_wise.rs:85-176: out = post(op(preA(a), preB(b))). */
int32_t wgf_launch_pairwise(wgf_device* dev, const wgf_tensor_desc* a, const wgf_tensor_desc* b,
                            const wgf_ew_op* pre_a, uint32_t n_pre_a, const wgf_ew_op* pre_b,
                            uint32_t n_pre_b, uint32_t opcode, const wgf_ew_op* post, uint32_t n_post,
                            wgf_tensor_desc* out, wgf_timing** timing);
/* UntypedReduceKernel::run_with_query, src/reduce.rs:283-386: out = post(reduce_axis(pre(in))). */
int32_t wgf_launch_reduce(wgf_device* dev, const wgf_tensor_desc* in, uint32_t axis,
                          const wgf_ew_op* pre, uint32_t n_pre, uint32_t reduce_opcode,
                          const wgf_ew_op* post, uint32_t n_post, wgf_tensor_desc* out,
                          wgf_timing** timing);
/* UntypedMatMul::run_with_query, src/matmul.rs:157-214.  Rank 2, or rank 3 = batched.
 * Strides and offsets are honoured.  `acc_dtype` names the accumulator type: WGF_F32 is the
 * one this backend has for every element type (fp32 accumulators in tensor memory for 16-bit
 * operands, FFMA for f32); anything else is WGF_ERR_UNSUPPORTED.  (The crate accumulates in
 * the element type, src/matmul.rs:87-149.) */
int32_t wgf_launch_matmul(wgf_device* dev, const wgf_tensor_desc* a, const wgf_tensor_desc* b,
                          uint32_t acc_dtype, wgf_tensor_desc* out, wgf_timing** timing);
/* UntypedResizeKernel::run_with_query, src/resize.rs:90-118: copy `in` into the leading
 * `fill_shape` box of a zero-filled tensor of `new_shape`. */
int32_t wgf_launch_resize(wgf_device* dev, const wgf_tensor_desc* in, uint32_t new_rank,
                          const int64_t* new_shape, const int64_t* fill_shape, wgf_tensor_desc* out,
                          wgf_timing** timing);
/* UntypedSliceAssignKernel::run_with_query, src/slice_assign.rs:39-74: writes `value` into
 * target[starts..ends) IN PLACE on the target's buffer. */
int32_t wgf_launch_slice_assign(wgf_device* dev, const wgf_tensor_desc* target, const int64_t* starts,
                                const int64_t* ends, const wgf_tensor_desc* value,
                                wgf_timing** timing);

/* ======================================================================================
 * Graph-level API: the crate's `Tensor<R, D>` (src/tensor.rs:418-644).  A wgf_tensor is a
 * handle on a node of the lazy compute graph (src/compute_graph/mod.rs:152-276); nothing
 * runs until wgf_tensor_materialize / wgf_tensor_download.
 * ==================================================================================== */
/* Tensor::new, src/tensor.rs:518-531 (row-major host data of `dtype`). */
int32_t wgf_tensor_from_host(wgf_device* dev, uint32_t dtype, uint32_t rank, const int64_t* shape,
                             const void* data, wgf_tensor** out);
/* Same, from PAGE-LOCKED host memory (wgf_host_alloc) without waiting: the copy runs on a
 * separate upload stream and overlaps kernels and downloads already queued; every consumer is
 * ordered behind it.  `data` must stay unchanged until a synchronising call (wgf_device_sync,
 * a download of a dependent tensor) has returned.  Pageable memory is rejected. */
int32_t wgf_tensor_from_host_pinned(wgf_device* dev, uint32_t dtype, uint32_t rank, const int64_t* shape,
                                    const void* data, wgf_tensor** out);
/* Wraps an existing buffer + layout as a graph leaf (TensorData::new_from_parts). */
int32_t wgf_tensor_from_desc(wgf_device* dev, const wgf_tensor_desc* desc, wgf_tensor** out);
/* Tensor::arange / arange_step, src/composite/arange.rs:4-23 (host loop + upload). */
int32_t wgf_tensor_arange(wgf_device* dev, uint32_t dtype, float start, float end, float step,
                          wgf_tensor** out);
/* Clone, src/tensor.rs:432-439: a second handle on the same node. */
int32_t wgf_tensor_clone(wgf_tensor* t, wgf_tensor** out);
int32_t wgf_tensor_release(wgf_tensor* t);
/* shape() / rank() / datatype(), src/tensor.rs:629-639 */
int32_t wgf_tensor_info(wgf_tensor* t, uint32_t* dtype, uint32_t* rank, int64_t* shape);

/* 19 unary functions + Neg, src/element_wise.rs:678-1380 */
int32_t wgf_tensor_unary(wgf_tensor* t, uint32_t opcode, wgf_tensor** out);
/* t+c, t-c, c-t, t*c, t/c, c/t, src/element_wise.rs:197-651 */
int32_t wgf_tensor_scalar(wgf_tensor* t, uint32_t opcode, float c, wgf_tensor** out);
/* CastTensor::cast, src/element_wise.rs:1408-1471 */
int32_t wgf_tensor_cast(wgf_tensor* t, uint32_t dtype, wgf_tensor** out);
/* + - * / pow on equal shapes and dtypes, src/pair_wise.rs:205-528 */
int32_t wgf_tensor_binary(wgf_tensor* a, wgf_tensor* b, uint32_t opcode, wgf_tensor** out);
/* sum / max / min / product over one axis, src/reduce.rs:433-815 */
int32_t wgf_tensor_reduce(wgf_tensor* t, uint32_t opcode, uint32_t axis, wgf_tensor** out);
/* mat_mul, src/matmul.rs:25-29 (rank 2; rank 3 = batched, an addition) */
int32_t wgf_tensor_matmul(wgf_tensor* a, wgf_tensor* b, wgf_tensor** out);
/* slice / transpose / broadcast, src/map_layout.rs:41-98 */
int32_t wgf_tensor_slice(wgf_tensor* t, const int64_t* starts, const int64_t* ends, wgf_tensor** out);
int32_t wgf_tensor_transpose(wgf_tensor* t, uint32_t axis_a, uint32_t axis_b, wgf_tensor** out);
/* Inserts ONE stride-0 axis; its position is the length of the common leading-dims prefix
 * of the two shapes (src/map_layout.rs:73-77). */
int32_t wgf_tensor_broadcast(wgf_tensor* t, uint32_t out_rank, const int64_t* out_shape,
                             wgf_tensor** out);
/* Same, with the position of the new axis stated (no counterpart in the crate). */
int32_t wgf_tensor_broadcast_axis(wgf_tensor* t, uint32_t axis, int64_t size, wgf_tensor** out);
/* Stride-0 expansion of size-1 axes to `out_shape` (no counterpart in the crate). */
int32_t wgf_tensor_expand(wgf_tensor* t, const int64_t* out_shape, wgf_tensor** out);
/* resize / reshape, src/resize.rs:121-144 */
int32_t wgf_tensor_resize(wgf_tensor* t, const int64_t* new_shape, wgf_tensor** out);
int32_t wgf_tensor_reshape(wgf_tensor* t, uint32_t new_rank, const int64_t* new_shape, wgf_tensor** out);
/* slice_assign, src/slice_assign.rs:76-79 */
int32_t wgf_tensor_slice_assign(wgf_tensor* target, const int64_t* starts, const int64_t* ends,
                                wgf_tensor* value, wgf_tensor** out);
/* Composites (graph recipes, no kernels of their own), src/composite/ */
int32_t wgf_tensor_cat(wgf_tensor* const* parts, uint32_t n_parts, uint32_t dim, wgf_tensor** out); /* cat.rs:4-40 */
int32_t wgf_tensor_narrow(wgf_tensor* t, uint32_t axis, int64_t start, int64_t length, wgf_tensor** out); /* narrow.rs:4-15 */
int32_t wgf_tensor_unsqueeze(wgf_tensor* t, uint32_t axis, wgf_tensor** out);                       /* unsqueeze.rs:16-53 */
int32_t wgf_tensor_silu(wgf_tensor* t, wgf_tensor** out);                                           /* silu.rs:4-7 */
int32_t wgf_tensor_layer_norm(wgf_tensor* t, wgf_tensor* weight, float eps, wgf_tensor** out);      /* rms_norm.rs:8-15 */
int32_t wgf_tensor_softmax(wgf_tensor* t, wgf_tensor** out);                                        /* softmax.rs:4-10, rank 1, no max-subtract */
/* Max-subtracted softmax over the last axis of any rank (no counterpart in the crate). */
int32_t wgf_tensor_softmax_last_dim(wgf_tensor* t, wgf_tensor** out);
int32_t wgf_tensor_rope(wgf_tensor* t, wgf_tensor* cos, wgf_tensor* sin, wgf_tensor** out);         /* rope.rs:13-22 */
/* softmax(scale * q k^T + mask) v for q [n, seq_q, d], k and v [n, seq_k, d] (n = batch * heads).
 * `mask` is an additive [seq_q, seq_k] tensor or NULL.  With mask == NULL, `causal` != 0 masks the
 * keys after each query; for 16-bit elements, d == 128 and seq_q == seq_k a multiple of 128 this
 * runs as ONE fused tensor-core kernel that keeps the scores in tensor memory.  Other shapes
 * (and any explicit mask) run as mat_mul, scale, add, softmax_last_dim, mat_mul; a causal
 * request that cannot be fused fails with WGF_ERR_UNSUPPORTED and asks for a mask.  No
 * counterpart in the crate. */
int32_t wgf_tensor_attention(wgf_tensor* q, wgf_tensor* k, wgf_tensor* v, wgf_tensor* mask, int32_t causal, float scale,
                             wgf_tensor** out);
/* Llama-style decoder block forward, composed from the primitives above (no counterpart in the
 * crate; its README lists the ops such a block needs, README.md:24-38).
 *   h = x + Wo.attn(rope(Wq.n1), rope(Wk.n1), Wv.n1), n1 = rms_norm(x, norm1);
 *   out = h + Wd.(silu(Wg.n2) * (Wu.n2)),             n2 = rms_norm(h, norm2).
 * x [batch, seq, hidden]; weights[7] = {Wq, Wk, Wv, Wo, Wg, Wu, Wd}, each stored
 * [out_features, in_features]; norm1/norm2 [hidden]; cos/sin [>= seq, head_dim/2];
 * mask [seq, seq] additive (0 where attended, -inf where not), or NULL for causal attention
 * through wgf_tensor_attention's fused kernel. */
int32_t wgf_tensor_llama_block(wgf_tensor* x, wgf_tensor* const* weights, wgf_tensor* norm1, wgf_tensor* norm2,
                               wgf_tensor* cos, wgf_tensor* sin, wgf_tensor* mask, uint32_t n_heads, float eps,
                               wgf_tensor** out);

/* LazyTensorData::materialize, src/tensor.rs:286-288: resolves the graph below `t`
 * (src/compute_graph/resolve.rs:16-248) and queues its kernels; does not wait. */
int32_t wgf_tensor_materialize(wgf_tensor* t);
/* Materialises `n` tensors as one request.  Same results as n calls of wgf_tensor_materialize;
 * in addition, a reduction of a whole tensor to a scalar (e.g. t.sum(0).sum(0), also below
 * wgf_tensor_all_reduce) that is requested together with a row-fused tensor over the same
 * index space (layer_norm, softmax_last_dim, ...) is computed inside that tensor's kernel and
 * reads nothing from memory a second time.  No counterpart in the crate, which resolves one
 * tensor per call (src/tensor.rs:551-554) and names sibling-reduce fusion as future work
 * (README.md:19-22). */
int32_t wgf_tensor_materialize_many(wgf_tensor* const* tensors, uint32_t n);
/* The layout and buffer of the materialised result (TensorData, src/tensor.rs:300-306).
 * `out->buf` is a new reference. */
int32_t wgf_tensor_desc_of(wgf_tensor* t, wgf_tensor_desc* out);
/* Tensor::as_slice, src/tensor.rs:551-554, compacted: materialises, waits, and copies the
 * logical elements in row-major order to `dst` (`bytes` must equal numel * sizeof(dtype)). */
int32_t wgf_tensor_download(wgf_tensor* t, void* dst, uint64_t bytes);
/* Tensor::all_timing_information, src/tensor.rs:556-558: device time in ns of each kernel
 * launched while resolving `t`'s graph.  Call with out_ns == NULL to get the count. */
int32_t wgf_tensor_timing(wgf_tensor* t, uint64_t* out_ns, uint32_t capacity, uint32_t* count);
/* Kernel names matching wgf_tensor_timing, one per line (elementwise, rows, stream_reduce,
 * col_reduce, copy, sgemm, matmul_tc, gemv_kn, ...).  Same size protocol as wgf_tensor_graphviz. */
int32_t wgf_tensor_timing_labels(wgf_tensor* t, char* dst, uint64_t capacity, uint64_t* needed);
/* Graphviz DOT text of the graph below `t` (Tensor::graphvis, src/tensor.rs:641-643). */
int32_t wgf_tensor_graphviz(wgf_tensor* t, char* dst, uint64_t capacity, uint64_t* needed);
/* Number of live graph nodes reachable from the graph `t` belongs to (debug aid). */
int32_t wgf_tensor_graph_size(wgf_tensor* t, uint64_t* nodes);

/* ======================================================================================
 * Multi-GPU (no counterpart in the crate, which drives one device): one process per GPU;
 * rows or batches are sharded by the caller; the only exchange is the all-reduce that
 * closes a full-tensor reduction.
 * ==================================================================================== */
/* Contiguous block partition of `n_units` over `world` ranks: the first n_units % world
 * ranks get one extra unit. */
int32_t wgf_shard_range(int64_t n_units, int32_t world, int32_t rank, int64_t* begin, int64_t* end);
#define WGF_COMM_ID_BYTES 128
int32_t wgf_comm_unique_id(uint8_t id[WGF_COMM_ID_BYTES]);
int32_t wgf_comm_create(wgf_device* dev, int32_t world, int32_t rank,
                        const uint8_t id[WGF_COMM_ID_BYTES], wgf_comm** out);
int32_t wgf_comm_release(wgf_comm* comm);
/* Lazy node: all-reduce (WGF_OP_SUM / MAX / MIN / PRODUCT) of `t` over the communicator.
 * Every rank must request the same all-reduces in the same order.  When `t` is a whole-tensor
 * reduction, the exchange is done over peer memory by the kernels of this and the following
 * steps (no collective launch); the result is final for every reader that goes through this
 * library, and after wgf_device_sync.  The exchange makes progress on a rank when that rank
 * queues its next all-reduce of this kind, reads a result or synchronises: a rank that has
 * requested an all-reduce must not block on its peers by other means before it has done one of
 * these.  A peer that does not take part within the limit
 * (environment WGF_PEER_WAIT_MS, default 5000) makes the next synchronisation return
 * WGF_ERR_TIMEOUT; later all-reduces on that device are refused until a new communicator
 * has been created. */
int32_t wgf_tensor_all_reduce(wgf_tensor* t, wgf_comm* comm, uint32_t opcode, wgf_tensor** out);

/* ======================================================================================
 * Recorded schedules: the kernels of a materialisation, captured once as a CUDA graph and
 * replayed with one call.  The crate pays its whole host cost (graph walk, shader text,
 * bind groups, one submit per kernel: src/compute_graph/resolve.rs:16-248,
 * src/kernel.rs:244-389) on every materialisation; a replay pays one graph launch.
 *
 *   wgf_schedule_begin(dev);
 *   ... build tensors, wgf_tensor_materialize / _materialize_many ...   (captured, not run)
 *   wgf_schedule_end(dev, &s);     (instantiates and runs the schedule once)
 *   loop: write new input data into the input tensors' buffers (wgf_tensor_desc_of +
 *         wgf_buffer_upload), wgf_schedule_launch(s), read the results' buffers.
 *
 * Inputs are the tensors that existed before wgf_schedule_begin; the schedule reads their
 * buffers at every launch and never overwrites them.  Tensors materialised while recording
 * keep their buffers for the life of the schedule and hold the values of the latest launch.
 * While recording, calls that wait for the device or copy between host and device (sync,
 * uploads, downloads, tensor creation from host data) and all-reduces fail with
 * WGF_ERR_UNSUPPORTED; constants of scalar ops are recorded by value.  One recording at a
 * time per device.  Memory taken while recording returns to the device's pool when the
 * schedule is destroyed.
 * ==================================================================================== */
typedef struct wgf_schedule wgf_schedule;
int32_t wgf_schedule_begin(wgf_device* dev);
/* Ends the recording started by wgf_schedule_begin.  On failure the recording is over as
 * well and *out is NULL. */
int32_t wgf_schedule_end(wgf_device* dev, wgf_schedule** out);
/* Queues one replay on the device's stream; does not wait. */
int32_t wgf_schedule_launch(wgf_schedule* s);
/* Kernels (and copies) one launch runs. */
int32_t wgf_schedule_kernel_count(wgf_schedule* s, uint64_t* out);
/* Waits for replays in flight, then frees the graph and returns its memory to the pool. */
int32_t wgf_schedule_destroy(wgf_schedule* s);

/* ======================================================================================
 * Reduction for callers that must not allocate.  (No counterpart in the crate: this entry
 * point exists for hosts of THIS library that cannot let a compute call reach the device
 * allocator -- real-time loops that rule out calls of unbounded latency, embedders with a
 * device-memory budget fixed up front, in which a hidden cudaMalloc would break the budget.)
 *
 * out[0] = reduce(pre(x[0..n))): x, out are DEVICE pointers owned by the caller, n <=
 * 2^31 f32 elements (more is rejected with WGF_ERR_UNSUPPORTED); `pre_opcode` is WGF_OP_EXP,
 * WGF_OP_SQR, WGF_OP_ABS or 0xFFFFFFFF for none; `reduce_opcode` is WGF_OP_SUM/MAX/MIN/PRODUCT;
 * `cuda_stream` is a cudaStream_t (NULL = default stream) the work is queued on.
 * Scratch (per-CTA partials and a ticket) is a fixed 16 KiB array inside the library image:
 * each GPU that loads the library holds it until the process ends; all calls on a GPU share
 * it, so calls that could overlap on the GPU race -- order them on one stream.  The first
 * call on each GPU resolves the array's device address; issue it outside stream capture.
 * Calls no cudaMalloc/cudaFree.
 * ==================================================================================== */
int32_t wgf_full_reduce_f32_noalloc(const float* x, uint64_t n, uint32_t pre_opcode,
                                    uint32_t reduce_opcode, float* out, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* WGF_H */
