// extern "C" boundary (include/wgf.h).  Handles are small heap objects around the C++
// objects; every entry point converts exceptions into status codes.
#include <nvtx3/nvToolsExt.h>
#include <mutex>

#include "comm.hpp"
#include "graph.hpp"
#include "half.hpp"

using namespace wgf;

struct wgf_device {
    DeviceRef ref;
    std::atomic<int> rc{1};
};
struct wgf_buffer {
    BufferRef ref;
    std::atomic<int> rc{1};
};
struct wgf_tensor {
    NodeRef node;
};
struct wgf_comm {
    std::shared_ptr<Comm> ref;
};
// Event pairs of the kernels (or the copy) one call queued; read with wgf_timing_elapsed_ns.
struct wgf_timing {
    DeviceRef dev;
    std::vector<TimingRecord> recs;
};

namespace {

thread_local std::string g_last_error;
// Graph objects are not internally synchronised (neither are the crate's: its nodes hold
// non-Send closures); one lock serialises all graph-level calls.
std::recursive_mutex g_graph_mu;

template <typename F>
int32_t guard(F&& f) {
    try {
        f();
        return WGF_OK;
    } catch (const Error& e) {
        g_last_error = e.msg;
        return e.code;
    } catch (const std::bad_alloc&) {
        g_last_error = "host allocation failed";
        return WGF_ERR_OOM;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return WGF_ERR_INVALID_ARGUMENT;
    }
}

#define REQUIRE(p) WGF_CHECK((p) != nullptr, WGF_ERR_INVALID_HANDLE, "null handle or pointer: " #p)

wgf_tensor* wrap(const NodeRef& n) {
    auto* t = new wgf_tensor{n};
    n->handles++;
    return t;
}

std::vector<int64_t> vec(const int64_t* p, size_t n) { return std::vector<int64_t>(p, p + n); }

TensorData from_desc(const wgf_tensor_desc* d, bool owning) {
    REQUIRE(d);
    REQUIRE(d->buf);
    WGF_CHECK(valid_dtype(d->dtype), WGF_ERR_DTYPE, "unknown element type");
    WGF_CHECK(d->rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
    TensorData td;
    // A non-owning alias keeps the use count out of the in-place decision: at this level the
    // caller states whether the input may be overwritten.
    td.buf = owning ? d->buf->ref : BufferRef(BufferRef(), d->buf->ref.get());
    d->buf->ref->dev->note_recorded_buffer(d->buf->ref);   // a recording keeps the buffers its kernels touch
    td.dtype = (DType)d->dtype;
    td.layout.offset = d->offset;
    td.layout.shape = vec(d->shape, d->rank);
    td.layout.strides = vec(d->stride, d->rank);
    WGF_CHECK(d->offset >= 0, WGF_ERR_INVALID_ARGUMENT, "negative offset");
    for (uint32_t i = 0; i < d->rank; ++i)
        WGF_CHECK(d->shape[i] >= 0 && d->stride[i] >= 0, WGF_ERR_INVALID_ARGUMENT, "negative extent or stride");
    WGF_CHECK((uint64_t)td.layout.extent() * dtype_size(td.dtype) <= d->buf->ref->bytes, WGF_ERR_INVALID_ARGUMENT,
              "view reaches past the end of its buffer");
    return td;
}

void to_desc(const TensorData& td, wgf_buffer* reuse, wgf_tensor_desc* out) {
    std::memset(out, 0, sizeof *out);
    if (reuse) {
        reuse->rc++;
        out->buf = reuse;
    } else {
        out->buf = new wgf_buffer{td.buf};
    }
    out->dtype = (uint32_t)td.dtype;
    out->rank = (uint32_t)td.layout.rank();
    out->offset = td.layout.offset;
    for (int i = 0; i < td.layout.rank(); ++i) {
        out->shape[i] = td.layout.shape[i];
        out->stride[i] = td.layout.strides[i];
    }
}

int apply_chain(Program& p, int v, const wgf_ew_op* chain, uint32_t n) {
    WGF_CHECK(chain || !n, WGF_ERR_INVALID_ARGUMENT, "null chain with a non-zero length");
    for (uint32_t i = 0; i < n; ++i) {
        const wgf_ew_op& op = chain[i];
        if (op.opcode == WGF_OP_CAST) {
            WGF_CHECK(valid_dtype(op.out_dtype), WGF_ERR_DTYPE, "unknown element type in cast");
            v = p.cast(v, (DType)op.out_dtype);
        } else if (op.opcode >= WGF_OP_ADD_C && op.opcode <= WGF_OP_RDIV_C) {
            DType dt = p.ins[v].dtype;
            float c = dt == DType::F16 ? f16_to_f32(f32_to_f16(op.imm))
                                       : dt == DType::BF16 ? bf16_to_f32(f32_to_bf16(op.imm)) : op.imm;
            v = p.scalar(op.opcode, v, c);
        } else {
            WGF_CHECK(op.opcode <= WGF_OP_NEG, WGF_ERR_INVALID_ARGUMENT, "not an element-wise opcode");
            v = p.unary(op.opcode, v);
        }
    }
    return v;
}

// Runs `f` with a private timing sink.  With `timing` given, the event pairs of the kernels `f`
// queued go into a new handle; nothing waits (PerformanceQueries of the crate are read later too,
// src/query.rs:78-112).
template <typename F>
void timed(const DeviceRef& devref, wgf_timing** timing, F&& f) {
    Device& dev = *devref;
    std::unique_ptr<wgf_timing> t;
    if (timing) {
        *timing = nullptr;
        t.reset(new wgf_timing{devref, {}});
    }
    bool was = dev.timing;
    dev.timing = timing != nullptr;
    dev.sink = timing ? &t->recs : nullptr;
    try {
        f();
    } catch (...) {
        dev.sink = nullptr;
        dev.timing = was;
        if (t)
            for (auto& r : t->recs) {
                dev.recycle(r.start);
                dev.recycle(r.stop);
            }
        throw;
    }
    dev.sink = nullptr;
    dev.timing = was;
    if (timing) *timing = t.release();
}

}  // namespace

namespace wgf {
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace wgf

extern "C" {

const char* wgf_last_error(void) { return g_last_error.c_str(); }
int32_t wgf_abi_version(void) { return 2; }

// ---------------------------------------------------------------- device
int32_t wgf_device_create(int32_t ordinal, wgf_device** out) {
    return guard([&] {
        REQUIRE(out);
        *out = new wgf_device{Device::create(ordinal)};
    });
}
int32_t wgf_device_retain(wgf_device* dev) {
    return guard([&] {
        REQUIRE(dev);
        dev->rc++;
    });
}
int32_t wgf_device_release(wgf_device* dev) {
    return guard([&] {
        REQUIRE(dev);
        if (--dev->rc == 0) delete dev;
    });
}
int32_t wgf_device_sync(wgf_device* dev) {
    return guard([&] {
        REQUIRE(dev);
        dev->ref->sync();
    });
}
int32_t wgf_device_poll(wgf_device* dev) {
    return guard([&] { REQUIRE(dev); });
}
int32_t wgf_device_set_timing(wgf_device* dev, int32_t enabled) {
    return guard([&] {
        REQUIRE(dev);
        dev->ref->timing = enabled != 0;
    });
}
int32_t wgf_device_launch_count(wgf_device* dev, uint64_t* out) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        *out = dev->ref->launches.load();
    });
}
int32_t wgf_device_compile_count(wgf_device* dev, uint64_t* out) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        *out = dev->ref->compiles.load();
    });
}
int32_t wgf_device_memory(wgf_device* dev, uint64_t* reserved, uint64_t* in_use) {
    return guard([&] {
        REQUIRE(dev);
        if (reserved) *reserved = dev->ref->reserved_bytes();
        if (in_use) *in_use = dev->ref->in_use_bytes();
    });
}
int32_t wgf_device_info(wgf_device* dev, int32_t* sm_count, void** stream) {
    return guard([&] {
        REQUIRE(dev);
        if (sm_count) *sm_count = dev->ref->sm_count;
        if (stream) *stream = (void*)dev->ref->stream;
    });
}

// ---------------------------------------------------------------- buffers
int32_t wgf_buffer_alloc(wgf_device* dev, uint64_t bytes, int32_t zero, wgf_buffer** out) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        *out = new wgf_buffer{dev->ref->alloc((size_t)bytes, zero != 0)};
    });
}
int32_t wgf_buffer_retain(wgf_buffer* buf) {
    return guard([&] {
        REQUIRE(buf);
        buf->rc++;
    });
}
int32_t wgf_buffer_release(wgf_buffer* buf) {
    return guard([&] {
        REQUIRE(buf);
        if (--buf->rc == 0) delete buf;
    });
}
int32_t wgf_buffer_use_count(wgf_buffer* buf, int64_t* out) {
    return guard([&] {
        REQUIRE(buf);
        REQUIRE(out);
        *out = (int64_t)buf->ref.use_count() - 1 + buf->rc.load();
    });
}
int32_t wgf_buffer_upload(wgf_buffer* buf, uint64_t offset_bytes, const void* src, uint64_t bytes) {
    return guard([&] {
        REQUIRE(buf);
        WGF_CHECK(src || !bytes, WGF_ERR_INVALID_ARGUMENT, "null source");
        buf->ref->dev->upload(*buf->ref, offset_bytes, src, bytes);
    });
}
int32_t wgf_buffer_download(wgf_buffer* buf, uint64_t offset_bytes, void* dst, uint64_t bytes) {
    return guard([&] {
        REQUIRE(buf);
        WGF_CHECK(dst || !bytes, WGF_ERR_INVALID_ARGUMENT, "null destination");
        buf->ref->dev->download(*buf->ref, offset_bytes, dst, bytes);
    });
}
int32_t wgf_buffer_upload_async(wgf_buffer* buf, uint64_t offset_bytes, const void* src, uint64_t bytes,
                                wgf_timing** done) {
    return guard([&] {
        REQUIRE(buf);
        WGF_CHECK(src || !bytes, WGF_ERR_INVALID_ARGUMENT, "null source");
        if (done) *done = nullptr;
        Device& dev = *buf->ref->dev;
        TimingRecord rec;
        const bool copies = bytes && !dev.dry;
        dev.upload_async(*buf->ref, offset_bytes, src, bytes, done && copies ? &rec : nullptr);
        if (done) {
            std::unique_ptr<wgf_timing> t(new wgf_timing{buf->ref->dev, {}});
            if (copies) t->recs.push_back(rec);
            *done = t.release();
        }
    });
}
int32_t wgf_buffer_device_ptr(wgf_buffer* buf, void** ptr, uint64_t* bytes) {
    return guard([&] {
        REQUIRE(buf);
        // whoever uses the address works outside this library: what other streams still do to the
        // buffer is ordered before the device stream's next work, and an open all-reduce is finished
        if (buf->ref->dev && !buf->ref->dev->recording()) buf->ref->dev->wait_for(*buf->ref);
        if (ptr) *ptr = buf->ref->ptr;
        if (bytes) *bytes = buf->ref->bytes;
    });
}

int32_t wgf_host_alloc(uint64_t bytes, void** out) {
    return guard([&] {
        REQUIRE(out);
        WGF_CUDA(cudaHostAlloc(out, (size_t)std::max<uint64_t>(bytes, 1), cudaHostAllocDefault));
    });
}
int32_t wgf_host_free(void* ptr) {
    return guard([&] {
        if (ptr) WGF_CUDA(cudaFreeHost(ptr));
    });
}

// ---------------------------------------------------------------- timing handles
int32_t wgf_timing_elapsed_ns(wgf_timing* t, uint64_t* out_ns) {
    return guard([&] {
        REQUIRE(t);
        REQUIRE(out_ns);
        t->dev->make_current();
        double total = 0;
        for (auto& r : t->recs) {
            float ms = 0;
            WGF_CUDA(cudaEventSynchronize(r.stop));
            WGF_CUDA(cudaEventElapsedTime(&ms, r.start, r.stop));
            total += ms;
        }
        *out_ns = (uint64_t)(total * 1e6);
    });
}
int32_t wgf_timing_wait(wgf_timing* t) {
    return guard([&] {
        REQUIRE(t);
        t->dev->make_current();
        for (auto& r : t->recs) WGF_CUDA(cudaEventSynchronize(r.stop));
    });
}
int32_t wgf_timing_kernel_count(wgf_timing* t, uint32_t* out) {
    return guard([&] {
        REQUIRE(t);
        REQUIRE(out);
        *out = (uint32_t)t->recs.size();
    });
}
int32_t wgf_timing_release(wgf_timing* t) {
    return guard([&] {
        REQUIRE(t);
        for (auto& r : t->recs) {
            // an event still in flight may be re-recorded by its next user: wait for it first
            cudaEventSynchronize(r.stop);
            t->dev->recycle(r.start);
            t->dev->recycle(r.stop);
        }
        delete t;
    });
}

// ---------------------------------------------------------------- kernel-level launches
int32_t wgf_launch_elementwise(wgf_device* dev, const wgf_tensor_desc* in, const wgf_ew_op* chain,
                               uint32_t n_ops, int32_t inplace_ok, wgf_tensor_desc* out,
                               wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(chain || !n_ops, WGF_ERR_INVALID_ARGUMENT, "null chain");
        TensorData x = from_desc(in, !inplace_ok);
        Program p;
        int v = p.load(p.new_slot(x.dtype), x.dtype, VKind::Elem);
        p.result = apply_chain(p, v, chain, n_ops);
        TensorData y;
        timed(dev->ref, timing,
              [&] { y = run_elementwise(*dev->ref, p, {x}, x.layout.shape, inplace_ok ? 0 : -1); });
        bool aliased = y.buf.get() == in->buf->ref.get();
        to_desc(y, aliased ? in->buf : nullptr, out);
    });
}

int32_t wgf_launch_pairwise(wgf_device* dev, const wgf_tensor_desc* a, const wgf_tensor_desc* b,
                            const wgf_ew_op* pre_a, uint32_t n_pre_a, const wgf_ew_op* pre_b,
                            uint32_t n_pre_b, uint32_t opcode, const wgf_ew_op* post, uint32_t n_post,
                            wgf_tensor_desc* out, wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(opcode >= WGF_OP_ADD && opcode <= WGF_OP_POW, WGF_ERR_INVALID_ARGUMENT, "not a binary opcode");
        TensorData x = from_desc(a, true), y = from_desc(b, true);
        WGF_CHECK(x.layout.shape == y.layout.shape, WGF_ERR_SHAPE, "pairwise operands must have equal shapes");
        Program p;
        int va = apply_chain(p, p.load(p.new_slot(x.dtype), x.dtype, VKind::Elem), pre_a, n_pre_a);
        int vb = apply_chain(p, p.load(p.new_slot(y.dtype), y.dtype, VKind::Elem), pre_b, n_pre_b);
        WGF_CHECK(p.ins[va].dtype == p.ins[vb].dtype, WGF_ERR_DTYPE, "pairwise operands must have equal element types");
        p.result = apply_chain(p, p.binary((uint16_t)opcode, va, vb), post, n_post);
        TensorData z;
        timed(dev->ref, timing, [&] { z = run_elementwise(*dev->ref, p, {x, y}, x.layout.shape, -1); });
        to_desc(z, nullptr, out);
    });
}

int32_t wgf_launch_reduce(wgf_device* dev, const wgf_tensor_desc* in, uint32_t axis,
                          const wgf_ew_op* pre, uint32_t n_pre, uint32_t reduce_opcode,
                          const wgf_ew_op* post, uint32_t n_post, wgf_tensor_desc* out,
                          wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(reduce_opcode >= WGF_OP_SUM && reduce_opcode <= WGF_OP_PRODUCT, WGF_ERR_INVALID_ARGUMENT,
                  "not a reduce opcode");
        TensorData x = from_desc(in, true);
        WGF_CHECK((int)axis < x.layout.rank(), WGF_ERR_INVALID_ARGUMENT, "reduce axis out of range");
        // index space: reduced axis last
        Layout l = x.layout;
        l.shape.push_back(l.shape[axis]);
        l.strides.push_back(l.strides[axis]);
        l.shape.erase(l.shape.begin() + axis);
        l.strides.erase(l.strides.begin() + axis);
        x.layout = l;
        Program p;
        int v = apply_chain(p, p.load(p.new_slot(x.dtype), x.dtype, VKind::Elem), pre, n_pre);
        p.result = apply_chain(p, p.row_reduce((uint16_t)reduce_opcode, v), post, n_post);
        TensorData y;
        timed(dev->ref, timing, [&] { y = run_rows(*dev->ref, p, {x}, l.shape, false, -1); });
        to_desc(y, nullptr, out);
    });
}

int32_t wgf_launch_matmul(wgf_device* dev, const wgf_tensor_desc* a, const wgf_tensor_desc* b,
                          uint32_t acc_dtype, wgf_tensor_desc* out, wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(valid_dtype(acc_dtype), WGF_ERR_DTYPE, "unknown accumulator type");
        WGF_CHECK(acc_dtype == WGF_F32, WGF_ERR_UNSUPPORTED,
                  "matmul accumulates in f32 for every element type (tensor memory / FFMA): pass WGF_F32");
        TensorData x = from_desc(a, true), y = from_desc(b, true), z;
        timed(dev->ref, timing, [&] { z = run_matmul(*dev->ref, x, y); });
        to_desc(z, nullptr, out);
    });
}

int32_t wgf_launch_resize(wgf_device* dev, const wgf_tensor_desc* in, uint32_t new_rank,
                          const int64_t* new_shape, const int64_t* fill_shape, wgf_tensor_desc* out,
                          wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(out);
        REQUIRE(new_shape);
        REQUIRE(fill_shape);
        WGF_CHECK(new_rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
        TensorData x = from_desc(in, true);
        std::vector<int64_t> ns = vec(new_shape, new_rank), fs = vec(fill_shape, new_rank);
        int64_t nfill = 1;
        for (uint32_t i = 0; i < new_rank; ++i) {
            WGF_CHECK(fs[i] >= 0 && fs[i] <= ns[i], WGF_ERR_SHAPE, "fill box larger than the new shape");
            nfill *= fs[i];
        }
        WGF_CHECK(nfill == x.layout.numel(), WGF_ERR_SHAPE, "fill box and input differ in element count");
        Device& d = *dev->ref;
        TensorData y;
        timed(dev->ref, timing, [&] {
            y.dtype = x.dtype;
            y.layout = Layout::contiguous(ns);
            y.buf = d.alloc((size_t)std::max<int64_t>(y.layout.numel(), 1) * dtype_size(x.dtype), true);
            TensorData box = y;
            box.layout.shape = fs;
            TensorData src = x;
            if (src.layout.shape != fs) {  // reshape semantics: same row-major element order
                if (!src.layout.is_dense() || src.layout.allocation_overlaps()) src = run_compact(d, src);
                int64_t off = src.layout.offset;
                src.layout = Layout::contiguous(fs);
                src.layout.offset = off;
            }
            run_copy(d, box, src);
        });
        to_desc(y, nullptr, out);
    });
}

int32_t wgf_launch_slice_assign(wgf_device* dev, const wgf_tensor_desc* target, const int64_t* starts,
                                const int64_t* ends, const wgf_tensor_desc* value, wgf_timing** timing) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(starts);
        REQUIRE(ends);
        TensorData t = from_desc(target, true), v = from_desc(value, true);
        WGF_CHECK(t.layout.rank() == v.layout.rank(), WGF_ERR_RANK, "slice_assign ranks differ");
        ViewOp op;
        op.kind = ViewOp::Slice;
        op.starts = vec(starts, t.layout.rank());
        op.ends = vec(ends, t.layout.rank());
        for (int i = 0; i < t.layout.rank(); ++i)
            WGF_CHECK(starts[i] >= 0 && starts[i] <= ends[i] && ends[i] <= t.layout.shape[i], WGF_ERR_SHAPE,
                      "slice_assign range outside the target");
        TensorData window = t;
        window.layout = op.apply(t.layout);
        timed(dev->ref, timing, [&] { run_copy(*dev->ref, window, v); });
    });
}

// ---------------------------------------------------------------- graph-level
#define GRAPH_GUARD(...)                                        \
    return guard([&] {                                          \
        std::lock_guard<std::recursive_mutex> lk(g_graph_mu);   \
        __VA_ARGS__                                             \
    });

int32_t wgf_tensor_from_host(wgf_device* dev, uint32_t dtype, uint32_t rank, const int64_t* shape,
                             const void* data, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(valid_dtype(dtype), WGF_ERR_DTYPE, "unknown element type");
        WGF_CHECK(rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
        WGF_CHECK(shape || !rank, WGF_ERR_INVALID_ARGUMENT, "null shape");
        TensorData td;
        td.dtype = (DType)dtype;
        td.layout = Layout::contiguous(vec(shape, rank));
        for (auto s : td.layout.shape) WGF_CHECK(s >= 0, WGF_ERR_SHAPE, "negative extent");
        size_t bytes = (size_t)td.layout.numel() * dtype_size(td.dtype);
        WGF_CHECK(data || !bytes, WGF_ERR_INVALID_ARGUMENT, "null data");
        td.buf = dev->ref->alloc(std::max<size_t>(bytes, 1), false);
        if (bytes) dev->ref->upload(*td.buf, 0, data, bytes);
        *out = wrap(make_tensor(dev->ref, td));
    })
}

int32_t wgf_tensor_from_host_pinned(wgf_device* dev, uint32_t dtype, uint32_t rank, const int64_t* shape,
                                    const void* data, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(valid_dtype(dtype), WGF_ERR_DTYPE, "unknown element type");
        WGF_CHECK(rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
        WGF_CHECK(shape || !rank, WGF_ERR_INVALID_ARGUMENT, "null shape");
        TensorData td;
        td.dtype = (DType)dtype;
        td.layout = Layout::contiguous(vec(shape, rank));
        for (auto s : td.layout.shape) WGF_CHECK(s >= 0, WGF_ERR_SHAPE, "negative extent");
        size_t bytes = (size_t)td.layout.numel() * dtype_size(td.dtype);
        WGF_CHECK(data || !bytes, WGF_ERR_INVALID_ARGUMENT, "null data");
        td.buf = dev->ref->alloc(std::max<size_t>(bytes, 1), false);
        if (bytes) dev->ref->upload_async(*td.buf, 0, data, bytes);
        *out = wrap(make_tensor(dev->ref, td));
    })
}

int32_t wgf_tensor_from_desc(wgf_device* dev, const wgf_tensor_desc* desc, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(dev);
        REQUIRE(out);
        *out = wrap(make_tensor(dev->ref, from_desc(desc, true)));
    })
}

int32_t wgf_tensor_arange(wgf_device* dev, uint32_t dtype, float start, float end, float step,
                          wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(dev);
        REQUIRE(out);
        WGF_CHECK(valid_dtype(dtype), WGF_ERR_DTYPE, "unknown element type");
        WGF_CHECK(step != 0.f && step == step, WGF_ERR_INVALID_ARGUMENT, "arange step must be non-zero");
        // src/composite/arange.rs:8-23: accumulate in the tensor's own element type
        std::vector<float> vals;
        auto rnd = [&](float v) {
            return dtype == WGF_F16 ? f16_to_f32(f32_to_f16(v)) : dtype == WGF_BF16 ? bf16_to_f32(f32_to_bf16(v)) : v;
        };
        float cur = rnd(start), e = rnd(end), st = rnd(step);
        WGF_CHECK(st != 0.f, WGF_ERR_INVALID_ARGUMENT, "arange step rounds to zero in this element type");
        while (st >= 0 ? cur < e : cur > e) {
            vals.push_back(cur);
            float next = rnd(cur + st);
            WGF_CHECK(next != cur, WGF_ERR_INVALID_ARGUMENT, "arange step is absorbed by rounding");
            WGF_CHECK(vals.size() < (1u << 28), WGF_ERR_OOM, "arange too long");
            cur = next;
        }
        TensorData td;
        td.dtype = (DType)dtype;
        td.layout = Layout::contiguous({(int64_t)vals.size()});
        size_t bytes = vals.size() * dtype_size(td.dtype);
        td.buf = dev->ref->alloc(std::max<size_t>(bytes, 1), false);
        if (dtype == WGF_F32) {
            if (bytes) dev->ref->upload(*td.buf, 0, vals.data(), bytes);
        } else {
            std::vector<uint16_t> h(vals.size());
            for (size_t i = 0; i < vals.size(); ++i) h[i] = dtype == WGF_F16 ? f32_to_f16(vals[i]) : f32_to_bf16(vals[i]);
            if (bytes) dev->ref->upload(*td.buf, 0, h.data(), bytes);
        }
        *out = wrap(make_tensor(dev->ref, td));
    })
}

int32_t wgf_tensor_clone(wgf_tensor* t, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(t->node);
    })
}

int32_t wgf_tensor_release(wgf_tensor* t) {
    GRAPH_GUARD({
        REQUIRE(t);
        t->node->handles--;
        delete t;
    })
}

int32_t wgf_tensor_info(wgf_tensor* t, uint32_t* dtype, uint32_t* rank, int64_t* shape) {
    GRAPH_GUARD({
        REQUIRE(t);
        if (dtype) *dtype = (uint32_t)t->node->dtype;
        if (rank) *rank = (uint32_t)t->node->rank();
        if (shape)
            for (int i = 0; i < t->node->rank(); ++i) shape[i] = t->node->shape[i];
    })
}

int32_t wgf_tensor_unary(wgf_tensor* t, uint32_t opcode, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(make_unary(t->node, (uint16_t)opcode));
    })
}
int32_t wgf_tensor_scalar(wgf_tensor* t, uint32_t opcode, float c, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(make_scalar(t->node, (uint16_t)opcode, c));
    })
}
int32_t wgf_tensor_cast(wgf_tensor* t, uint32_t dtype, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        WGF_CHECK(valid_dtype(dtype), WGF_ERR_DTYPE, "unknown element type");
        *out = wrap(make_cast(t->node, (DType)dtype));
    })
}
int32_t wgf_tensor_binary(wgf_tensor* a, wgf_tensor* b, uint32_t opcode, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(a);
        REQUIRE(b);
        REQUIRE(out);
        *out = wrap(make_binary(a->node, b->node, (uint16_t)opcode));
    })
}
int32_t wgf_tensor_reduce(wgf_tensor* t, uint32_t opcode, uint32_t axis, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(make_reduce(t->node, (uint16_t)opcode, (int)axis));
    })
}
int32_t wgf_tensor_matmul(wgf_tensor* a, wgf_tensor* b, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(a);
        REQUIRE(b);
        REQUIRE(out);
        *out = wrap(make_matmul(a->node, b->node));
    })
}
int32_t wgf_tensor_slice(wgf_tensor* t, const int64_t* starts, const int64_t* ends, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(starts);
        REQUIRE(ends);
        REQUIRE(out);
        *out = wrap(view_slice(t->node, vec(starts, t->node->rank()), vec(ends, t->node->rank())));
    })
}
int32_t wgf_tensor_transpose(wgf_tensor* t, uint32_t axis_a, uint32_t axis_b, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(view_transpose(t->node, (int)axis_a, (int)axis_b));
    })
}
int32_t wgf_tensor_broadcast(wgf_tensor* t, uint32_t out_rank, const int64_t* out_shape, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out_shape);
        REQUIRE(out);
        WGF_CHECK(out_rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
        *out = wrap(view_broadcast(t->node, vec(out_shape, out_rank)));
    })
}
int32_t wgf_tensor_broadcast_axis(wgf_tensor* t, uint32_t axis, int64_t size, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(view_broadcast_axis(t->node, (int)axis, size));
    })
}
int32_t wgf_tensor_expand(wgf_tensor* t, const int64_t* out_shape, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out_shape);
        REQUIRE(out);
        *out = wrap(view_expand(t->node, vec(out_shape, t->node->rank())));
    })
}
int32_t wgf_tensor_resize(wgf_tensor* t, const int64_t* new_shape, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(new_shape);
        REQUIRE(out);
        std::vector<int64_t> ns = vec(new_shape, t->node->rank());
        for (int i = 0; i < t->node->rank(); ++i)
            WGF_CHECK(ns[i] >= t->node->shape[i], WGF_ERR_SHAPE, "resize cannot shrink an axis");
        *out = wrap(make_resize(t->node, ns, t->node->shape));
    })
}
int32_t wgf_tensor_reshape(wgf_tensor* t, uint32_t new_rank, const int64_t* new_shape, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        WGF_CHECK(new_shape || !new_rank, WGF_ERR_INVALID_ARGUMENT, "null shape");
        WGF_CHECK(new_rank <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
        *out = wrap(op_reshape(t->node, vec(new_shape, new_rank)));
    })
}
int32_t wgf_tensor_slice_assign(wgf_tensor* target, const int64_t* starts, const int64_t* ends,
                                wgf_tensor* value, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(target);
        REQUIRE(value);
        REQUIRE(starts);
        REQUIRE(ends);
        REQUIRE(out);
        int r = target->node->rank();
        *out = wrap(make_slice_assign(target->node, vec(starts, r), vec(ends, r), value->node));
    })
}
int32_t wgf_tensor_cat(wgf_tensor* const* parts, uint32_t n_parts, uint32_t dim, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(parts);
        REQUIRE(out);
        std::vector<NodeRef> v;
        for (uint32_t i = 0; i < n_parts; ++i) {
            REQUIRE(parts[i]);
            v.push_back(parts[i]->node);
        }
        *out = wrap(op_cat(v, (int)dim));
    })
}
int32_t wgf_tensor_narrow(wgf_tensor* t, uint32_t axis, int64_t start, int64_t length, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(op_narrow(t->node, (int)axis, start, length));
    })
}
int32_t wgf_tensor_unsqueeze(wgf_tensor* t, uint32_t axis, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(op_unsqueeze(t->node, (int)axis));
    })
}
int32_t wgf_tensor_silu(wgf_tensor* t, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(op_silu(t->node));
    })
}
int32_t wgf_tensor_layer_norm(wgf_tensor* t, wgf_tensor* weight, float eps, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(weight);
        REQUIRE(out);
        *out = wrap(op_layer_norm(t->node, weight->node, eps));
    })
}
int32_t wgf_tensor_softmax(wgf_tensor* t, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(op_softmax(t->node));
    })
}
int32_t wgf_tensor_softmax_last_dim(wgf_tensor* t, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        *out = wrap(op_softmax_last_dim(t->node));
    })
}
int32_t wgf_tensor_rope(wgf_tensor* t, wgf_tensor* cos, wgf_tensor* sin, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(cos);
        REQUIRE(sin);
        REQUIRE(out);
        *out = wrap(op_rope(t->node, cos->node, sin->node));
    })
}

int32_t wgf_tensor_llama_block(wgf_tensor* x, wgf_tensor* const* weights, wgf_tensor* norm1, wgf_tensor* norm2,
                               wgf_tensor* cos, wgf_tensor* sin, wgf_tensor* mask, uint32_t n_heads, float eps,
                               wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(x);
        REQUIRE(weights);
        REQUIRE(norm1);
        REQUIRE(norm2);
        REQUIRE(cos);
        REQUIRE(sin);
        REQUIRE(out);
        for (int i = 0; i < 7; ++i) REQUIRE(weights[i]);
        *out = wrap(op_llama_block(x->node, weights[0]->node, weights[1]->node, weights[2]->node, weights[3]->node,
                                   weights[4]->node, weights[5]->node, weights[6]->node, norm1->node, norm2->node,
                                   cos->node, sin->node, mask ? mask->node : NodeRef(), (int)n_heads, eps));
    })
}

int32_t wgf_tensor_attention(wgf_tensor* q, wgf_tensor* k, wgf_tensor* v, wgf_tensor* mask, int32_t causal, float scale,
                             wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(q);
        REQUIRE(k);
        REQUIRE(v);
        REQUIRE(out);
        *out = wrap(op_attention(q->node, k->node, v->node, mask ? mask->node : NodeRef(), causal != 0, scale));
    })
}

namespace {
// WGF_NVTX=1: one range per materialisation request around the ranges of its kernels.
struct NvtxRange {
    bool on;
    explicit NvtxRange(const char* name) {
        static const bool enabled = getenv("WGF_NVTX") != nullptr;
        on = enabled;
        if (on) nvtxRangePushA(name);
    }
    ~NvtxRange() {
        if (on) nvtxRangePop();
    }
};
}  // namespace

int32_t wgf_tensor_materialize(wgf_tensor* t) {
    NvtxRange range("wgf materialize");
    GRAPH_GUARD({
        REQUIRE(t);
        resolve(t->node);
    })
}

int32_t wgf_tensor_materialize_many(wgf_tensor* const* tensors, uint32_t n) {
    NvtxRange range("wgf materialize_many");
    GRAPH_GUARD({
        if (n > 0) REQUIRE(tensors);
        std::vector<NodeRef> nodes;
        for (uint32_t i = 0; i < n; ++i) {
            REQUIRE(tensors[i]);
            nodes.push_back(tensors[i]->node);
        }
        resolve_many(nodes);
    })
}

int32_t wgf_tensor_desc_of(wgf_tensor* t, wgf_tensor_desc* out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(out);
        TensorData td = resolve(t->node);
        to_desc(td, nullptr, out);
    })
}

int32_t wgf_tensor_download(wgf_tensor* t, void* dst, uint64_t bytes) {
    GRAPH_GUARD({
        REQUIRE(t);
        TensorData td = resolve(t->node);
        uint64_t need = (uint64_t)td.layout.numel() * dtype_size(td.dtype);
        WGF_CHECK(bytes == need, WGF_ERR_INVALID_ARGUMENT,
                  "destination size " + std::to_string(bytes) + " differs from the tensor's " + std::to_string(need));
        WGF_CHECK(dst || !need, WGF_ERR_INVALID_ARGUMENT, "null destination");
        Device& dev = *t->node->dev;
        if (!td.layout.is_dense() || td.layout.allocation_overlaps()) td = run_compact(dev, td);
        dev.download(*td.buf, (size_t)td.layout.offset * dtype_size(td.dtype), dst, (size_t)need);
    })
}

int32_t wgf_tensor_timing(wgf_tensor* t, uint64_t* out_ns, uint32_t capacity, uint32_t* count) {
    GRAPH_GUARD({
        REQUIRE(t);
        auto g = graph_of(t->node);
        if (count) *count = (uint32_t)g->timings.size();
        if (!out_ns) return;
        uint32_t n = std::min<uint32_t>(capacity, (uint32_t)g->timings.size());
        t->node->dev->make_current();
        for (uint32_t i = 0; i < n; ++i) {
            float ms = 0;
            WGF_CUDA(cudaEventSynchronize(g->timings[i].stop));
            WGF_CUDA(cudaEventElapsedTime(&ms, g->timings[i].start, g->timings[i].stop));
            out_ns[i] = (uint64_t)((double)ms * 1e6);
        }
    })
}

int32_t wgf_tensor_timing_labels(wgf_tensor* t, char* dst, uint64_t capacity, uint64_t* needed) {
    GRAPH_GUARD({
        REQUIRE(t);
        std::string s;
        for (auto& r : graph_of(t->node)->timings) {
            s += r.what;
            s += '\n';
        }
        if (needed) *needed = s.size() + 1;
        if (dst && capacity) {
            size_t n = std::min<size_t>(s.size(), (size_t)capacity - 1);
            std::memcpy(dst, s.data(), n);
            dst[n] = 0;
        }
    })
}

int32_t wgf_tensor_graphviz(wgf_tensor* t, char* dst, uint64_t capacity, uint64_t* needed) {
    GRAPH_GUARD({
        REQUIRE(t);
        std::string s = graphviz(t->node);
        if (needed) *needed = s.size() + 1;
        if (dst && capacity) {
            size_t n = std::min<size_t>(s.size(), (size_t)capacity - 1);
            std::memcpy(dst, s.data(), n);
            dst[n] = 0;
        }
    })
}

int32_t wgf_tensor_graph_size(wgf_tensor* t, uint64_t* nodes) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(nodes);
        *nodes = graph_of(t->node)->live_nodes;
    })
}

// ---------------------------------------------------------------- multi-GPU
int32_t wgf_shard_range(int64_t n_units, int32_t world, int32_t rank, int64_t* begin, int64_t* end) {
    return guard([&] {
        REQUIRE(begin);
        REQUIRE(end);
        WGF_CHECK(n_units >= 0 && world >= 1 && rank >= 0 && rank < world, WGF_ERR_INVALID_ARGUMENT,
                  "bad unit count / world size / rank");
        shard_range(n_units, world, rank, *begin, *end);
    });
}
int32_t wgf_comm_unique_id(uint8_t id[WGF_COMM_ID_BYTES]) {
    return guard([&] {
        REQUIRE(id);
        comm_unique_id(id);
    });
}
int32_t wgf_comm_create(wgf_device* dev, int32_t world, int32_t rank, const uint8_t id[WGF_COMM_ID_BYTES],
                        wgf_comm** out) {
    return guard([&] {
        REQUIRE(dev);
        REQUIRE(id);
        REQUIRE(out);
        *out = new wgf_comm{comm_create(dev->ref, world, rank, id)};
    });
}
int32_t wgf_comm_release(wgf_comm* comm) {
    return guard([&] {
        REQUIRE(comm);
        delete comm;
    });
}
// ---- recorded schedules --------------------------------------------------------------------
struct wgf_schedule {
    DeviceRef dev;
    Device::Recorded rec;
};

int32_t wgf_schedule_begin(wgf_device* dev) {
    GRAPH_GUARD({
        REQUIRE(dev);
        dev->ref->begin_recording();
    })
}
int32_t wgf_schedule_end(wgf_device* dev, wgf_schedule** out) {
    GRAPH_GUARD({
        REQUIRE(dev);
        REQUIRE(out);
        *out = nullptr;
        Device::Recorded rec = dev->ref->end_recording();
        *out = new wgf_schedule{dev->ref, rec};
    })
}
int32_t wgf_schedule_launch(wgf_schedule* s) {
    GRAPH_GUARD({
        REQUIRE(s);
        s->dev->replay(s->rec);
    })
}
int32_t wgf_schedule_kernel_count(wgf_schedule* s, uint64_t* out) {
    return guard([&] {
        REQUIRE(s);
        REQUIRE(out);
        *out = s->rec.kernels;
    });
}
int32_t wgf_schedule_destroy(wgf_schedule* s) {
    GRAPH_GUARD({
        REQUIRE(s);
        s->dev->destroy_recorded(s->rec);
        delete s;
    })
}

int32_t wgf_tensor_all_reduce(wgf_tensor* t, wgf_comm* comm, uint32_t opcode, wgf_tensor** out) {
    GRAPH_GUARD({
        REQUIRE(t);
        REQUIRE(comm);
        REQUIRE(out);
        *out = wrap(make_all_reduce(t->node, comm->ref, (uint16_t)opcode));
    })
}

}  // extern "C"
