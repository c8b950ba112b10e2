// C++17 mirror of the crate's public API (`Tensor<R, D>`, `Device`, `TensorSlice`; src/lib.rs:1-11)
// over the C ABI in wgf.h.  Header only; link with libwgf.so.  Rank and element type are
// compile-time parameters as in the crate (`Tensor<const R: usize, D: DataType>`,
// src/tensor.rs:418-430); misuse that the crate rejects with `assert!` throws wgf::Error here.
//
//   wgf::Device dev;                                       // Device::new().await
//   auto t = wgf::Tensor<2, float>::from_rows(dev, {{1, 2}, {3, 4}});
//   auto y = (t + 1.0f).sum(0);                            // lazy
//   auto s = y.as_slice();                                 // resolves, downloads
//   float v = s[{0}];
#pragma once
#include <array>
#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../wgf.h"

namespace wgf {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
inline void check(int32_t status) {
    if (status != WGF_OK) throw Error(status, wgf_last_error());
}

// IEEE binary16 / bfloat16 storage types (the crate uses half::f16; values are bit patterns).
struct f16 { uint16_t bits; };
struct bf16 { uint16_t bits; };

// DataType trait, src/tensor.rs:22-65
template <typename D> struct DataType;
template <> struct DataType<float> { static constexpr uint32_t code = WGF_F32; };
template <> struct DataType<f16> { static constexpr uint32_t code = WGF_F16; };
template <> struct DataType<bf16> { static constexpr uint32_t code = WGF_BF16; };

// Device, src/device.rs:8-52
class Device {
   public:
    explicit Device(int ordinal = 0) { check(wgf_device_create(ordinal, &h_)); }
    Device(const Device& o) : h_(o.h_) { check(wgf_device_retain(h_)); }
    Device& operator=(const Device& o) {
        if (this != &o) {
            check(wgf_device_retain(o.h_));
            if (h_) wgf_device_release(h_);
            h_ = o.h_;
        }
        return *this;
    }
    ~Device() {
        if (h_) wgf_device_release(h_);
    }
    void sync() const { check(wgf_device_sync(h_)); }
    void poll() const { check(wgf_device_poll(h_)); }   // kept for callers of wgpu_device().poll()
    uint64_t launch_count() const {
        uint64_t n = 0;
        check(wgf_device_launch_count(h_, &n));
        return n;
    }
    wgf_device* raw() const { return h_; }

   private:
    wgf_device* h_ = nullptr;
};

// A recorded schedule (wgf_schedule_*).  Everything materialised between construction and
// finish() is captured instead of run; launch() replays it with one call.
//     wgf::Schedule s(dev);  auto y = f(x);  y.materialize();  s.finish();
//     for (...) { x.write(host_data);  s.launch();  y.as_slice(); }
class Schedule {
   public:
    explicit Schedule(const Device& dev) : dev_(dev) { check(wgf_schedule_begin(dev_.raw())); }
    Schedule(const Schedule&) = delete;
    Schedule& operator=(const Schedule&) = delete;
    ~Schedule() {
        if (recording_) {
            wgf_schedule* dropped = nullptr;
            if (wgf_schedule_end(dev_.raw(), &dropped) == WGF_OK) wgf_schedule_destroy(dropped);
        }
        if (h_) wgf_schedule_destroy(h_);
    }
    void finish() {
        recording_ = false;
        check(wgf_schedule_end(dev_.raw(), &h_));
    }
    void launch() const { check(wgf_schedule_launch(h_)); }
    uint64_t kernel_count() const {
        uint64_t n = 0;
        check(wgf_schedule_kernel_count(h_, &n));
        return n;
    }

   private:
    Device dev_;
    wgf_schedule* h_ = nullptr;
    bool recording_ = true;
};

// TensorSlice, src/tensor.rs:669-855: host copy of a materialised tensor with index access.
template <int R, typename D>
class TensorSlice {
   public:
    TensorSlice(std::array<int64_t, R> shape, std::vector<D> data) : shape_(shape), data_(std::move(data)) {}
    const std::array<int64_t, R>& shape() const { return shape_; }
    const D& operator[](const std::array<int64_t, R>& idx) const { return data_[offset(idx)]; }
    const D* get(const std::array<int64_t, R>& idx) const {
        for (int i = 0; i < R; ++i)
            if (idx[i] < 0 || idx[i] >= shape_[i]) return nullptr;
        return &data_[offset(idx)];
    }
    const std::vector<D>& data() const { return data_; }
    bool operator==(const TensorSlice& o) const {
        if (shape_ != o.shape_) return false;
        for (size_t i = 0; i < data_.size(); ++i)
            if (!same(data_[i], o.data_[i])) return false;
        return true;
    }

   private:
    static bool same(float a, float b) { return a == b; }
    static bool same(f16 a, f16 b) { return a.bits == b.bits; }
    static bool same(bf16 a, bf16 b) { return a.bits == b.bits; }
    size_t offset(const std::array<int64_t, R>& idx) const {
        size_t off = 0;
        for (int i = 0; i < R; ++i) off = off * (size_t)shape_[i] + (size_t)idx[i];
        return off;
    }
    std::array<int64_t, R> shape_;
    std::vector<D> data_;
};

template <int R, typename D>
class Tensor {
    static_assert(R >= 0 && R <= WGF_MAX_RANK, "rank 0..8");

   public:
    using Shape = std::array<int64_t, R>;
    using Range = std::pair<int64_t, int64_t>;   // start..end, as Rust's Range<usize>

    // ---- construction: Tensor::new, src/tensor.rs:518-531 (row-major data) --------------
    Tensor(const Device& dev, const Shape& shape, const D* data) {
        check(wgf_tensor_from_host(dev.raw(), DataType<D>::code, R, shape.data(), data, &h_));
    }
    static Tensor from_values(const Device& dev, std::initializer_list<D> v) {
        static_assert(R == 1, "flat list makes a rank-1 tensor");
        std::vector<D> d(v);
        return Tensor(dev, Shape{(int64_t)d.size()}, d.data());
    }
    static Tensor from_rows(const Device& dev, std::initializer_list<std::initializer_list<D>> v) {
        static_assert(R == 2, "nested list of depth 2 makes a rank-2 tensor");
        std::vector<D> d;
        int64_t cols = v.size() ? (int64_t)v.begin()->size() : 0;
        for (auto& row : v) {
            if ((int64_t)row.size() != cols) throw Error(WGF_ERR_SHAPE, "ragged rows");
            d.insert(d.end(), row.begin(), row.end());
        }
        return Tensor(dev, Shape{(int64_t)v.size(), cols}, d.data());
    }
    // Tensor::arange / arange_step, src/composite/arange.rs:4-23
    static Tensor arange(const Device& dev, float start, float end, float step = 1.f) {
        static_assert(R == 1, "arange makes a rank-1 tensor");
        wgf_tensor* out = nullptr;
        check(wgf_tensor_arange(dev.raw(), DataType<D>::code, start, end, step, &out));
        return Tensor(out);
    }

    Tensor(const Tensor& o) { check(wgf_tensor_clone(o.h_, &h_)); }   // Clone, src/tensor.rs:432-439
    Tensor(Tensor&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    Tensor& operator=(Tensor o) noexcept {
        std::swap(h_, o.h_);
        return *this;
    }
    ~Tensor() {
        if (h_) wgf_tensor_release(h_);
    }

    // ---- introspection: src/tensor.rs:629-643 -------------------------------------------
    Shape shape() const {
        Shape s{};
        int64_t tmp[WGF_MAX_RANK];
        uint32_t rank = 0;
        check(wgf_tensor_info(h_, nullptr, &rank, tmp));
        for (int i = 0; i < R; ++i) s[i] = tmp[i];
        return s;
    }
    static constexpr int rank() { return R; }
    std::string graphvis() const {
        uint64_t need = 0;
        check(wgf_tensor_graphviz(h_, nullptr, 0, &need));
        std::string s(need, '\0');
        check(wgf_tensor_graphviz(h_, &s[0], need, &need));
        s.resize(need ? need - 1 : 0);
        return s;
    }

    // ---- materialise: as_slice / all_timing_information, src/tensor.rs:551-558 -----------
    TensorSlice<R, D> as_slice() const {
        Shape s = shape();
        size_t n = 1;
        for (auto v : s) n *= (size_t)v;
        std::vector<D> host(n);
        check(wgf_tensor_download(h_, host.data(), n * sizeof(D)));
        return TensorSlice<R, D>(s, std::move(host));
    }
    // New contents (row-major, numel values) for a materialised contiguous tensor, written into
    // the buffer it already has: the way to feed the inputs of a recorded schedule.
    void write(const D* values) const {
        wgf_tensor_desc d;
        check(wgf_tensor_desc_of(h_, &d));
        size_t n = 1;
        bool dense = true;
        for (int i = R - 1; i >= 0; --i) {
            dense = dense && (d.shape[i] <= 1 || d.stride[i] == (int64_t)n);
            n *= (size_t)d.shape[i];
        }
        int32_t st = dense ? wgf_buffer_upload(d.buf, (uint64_t)d.offset * sizeof(D), values, n * sizeof(D))
                           : (int32_t)WGF_ERR_UNSUPPORTED;
        wgf_buffer_release(d.buf);
        if (!dense) throw Error(WGF_ERR_UNSUPPORTED, "write needs a contiguous tensor");
        check(st);
    }
    std::vector<uint64_t> all_timing_information() const {
        uint32_t n = 0;
        check(wgf_tensor_timing(h_, nullptr, 0, &n));
        std::vector<uint64_t> ns(n);
        if (n) check(wgf_tensor_timing(h_, ns.data(), n, &n));
        return ns;
    }

    // ---- scalar ops: src/element_wise.rs:197-651 ------------------------------------------
    friend Tensor operator+(const Tensor& t, float c) { return t.scalar(WGF_OP_ADD_C, c); }
    friend Tensor operator+(float c, const Tensor& t) { return t.scalar(WGF_OP_ADD_C, c); }
    friend Tensor operator-(const Tensor& t, float c) { return t.scalar(WGF_OP_SUB_C, c); }
    friend Tensor operator-(float c, const Tensor& t) { return t.scalar(WGF_OP_RSUB_C, c); }
    friend Tensor operator*(const Tensor& t, float c) { return t.scalar(WGF_OP_MUL_C, c); }
    friend Tensor operator*(float c, const Tensor& t) { return t.scalar(WGF_OP_MUL_C, c); }
    friend Tensor operator/(const Tensor& t, float c) { return t.scalar(WGF_OP_DIV_C, c); }
    friend Tensor operator/(float c, const Tensor& t) { return t.scalar(WGF_OP_RDIV_C, c); }
    Tensor operator-() const { return unary(WGF_OP_NEG); }   // Neg, :1370-1380

    // ---- unary: src/element_wise.rs:678-1342 ----------------------------------------------
    Tensor exp() const { return unary(WGF_OP_EXP); }
    Tensor exp2() const { return unary(WGF_OP_EXP2); }
    Tensor log() const { return unary(WGF_OP_LOG); }
    Tensor log2() const { return unary(WGF_OP_LOG2); }
    Tensor sqr() const { return unary(WGF_OP_SQR); }
    Tensor sqrt() const { return unary(WGF_OP_SQRT); }
    Tensor sin() const { return unary(WGF_OP_SIN); }
    Tensor cos() const { return unary(WGF_OP_COS); }
    Tensor tan() const { return unary(WGF_OP_TAN); }
    Tensor asin() const { return unary(WGF_OP_ASIN); }
    Tensor acos() const { return unary(WGF_OP_ACOS); }
    Tensor atan() const { return unary(WGF_OP_ATAN); }
    Tensor sinh() const { return unary(WGF_OP_SINH); }
    Tensor cosh() const { return unary(WGF_OP_COSH); }
    Tensor tanh() const { return unary(WGF_OP_TANH); }
    Tensor asinh() const { return unary(WGF_OP_ASINH); }
    Tensor acosh() const { return unary(WGF_OP_ACOSH); }
    Tensor atanh() const { return unary(WGF_OP_ATANH); }
    Tensor abs() const { return unary(WGF_OP_ABS); }

    // CastTensor::cast, src/element_wise.rs:1408-1471
    template <typename D2> Tensor<R, D2> cast() const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_cast(h_, DataType<D2>::code, &out));
        return Tensor<R, D2>(out);
    }

    // ---- pair-wise: src/pair_wise.rs:205-528 ----------------------------------------------
    friend Tensor operator+(const Tensor& a, const Tensor& b) { return a.binary(b, WGF_OP_ADD); }
    friend Tensor operator-(const Tensor& a, const Tensor& b) { return a.binary(b, WGF_OP_SUB); }
    friend Tensor operator*(const Tensor& a, const Tensor& b) { return a.binary(b, WGF_OP_MUL); }
    friend Tensor operator/(const Tensor& a, const Tensor& b) { return a.binary(b, WGF_OP_DIV); }
    Tensor pow(const Tensor& o) const { return binary(o, WGF_OP_POW); }

    // ---- reductions to rank R-1: src/reduce.rs:433-815 -------------------------------------
    Tensor<R - 1, D> sum(int axis) const { return reduce(WGF_OP_SUM, axis); }
    Tensor<R - 1, D> max(int axis) const { return reduce(WGF_OP_MAX, axis); }
    Tensor<R - 1, D> min(int axis) const { return reduce(WGF_OP_MIN, axis); }
    Tensor<R - 1, D> product(int axis) const { return reduce(WGF_OP_PRODUCT, axis); }

    // mat_mul, src/matmul.rs:25-29 (rank 2; rank 3 = batched)
    Tensor mat_mul(const Tensor& o) const {
        static_assert(R == 2 || R == 3, "mat_mul takes rank 2, or rank 3 (batched)");
        wgf_tensor* out = nullptr;
        check(wgf_tensor_matmul(h_, o.h_, &out));
        return Tensor(out);
    }

    // ---- views: src/map_layout.rs:41-98 ----------------------------------------------------
    Tensor slice(const std::array<Range, R>& ranges) const {
        int64_t s[R > 0 ? R : 1], e[R > 0 ? R : 1];
        for (int i = 0; i < R; ++i) {
            s[i] = ranges[i].first;
            e[i] = ranges[i].second;
        }
        wgf_tensor* out = nullptr;
        check(wgf_tensor_slice(h_, s, e, &out));
        return Tensor(out);
    }
    Tensor transpose(int a, int b) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_transpose(h_, (uint32_t)a, (uint32_t)b, &out));
        return Tensor(out);
    }
    Tensor<R + 1, D> broadcast(const std::array<int64_t, R + 1>& out_shape) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_broadcast(h_, R + 1, out_shape.data(), &out));
        return Tensor<R + 1, D>(out);
    }
    Tensor narrow(int axis, int64_t start, int64_t length) const {   // src/composite/narrow.rs:4-15
        wgf_tensor* out = nullptr;
        check(wgf_tensor_narrow(h_, (uint32_t)axis, start, length, &out));
        return Tensor(out);
    }

    // ---- moves: src/resize.rs:121-144, src/slice_assign.rs:76-79, src/composite/ -------------
    Tensor resize(const Shape& new_shape) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_resize(h_, new_shape.data(), &out));
        return Tensor(out);
    }
    template <size_t R2> Tensor<(int)R2, D> reshape(const std::array<int64_t, R2>& new_shape) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_reshape(h_, (uint32_t)R2, new_shape.data(), &out));
        return Tensor<(int)R2, D>(out);
    }
    Tensor slice_assign(const std::array<Range, R>& ranges, const Tensor& value) const {
        int64_t s[R > 0 ? R : 1], e[R > 0 ? R : 1];
        for (int i = 0; i < R; ++i) {
            s[i] = ranges[i].first;
            e[i] = ranges[i].second;
        }
        wgf_tensor* out = nullptr;
        check(wgf_tensor_slice_assign(h_, s, e, value.h_, &out));
        return Tensor(out);
    }
    static Tensor cat(const std::vector<Tensor>& parts, int dim) {   // src/composite/cat.rs:4-40
        std::vector<wgf_tensor*> raw;
        for (auto& p : parts) raw.push_back(p.h_);
        wgf_tensor* out = nullptr;
        check(wgf_tensor_cat(raw.data(), (uint32_t)raw.size(), (uint32_t)dim, &out));
        return Tensor(out);
    }
    Tensor<R + 1, D> unsqueeze(int axis) const {   // src/composite/unsqueeze.rs:16-53
        wgf_tensor* out = nullptr;
        check(wgf_tensor_unsqueeze(h_, (uint32_t)axis, &out));
        return Tensor<R + 1, D>(out);
    }

    // ---- composites: src/composite/ ----------------------------------------------------------
    Tensor silu() const { return unary_call(wgf_tensor_silu); }
    Tensor layer_norm(const Tensor<1, D>& weight, float eps) const {   // RmsNorm, rms_norm.rs:8-15
        wgf_tensor* out = nullptr;
        check(wgf_tensor_layer_norm(h_, weight.raw(), eps, &out));
        return Tensor(out);
    }
    Tensor rms_norm(const Tensor<1, D>& weight, float eps) const { return layer_norm(weight, eps); }
    Tensor softmax() const {   // softmax.rs:4-10
        static_assert(R == 1, "softmax takes rank 1 (see softmax_last_dim)");
        return unary_call(wgf_tensor_softmax);
    }
    Tensor softmax_last_dim() const { return unary_call(wgf_tensor_softmax_last_dim); }
    Tensor rope(const Tensor<2, D>& cos, const Tensor<2, D>& sin) const {   // rope.rs:13-22
        static_assert(R == 3, "rope takes [heads, sequence, embed]");
        wgf_tensor* out = nullptr;
        check(wgf_tensor_rope(h_, cos.raw(), sin.raw(), &out));
        return Tensor(out);
    }
    // ---- beyond the crate's API ---------------------------------------------------------------
    // softmax(scale * this k^T [+ mask]) v for [batch*heads, seq, head_dim] tensors; mask may be null.
    Tensor attention(const Tensor& k, const Tensor& v, const Tensor<2, D>* mask, bool causal, float scale) const {
        static_assert(R == 3, "attention takes [batch*heads, sequence, head_dim]");
        wgf_tensor* out = nullptr;
        check(wgf_tensor_attention(h_, k.raw(), v.raw(), mask ? mask->raw() : nullptr, causal ? 1 : 0, scale, &out));
        return Tensor(out);
    }
    // Queues the kernels of this tensor's graph without downloading (LazyTensorData::materialize).
    void materialize() const { check(wgf_tensor_materialize(h_)); }

    explicit Tensor(wgf_tensor* raw) : h_(raw) {}
    wgf_tensor* raw() const { return h_; }

   private:
    Tensor unary(uint32_t op) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_unary(h_, op, &out));
        return Tensor(out);
    }
    Tensor scalar(uint32_t op, float c) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_scalar(h_, op, c, &out));
        return Tensor(out);
    }
    Tensor binary(const Tensor& o, uint32_t op) const {
        wgf_tensor* out = nullptr;
        check(wgf_tensor_binary(h_, o.h_, op, &out));
        return Tensor(out);
    }
    Tensor<R - 1, D> reduce(uint32_t op, int axis) const {
        static_assert(R >= 1, "cannot reduce a rank-0 tensor");
        wgf_tensor* out = nullptr;
        check(wgf_tensor_reduce(h_, op, (uint32_t)axis, &out));
        return Tensor<R - 1, D>(out);
    }
    Tensor unary_call(int32_t (*fn)(wgf_tensor*, wgf_tensor**)) const {
        wgf_tensor* out = nullptr;
        check(fn(h_, &out));
        return Tensor(out);
    }
    wgf_tensor* h_ = nullptr;
};

// One request for several tensors of any rank and type (wgf_tensor_materialize_many): a
// whole-tensor reduction among them is computed inside the row kernel of another one.
template <typename... Ts>
void materialize_all(const Ts&... tensors) {
    wgf_tensor* raw[] = {tensors.raw()...};
    check(wgf_tensor_materialize_many(raw, (uint32_t)sizeof...(Ts)));
}

}  // namespace wgf
