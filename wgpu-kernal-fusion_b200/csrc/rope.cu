// Rotary position embedding as one kernel (the crate composes it from cat / narrow / broadcast
// / mul / add, src/composite/rope.rs:13-22):
//   out[.., s, j] = x[.., s, j] * cos2[s, j] + rot[.., s, j] * sin2[s, j]
//   cos2 = cat(cos, cos) along the last axis, rot = cat(-x[.., D/2:], x[.., :D/2])
// Every product and the sum are rounded to the element type on their own, exactly as the
// chain of separate ops does, so the results are bit-identical to the composed form.  The
// input may be any view whose last axis is contiguous (e.g. the [batch, heads, seq, head_dim]
// transpose of a projection output); the output is contiguous, so splitting heads costs no
// copy of its own.  A thread handles VEC elements of the first half of a row and their
// partners in the second half.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "launch.hpp"

namespace wgf {

namespace {

struct RopeParams {
    long long rows;          // product of the outer extents times S
    long long xs_o1, xs_o0, xs_s;   // strides of x in elements: two outer axes, sequence axis
    long long cs;            // row stride of cos / sin in elements
    int S, half, o0;         // sequence length, D / 2, extent of the inner outer axis
};

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
// round a float to the element type and back
template <typename T> __device__ __forceinline__ float rnd(float v);
template <> __device__ __forceinline__ float rnd<float>(float v) { return v; }
template <> __device__ __forceinline__ float rnd<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack {
    T v[VEC];
};

template <typename T, int VEC>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ cosp,
                                                   const T* __restrict__ sinp, const __grid_constant__ RopeParams p) {
    typedef Pack<T, VEC> V;
    const int vper = p.half / VEC;
    const long long total = p.rows * vper;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
        const long long row = t / vper;
        const int j = (int)(t - row * vper) * VEC;
        const int s = (int)(row % p.S);
        const long long o = row / p.S;
        const long long i0 = o % p.o0, i1 = o / p.o0;
        const T* xr = x + i1 * p.xs_o1 + i0 * p.xs_o0 + (long long)s * p.xs_s;
        const V a = *reinterpret_cast<const V*>(xr + j), b = *reinterpret_cast<const V*>(xr + p.half + j);
        const V c = *reinterpret_cast<const V*>(cosp + (long long)s * p.cs + j);
        const V sn = *reinterpret_cast<const V*>(sinp + (long long)s * p.cs + j);
        V lo, hi;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float x1 = to_f<T>(a.v[e]), x2 = to_f<T>(b.v[e]), cc = to_f<T>(c.v[e]), ss = to_f<T>(sn.v[e]);
            // first half: x1 * cos + (-x2) * sin;  second half: x2 * cos + x1 * sin
            lo.v[e] = from_f<T>(__fadd_rn(rnd<T>(__fmul_rn(x1, cc)), rnd<T>(__fmul_rn(-x2, ss))));
            hi.v[e] = from_f<T>(__fadd_rn(rnd<T>(__fmul_rn(x2, cc)), rnd<T>(__fmul_rn(x1, ss))));
        }
        T* orow = out + row * (2ll * p.half);
        *reinterpret_cast<V*>(orow + j) = lo;
        *reinterpret_cast<V*>(orow + p.half + j) = hi;
    }
}

template <typename T>
void launch_rope(Device& dev, void* out, const void* x, const void* c, const void* s, const RopeParams& p, int vec) {
    const long long total = p.rows * (p.half / vec);
    const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, (long long)dev.sm_count * 16);
    dev.begin_launch("rope");
    if (!dev.dry) {
        if (vec == 8) rope_kernel<T, 8><<<blocks, 256, 0, dev.stream>>>((T*)out, (const T*)x, (const T*)c, (const T*)s, p);
        else if (vec == 4) rope_kernel<T, 4><<<blocks, 256, 0, dev.stream>>>((T*)out, (const T*)x, (const T*)c, (const T*)s, p);
        else rope_kernel<T, 1><<<blocks, 256, 0, dev.stream>>>((T*)out, (const T*)x, (const T*)c, (const T*)s, p);
    }
    dev.end_launch();
}

}  // namespace

TensorData run_rope(Device& dev, const TensorData& x_in, const TensorData& cos_in, const TensorData& sin_in) {
    const int r = x_in.layout.rank();
    WGF_CHECK(r == 3 || r == 4, WGF_ERR_RANK, "rope takes [heads, seq, embed] or [batch, heads, seq, embed]");
    const int64_t S = x_in.layout.shape[r - 2], D = x_in.layout.shape[r - 1];
    WGF_CHECK(D % 2 == 0 && cos_in.layout.rank() == 2 && cos_in.layout.shape == sin_in.layout.shape &&
                  cos_in.layout.shape[1] * 2 == D && cos_in.layout.shape[0] >= S,
              WGF_ERR_SHAPE, "rope cos/sin must be [>= sequence, embed / 2]");
    dev.make_current();
    TensorData x = x_in.layout.strides[r - 1] == 1 || D == 1 ? x_in : run_compact(dev, x_in);
    auto rows_ok = [](const TensorData& t) { return t.layout.strides[1] == 1 || t.layout.shape[1] == 1; };
    const bool cs_ok = rows_ok(cos_in) && rows_ok(sin_in) && cos_in.layout.strides[0] == sin_in.layout.strides[0];
    TensorData c = cs_ok ? cos_in : run_compact(dev, cos_in);
    TensorData s = cs_ok ? sin_in : run_compact(dev, sin_in);
    for (const TensorData* t : {&x, &c, &s}) dev.wait_for(*t->buf);
    TensorData out;
    out.dtype = x.dtype;
    out.layout = Layout::contiguous(x.layout.shape);
    const int64_t n = out.layout.numel();
    out.buf = dev.alloc((size_t)std::max<int64_t>(n, 1) * dtype_size(x.dtype), false);
    if (n == 0) return out;
    RopeParams p{};
    p.S = (int)S;
    p.half = (int)(D / 2);
    p.o0 = (int)x.layout.shape[r - 3];
    p.rows = n / D;
    p.xs_s = x.layout.strides[r - 2];
    p.xs_o0 = x.layout.strides[r - 3];
    p.xs_o1 = r == 4 ? x.layout.strides[0] : 0;
    p.cs = c.layout.strides[0];
    WGF_CHECK(S < (1ll << 31) && D < (1ll << 31) && x.layout.shape[r - 3] < (1ll << 31), WGF_ERR_UNSUPPORTED, "rope extents too large");
    // widest vector every row start allows
    const int64_t es = (int64_t)dtype_size(x.dtype);
    int vec = 1;
    for (int v : {8, 4}) {
        if (v * es > 16 || p.half % v) continue;
        bool ok = p.xs_s % v == 0 && p.xs_o0 % v == 0 && p.xs_o1 % v == 0 && p.cs % v == 0;
        for (const TensorData* t : {&x, &c, &s, &out}) ok = ok && ((uintptr_t)t->base_ptr() % (uintptr_t)(v * es)) == 0;
        if (ok) {
            vec = v;
            break;
        }
    }
    if (x.dtype == DType::F32) launch_rope<float>(dev, out.base_ptr(), x.base_ptr(), c.base_ptr(), s.base_ptr(), p, vec);
    else if (x.dtype == DType::F16) launch_rope<__half>(dev, out.base_ptr(), x.base_ptr(), c.base_ptr(), s.base_ptr(), p, vec);
    else launch_rope<__nv_bfloat16>(dev, out.base_ptr(), x.base_ptr(), c.base_ptr(), s.base_ptr(), p, vec);
    return out;
}

}  // namespace wgf
