// MatMul dispatch (UntypedMatMul::run_with_query, src/matmul.rs:157-214 of the crate) and
// the strided fallback kernel: any element type, any strides/offsets, batched, fp32
// accumulate.  The crate's kernel ignores strides and is only right for tiny shapes; the
// definition implemented here is C[b,m,n] = sum_k A[b,m,k] * B[b,k,n].
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "launch.hpp"
#include "matmul.hpp"

namespace wgf {

namespace {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 64x64 output tile, 16-deep k-steps, 256 threads, 4x4 outputs per thread.
template <typename T>
__global__ void __launch_bounds__(256) matmul_strided_kernel(const T* __restrict__ A, const T* __restrict__ B,
                                                             T* __restrict__ C, const __grid_constant__ MatmulDims d) {
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.y * 64, n0 = (long long)blockIdx.x * 64;
    const long long bz = blockIdx.z;
    const T* Ab = A + bz * d.a_bs;
    const T* Bb = B + bz * d.b_bs;
    T* Cb = C + bz * d.c_bs;
    float acc[4][4] = {};
    for (long long k0 = 0; k0 < d.K; k0 += 16) {
        // A tile: 64 rows x 16 k; B tile: 16 k x 64 cols; 4 elements per thread each
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int e = tid + i * 256;
            int ak = e % 16, am = e / 16;
            long long m = m0 + am, k = k0 + ak;
            As[ak][am] = (m < d.M && k < d.K) ? to_f32<T>(Ab[m * d.a_rs + k * d.a_cs]) : 0.f;
            int bn = e % 64, bk = e / 64;
            long long n = n0 + bn;
            k = k0 + bk;
            Bs[bk][bn] = (n < d.N && k < d.K) ? to_f32<T>(Bb[k * d.b_rs + n * d.b_cs]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        long long m = m0 + ty * 4 + i;
        if (m >= d.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            long long n = n0 + tx * 4 + j;
            if (n < d.N) Cb[m * d.c_rs + n] = from_f32<T>(acc[i][j]);
        }
    }
}

template <typename T>
void launch_strided(Device& dev, const void* a, const void* b, void* c, const MatmulDims& d) {
    dim3 grid((unsigned)((d.N + 63) / 64), (unsigned)((d.M + 63) / 64), (unsigned)d.batch);
    dev.begin_launch("matmul_strided");
    if (!dev.dry) matmul_strided_kernel<T><<<grid, 256, 0, dev.stream>>>((const T*)a, (const T*)b, (T*)c, d);
    dev.end_launch();
}

}  // namespace

namespace {
// Shapes and strides of C = A B in elements; checks what the crate's front-end asserts.
MatmulDims dims_of(const TensorData& a, const TensorData& b) {
    const int r = a.layout.rank();
    WGF_CHECK(r == b.layout.rank() && (r == 2 || r == 3), WGF_ERR_RANK, "matmul takes rank 2, or rank 3 (batched)");
    WGF_CHECK(a.dtype == b.dtype, WGF_ERR_DTYPE, "matmul operands must have equal element types");
    MatmulDims d{};
    d.batch = r == 3 ? a.layout.shape[0] : 1;
    d.M = a.layout.shape[r - 2];
    d.K = a.layout.shape[r - 1];
    d.N = b.layout.shape[r - 1];
    WGF_CHECK(b.layout.shape[r - 2] == d.K, WGF_ERR_SHAPE, "matmul inner dimensions differ");
    if (r == 3) WGF_CHECK(b.layout.shape[0] == d.batch, WGF_ERR_SHAPE, "matmul batch sizes differ");
    d.a_bs = r == 3 ? a.layout.strides[0] : 0;
    d.a_rs = a.layout.strides[r - 2];
    d.a_cs = a.layout.strides[r - 1];
    d.b_bs = r == 3 ? b.layout.strides[0] : 0;
    d.b_rs = b.layout.strides[r - 2];
    d.b_cs = b.layout.strides[r - 1];
    d.c_rs = d.N;
    d.c_bs = d.M * d.N;
    return d;
}
}  // namespace

bool matmul_tc_pair_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d,
                         const MatmulEpilogue* epi);

TensorData run_matmul(Device& dev, const TensorData& a, const TensorData& b) {
    const int r = a.layout.rank();
    const MatmulDims d = dims_of(a, b);
    std::vector<int64_t> oshape = a.layout.shape;
    oshape[r - 1] = d.N;
    TensorData out;
    out.dtype = a.dtype;
    out.layout = Layout::contiguous(oshape);
    const int64_t n_out = out.layout.numel();
    out.buf = dev.alloc((size_t)std::max<int64_t>(n_out, 1) * dtype_size(a.dtype), d.K == 0);
    if (n_out == 0 || d.K == 0) return out;
    WGF_CHECK(d.batch <= 65535 && (d.M + 63) / 64 <= 65535, WGF_ERR_UNSUPPORTED, "matmul grid too large");
    dev.make_current();
    dev.wait_for(*a.buf);
    dev.wait_for(*b.buf);

    if (matmul_fast_path(dev, a.base_ptr(), b.base_ptr(), out.base_ptr(), a.dtype, d)) return out;

    switch (a.dtype) {
        case DType::F32: launch_strided<float>(dev, a.base_ptr(), b.base_ptr(), out.base_ptr(), d); break;
        case DType::F16: launch_strided<__half>(dev, a.base_ptr(), b.base_ptr(), out.base_ptr(), d); break;
        default: launch_strided<__nv_bfloat16>(dev, a.base_ptr(), b.base_ptr(), out.base_ptr(), d); break;
    }
    return out;
}

// C = round(A B) + R in one kernel, or false (nothing launched) when the tensor-core CTA-pair kernel
// does not take this problem; the caller then runs the product and the addition as separate kernels.
bool run_matmul_residual(Device& dev, const TensorData& a, const TensorData& b, const TensorData& resid, TensorData& out) {
    const int r = a.layout.rank();
    if (a.dtype == DType::F32 || resid.dtype != a.dtype) return false;
    const MatmulDims d = dims_of(a, b);
    std::vector<int64_t> oshape = a.layout.shape;
    oshape[r - 1] = d.N;
    if (resid.layout.shape != oshape || resid.layout.strides[r - 1] != 1 || d.K == 0) return false;
    if (Layout::contiguous(oshape).numel() == 0) return false;
    MatmulEpilogue epi;
    epi.kind = MatmulEpilogue::RESIDUAL;
    epi.resid = resid.base_ptr();
    epi.r_rs = resid.layout.strides[r - 2];
    epi.r_bs = r == 3 ? resid.layout.strides[0] : 0;
    TensorData c;
    c.dtype = a.dtype;
    c.layout = Layout::contiguous(oshape);
    c.buf = dev.alloc((size_t)c.layout.numel() * dtype_size(a.dtype), false);
    dev.make_current();
    dev.wait_for(*a.buf);
    dev.wait_for(*b.buf);
    dev.wait_for(*resid.buf);
    if (!matmul_tc_pair_path(dev, a.base_ptr(), b.base_ptr(), c.base_ptr(), a.dtype, d, &epi)) return false;
    out = c;
    return true;
}

// C = silu(A Bg) * (A Bu) in one kernel (Bg and Bu of one shape and one set of strides), or false.
bool run_matmul_silu_mul(Device& dev, const TensorData& a, const TensorData& bg, const TensorData& bu, TensorData& out) {
    const int r = a.layout.rank();
    if (a.dtype == DType::F32 || bg.dtype != a.dtype || bu.dtype != a.dtype) return false;
    if (bg.layout.shape != bu.layout.shape || bg.layout.strides != bu.layout.strides) return false;
    const MatmulDims d = dims_of(a, bg);
    if (d.K == 0) return false;
    std::vector<int64_t> oshape = a.layout.shape;
    oshape[r - 1] = d.N;
    if (Layout::contiguous(oshape).numel() == 0) return false;
    MatmulEpilogue epi;
    epi.kind = MatmulEpilogue::SILU_MUL;
    epi.b2 = bu.base_ptr();
    TensorData c;
    c.dtype = a.dtype;
    c.layout = Layout::contiguous(oshape);
    c.buf = dev.alloc((size_t)c.layout.numel() * dtype_size(a.dtype), false);
    dev.make_current();
    dev.wait_for(*a.buf);
    dev.wait_for(*bg.buf);
    dev.wait_for(*bu.buf);
    if (!matmul_tc_pair_path(dev, a.base_ptr(), bg.base_ptr(), c.base_ptr(), a.dtype, d, &epi)) return false;
    out = c;
    return true;
}

}  // namespace wgf
