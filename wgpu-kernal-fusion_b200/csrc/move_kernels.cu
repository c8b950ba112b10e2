// Bit-exact data movement between strided views: the one kernel behind resize, reshape of
// non-row-major inputs, slice_assign, cat and the compaction done before a download
// (src/resize.rs:43-118, src/slice_assign.rs:39-74, src/composite/cat.rs:4-40 of the crate).
// Threads run along the innermost axis of the collapsed index space; when both views are
// stride-1 there and 16-byte aligned, each thread moves 16 bytes.
#include <algorithm>

#include "launch.hpp"

namespace wgf {

namespace {

struct CopyParams {
    long long n;       // number of units (elements or vectors)
    int rank;
    long long shape[WGF_MAX_RANK];   // in units along the innermost axis
    long long dstride[WGF_MAX_RANK]; // in elements
    long long sstride[WGF_MAX_RANK];
};

template <typename T, typename IDX>
__global__ void __launch_bounds__(256) copy_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                   const __grid_constant__ CopyParams p) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += stride) {
        IDX rem = (IDX)i;
        long long doff = 0, soff = 0;
#pragma unroll 1
        for (int d = p.rank - 1; d >= 1; --d) {
            IDX q = rem / (IDX)p.shape[d];
            long long c = (long long)(rem - q * (IDX)p.shape[d]);
            rem = q;
            doff += c * p.dstride[d];
            soff += c * p.sstride[d];
        }
        doff += (long long)rem * p.dstride[0];
        soff += (long long)rem * p.sstride[0];
        dst[doff] = src[soff];
    }
}

// Transposing copy: the destination is contiguous along the last axis, the source along axis
// `pax`.  A CTA moves a 32 x 32 tile of the (pax, last) plane through shared memory so that
// both its reads and its writes are coalesced (the crate's strided kernel walks the source
// with adjacent threads a whole row apart, src/visit_tiled.rs:100-144).
struct TransposeParams {
    int rank, pax;
    long long tiles_p, tiles_l, total_tiles;
    long long shape[WGF_MAX_RANK];
    long long dstride[WGF_MAX_RANK];
    long long sstride[WGF_MAX_RANK];
};

template <typename T>
__global__ void __launch_bounds__(256) transpose_copy_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                             const __grid_constant__ TransposeParams p) {
    __shared__ T tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;   // 32 x 8
    const int last = p.rank - 1;
    for (long long t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
        long long rem = t;
        const long long tl = rem % p.tiles_l;
        rem /= p.tiles_l;
        const long long tp = rem % p.tiles_p;
        rem /= p.tiles_p;
        long long doff = 0, soff = 0;
#pragma unroll 1
        for (int d = last - 1; d >= 0; --d) {
            if (d == p.pax) continue;
            const long long c = rem % p.shape[d];
            rem /= p.shape[d];
            doff += c * p.dstride[d];
            soff += c * p.sstride[d];
        }
        const long long p0 = tp * 32, l0 = tl * 32;
        // read: x along pax (source contiguous), rows along last
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            const long long pi = p0 + tx, li = l0 + ty + i;
            if (pi < p.shape[p.pax] && li < p.shape[last])
                tile[ty + i][tx] = src[soff + pi * p.sstride[p.pax] + li * p.sstride[last]];
        }
        __syncthreads();
        // write: x along last (destination contiguous), rows along pax
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            const long long pi = p0 + ty + i, li = l0 + tx;
            if (pi < p.shape[p.pax] && li < p.shape[last])
                dst[doff + pi * p.dstride[p.pax] + li * p.dstride[last]] = tile[tx][ty + i];
        }
        __syncthreads();
    }
}

// The same move on 64 x 64 tiles with 4-element vector accesses on both sides (16 bytes for
// 4-byte elements, 8 for 2-byte): every thread has four vector loads in flight before it
// touches shared memory.  Needs both extents, every other stride and both base addresses
// to be multiples of 4 elements; tiles_p / tiles_l count 64-wide tiles here.
template <typename T, typename V>
__global__ void __launch_bounds__(256) transpose_copy_vec_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                                 const __grid_constant__ TransposeParams p) {
    constexpr int PAD = 4 / (int)sizeof(T);       // rows start one 32-bit bank further each
    __shared__ T tile[64][64 + PAD];              // [pax index][last index]
    const int c = threadIdx.x & 15, r = threadIdx.x >> 4;   // 16 vectors per 64-wide row, 16 rows per pass
    const int last = p.rank - 1;
    const long long P = p.shape[p.pax], L = p.shape[last];
    const long long sl = p.sstride[last], dp = p.dstride[p.pax];
    for (long long t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
        long long rem = t;
        const long long tl = rem % p.tiles_l;
        rem /= p.tiles_l;
        const long long tp = rem % p.tiles_p;
        rem /= p.tiles_p;
        long long doff = 0, soff = 0;
#pragma unroll 1
        for (int d = last - 1; d >= 0; --d) {
            if (d == p.pax) continue;
            const long long q = rem % p.shape[d];
            rem /= p.shape[d];
            doff += q * p.dstride[d];
            soff += q * p.sstride[d];
        }
        const long long p0 = tp * 64, l0 = tl * 64;
        V v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long li = l0 + r + 16 * i, pi = p0 + 4 * c;
            if (li < L && pi < P) v[i] = *(const V*)(src + soff + pi + li * sl);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const T* e = (const T*)&v[i];
            if (l0 + r + 16 * i < L && p0 + 4 * c < P) {
#pragma unroll
                for (int k = 0; k < 4; ++k) tile[4 * c + k][r + 16 * i] = e[k];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long pi = p0 + r + 16 * i, li = l0 + 4 * c;
            if (pi < P && li < L) {
                V o;
                T* e = (T*)&o;
#pragma unroll
                for (int k = 0; k < 4; ++k) e[k] = tile[r + 16 * i][4 * c + k];
                *(V*)(dst + doff + pi * dp + li) = o;
            }
        }
        __syncthreads();
    }
}

template <typename T>
void launch_transpose(Device& dev, void* dst, const void* src, const TransposeParams& p) {
    long long blocks = std::min<long long>(p.total_tiles, (long long)dev.sm_count * 16);
    dev.begin_launch("transpose_copy");
    if (!dev.dry)
        transpose_copy_kernel<T><<<(unsigned)blocks, dim3(32, 8), 0, dev.stream>>>((T*)dst, (const T*)src, p);
    dev.end_launch();
}

template <typename T, typename V>
void launch_transpose_vec(Device& dev, void* dst, const void* src, const TransposeParams& p) {
    long long blocks = std::min<long long>(p.total_tiles, (long long)dev.sm_count * 8);
    dev.begin_launch("transpose_copy");
    if (!dev.dry)
        transpose_copy_vec_kernel<T, V><<<(unsigned)blocks, 256, 0, dev.stream>>>((T*)dst, (const T*)src, p);
    dev.end_launch();
}

template <typename T>
void launch_copy(Device& dev, void* dst, const void* src, const CopyParams& p) {
    long long blocks = std::min<long long>((p.n + 255) / 256, (long long)dev.sm_count * 32);
    dev.begin_launch("copy");
    if (dev.dry) {
        dev.end_launch();
        return;
    }
    if (p.n < (1ll << 31))
        copy_kernel<T, unsigned><<<(unsigned)blocks, 256, 0, dev.stream>>>((T*)dst, (const T*)src, p);
    else
        copy_kernel<T, unsigned long long><<<(unsigned)blocks, 256, 0, dev.stream>>>((T*)dst, (const T*)src, p);
    dev.end_launch();
}

}  // namespace

void run_copy(Device& dev, const TensorData& dst, const TensorData& src) {
    WGF_CHECK(dst.layout.shape == src.layout.shape, WGF_ERR_SHAPE, "copy between different shapes");
    WGF_CHECK(dst.dtype == src.dtype, WGF_ERR_DTYPE, "copy between different element types");
    WGF_CHECK(!dst.layout.allocation_overlaps(), WGF_ERR_INVALID_ARGUMENT, "copy into an overlapping view");
    const int64_t n = src.layout.numel();
    if (n == 0) return;
    dev.make_current();
    dev.wait_for(*dst.buf);
    dev.wait_for(*src.buf);
    const int64_t esize = (int64_t)dtype_size(src.dtype);
    // collapse
    std::vector<int64_t> shape, ds, ss;
    for (int d = 0; d < src.layout.rank(); ++d) {
        int64_t e = src.layout.shape[d];
        if (e == 1) continue;
        int64_t a = dst.layout.strides[d], b = src.layout.strides[d];
        if (!shape.empty() && ds.back() == a * e && ss.back() == b * e) {
            shape.back() *= e;
            ds.back() = a;
            ss.back() = b;
        } else {
            shape.push_back(e);
            ds.push_back(a);
            ss.push_back(b);
        }
    }
    if (shape.empty()) {
        shape.push_back(1);
        ds.push_back(1);
        ss.push_back(1);
    }
    const int R = (int)shape.size();
    // transposed source: contiguous along another axis than the destination -> tiled transpose
    if (R >= 2 && ds[R - 1] == 1 && ss[R - 1] != 1 && n >= 4096) {
        int pax = -1;
        for (int d = 0; d < R - 1; ++d)
            if (ss[d] == 1 && shape[d] >= 8) pax = d;
        if (pax >= 0) {
            TransposeParams tp{};
            tp.rank = R;
            tp.pax = pax;
            tp.tiles_p = (shape[pax] + 31) / 32;
            tp.tiles_l = (shape[R - 1] + 31) / 32;
            tp.total_tiles = tp.tiles_p * tp.tiles_l;
            for (int d = 0; d < R; ++d) {
                tp.shape[d] = shape[d];
                tp.dstride[d] = ds[d];
                tp.sstride[d] = ss[d];
                if (d != pax && d != R - 1) tp.total_tiles *= shape[d];
            }
            bool vec_ok = shape[pax] % 4 == 0 && shape[R - 1] % 4 == 0 && n >= (1 << 16) &&
                          (uintptr_t)dst.base_ptr() % (4 * esize) == 0 && (uintptr_t)src.base_ptr() % (4 * esize) == 0;
            for (int d = 0; d < R && vec_ok; ++d) {
                if (d != pax && ss[d] % 4 != 0) vec_ok = false;
                if (d != R - 1 && ds[d] % 4 != 0) vec_ok = false;
            }
            if (vec_ok) {
                tp.total_tiles /= tp.tiles_p * tp.tiles_l;
                tp.tiles_p = (shape[pax] + 63) / 64;
                tp.tiles_l = (shape[R - 1] + 63) / 64;
                tp.total_tiles *= tp.tiles_p * tp.tiles_l;
                if (esize == 4) launch_transpose_vec<uint32_t, uint4>(dev, dst.base_ptr(), src.base_ptr(), tp);
                else launch_transpose_vec<uint16_t, uint2>(dev, dst.base_ptr(), src.base_ptr(), tp);
                return;
            }
            if (esize == 4) launch_transpose<uint32_t>(dev, dst.base_ptr(), src.base_ptr(), tp);
            else launch_transpose<uint16_t>(dev, dst.base_ptr(), src.base_ptr(), tp);
            return;
        }
    }
    // vector width: 16, 8 or 4 bytes per thread when the innermost axis allows it
    int64_t vec = 1;
    if (ds[R - 1] == 1 && ss[R - 1] == 1) {
        for (int64_t v = 16 / esize; v > 1; v /= 2) {
            bool ok = shape[R - 1] % v == 0 && (uintptr_t)dst.base_ptr() % (v * esize) == 0 &&
                      (uintptr_t)src.base_ptr() % (v * esize) == 0;
            for (int d = 0; d < R - 1 && ok; ++d) ok = ds[d] % v == 0 && ss[d] % v == 0;
            if (ok) {
                vec = v;
                break;
            }
        }
    }
    CopyParams p{};
    p.rank = R;
    p.n = n / vec;
    for (int d = 0; d < R; ++d) {
        p.shape[d] = d == R - 1 ? shape[d] / vec : shape[d];
        p.dstride[d] = d == R - 1 ? 1 : ds[d] / vec;
        p.sstride[d] = d == R - 1 ? 1 : ss[d] / vec;
    }
    if (vec == 1) {
        p.dstride[R - 1] = ds[R - 1];
        p.sstride[R - 1] = ss[R - 1];
    }
    const int64_t unit = vec * esize;
    if (unit == 16) launch_copy<uint4>(dev, dst.base_ptr(), src.base_ptr(), p);
    else if (unit == 8) launch_copy<uint2>(dev, dst.base_ptr(), src.base_ptr(), p);
    else if (unit == 4) launch_copy<uint32_t>(dev, dst.base_ptr(), src.base_ptr(), p);
    else launch_copy<uint16_t>(dev, dst.base_ptr(), src.base_ptr(), p);
}

TensorData run_compact(Device& dev, const TensorData& src) {
    TensorData out;
    out.dtype = src.dtype;
    out.layout = Layout::contiguous(src.layout.shape);
    out.buf = dev.alloc((size_t)std::max<int64_t>(out.layout.numel(), 1) * dtype_size(src.dtype), false);
    run_copy(dev, out, src);
    return out;
}

}  // namespace wgf
