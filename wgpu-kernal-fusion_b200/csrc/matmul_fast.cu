// Specialised matmul kernels and their dispatch (the crate has one shared-memory kernel for
// everything, src/matmul.rs:56-155):
//   * sgemm_kernel       f32, 128x128x16 tiles, 8x8 register tile per thread, FFMA pipe;
//   * gemv_kn_kernel     skinny M (decode GEMV) with B stored [K,N]: streams B once at HBM speed,
//                        16-byte loads along N, split over K, fp32 partials combined by the last CTA
//                        of each column block (ticket);
//   * gemv_nk_kernel     skinny M with B stored [N,K] (a transposed view): one warp per output column;
//   * f16 / bf16 large:  tcgen05 kernel in matmul_tc.cu.
// All accumulate in fp32 and round once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <mutex>

#include "matmul.hpp"

namespace wgf {

bool matmul_tc_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d);
bool matmul_tc_pair_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d,
                         const MatmulEpilogue* epi = nullptr);

namespace {

// ---------------------------------------------------------------------------------------
// f32 SGEMM.  A is [M,K] row-major (lda), B is [K,N] row-major (B_NK = false) or [N,K]
// row-major (B_NK = true, i.e. a transposed view), C is [M,N] row-major.
// ---------------------------------------------------------------------------------------
constexpr int SG_BM = 128, SG_BN = 128, SG_BK = 16, SG_PAD = 4;

template <bool B_NK>
__global__ void __launch_bounds__(256, 2)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
             const __grid_constant__ MatmulDims d) {
    __shared__ __align__(16) float As[2][SG_BK][SG_BM + SG_PAD];
    __shared__ __align__(16) float Bs[2][SG_BK][SG_BN + SG_PAD];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.y * SG_BM, n0 = (long long)blockIdx.x * SG_BN;
    const float* Ab = A + (long long)blockIdx.z * d.a_bs;
    const float* Bb = B + (long long)blockIdx.z * d.b_bs;
    float* Cb = C + (long long)blockIdx.z * d.c_bs;
    const long long lda = d.a_rs, ldb = B_NK ? d.b_cs : d.b_rs;

    float4 ra[2], rb[2];
    auto load_tiles = [&](long long k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 256;
            {   // A: 128 rows x 16 k, float4 along k
                const int r = idx / 4, c4 = idx % 4;
                const long long m = m0 + r, k = k0 + c4 * 4;
                ra[i] = (m < d.M && k < d.K) ? *reinterpret_cast<const float4*>(Ab + m * lda + k) : make_float4(0, 0, 0, 0);
            }
            if (B_NK) {  // B^T: 128 n-rows x 16 k, float4 along k
                const int r = idx / 4, c4 = idx % 4;
                const long long n = n0 + r, k = k0 + c4 * 4;
                rb[i] = (n < d.N && k < d.K) ? *reinterpret_cast<const float4*>(Bb + n * ldb + k) : make_float4(0, 0, 0, 0);
            } else {     // B: 16 k-rows x 128 n, float4 along n
                const int kr = idx / 32, c4 = idx % 32;
                const long long k = k0 + kr, n = n0 + c4 * 4;
                rb[i] = (k < d.K && n < d.N) ? *reinterpret_cast<const float4*>(Bb + k * ldb + n) : make_float4(0, 0, 0, 0);
            }
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 256;
            {
                const int r = idx / 4, c4 = idx % 4;
                As[buf][c4 * 4 + 0][r] = ra[i].x;
                As[buf][c4 * 4 + 1][r] = ra[i].y;
                As[buf][c4 * 4 + 2][r] = ra[i].z;
                As[buf][c4 * 4 + 3][r] = ra[i].w;
            }
            if (B_NK) {
                const int r = idx / 4, c4 = idx % 4;
                Bs[buf][c4 * 4 + 0][r] = rb[i].x;
                Bs[buf][c4 * 4 + 1][r] = rb[i].y;
                Bs[buf][c4 * 4 + 2][r] = rb[i].z;
                Bs[buf][c4 * 4 + 3][r] = rb[i].w;
            } else {
                const int kr = idx / 32, c4 = idx % 32;
                *reinterpret_cast<float4*>(&Bs[buf][kr][c4 * 4]) = rb[i];
            }
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    int buf = 0;
    for (long long k0 = 0; k0 < d.K; k0 += SG_BK) {
        const bool more = k0 + SG_BK < d.K;
        if (more) load_tiles(k0 + SG_BK);   // global loads of the next tile overlap the FMAs below
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) {
            store_tiles(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }
    const bool vec_ok = (d.N % 4 == 0) && (d.c_rs % 4 == 0) && ((reinterpret_cast<uintptr_t>(Cb) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= d.M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long n = n0 + h * 64 + tx * 4;
            if (vec_ok && n + 3 < d.N) {
                *reinterpret_cast<float4*>(Cb + m * d.c_rs + n) =
                    make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < d.N) Cb[m * d.c_rs + n + j] = acc[i][h * 4 + j];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Skinny-M kernels.  T = float / __half / __nv_bfloat16; VEC = elements per 16 bytes.
// ---------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T st_from(float v);
template <> __device__ __forceinline__ float st_from<float>(float v) { return v; }
template <> __device__ __forceinline__ __half st_from<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 st_from<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ void unpack16(const uint4& raw, float* out) {
    const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; ++j) out[j] = ld_f32<T>(p + j);
}

constexpr int GV_MAXM = 8;

// B is [K,N] row-major.  Each lane owns VEC consecutive columns; the 8 warps of a CTA take
// interleaved k rows of the CTA's k range; partial[ksplit][M][N] in fp32.  With `counters`
// (one zeroed word per column block) the last CTA to arrive for a column block adds the
// k-split partials in split order and stores C, so no finishing launch is needed.
template <typename T, int MM>
__global__ void __launch_bounds__(256)
gemv_kn_kernel(const T* __restrict__ A, const T* __restrict__ B, float* __restrict__ partial, T* __restrict__ C,
               unsigned* __restrict__ counters, const __grid_constant__ MatmulDims d, int k_per_cta) {
    constexpr int VEC = Vec16<T>::N;
    __shared__ float red[8][32 * VEC + 1];
    __shared__ unsigned is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long n = ((long long)blockIdx.x * 32 + lane) * VEC;
    const long long kbeg = (long long)blockIdx.y * k_per_cta;
    const long long kend = min(kbeg + (long long)k_per_cta, d.K);
    float acc[MM][VEC];
#pragma unroll
    for (int m = 0; m < MM; ++m)
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[m][j] = 0.f;
    if (n < d.N) {
        constexpr int UN = MM <= 2 ? 8 : 4;     // k rows in flight per lane (16-byte loads)
        for (long long k = kbeg + warp; k < kend; k += 8 * UN) {
            uint4 raw[UN];
            float av[UN][MM];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const long long kk = k + u * 8;
                if (kk < kend) {
                    raw[u] = *reinterpret_cast<const uint4*>(B + kk * d.b_rs + n);
#pragma unroll
                    for (int m = 0; m < MM; ++m) av[u][m] = ld_f32<T>(A + m * d.a_rs + kk * d.a_cs);
                } else {
                    raw[u] = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int m = 0; m < MM; ++m) av[u][m] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                float bv[VEC];
                unpack16<T>(raw[u], bv);
#pragma unroll
                for (int m = 0; m < MM; ++m)
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc[m][j] = fmaf(av[u][m], bv[j], acc[m][j]);
            }
        }
    }
    // the 8 warps' partial sums are added in warp order, one output row at a time
#pragma unroll
    for (int m = 0; m < MM; ++m) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) red[warp][lane * VEC + j] = acc[m][j];
        __syncthreads();
        for (int c = threadIdx.x; c < 32 * VEC; c += 256) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += red[w][c];
            const long long col = (long long)blockIdx.x * 32 * VEC + c;
            if (col < d.N) partial[((long long)blockIdx.y * MM + m) * d.N + col] = s;
        }
        __syncthreads();
    }
    if (counters == nullptr) return;
    // ticket: the last CTA of this column block combines the splits
    __threadfence();            // every thread's partial sums are visible device-wide ...
    __syncthreads();            // ... before thread 0 takes the ticket
    if (threadIdx.x == 0) {
        const unsigned ticket = atomicAdd(counters + blockIdx.x, 1u);
        is_last = ticket == gridDim.y - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int c = threadIdx.x; c < 32 * VEC; c += 256) {
        const long long col = (long long)blockIdx.x * 32 * VEC + c;
        if (col >= d.N) continue;
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            float s = 0.f;
            for (unsigned k = 0; k < gridDim.y; ++k) s += __ldcg(partial + ((long long)k * MM + m) * d.N + col);
            C[(long long)m * d.c_rs + col] = st_from<T>(s);
        }
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;
}

template <typename T>
__global__ void __launch_bounds__(256)
gemv_finish_kernel(const float* __restrict__ partial, T* __restrict__ C, long long M, long long N, int splits, long long c_rs) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= M * N) return;
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(long long)k * M * N + i];
    C[(i / N) * c_rs + (i % N)] = st_from<T>(s);
}

// B is [N,K] row-major (b_cs == K-stride == 1 along k): one warp per output column n, 16-byte
// loads along k, shuffle reduction.
template <typename T, int MM>
__global__ void __launch_bounds__(256)
gemv_nk_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, const __grid_constant__ MatmulDims d) {
    constexpr int VEC = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long n = (long long)blockIdx.x * 8 + warp;
    if (n >= d.N) return;
    const T* brow = B + n * d.b_cs;
    float acc[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[m] = 0.f;
    for (long long k = (long long)lane * VEC; k < d.K; k += 32 * VEC * 2) {
        uint4 rb[2];
        bool ok[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const long long kk = k + u * 32 * VEC;
            ok[u] = kk < d.K;
            rb[u] = ok[u] ? *reinterpret_cast<const uint4*>(brow + kk) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!ok[u]) continue;
            const long long kk = k + u * 32 * VEC;
            float bv[VEC];
            unpack16<T>(rb[u], bv);
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                const uint4 ar = *reinterpret_cast<const uint4*>(A + m * d.a_rs + kk);
                float av[VEC];
                unpack16<T>(ar, av);
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[m] = fmaf(av[j], bv[j], acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        float v = acc[m];
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) C[m * d.c_rs + n] = st_from<T>(v);
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
bool run_gemv(Device& dev, const void* a, const void* b, void* c, const MatmulDims& d) {
    constexpr int VEC = Vec16<T>::N;
    if (d.batch != 1 || d.M > GV_MAXM) return false;
    auto pick = [&](auto fn) {
        switch (d.M) {
            case 1: fn(std::integral_constant<int, 1>()); break;
            case 2: fn(std::integral_constant<int, 2>()); break;
            case 3: case 4: fn(std::integral_constant<int, 4>()); break;
            default: fn(std::integral_constant<int, 8>()); break;
        }
    };
    // rows of A beyond M must not be read: only exact instantiations are used
    if (d.M != 1 && d.M != 2 && d.M != 4 && d.M != 8) return false;
    if (d.b_cs == 1 && d.b_rs % VEC == 0 && d.N % VEC == 0 && aligned16(b) && d.K >= 64) {
        // [K,N] row-major
        const long long nblocks = (d.N + 32 * VEC - 1) / (32 * VEC);
        long long splits = std::max<long long>(1, (long long)dev.sm_count * 4 / nblocks);
        splits = std::min<long long>(splits, std::max<long long>(1, d.K / 64));
        const int k_per_cta = (int)((d.K + splits - 1) / splits);
        splits = (d.K + k_per_cta - 1) / k_per_cta;
        BufferRef scratch = dev.alloc((size_t)(splits * d.M * d.N) * sizeof(float), false);
        static const bool finish_kernel = getenv("WGF_GEMV_FINISH_KERNEL") != nullptr;   // diagnostic switch, read once
        const bool ticketed = nblocks <= Device::kCounters && !finish_kernel;
        pick([&](auto mm) {
            constexpr int MM = decltype(mm)::value;
            dev.begin_launch("gemv_kn");
            if (!dev.dry)
                gemv_kn_kernel<T, MM><<<dim3((unsigned)nblocks, (unsigned)splits), 256, 0, dev.stream>>>(
                    (const T*)a, (const T*)b, (float*)scratch->ptr, (T*)c, ticketed ? (unsigned*)dev.counters() : (unsigned*)nullptr, d, k_per_cta);
            dev.end_launch();
        });
        if (ticketed) return true;
        dev.begin_launch("gemv_finish");
        if (!dev.dry)
            gemv_finish_kernel<T><<<(unsigned)((d.M * d.N + 255) / 256), 256, 0, dev.stream>>>(
                (const float*)scratch->ptr, (T*)c, d.M, d.N, (int)splits, d.c_rs);
        dev.end_launch();
        return true;
    }
    if (d.b_rs == 1 && d.a_cs == 1 && d.b_cs % VEC == 0 && d.a_rs % VEC == 0 && d.K % VEC == 0 && aligned16(a) && aligned16(b)) {
        // [N,K] row-major (transposed view)
        pick([&](auto mm) {
            constexpr int MM = decltype(mm)::value;
            dev.begin_launch("gemv_nk");
            if (!dev.dry)
                gemv_nk_kernel<T, MM><<<(unsigned)((d.N + 7) / 8), 256, 0, dev.stream>>>((const T*)a, (const T*)b, (T*)c, d);
            dev.end_launch();
        });
        return true;
    }
    return false;
}

// ---------------------------------------------------------------------------------------
// f32 SGEMM for large problems with B stored [K,N]: 128x256x16 tiles, 8x16 register tile per
// thread, one CTA of 256 threads per SM, tiles brought into a 4-stage shared-memory ring with
// cp.async (no staging registers, no shared-memory stores, one barrier per k-tile).
// Why this shape: an FFMA kernel on this SM (128 fp32 lanes, 128 bytes of shared memory per clock)
// with an 8x8 register tile needs a byte of shared memory per FFMA lane -- exactly all there is --
// so fragment loads and FFMAs have to overlap perfectly; 8x16 needs 0.75.  A is kept [m][k] in
// shared memory as it comes from global memory (rows of 16 floats padded to 20: the two rows a
// warp reads are broadcast), and a thread takes four k steps of a row with one 16-byte load.
// ---------------------------------------------------------------------------------------
constexpr int SW_BM = 128, SW_BN = 256, SW_BK = 16, SW_STAGES = 4, SW_LDA = SW_BK + 4;
constexpr int SW_A_FLOATS = SW_BM * SW_LDA, SW_B_FLOATS = SW_BK * SW_BN;
constexpr size_t SW_SMEM = (size_t)SW_STAGES * (SW_A_FLOATS + SW_B_FLOATS) * sizeof(float);

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}

// Two fp32 FMAs in one instruction on a register pair (fma.rn.f32x2, sm_100): the FMA pipe does the
// same work per clock, but the scheduler dispatches half as many instructions, and what limited
// the scalar form of this kernel were dispatch stalls (66 % of the pipe at 0.5 stalls per issue).
// Every lane rounds like a scalar fmaf.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void ffma2(unsigned long long& d, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

// Work items: tile t (0 <= t < tiles) in full for CTAs below `whole`; the remaining tiles -- the part
// of the last wave that would leave most SMs idle -- are computed as two halves of the k range by
// two CTAs each, which add their halves to a zeroed C with atomics (x + y on 0 is the same bits in
// either order, so the result does not depend on which half arrives first).
struct WideSplit {
    int tn, tm;        // tiles along N and M
    int whole;         // CTAs [0, whole) own a full tile; CTA whole + 2 i + h owns half h of tile whole + i
};

__global__ void __launch_bounds__(256, 1)
sgemm_wide_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                  const __grid_constant__ MatmulDims d, const WideSplit ws) {
    extern __shared__ __align__(16) float sw_smem[];
    float* As = sw_smem;                                   // [stage][128][20]
    float* Bs = sw_smem + SW_STAGES * SW_A_FLOATS;         // [stage][16][256]
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const bool halved = (int)blockIdx.x >= ws.whole;
    const int tile = halved ? ws.whole + ((int)blockIdx.x - ws.whole) / 2 : (int)blockIdx.x;
    const int bx = tile % ws.tn, by = (tile / ws.tn) % ws.tm, bz = tile / (ws.tn * ws.tm);
    const long long m0 = (long long)by * SW_BM, n0 = (long long)bx * SW_BN;
    const float* Ab = A + (long long)bz * d.a_bs;
    const float* Bb = B + (long long)bz * d.b_bs;
    float* Cb = C + (long long)bz * d.c_bs;
    const long long lda = d.a_rs, ldb = d.b_rs;
    const int all_tiles = (int)((d.K + SW_BK - 1) / SW_BK);
    // k tiles [kt0, kt0 + n_tiles) of this work item
    const int kt0 = halved && (((int)blockIdx.x - ws.whole) & 1) ? all_tiles / 2 : 0;
    const int n_tiles = !halved ? all_tiles : kt0 ? all_tiles - all_tiles / 2 : all_tiles / 2;

    // K, N, lda, ldb are multiples of 4 and the bases 16-byte aligned (the launcher checks), so a
    // 16-byte piece is either wholly inside the matrix or wholly outside (then zero-filled; the
    // source address of such a piece is the matrix base, never dereferenced)
    auto load_tile = [&](int kt, int stage) {
        const long long k0 = (long long)(kt0 + kt) * SW_BK;
        float* as = As + stage * SW_A_FLOATS;
        float* bs = Bs + stage * SW_B_FLOATS;
#pragma unroll
        for (int i = 0; i < 2; ++i) {          // A: 128 rows x 4 pieces
            const int idx = tid + i * 256, r = idx / 4, c4 = idx % 4;
            const long long m = m0 + r, k = k0 + c4 * 4;
            const bool in = m < d.M && k < d.K;
            cp_async16(as + r * SW_LDA + c4 * 4, in ? Ab + m * lda + k : Ab, in ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {          // B: 16 k-rows x 64 pieces
            const int idx = tid + i * 256, kr = idx / 64, c4 = idx % 64;
            const long long k = k0 + kr, n = n0 + c4 * 4;
            const bool in = k < d.K && n < d.N;
            cp_async16(bs + kr * SW_BN + c4 * 4, in ? Bb + k * ldb + n : Bb, in ? 16 : 0);
        }
    };

    unsigned long long acc[8][8];   // acc[i][jj] = columns 2 jj, 2 jj + 1 of row i of the thread's 8 x 16 tile
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0ull;

#pragma unroll
    for (int s = 0; s < SW_STAGES - 1; ++s) {
        if (s < n_tiles) load_tile(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < n_tiles; ++kt) {
        // tile kt has landed (all but the newest STAGES-2 groups are complete) and every thread is
        // done with the stage that the load below overwrites (tile kt-1's)
        asm volatile("cp.async.wait_group %0;" ::"n"(SW_STAGES - 2) : "memory");
        __syncthreads();
        if (kt + SW_STAGES - 1 < n_tiles) load_tile(kt + SW_STAGES - 1, (kt + SW_STAGES - 1) % SW_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float* as = As + (kt % SW_STAGES) * SW_A_FLOATS;
        const float* bs = Bs + (kt % SW_STAGES) * SW_B_FLOATS;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float4 av[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = (i < 4 ? 0 : 64) + ty * 4 + (i & 3);
                av[i] = *reinterpret_cast<const float4*>(as + r * SW_LDA + g * 4);
            }
#pragma unroll
            for (int kq = 0; kq < 4; ++kq) {
                unsigned long long b[8];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float4 t = *reinterpret_cast<const float4*>(bs + (g * 4 + kq) * SW_BN + h * 64 + tx * 4);
                    b[h * 2] = pack2(t.x, t.y);
                    b[h * 2 + 1] = pack2(t.z, t.w);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = kq == 0 ? av[i].x : kq == 1 ? av[i].y : kq == 2 ? av[i].z : av[i].w;
                    const unsigned long long aa = pack2(a, a);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ffma2(acc[i][j], aa, b[j]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const bool vec_ok = (d.c_rs % 4 == 0) && ((reinterpret_cast<uintptr_t>(Cb) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long m = m0 + (i < 4 ? 0 : 64) + ty * 4 + (i & 3);
        if (m >= d.M) continue;
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const long long n = n0 + h * 64 + tx * 4;
            float v[4];
            asm("mov.b64 {%0, %1}, %2;" : "=f"(v[0]), "=f"(v[1]) : "l"(acc[i][h * 2]));
            asm("mov.b64 {%0, %1}, %2;" : "=f"(v[2]), "=f"(v[3]) : "l"(acc[i][h * 2 + 1]));
            if (halved) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < d.N) atomicAdd(Cb + m * d.c_rs + n + j, v[j]);
            } else if (vec_ok && n + 3 < d.N) {
                *reinterpret_cast<float4*>(Cb + m * d.c_rs + n) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < d.N) Cb[m * d.c_rs + n + j] = v[j];
            }
        }
    }
}

bool run_sgemm(Device& dev, const void* a, const void* b, void* c, const MatmulDims& d) {
    if (d.a_cs != 1 || d.a_rs % 4 || d.K % 4 || !aligned16(a) || !aligned16(b)) return false;
    if (d.a_bs % 4 || d.b_bs % 4) return false;
    const bool b_kn = d.b_cs == 1 && d.b_rs % 4 == 0 && d.N % 4 == 0;
    const bool b_nk = d.b_rs == 1 && d.b_cs % 4 == 0;
    if (!b_kn && !b_nk) return false;
    // the wide kernel pays where its 128x256 tiles fill the machine more than once
    static const bool no_wide = getenv("WGF_SGEMM_NO_WIDE") != nullptr;   // diagnostic switch, read once
    const long long wide_tiles = ((d.M + SW_BM - 1) / SW_BM) * ((d.N + SW_BN - 1) / SW_BN) * d.batch;
    // C as one dense block [batch, M, N]: what the memset before a split launch assumes
    const bool wide_rows_dense = d.c_rs == d.N && (d.batch == 1 || d.c_bs == d.M * d.N);
    if (b_kn && !no_wide && d.M >= 512 && d.N >= 512 && d.K >= 256 && wide_tiles >= 2ll * dev.sm_count &&
        wide_tiles < (1ll << 30)) {
        dev.begin_launch("sgemm_wide");
        if (!dev.dry) {
            static std::mutex mu;
            static bool attr_set[64] = {};
            {
                std::lock_guard<std::mutex> g(mu);
                if (dev.ordinal >= 0 && dev.ordinal < 64 && !attr_set[dev.ordinal]) {
                    cudaFuncSetAttribute(sgemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SW_SMEM);
                    attr_set[dev.ordinal] = true;
                }
            }
            WideSplit ws;
            ws.tn = (int)((d.N + SW_BN - 1) / SW_BN);
            ws.tm = (int)((d.M + SW_BM - 1) / SW_BM);
            const long long tail = wide_tiles % dev.sm_count;
            const bool split = tail > 0 && 2 * tail <= dev.sm_count && d.K >= 4 * SW_BK && wide_rows_dense;
            ws.whole = (int)(split ? wide_tiles - tail : wide_tiles);
            if (split) {
                // the halved tiles are added into C: rows of C are dense here, so one memset covers it
                WGF_CUDA(cudaMemsetAsync(c, 0, (size_t)d.batch * d.M * d.N * sizeof(float), dev.stream));
            }
            const unsigned ctas = (unsigned)(ws.whole + (split ? 2 * tail : 0));
            sgemm_wide_kernel<<<ctas, 256, SW_SMEM, dev.stream>>>((const float*)a, (const float*)b, (float*)c, d, ws);
        }
        dev.end_launch();
        return true;
    }
    dim3 grid((unsigned)((d.N + SG_BN - 1) / SG_BN), (unsigned)((d.M + SG_BM - 1) / SG_BM), (unsigned)d.batch);
    if (grid.y > 65535) return false;
    dev.begin_launch("sgemm");
    if (!dev.dry) {
        if (b_kn) sgemm_kernel<false><<<grid, 256, 0, dev.stream>>>((const float*)a, (const float*)b, (float*)c, d);
        else sgemm_kernel<true><<<grid, 256, 0, dev.stream>>>((const float*)a, (const float*)b, (float*)c, d);
    }
    dev.end_launch();
    return true;
}

}  // namespace

bool matmul_fast_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d) {
    static const bool fallback_only = getenv("WGF_MATMUL_FALLBACK") != nullptr;   // diagnostic switch, read once
    if (fallback_only) return false;
    switch (dt) {
        case DType::F32:
            if (run_gemv<float>(dev, a, b, c, d)) return true;
            if (d.M >= 32 && d.N >= 32) return run_sgemm(dev, a, b, c, d);
            return false;
        case DType::F16:
            if (run_gemv<__half>(dev, a, b, c, d)) return true;
            if (matmul_tc_pair_path(dev, a, b, c, dt, d)) return true;
            return matmul_tc_path(dev, a, b, c, dt, d);
        default:
            if (run_gemv<__nv_bfloat16>(dev, a, b, c, d)) return true;
            if (matmul_tc_pair_path(dev, a, b, c, dt, d)) return true;
            return matmul_tc_path(dev, a, b, c, dt, d);
    }
}

}  // namespace wgf
