// Full-tensor reduction for callers that must not allocate.
//
// Some hosts of this library cannot tolerate an allocation inside a compute call: real-time
// loops that forbid anything with unbounded latency (cudaMalloc may synchronise the device),
// and embedders whose memory budget is fixed up front so that every byte on the device is
// accounted for by them.  wgf_full_reduce_f32_noalloc gives those callers the streaming
// reduction (the kernel behind `t.exp().sum(0).sum(0)` and friends) without the pool: its
// scratch -- one partial result per CTA and the ticket that elects the last CTA -- lives in a
// fixed array inside the library image instead of a buffer taken from the device allocator.
//
// Consequences of the fixed array, all part of the contract:
//   * every GPU that loads the library holds the 16 KiB array until the process exits;
//   * all calls on one GPU share it, and it keeps what the previous call left there, so the
//     ticket is cleared on the stream before each launch; two calls that overlap on the GPU
//     (different streams, no dependency) race on it and must not be issued;
//   * the first call on a GPU looks the array's device address up (cudaGetSymbolAddress);
//     make that first call outside any stream capture.
// Inputs and outputs are the caller's device pointers; nothing here calls cudaMalloc,
// cudaFree or any allocating library routine.
#include <cuda_runtime.h>

#include <mutex>

#include "common.hpp"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxCtas = 3840;                        // partial slots in the fixed array
constexpr size_t kTicketBytes = 256;                  // first 256 bytes: the ticket counter
constexpr size_t kScratchBytes = kTicketBytes + sizeof(float) * kMaxCtas;  // 15 616 bytes
constexpr unsigned long long kMaxElems = 1ull << 31;  // 8 GiB of f32 per call

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device
// address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[16384];
static_assert(kScratchBytes <= sizeof(g_noalloc_scratch), "scratch layout exceeds the fixed array");

enum Pre { PRE_NONE = 0, PRE_EXP, PRE_SQR, PRE_ABS };
enum Red { R_SUM = 0, R_MAX, R_MIN, R_PROD };

template <int PRE> __device__ __forceinline__ float pre_op(float x) {
    return PRE == PRE_EXP ? expf(x) : PRE == PRE_SQR ? __fmul_rn(x, x) : PRE == PRE_ABS ? fabsf(x) : x;
}
template <int RED> __device__ __forceinline__ float ident() {
    return RED == R_SUM ? 0.f : RED == R_PROD ? 1.f : RED == R_MAX ? -3.40282e+38f : 3.40282e+38f;
}
template <int RED> __device__ __forceinline__ float comb(float a, float b) {
    return RED == R_SUM ? __fadd_rn(a, b) : RED == R_PROD ? __fmul_rn(a, b) : RED == R_MAX ? fmaxf(a, b) : fminf(a, b);
}
template <int RED> __device__ __forceinline__ float block_reduce(float v, float* smem) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = comb<RED>(v, __shfl_xor_sync(0xffffffffu, v, m));
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    v = smem[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) v = comb<RED>(v, smem[w]);
    __syncthreads();
    return v;
}

// Grid-stride over float4 chunks (scalar head/tail when the pointer or length is ragged);
// per-CTA partials go to the fixed scratch, the last CTA to take a ticket combines them in
// index order and writes the result.
template <int PRE, int RED>
__global__ void __launch_bounds__(kThreads, 4)
noalloc_reduce_kernel(const float* __restrict__ x, unsigned long long n, float* __restrict__ out,
                      unsigned char* scratch) {
    __shared__ float smem[kThreads / 32];
    __shared__ unsigned is_last;
    unsigned* ticket = reinterpret_cast<unsigned*>(scratch);
    float* partials = reinterpret_cast<float*>(scratch + kTicketBytes);
    float acc = ident<RED>();
    const unsigned long long tid = (unsigned long long)blockIdx.x * kThreads + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * kThreads;
    // elements before the first 16-byte boundary
    unsigned long long head = ((16 - ((unsigned long long)x & 15)) & 15) / 4;
    if (head > n) head = n;
    if (tid < head) acc = comb<RED>(acc, pre_op<PRE>(x[tid]));
    const float4* x4 = reinterpret_cast<const float4*>(x + head);
    const unsigned long long n4 = (n - head) / 4;
    for (unsigned long long i = tid; i < n4; i += 2 * nthreads) {
        float4 a = x4[i];
        const unsigned long long j = i + nthreads;
        float4 b = make_float4(0, 0, 0, 0);
        const bool hb = j < n4;
        if (hb) b = x4[j];
        acc = comb<RED>(acc, pre_op<PRE>(a.x));
        acc = comb<RED>(acc, pre_op<PRE>(a.y));
        acc = comb<RED>(acc, pre_op<PRE>(a.z));
        acc = comb<RED>(acc, pre_op<PRE>(a.w));
        if (hb) {
            acc = comb<RED>(acc, pre_op<PRE>(b.x));
            acc = comb<RED>(acc, pre_op<PRE>(b.y));
            acc = comb<RED>(acc, pre_op<PRE>(b.z));
            acc = comb<RED>(acc, pre_op<PRE>(b.w));
        }
    }
    const unsigned long long tail0 = head + n4 * 4;
    if (tail0 + tid < n) acc = comb<RED>(acc, pre_op<PRE>(x[tail0 + tid]));
    acc = block_reduce<RED>(acc, smem);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = acc;
        __threadfence();
        is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    acc = ident<RED>();
    for (unsigned i = threadIdx.x; i < gridDim.x; i += kThreads) acc = comb<RED>(acc, __ldcg(partials + i));
    acc = block_reduce<RED>(acc, smem);
    if (threadIdx.x == 0) {
        out[0] = acc;
        *ticket = 0;
    }
}

template <int PRE>
cudaError_t launch_red(int red, int grid, cudaStream_t s, const float* x, unsigned long long n, float* out,
                       unsigned char* scratch) {
    switch (red) {
        case R_SUM: noalloc_reduce_kernel<PRE, R_SUM><<<grid, kThreads, 0, s>>>(x, n, out, scratch); break;
        case R_MAX: noalloc_reduce_kernel<PRE, R_MAX><<<grid, kThreads, 0, s>>>(x, n, out, scratch); break;
        case R_MIN: noalloc_reduce_kernel<PRE, R_MIN><<<grid, kThreads, 0, s>>>(x, n, out, scratch); break;
        default: noalloc_reduce_kernel<PRE, R_PROD><<<grid, kThreads, 0, s>>>(x, n, out, scratch); break;
    }
    return cudaGetLastError();
}

struct PerDevice {
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this GPU
    int sm_count = 0;
};
std::mutex g_mu;
PerDevice g_dev[64];

}  // namespace

extern "C" int32_t wgf_full_reduce_f32_noalloc(const float* x, uint64_t n, uint32_t pre_opcode,
                                               uint32_t reduce_opcode, float* out, void* cuda_stream) {
    auto fail_with = [&](int code, const std::string& m) {
        wgf::set_last_error(m);
        return code;
    };
    if (!x || !out) return fail_with(WGF_ERR_INVALID_HANDLE, "wgf_full_reduce_f32_noalloc: null device pointer");
    if (n > kMaxElems)
        return fail_with(WGF_ERR_UNSUPPORTED,
                         "wgf_full_reduce_f32_noalloc: " + std::to_string(n) +
                             " elements exceed the maximum of 2147483648 per call; split the input");
    int pre;
    switch (pre_opcode) {
        case 0xFFFFFFFFu: pre = PRE_NONE; break;
        case WGF_OP_EXP: pre = PRE_EXP; break;
        case WGF_OP_SQR: pre = PRE_SQR; break;
        case WGF_OP_ABS: pre = PRE_ABS; break;
        default:
            return fail_with(WGF_ERR_INVALID_ARGUMENT,
                             "wgf_full_reduce_f32_noalloc: prologue must be WGF_OP_EXP, WGF_OP_SQR, WGF_OP_ABS or 0xFFFFFFFF (none)");
    }
    if (reduce_opcode < WGF_OP_SUM || reduce_opcode > WGF_OP_PRODUCT)
        return fail_with(WGF_ERR_INVALID_ARGUMENT, "wgf_full_reduce_f32_noalloc: not a reduce opcode");
    const int red = reduce_opcode == WGF_OP_SUM ? R_SUM : reduce_opcode == WGF_OP_MAX ? R_MAX
                    : reduce_opcode == WGF_OP_MIN ? R_MIN : R_PROD;

    // the GPU that owns the input becomes current for the duration of the call
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, x);
    if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        return fail_with(WGF_ERR_INVALID_ARGUMENT, "wgf_full_reduce_f32_noalloc: x is not a device pointer");
    }
    const int ordinal = attr.device;
    if (ordinal < 0 || ordinal >= 64) return fail_with(WGF_ERR_UNSUPPORTED, "wgf_full_reduce_f32_noalloc: device ordinal above 63");
    int previous = 0;
    cudaGetDevice(&previous);
    if ((e = cudaSetDevice(ordinal)) != cudaSuccess)
        return fail_with(WGF_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));

    PerDevice pd;
    {
        // one-time set-up per GPU, with that GPU current: the device address of the array
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_dev[ordinal].scratch) {
            unsigned char* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                cudaSetDevice(previous);
                return fail_with(WGF_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
            }
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal);
            if (e != cudaSuccess || sms <= 0) {
                cudaSetDevice(previous);
                return fail_with(WGF_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
            }
            g_dev[ordinal].scratch = p;
            g_dev[ordinal].sm_count = sms;
        }
        pd = g_dev[ordinal];
    }
    cudaStream_t s = (cudaStream_t)cuda_stream;
    // four resident CTAs per SM, never more partial slots than the array holds, never more
    // CTAs than there are 2 KiB pieces of input
    unsigned long long want = (n + 2047) / 2048;
    int grid = pd.sm_count * 4;
    if (grid > kMaxCtas) grid = kMaxCtas;
    if ((unsigned long long)grid > want) grid = (int)(want ? want : 1);
    // the array keeps the previous call's contents: the ticket has to start at zero
    e = cudaMemsetAsync(pd.scratch, 0, kTicketBytes, s);
    if (e == cudaSuccess) {
        switch (pre) {
            case PRE_NONE: e = launch_red<PRE_NONE>(red, grid, s, x, n, out, pd.scratch); break;
            case PRE_EXP: e = launch_red<PRE_EXP>(red, grid, s, x, n, out, pd.scratch); break;
            case PRE_SQR: e = launch_red<PRE_SQR>(red, grid, s, x, n, out, pd.scratch); break;
            default: e = launch_red<PRE_ABS>(red, grid, s, x, n, out, pd.scratch); break;
        }
    }
    cudaSetDevice(previous);
    if (e != cudaSuccess) return fail_with(WGF_ERR_CUDA, std::string("wgf_full_reduce_f32_noalloc: ") + cudaGetErrorString(e));
    return WGF_OK;
}
