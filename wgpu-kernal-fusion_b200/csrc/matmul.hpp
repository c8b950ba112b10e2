// Shared between the matmul kernels: problem description in elements.
#pragma once
#include "runtime.hpp"

namespace wgf {

struct MatmulDims {
    long long batch, M, N, K;
    long long a_bs, a_rs, a_cs;  // A[b, m, k] strides
    long long b_bs, b_rs, b_cs;  // B[b, k, n] strides
    long long c_bs, c_rs;        // C is row-major: column stride 1
};

// Tries the specialised kernels (f32 tiled FFMA, f16/bf16 tcgen05, GEMV).  Returns false if
// none applies to this layout, in which case the strided fallback runs.
bool matmul_fast_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d);

}  // namespace wgf
