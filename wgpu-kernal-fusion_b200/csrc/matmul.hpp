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

// What the tcgen05 CTA-pair kernel can do to the product before it is stored (matmul_tc2.cu).
struct MatmulEpilogue {
    enum Kind { NONE = 0, RESIDUAL = 1, SILU_MUL = 2 };
    int kind = NONE;
    const void* resid = nullptr;   // RESIDUAL: [batch, M, N] of C's element type, added to the rounded product
    long long r_rs = 0, r_bs = 0;  //           its row / batch strides in elements (column stride 1)
    const void* b2 = nullptr;      // SILU_MUL: the second B operand, same shape and strides as b: C = silu(A b) * (A b2)
};

// Tries the specialised kernels (f32 tiled FFMA, f16/bf16 tcgen05, GEMV).  Returns false if
// none applies to this layout, in which case the strided fallback runs.
bool matmul_fast_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d);

}  // namespace wgf
