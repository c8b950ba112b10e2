/*
 * oracle.c -- CPU restatement of the shader math of the crate `wgpu-compute`
 * (ealmloff/wgpu-kernal-fusion).  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA
 * path (tests/, the smoke test, and the cpu_baseline / reference arm of bench.py); nothing
 * in the product may call it.
 *
 * The crate has no CPU code for its ops: every op is a WGSL snippet evaluated by the GPU
 * driver's shader compiler, whose precision is implementation-defined.  This file restates
 * each snippet with these rules (the reference cannot be built or run here, so the values
 * are pinned by the known answers in the crate's own tests, see tests/test_reference_kats.py;
 * past those answers and their tolerances -- the last bits a particular shader compiler gives
 * a transcendental op -- PARITY IS UNPINNED, because no run of the crate exists to compare with):
 *   - element-wise / pair-wise: evaluate in double, round ONCE to the op's element type;
 *     chains apply op after op, each rounding on its own (src/element_wise.rs:64-79 emits one
 *     WGSL function per op, so no contraction across ops);
 *   - casts: f32->f16 round-to-nearest-even (half::f16::from_f32, src/element_wise.rs:1455),
 *     f16->f32 exact;
 *   - reduce: double accumulation in index order, rounded once (src/reduce.rs:83-281 leaves
 *     the order to the hardware; tolerance in the tests covers that);
 *   - matmul: the mathematical definition with double accumulation (the crate's kernel,
 *     src/matmul.rs:56-155, is only correct up to 8x8).
 * The "fast" functions at the end are the timed CPU baseline: plain float arithmetic with
 * libm, one memory pass per kernel the crate's resolver would launch
 * (src/compute_graph/resolve.rs:63-196), OpenMP over rows.
 *
 * Element type codes: 0 = f32 (float), 1 = f16 and 2 = bf16 (uint16_t bit patterns).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* opcodes: identical to include/wgf.h */
enum {
    OP_EXP = 0, OP_EXP2, OP_LOG, OP_LOG2, OP_SQR, OP_SQRT, OP_SIN, OP_COS, OP_TAN, OP_ASIN, OP_ACOS,
    OP_ATAN, OP_SINH, OP_COSH, OP_TANH, OP_ASINH, OP_ACOSH, OP_ATANH, OP_ABS, OP_NEG,
    OP_ADD_C = 32, OP_SUB_C, OP_RSUB_C, OP_MUL_C, OP_DIV_C, OP_RDIV_C,
    OP_ADD = 64, OP_SUB, OP_MUL, OP_DIV, OP_POW,
    OP_SUM = 96, OP_MAX, OP_MIN, OP_PRODUCT
};

/* ---- rounding a double to f16 / bf16 in one step (round to nearest even) ---------------- */
static double round_to_grid(double x, int mant_bits, int min_exp, double max_finite) {
    if (x == 0.0 || isnan(x) || isinf(x)) return x;
    int e;
    frexp(x, &e);          /* |x| = f * 2^e, f in [0.5, 1) -> exponent of the leading bit is e-1 */
    int lead = e - 1;
    if (lead < min_exp) lead = min_exp;             /* subnormal range: fixed spacing */
    double ulp = ldexp(1.0, lead - mant_bits);
    double q = nearbyint(x / ulp) * ulp;            /* default rounding mode: ties to even */
    if (fabs(q) > max_finite) return x > 0 ? INFINITY : -INFINITY;
    return q;
}
static double round_f16(double x) { return round_to_grid(x, 10, -14, 65504.0); }
static double round_bf16(double x) { return round_to_grid(x, 7, -126, 3.3895313892515355e38); }

static uint16_t f16_bits(double v) { /* v is already on the f16 grid (or inf/nan) */
    uint16_t sign = signbit(v) ? 0x8000u : 0;
    double a = fabs(v);
    if (isnan(v)) return sign | 0x7e00u;
    if (isinf(v)) return sign | 0x7c00u;
    if (a == 0.0) return sign;
    int e;
    double f = frexp(a, &e); /* a = f * 2^e */
    int lead = e - 1;
    if (lead < -14) return sign | (uint16_t)(a / ldexp(1.0, -24));
    uint16_t man = (uint16_t)((f * 2.0 - 1.0) * 1024.0);
    return sign | (uint16_t)((lead + 15) << 10) | man;
}
static double f16_value(uint16_t h) {
    int sign = h >> 15, exp = (h >> 10) & 31, man = h & 1023;
    double v;
    if (exp == 0) v = ldexp((double)man, -24);
    else if (exp == 31) v = man ? NAN : INFINITY;
    else v = ldexp(1.0 + man / 1024.0, exp - 15);
    return sign ? -v : v;
}
static uint16_t bf16_bits(double v) {
    float f = (float)v; /* v is on the bf16 grid, hence exact in float */
    uint32_t u;
    memcpy(&u, &f, 4);
    if (isnan(v)) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)(u >> 16);
}
static double bf16_value(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return (double)f;
}

static double load(const void* p, int dt, int64_t i) {
    if (dt == 0) return (double)((const float*)p)[i];
    if (dt == 1) return f16_value(((const uint16_t*)p)[i]);
    return bf16_value(((const uint16_t*)p)[i]);
}
static void store(void* p, int dt, int64_t i, double v) {
    if (dt == 0) ((float*)p)[i] = (float)v;
    else if (dt == 1) ((uint16_t*)p)[i] = f16_bits(round_f16(v));
    else ((uint16_t*)p)[i] = bf16_bits(round_bf16(v));
}
/* a float constant as the shader of an f16 / bf16 tensor sees it (src/element_wise.rs:70-74) */
static double imm_as(int dt, float c) { return dt == 0 ? (double)c : dt == 1 ? round_f16(c) : round_bf16(c); }

/* ---- WGSL snippets: src/element_wise.rs:678-1380 ---------------------------------------- */
static double unary(int op, double x) {
    switch (op) {
        case OP_EXP: return exp(x);      /* "let output = exp(input);"   :682 */
        case OP_EXP2: return exp2(x);    /* :717 */
        case OP_LOG: return log(x);      /* :752 */
        case OP_LOG2: return log2(x);    /* :787 */
        case OP_SQR: return x * x;       /* "input * input" :823 */
        case OP_SQRT: return sqrt(x);    /* :863 */
        case OP_SIN: return sin(x);      /* :898 */
        case OP_COS: return cos(x);      /* :933 */
        case OP_TAN: return tan(x);      /* :968 */
        case OP_ASIN: return asin(x);    /* :1003 */
        case OP_ACOS: return acos(x);    /* :1042 */
        case OP_ATAN: return atan(x);    /* :1081 */
        case OP_SINH: return sinh(x);    /* :1116 */
        case OP_COSH: return cosh(x);    /* :1151 */
        case OP_TANH: return tanh(x);    /* :1186 */
        case OP_ASINH: return asinh(x);  /* :1221 */
        case OP_ACOSH: return acosh(x);  /* :1260 */
        case OP_ATANH: return atanh(x);  /* :1299 */
        case OP_ABS: return fabs(x);     /* :1338 */
        case OP_NEG: return -x;          /* :1376 */
    }
    return NAN;
}
/* src/element_wise.rs:204, 452, 492, 532, 605, 645 */
static double scalar(int op, double x, double c) {
    switch (op) {
        case OP_ADD_C: return x + c;
        case OP_SUB_C: return x - c;
        case OP_RSUB_C: return c - x;
        case OP_MUL_C: return x * c;
        case OP_DIV_C: return x / c;
        case OP_RDIV_C: return c / x;
    }
    return NAN;
}
/* src/pair_wise.rs:219, 390, 438, 486, 524 */
static double binary(int op, double a, double b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_SUB: return a - b;
        case OP_MUL: return a * b;
        case OP_DIV: return a / b;
        case OP_POW: return pow(a, b);
    }
    return NAN;
}

void orc_unary(int op, int dt, const void* in, void* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) store(out, dt, i, unary(op, load(in, dt, i)));
}
void orc_scalar(int op, int dt, const void* in, float c, void* out, int64_t n) {
    double cc = imm_as(dt, c);
    for (int64_t i = 0; i < n; ++i) store(out, dt, i, scalar(op, load(in, dt, i), cc));
}
/* src/element_wise.rs:1408-1471 */
void orc_cast(int from, int to, const void* in, void* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) store(out, to, i, load(in, from, i));
}
void orc_binary(int op, int dt, const void* a, const void* b, void* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) store(out, dt, i, binary(op, load(a, dt, i), load(b, dt, i)));
}

/* src/reduce.rs:439-448 (sum, init 0), :633-646 (max, init -3.40282e+38), :706-719 (min),
 * :779-788 (product, init 1).  in = [outer, k, inner] row-major, out = [outer, inner]. */
void orc_reduce(int op, int dt, const void* in, void* out, int64_t outer, int64_t k, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            double acc = op == OP_SUM ? 0.0 : op == OP_PRODUCT ? 1.0
                         : op == OP_MAX ? (double)-3.40282e+38f : (double)3.40282e+38f;
            for (int64_t j = 0; j < k; ++j) {
                double v = load(in, dt, (o * k + j) * inner + i);
                if (op == OP_SUM) acc += v;
                else if (op == OP_PRODUCT) acc *= v;
                else if (op == OP_MAX) acc = v > acc ? v : acc;
                else acc = v < acc ? v : acc;
            }
            store(out, dt, o * inner + i, acc);
        }
}

/* C[b,m,n] = sum_k A[b,m,k] B[b,k,n], double accumulation, one rounding. */
void orc_matmul(int dt, const void* a, const void* b, void* c, int64_t batch, int64_t M, int64_t N, int64_t K) {
    double* row = (double*)malloc(sizeof(double) * (size_t)(N > 0 ? N : 1));
    for (int64_t z = 0; z < batch; ++z)
        for (int64_t m = 0; m < M; ++m) {
            for (int64_t n = 0; n < N; ++n) row[n] = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                double av = load(a, dt, (z * M + m) * K + k);
                for (int64_t n = 0; n < N; ++n) row[n] += av * load(b, dt, (z * K + k) * N + n);
            }
            for (int64_t n = 0; n < N; ++n) store(c, dt, (z * M + m) * N + n, row[n]);
        }
    free(row);
}

/* Units in the last place between two floats of the same sign region (for reports). */
int64_t orc_ulp_diff_f32(float a, float b) {
    if (isnan(a) || isnan(b)) return (isnan(a) && isnan(b)) ? 0 : INT64_MAX;
    int32_t ia, ib;
    memcpy(&ia, &a, 4);
    memcpy(&ib, &b, 4);
    if (ia < 0) ia = (int32_t)0x80000000 - ia;
    if (ib < 0) ib = (int32_t)0x80000000 - ib;
    int64_t d = (int64_t)ia - (int64_t)ib;
    return d < 0 ? -d : d;
}

/* =========================================================================================
 * Timed CPU baseline ("fast mode"): float arithmetic + libm, one pass over memory per kernel
 * the crate would launch, all host threads.
 * ======================================================================================= */
int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the thread count of the timed functions, whatever OMP_NUM_THREADS says (process
 * launchers export OMP_NUM_THREADS=1 for their children; the CPU baseline is meant to use
 * every host core).  Returns the count now in effect. */
int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) {
        omp_set_dynamic(0);
        omp_set_num_threads(n);
    }
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* layer_norm (src/composite/rms_norm.rs:8-15) resolves to 3 kernels: reduce(sum, pre sqr,
 * post /H +eps sqrt), pairwise div by the broadcast norm, pairwise mul by the broadcast weight. */
void orc_fast_rms_norm(const float* x, const float* w, float eps, float* norm, float* tmp, float* out,
                       int64_t rows, int64_t h) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float s = 0.f;
        for (int64_t i = 0; i < h; ++i) s += x[r * h + i] * x[r * h + i];
        norm[r] = sqrtf(s / (float)h + eps);
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < h; ++i) tmp[r * h + i] = x[r * h + i] / norm[r];
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < h; ++i) out[r * h + i] = tmp[r * h + i] * w[i];
}

/* Max-subtracted row softmax composed from max(1), broadcast, -, exp, sum(1), /.  The crate's
 * resolver keeps no memo of shared nodes (src/compute_graph/resolve.rs:16-47), so the
 * (x - max) node is computed once per consumer: 6 kernels. */
void orc_fast_softmax_rows(const float* x, float* m, float* t1, float* t2, float* s, float* out,
                           int64_t rows, int64_t h) {
    for (int rep = 0; rep < 2; ++rep) { /* max reduce + subtract, once for each consumer of exp(x - max) */
        float* t = rep ? t2 : t1;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float mx = -3.40282e+38f;
            for (int64_t i = 0; i < h; ++i) mx = fmaxf(mx, x[r * h + i]);
            m[r] = mx;
        }
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t i = 0; i < h; ++i) t[r * h + i] = x[r * h + i] - m[r];
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) { /* sum reduce with exp as prologue */
        float acc = 0.f;
        for (int64_t i = 0; i < h; ++i) acc += expf(t2[r * h + i]);
        s[r] = acc;
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) /* pairwise div with exp as prologue of operand 0 */
        for (int64_t i = 0; i < h; ++i) out[r * h + i] = expf(t1[r * h + i]) / s[r];
}

/* exp(x).sum(0).sum(0): reduce over axis 0 with exp as prologue, then a second reduce. */
float orc_fast_sum_exp(const float* x, float* col, int64_t rows, int64_t h) {
#pragma omp parallel for schedule(static)
    for (int64_t i0 = 0; i0 < h; i0 += 64) {
        int64_t i1 = i0 + 64 < h ? i0 + 64 : h;
        for (int64_t i = i0; i < i1; ++i) col[i] = 0.f;
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t i = i0; i < i1; ++i) col[i] += expf(x[r * h + i]);
    }
    float acc = 0.f;
    for (int64_t i = 0; i < h; ++i) acc += col[i];
    return acc;
}

/* C1 chain as one element-wise pass (the crate would need one pair-wise kernel). */
void orc_fast_chain_c1(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        y[i] = cosf(sinf(v * 2.0f + 1.0f)) * 0.5f + expf(-(v * v));
    }
}
