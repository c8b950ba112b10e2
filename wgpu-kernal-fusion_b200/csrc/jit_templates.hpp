// Hand-written CUDA kernel templates for the fused element-wise / pair-wise / reduce family.
// codegen.cpp prepends `#define`s and the generated per-program functions, then hands the
// text to NVRTC (the analogue of the crate's WGSL assembly in src/kernel.rs:391-495 and
// src/visit_tiled.rs:63-147, but the kernels themselves are written for sm_100a: 128-bit
// coalesced accesses along the innermost stride-1 axis, rows kept in registers across
// reductions, warp-shuffle + shared-memory block reductions).
#pragma once

namespace wgf {

// Common device helpers.  No CUDA headers are included: conversions use PTX directly.
static const char* const JIT_PRELUDE = R"CUDA(
typedef unsigned short u16;
typedef unsigned int u32;
typedef long long i64;
typedef unsigned long long u64;
#define DEV __device__ __forceinline__

// Checked build (environment WGF_CHECKED=1; the device puts the three defines in front of this
// text): every access of a generated kernel to tensor memory is tested against the extents of the
// buffers that the host bound to the launch.  An access outside all of them is NOT made: the first
// one is recorded (error word = 61, then the address and the byte count) and the host reports it
// at its next synchronisation.  The stand-in for a memory checker where none can be run; several
// times slower than the normal build.
#ifndef WGF_CHECKED
#define WGF_CHECKED 0
#endif
#if WGF_CHECKED
struct ChkTable { u64 n; u64 lo[24]; u64 hi[24]; };
__device__ __noinline__ bool chk(const void* base, i64 elem, int esize, int n) {
    const ChkTable* t = (const ChkTable*)WGF_CHK_TABLE;
    const u64 a = (u64)base + (u64)(elem * esize), e = a + (u64)(n * esize);
    for (u64 k = 0; k < t->n; ++k)
        if (a >= t->lo[k] && e <= t->hi[k]) return true;
    u32* err = (u32*)WGF_CHK_ERR;
    if (atomicCAS(err, 0u, 61u) == 0u) {
        ((u64*)err)[1] = a;
        ((u64*)err)[2] = e - a;
    }
    return false;
}
#define CHK_FAILS(base, i, esize, n) (!chk(base, i, esize, n))
#else
#define CHK_FAILS(base, i, esize, n) false
#endif

DEV float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
DEV float b2f(u16 b) { return __uint_as_float(((u32)b) << 16); }
// two floats -> packed pair of 16-bit values (lo in bits 0-15), round to nearest even
DEV u32 f2h2(float lo, float hi) { u32 r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
DEV u32 f2b2(float lo, float hi) { u32 r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
DEV u16 f2h(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
DEV u16 f2b(float f) { u16 b; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(b) : "f"(f)); return b; }
// round a float to the nearest f16 / bf16 value (every op of a 16-bit tensor rounds once)
DEV float rh(float x) { return h2f(f2h(x)); }
DEV float rb(float x) { return b2f(f2b(x)); }

// Unary functions.  Single-precision CUDA functions documented at <= 2 ulp are used as they
// are; the ones documented above that (tan, sinh, asinh, acosh, atanh, pow) go through double.
DEV float op_exp(float x) { return expf(x); }
// 2^(x * log2 e) by the special-function unit (about 1e-6 relative): for results that are rounded to a
// 16-bit type, and for f32 values that only feed sums
DEV float op_exp_sfu(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f)); return y; }
// a / b to 2 ulp over the full range (div.full.f32): for quotients whose divisor is itself the result
// of an approximated function (Instr::fast_div); exact quotients use the IEEE `/`
DEV float op_div_full(float a, float b) { float q; asm("div.full.f32 %0, %1, %2;" : "=f"(q) : "f"(a), "f"(b)); return q; }
DEV float op_exp2(float x) { return exp2f(x); }
DEV float op_log(float x) { return logf(x); }
DEV float op_log2(float x) { return log2f(x); }
DEV float op_sqrt(float x) { return sqrtf(x); }
DEV float op_sin(float x) { return sinf(x); }
DEV float op_cos(float x) { return cosf(x); }
// sin / cos of an argument in [-1, 1] (Instr::arg_unit: the argument is itself a sine, cosine or
// tanh): the Taylor polynomial on the whole interval, no range reduction, no slow path.  Truncation
// error at |x| = 1: 1.6e-10 (sin, degree 11), 2.1e-9 (cos, degree 10); with the rounding of the
// Horner steps the results stay within 1 ulp of the correctly rounded value over all of [-1, 1]
// (checked against float64 over the sampled interval in the parity tests).  NaN gives NaN.
DEV float op_sin_unit(float x) {
    const float s = x * x;
    float p = fmaf(s, -2.50521084e-08f, 2.75573192e-06f);
    p = fmaf(p, s, -1.98412698e-04f);
    p = fmaf(p, s, 8.33333333e-03f);
    p = fmaf(p, s, -1.66666667e-01f);
    return fmaf(x, p * s, x);
}
DEV float op_cos_unit(float x) {
    const float s = x * x;
    float p = fmaf(s, -2.75573192e-07f, 2.48015873e-05f);
    p = fmaf(p, s, -1.38888889e-03f);
    p = fmaf(p, s, 4.16666667e-02f);
    p = fmaf(p, s, -0.5f);
    return fmaf(p, s, 1.0f);
}
DEV float op_tan(float x) { return (float)tan((double)x); }
DEV float op_asin(float x) { return asinf(x); }
DEV float op_acos(float x) { return acosf(x); }
DEV float op_atan(float x) { return atanf(x); }
DEV float op_sinh(float x) { return (float)sinh((double)x); }
DEV float op_cosh(float x) { return coshf(x); }
DEV float op_tanh(float x) { return tanhf(x); }
DEV float op_asinh(float x) { return (float)asinh((double)x); }
DEV float op_acosh(float x) { return (float)acosh((double)x); }
DEV float op_atanh(float x) { return (float)atanh((double)x); }
DEV float op_pow(float a, float b) { return (float)pow((double)a, (double)b); }

// n / d for n < 2^31 with a precomputed multiplier (m == 0 encodes d == 1)
DEV u32 fastdiv(u32 n, u32 m, u32 s) { return m ? (__umulhi(n, m) >> s) : n; }

template <int DT> DEV float load1(const void* base, i64 i) {
    if (CHK_FAILS(base, i, DT == 0 ? 4 : 2, 1)) return 0.f;
    if (DT == 0) return ((const float*)base)[i];
    u16 v = ((const u16*)base)[i];
    return DT == 1 ? h2f(v) : b2f(v);
}
template <int DT> DEV void store1(void* base, i64 i, float v) {
    if (CHK_FAILS(base, i, DT == 0 ? 4 : 2, 1)) return;
    if (DT == 0) ((float*)base)[i] = v;
    else ((u16*)base)[i] = DT == 1 ? f2h(v) : f2b(v);
}
// four consecutive f32 at element index i (16-byte aligned), zeros where the checked build refuses
DEV float4 load_f4(const void* base, i64 i) {
    if (CHK_FAILS(base, i, 4, 4)) return make_float4(0.f, 0.f, 0.f, 0.f);
    return *(const float4*)((const float*)base + i);
}
template <int DT> DEV float cvt16(u16 v) { return DT == 1 ? h2f(v) : b2f(v); }
template <int DT> DEV u32 pack16(float lo, float hi) {
    return DT == 1 ? f2h2(lo, hi) : f2b2(lo, hi);
}

// C consecutive elements starting at element index i; (base + i) is aligned to the vector.
template <int DT, int C> DEV void load_vec(const void* base, i64 i, float* out) {
    if (CHK_FAILS(base, i, DT == 0 ? 4 : 2, C)) {
#pragma unroll
        for (int j = 0; j < C; ++j) out[j] = 0.f;
        return;
    }
    if (DT == 0) {
        if (C % 4 == 0) {
            const float4* p = (const float4*)((const float*)base + i);
#pragma unroll
            for (int q = 0; q < C / 4; ++q) {
                float4 t = p[q];
                out[4 * q] = t.x; out[4 * q + 1] = t.y; out[4 * q + 2] = t.z; out[4 * q + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) out[j] = ((const float*)base)[i + j];
        }
    } else {
        if (C == 8) {
            uint4 t = *(const uint4*)((const u16*)base + i);
            u32 w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                out[2 * q] = cvt16<DT>((u16)(w[q] & 0xffff));
                out[2 * q + 1] = cvt16<DT>((u16)(w[q] >> 16));
            }
        } else if (C == 4) {
            uint2 t = *(const uint2*)((const u16*)base + i);
            out[0] = cvt16<DT>((u16)(t.x & 0xffff)); out[1] = cvt16<DT>((u16)(t.x >> 16));
            out[2] = cvt16<DT>((u16)(t.y & 0xffff)); out[3] = cvt16<DT>((u16)(t.y >> 16));
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) out[j] = cvt16<DT>(((const u16*)base)[i + j]);
        }
    }
}
template <int DT, int C> DEV void store_vec(void* base, i64 i, const float* v) {
    if (CHK_FAILS(base, i, DT == 0 ? 4 : 2, C)) return;
    if (DT == 0) {
        if (C % 4 == 0) {
            float4* p = (float4*)((float*)base + i);
#pragma unroll
            for (int q = 0; q < C / 4; ++q) p[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) ((float*)base)[i + j] = v[j];
        }
    } else {
        if (C == 8) {
            uint4 t;
            t.x = pack16<DT>(v[0], v[1]); t.y = pack16<DT>(v[2], v[3]);
            t.z = pack16<DT>(v[4], v[5]); t.w = pack16<DT>(v[6], v[7]);
            *(uint4*)((u16*)base + i) = t;
        } else if (C == 4) {
            uint2 t;
            t.x = pack16<DT>(v[0], v[1]); t.y = pack16<DT>(v[2], v[3]);
            *(uint2*)((u16*)base + i) = t;
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) store1<DT>(base, i + j, v[j]);
        }
    }
}

// MODE 0: aligned vector, 1: contiguous scalars, 2: one element broadcast, 3: strided.
template <int DT, int C, int MODE>
DEV void load_chunk(const void* base, i64 off, i64 cs, int nvalid, float* out) {
    if (MODE == 2) {
        float v = load1<DT>(base, off);
#pragma unroll
        for (int j = 0; j < C; ++j) out[j] = v;
    } else if (MODE == 0 && C > 1) {
        if (nvalid == C) {
            load_vec<DT, C>(base, off, out);
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) out[j] = j < nvalid ? load1<DT>(base, off + j) : 0.f;
        }
    } else {
        const i64 st = MODE == 3 ? cs : 1;
#pragma unroll
        for (int j = 0; j < C; ++j) out[j] = j < nvalid ? load1<DT>(base, off + j * st) : 0.f;
    }
}
template <int DT, int C, int MODE>
DEV void store_chunk(void* base, i64 off, int nvalid, const float* v) {
    if (MODE == 0 && C > 1 && nvalid == C) {
        store_vec<DT, C>(base, off, v);
    } else {
#pragma unroll
        for (int j = 0; j < C; ++j)
            if (j < nvalid) store1<DT>(base, off + j, v[j]);
    }
}

// Reductions (identities follow src/reduce.rs:444, 638-642, 711-715, 784).
#define RED_SUM 0
#define RED_MAX 1
#define RED_MIN 2
#define RED_PROD 3
template <int OP> DEV float red_ident() {
    return OP == RED_SUM ? 0.f : OP == RED_PROD ? 1.f : OP == RED_MAX ? -3.40282e+38f : 3.40282e+38f;
}
template <int OP> DEV float red_comb(float a, float b) {
    return OP == RED_SUM ? a + b : OP == RED_PROD ? a * b : OP == RED_MAX ? fmaxf(a, b) : fminf(a, b);
}
// All-lanes reduction over the `GROUP` consecutive threads that share a row.  `slot` points
// at GROUP/32 floats of shared memory private to this (reduction, row) pair, 16-byte aligned
// when GROUP >= 128.  The warps' values are combined in warp order whichever way they are read.
template <int OP, int GROUP> DEV float group_reduce(float v, float* slot, int t) {
#if WGF_REDUX
    // max / min of a warp in one instruction (redux.sync on f32, sm_100a); NaN operands are
    // skipped exactly as fmaxf / fminf skip them
    if (OP == RED_MAX) asm volatile("redux.sync.max.f32 %0, %0, 0xffffffff;" : "+f"(v));
    else if (OP == RED_MIN) asm volatile("redux.sync.min.f32 %0, %0, 0xffffffff;" : "+f"(v));
    else
#endif
    {
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) v = red_comb<OP>(v, __shfl_xor_sync(0xffffffffu, v, m));
    }
    if (GROUP > 32) {
        if ((t & 31) == 0) slot[t >> 5] = v;
        __syncthreads();
        if (GROUP >= 128) {
            const float4* s4 = (const float4*)slot;
#pragma unroll
            for (int w = 0; w < GROUP / 128; ++w) {
                const float4 q = s4[w];
                v = w == 0 ? q.x : red_comb<OP>(v, q.x);
                v = red_comb<OP>(red_comb<OP>(red_comb<OP>(v, q.y), q.z), q.w);
            }
        } else {
            v = slot[0];
#pragma unroll
            for (int w = 1; w < GROUP / 32; ++w) v = red_comb<OP>(v, slot[w]);
        }
    }
    return v;
}

// All-reduce of a few scalars across the GPUs of a communicator without a collective launch, as
// a pipeline over three kernels of the same stream that all belong to this path (see Comm).
// Mailboxes hold words {sequence << 32 | value bits} at
// [sequence % PEER_SLOTS][source rank][value index]; a single 64-bit store is atomic, so a word
// that carries the expected sequence number carries the value that belongs to it.
//
// The kernel that PRODUCES exchange k only stores this GPU's values to the result buffers.
// The next such kernel POSTS them first thing (one thread per value of its last CTA): it reads
// the value back from the result buffer and sends it to every rank's mailbox, this GPU's own
// included, by one 64-bit store each (over NVLink for the peers).  Nothing here waits.  Stores
// to memory that peers have mapped delay the end of the kernel that issues them by about 2 us
// when they are its last instructions; issued at the start they cost nothing.
#define PEER_SLOTS 16u
#define PEER_ST(ptr, v) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(ptr), "l"(v) : "memory")
#define PEER_LD(w, ptr) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(ptr) : "memory")
// meta = dtype << 8 | value index << 16 (the low byte, the settling side's op code, is not used here)
DEV void peer_post(u64 src, u32 meta, u64 peers, u32 world, u32 rank, u32 seq) {
    const u32 dt = (meta >> 8) & 255u;
    const float mine = dt == 0 ? *(const float*)src : dt == 1 ? h2f(*(const u16*)src) : b2f(*(const u16*)src);
    const u64* table = (const u64*)peers;
    const u64 word = ((u64)seq << 32) | (u64)__float_as_uint(mine);
    const u64 at = ((u64)((seq % PEER_SLOTS) * world + rank)) * 4 + (u64)(meta >> 16);
    for (u32 r = 0; r < world; ++r) {
        u64* slot = (u64*)table[r] + at;
        PEER_ST(slot, word);
    }
}

// SETTLING exchange k: wait (bounded by wait_ns) until this GPU's own mailbox holds every rank's
// word of it, combine the words in rank order -- every rank ends with the same bits -- and write
// the n results over this GPU's own values.  The kernel that produces exchange k + 6 does it (the
// lag of the pipeline, see Comm): the peers posted k at the start of their kernel k + 1, several
// kernels earlier for ranks that run the same program, so nothing waits even when the ranks have
// drifted apart by a few kernels, and no launch, event or second stream is spent on the
// exchange.  All threads of the kernel's LAST CTA take part: peer_peek issues the loads when the
// CTA starts, peer_settle takes the words when the CTA is done with its own rows, polls for the
// ones that had not arrived, and combines by shuffles.  Warp w serves value w (w + warps, ... if
// the CTA has fewer warps than there are values); lane l holds rank l's word (at most 32 ranks).
// A wait that runs out sets the error word (51) and leaves this GPU's own value as the result:
// the kernel always returns and the host sees a timeout status at its next synchronisation.
// meta[v] = op (0 sum, 1 product, 2 max, 3 min) | dtype << 8 | value index << 16.
DEV const u64* peer_word(u64 mailbox, u32 world, u32 seq, u32 m, u32 r) {
    return (const u64*)mailbox + ((u64)((seq % PEER_SLOTS) * world + r)) * 4 + (u64)(m >> 16);
}
DEV u64 peer_peek(u64 mailbox, u32 world, u32 seq, u32 n, const u32* meta) {
    const u32 v = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    u64 w = 0;
    if (v < n && lane < world)
        PEER_LD(w, peer_word(mailbox, world, seq, meta[v], lane));
    return w;
}
DEV void peer_settle(u64 peeked, u64 mailbox, u64 err, u64 wait_ns, u32 world, u32 rank, u32 seq, u32 n, const u32* meta, const u64* out) {
    const u32 first = threadIdx.x >> 5, lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    for (u32 v = first; v < n; v += warps) {
        const u32 m = meta[v], op = m & 255u, dt = (m >> 8) & 255u;
        u64 w = v == first ? peeked : 0;
        bool got = lane >= world || (u32)(w >> 32) == seq;
        if (!got) {
            const u64* slot = peer_word(mailbox, world, seq, m, lane);
            u64 start = 0;
            for (u32 spin = 0; spin < (1u << 30) && !got; ++spin) {
                PEER_LD(w, slot);
                got = (u32)(w >> 32) == seq;
                if (!got && (spin & 63u) == 63u) {
                    u64 now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (start == 0) start = now;
                    else if (now - start > wait_ns) break;
                }
            }
        }
        const bool all_here = __all_sync(0xffffffffu, got);
        const float x = __uint_as_float((u32)w);
        float acc = __shfl_sync(0xffffffffu, x, all_here ? 0 : (int)rank);
        if (all_here)
            for (u32 r = 1; r < world; ++r) {
                const float y = __shfl_sync(0xffffffffu, x, (int)r);
                acc = op == 0 ? acc + y : op == 1 ? acc * y : op == 2 ? fmaxf(acc, y) : fminf(acc, y);
            }
        if (lane == 0) {
            if (!all_here) atomicExch((u32*)err, 51u);
            if (dt == 0) *(float*)out[v] = acc;
            else if (dt == 1) *(u16*)out[v] = f2h(acc);
            else *(u16*)out[v] = f2b(acc);
        }
    }
}
// The two earlier exchanges a kernel of this path works on: the one it posts (gpost_n == 0: none)
// and the one it settles (gprev_n == 0: none).
#define PEER_SETTLE_PARAMS u64 gmailbox; u64 gwait_ns; u64 gprev_out[4]; u64 gpost_src[4]; u32 gprev_meta[4]; u32 gpost_meta[4]; u32 gprev_seq, gprev_n, gpost_seq, gpost_n;
#define PEER_POST(p) if (blockIdx.x == gridDim.x - 1 && threadIdx.x < p.gpost_n) peer_post(p.gpost_src[threadIdx.x], p.gpost_meta[threadIdx.x], p.gpeers, p.gworld, p.grank, p.gpost_seq);
// One CTA does both, and the settling around its own share of the work: the loads of the peers'
// words are issued when it starts and consumed when it is done with its rows, so their latency is
// hidden and the end of the kernel is not held up.  It is the LAST CTA of the grid: when the rows do
// not divide evenly over the CTAs it is the one with a round less to do, which gives it the time.
#define PEER_PEEK(p) u64 peeked_ = 0; if (blockIdx.x == gridDim.x - 1) peeked_ = peer_peek(p.gmailbox, p.gworld, p.gprev_seq, p.gprev_n, p.gprev_meta);
#define PEER_SETTLE(p) if (blockIdx.x == gridDim.x - 1) peer_settle(peeked_, p.gmailbox, p.gerr, p.gwait_ns, p.gworld, p.grank, p.gprev_seq, p.gprev_n, p.gprev_meta, p.gprev_out);
)CUDA";

// ---------------------------------------------------------------------------------------
// Element-wise template.  Defines expected: R NIN C U IDX64 NIMM OUT_DT OUT_MODE, macro
// LOAD_INPUTS(off, nvalid, x) and function prog(x, j, imm).
// ---------------------------------------------------------------------------------------
static const char* const JIT_EW_KERNEL = R"CUDA(
struct Params {
    u64 n;
    u64 ptr[NIN + 1];
    i64 stride[NIN * R];
    u32 shape[R];
    u32 mm[R];
    u32 ms[R];
    float imm[NIMM > 0 ? NIMM : 1];
};

DEV void offsets(const Params& p, u64 e, i64* off) {
#if R == 1
#pragma unroll
    for (int s = 0; s < NIN; ++s) off[s] = (i64)e * p.stride[s];
#else
#pragma unroll
    for (int s = 0; s < NIN; ++s) off[s] = 0;
#if IDX64
    u64 rem = e;
#pragma unroll
    for (int d = R - 1; d >= 1; --d) {
        u64 q = rem / p.shape[d];
        i64 c = (i64)(rem - q * p.shape[d]);
        rem = q;
#pragma unroll
        for (int s = 0; s < NIN; ++s) off[s] += c * p.stride[s * R + d];
    }
#else
    u32 rem = (u32)e;
#pragma unroll
    for (int d = R - 1; d >= 1; --d) {
        u32 q = fastdiv(rem, p.mm[d], p.ms[d]);
        i64 c = (i64)(rem - q * p.shape[d]);
        rem = q;
#pragma unroll
        for (int s = 0; s < NIN; ++s) off[s] += c * p.stride[s * R + d];
    }
#endif
#pragma unroll
    for (int s = 0; s < NIN; ++s) off[s] += (i64)rem * p.stride[s * R];
#endif
}

extern "C" __global__ void __launch_bounds__(256, MINB) wgf_elementwise(const __grid_constant__ Params p) {
    const u64 nchunks = (p.n + C - 1) / C;
    const u64 chunk0 = (u64)blockIdx.x * (256 * U) + threadIdx.x;
    float x[U][NIN][C];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const u64 chunk = chunk0 + (u64)u * 256;
        if (chunk < nchunks) {
            const u64 e = chunk * C;
            const u64 left = p.n - e;
            const int nvalid = left < (u64)C ? (int)left : C;
            i64 off[NIN];
            offsets(p, e, off);
            LOAD_INPUTS(off, nvalid, x[u])
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const u64 chunk = chunk0 + (u64)u * 256;
        if (chunk < nchunks) {
            const u64 e = chunk * C;
            const u64 left = p.n - e;
            const int nvalid = left < (u64)C ? (int)left : C;
            float y[C];
#pragma unroll
            for (int j = 0; j < C; ++j) y[j] = prog(x[u], j, p.imm);
            store_chunk<OUT_DT, C, OUT_MODE>((void*)p.ptr[NIN], (i64)e, nvalid, y);
        }
    }
}
)CUDA";

// ---------------------------------------------------------------------------------------
// Element-wise template for operands that are contiguous along ANOTHER axis than the output
// (transposed views).  A CTA works on a tile of TP x TL elements of the plane (PAX, last
// axis): it first brings the tile of every such operand into shared memory with the threads
// running along PAX, where that operand is contiguous (16-byte loads, four in flight per
// thread and operand), then computes with the threads running along the last axis, where the
// output and the other operands are contiguous, taking the staged operands from shared
// memory (rows padded by one word: two-way bank conflicts at most on either side).  Nothing is
// read with adjacent threads a row apart (the crate's strided kernel,
// src/visit_tiled.rs:100-144) and no transposed copy goes through HBM first.  4-byte elements,
// chunks of 4; the staged operands' extents along PAX, their other strides and their base
// addresses are multiples of 4 elements (the launcher checks).
// Defines expected: R NIN C (= 4) NIMM OUT_DT OUT_MODE PAX NSTAGED; macros TILE_STAGE (loads of
// the staged operands) and TILE_INPUTS(X) (fills X[NIN][C] for one chunk); function prog.
// ---------------------------------------------------------------------------------------
static const char* const JIT_EW_TILE_KERNEL = R"CUDA(
#define TP 64
#define TL 64
struct Params {
    u64 ptr[NIN + 1];
    i64 stride[(NIN + 1) * R];
    u32 shape[R];
    u32 tiles_p, tiles_l;
    float imm[NIMM > 0 ? NIMM : 1];
};

extern "C" __global__ void __launch_bounds__(256) wgf_elementwise_tiled(const __grid_constant__ Params p) {
    __shared__ float stage[NSTAGED][TP][TL + 1];
    const int tid = threadIdx.x;
    const int c16 = tid & 15, r16 = tid >> 4;   // 16 vectors / chunks along one tile axis, 16 rows along the other
    u32 id = blockIdx.x;
    const u32 tl = id % p.tiles_l;
    id /= p.tiles_l;
    const u32 tp = id % p.tiles_p;
    id /= p.tiles_p;
    i64 base[NIN + 1];
#pragma unroll
    for (int s = 0; s <= NIN; ++s) base[s] = 0;
#pragma unroll
    for (int d = R - 2; d >= 0; --d) {
        if (d == PAX) continue;
        const u32 c = id % p.shape[d];
        id /= p.shape[d];
#pragma unroll
        for (int s = 0; s <= NIN; ++s) base[s] += (i64)c * p.stride[s * R + d];
    }
    const u32 P = p.shape[PAX], L = p.shape[R - 1];
    const u32 p0 = tp * TP, l0 = tl * TL;
    // stage: a thread loads 4 consecutive elements along PAX for 4 indices of the last axis
    {
        const u32 pp = p0 + 4 * c16;
        TILE_STAGE
    }
    __syncthreads();
    const int tx = c16, ty = r16;               // 16 chunks along the last axis, 16 rows of PAX per pass
    const u32 l = l0 + tx * C;
#pragma unroll 1
    for (int pass = 0; pass < TP / 16; ++pass) {
        const int pi = ty + pass * 16;
        const u32 pp = p0 + pi;
        if (pp >= P || l >= L) continue;
        const int nvalid = L - l < (u32)C ? (int)(L - l) : C;
        float x[NIN][C];
        TILE_INPUTS(x)
        float y[C];
#pragma unroll
        for (int j = 0; j < C; ++j) y[j] = prog(x, j, p.imm);
        store_chunk<OUT_DT, C, OUT_MODE>((void*)p.ptr[NIN], base[NIN] + (i64)pp * p.stride[NIN * R + PAX] + (i64)l, nvalid, y);
    }
}
)CUDA";

// ---------------------------------------------------------------------------------------
// Row template: index space [outer..., H]; GROUP threads share a row, RPC rows per CTA;
// each thread keeps EPT = NCH*C elements of the row in registers across all reductions.
// CTAs are persistent: each walks rows blockIdx.x*RPC + g, + gridDim.x*RPC, ... and loads
// the next row's inputs before it reduces the current one, so HBM requests stay in flight
// during the barrier phases.  Inputs that do not depend on the row are loaded once.
// Defines expected: RO NIN C NCH GROUP RPC NRED NIMM MINB; text markers ROW_INVARIANT,
// ROW_NEXT_DECL, ROW_PREFETCH, ROW_TAKE, ROW_BODY are replaced by generated code.
// ---------------------------------------------------------------------------------------
static const char* const JIT_ROW_KERNEL = R"CUDA(
#define THREADS (GROUP * RPC)
#define EPT (NCH * C)
struct Params {
    u64 rows;
    u64 ptr[NIN + 1];
    i64 rstride[(NIN + 1) * RO];
    i64 cstride[NIN + 1];
    u32 H;
    u32 pad_;
#if NGRAND > 0
    u64 gpartials;      // float [gridDim.x][NGRAND]
    u64 gcounter;       // u32, zero on entry, zero again on exit
    u64 gout[NGRAND];   // one scalar each
    u64 gpeers;         // all-reduce inside this kernel: device array of every rank's mailbox address
    u64 gerr;           // u32 device error word
    u32 gworld, grank, gseq, gpad_;   // gseq: number of the exchange this kernel produces (for inspection; the kernel does not use it)
    PEER_SETTLE_PARAMS
#endif
    u32 oshape[RO];
    u32 mm[RO];
    u32 ms[RO];
    float imm[NIMM > 0 ? NIMM : 1];
};

DEV void row_offsets(const Params& p, u64 row, bool rv, i64* roff) {
#pragma unroll
    for (int s = 0; s <= NIN; ++s) roff[s] = 0;
    if (rv) {
        u32 rem = (u32)row;
#pragma unroll
        for (int d = RO - 1; d >= 1; --d) {
            u32 q = fastdiv(rem, p.mm[d], p.ms[d]);
            i64 c = (i64)(rem - q * p.oshape[d]);
            rem = q;
#pragma unroll
            for (int s = 0; s <= NIN; ++s) roff[s] += c * p.rstride[s * RO + d];
        }
#pragma unroll
        for (int s = 0; s <= NIN; ++s) roff[s] += (i64)rem * p.rstride[s * RO];
    }
}

extern "C" __global__ void __launch_bounds__(THREADS, MINB) wgf_rows(const __grid_constant__ Params p) {
#if GROUP > 32 && NRED > 0
    __shared__ __align__(16) float red_smem[NRED][RPC][GROUP / 32];
#endif
    const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
    ROW_GRAND_POST
    const float* imm = p.imm;
    bool cv[NCH];
#pragma unroll
    for (int k = 0; k < NCH; ++k) cv[k] = (u32)((k * GROUP + t) * C) < p.H;
    ROW_INVARIANT
    const u64 row_step = (u64)gridDim.x * RPC;
    u64 row0 = (u64)blockIdx.x * RPC;   // first row of this CTA in the current iteration
    u64 row = row0 + g;
    bool rv = row < p.rows;
    i64 roff[NIN + 1];
    row_offsets(p, row, rv, roff);
    ROW_NEXT_DECL
    ROW_PREFETCH
    while (row0 < p.rows) {
        const bool crv = rv;
        i64 coff[NIN + 1];
#pragma unroll
        for (int s = 0; s <= NIN; ++s) coff[s] = roff[s];
        bool kv[NCH];
#pragma unroll
        for (int k = 0; k < NCH; ++k) kv[k] = crv && cv[k];
        ROW_TAKE
        row0 += row_step;
        row += row_step;
        rv = row < p.rows;
        row_offsets(p, row, rv, roff);
        ROW_PREFETCH
        ROW_BODY
    }
    ROW_GRAND_SETTLE
#if NGRAND > 0
    // Companion whole-tensor reductions: CTA partial -> scratch; the last CTA to arrive
    // (ticket) combines all partials in index order and stores the scalars.
    __shared__ __align__(16) float g_smem[NGRAND][THREADS / 32];
    __shared__ u32 g_last;
    float* gpart = (float*)p.gpartials;
    ROW_GRAND_BLOCK
    if (threadIdx.x == 0) {
        ROW_GRAND_PUT
        __threadfence();
        const u32 ticket = atomicAdd((u32*)p.gcounter, 1u);
        g_last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (!g_last) return;
    __threadfence();
    ROW_GRAND_FINISH
    if (threadIdx.x == 0) *(u32*)p.gcounter = 0;
#endif
}
)CUDA";

// ---------------------------------------------------------------------------------------
// Streaming reduce template: single-phase programs with a Row result, any row length.
// A row is split over p.split CTAs; each CTA streams its share with the next tile's loads
// issued before the current tile is reduced; partials go to scratch and the last CTA to
// arrive for a row combines them in a fixed order, runs the row phase and stores.
// Defines expected: RO NIN NINE C U NRED NIMM MINB, macros STREAM_PRE, STREAM_INIT,
// STREAM_LOAD(COL, NV, X), STREAM_COMBINE_PARTIAL(PP), STREAM_BLOCK_REDUCE, STREAM_POST and
// function elem_phase(x, rowv, imm, nvalid, acc).
// ---------------------------------------------------------------------------------------
static const char* const JIT_STREAM_KERNEL = R"CUDA(
#define THREADS 256
struct Params {
    u64 rows;
    u64 ptr[NIN + 1];
    i64 rstride[(NIN + 1) * RO];
    i64 cstride[NIN + 1];
    u64 partials;   // float [rows][split][NRED]
    u64 counters;   // u32 [rows], zero on entry, zero again on exit
    u64 H;
    u32 split;
    u32 pad_;
#if STREAM_AR
    u64 gpeers;         // all-reduce of the result inside this kernel: the ranks' mailbox addresses
    u64 gerr;           // u32 device error word
    u32 gworld, grank, gseq, gpad_;   // gseq: number of the exchange this kernel produces (for inspection; the kernel does not use it)
    PEER_SETTLE_PARAMS
#endif
    u32 oshape[RO];
    u32 mm[RO];
    u32 ms[RO];
    float imm[NIMM > 0 ? NIMM : 1];
};

typedef float Tile[U][NINE > 0 ? NINE : 1][C];

DEV void load_tile(const Params& p, const i64* roff, u64 base, u64 nch, int t, Tile& x, int* nval) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const u64 chunk = base + (u64)u * THREADS + t;
        nval[u] = 0;
        if (chunk < nch) {
            const u64 col = chunk * C;
            const u64 left = p.H - col;
            nval[u] = left < (u64)C ? (int)left : C;
            STREAM_LOAD(col, nval[u], x[u])
        }
    }
}

extern "C" __global__ void __launch_bounds__(THREADS, MINB) wgf_stream_reduce(const __grid_constant__ Params p) {
    __shared__ __align__(16) float red_smem[NRED][THREADS / 32];
    __shared__ u32 is_last;
    const int t = threadIdx.x;
#if STREAM_AR
    PEER_POST(p)
    PEER_PEEK(p)
#endif
    const u32 sp = blockIdx.x % p.split;
    const u64 row = blockIdx.x / p.split;
    i64 roff[NIN + 1];
#pragma unroll
    for (int s = 0; s <= NIN; ++s) roff[s] = 0;
    {
        u32 rem = (u32)row;
#pragma unroll
        for (int d = RO - 1; d >= 1; --d) {
            u32 q = fastdiv(rem, p.mm[d], p.ms[d]);
            i64 c = (i64)(rem - q * p.oshape[d]);
            rem = q;
#pragma unroll
            for (int s = 0; s <= NIN; ++s) roff[s] += c * p.rstride[s * RO + d];
        }
#pragma unroll
        for (int s = 0; s <= NIN; ++s) roff[s] += (i64)rem * p.rstride[s * RO];
    }
    const float* imm = p.imm;
    STREAM_PRE
    float acc[NRED];
    STREAM_INIT
    const u64 nch = (p.H + C - 1) / C;
    const u64 step = (u64)p.split * (THREADS * U);
    u64 base = (u64)sp * (THREADS * U);
    Tile xa, xb;
    int na[U], nb[U];
    if (base < nch) load_tile(p, roff, base, nch, t, xa, na);
    while (base < nch) {
        // ping: fetch the next tile into b, reduce a
        if (base + step < nch) load_tile(p, roff, base + step, nch, t, xb, nb);
#pragma unroll
        for (int u = 0; u < U; ++u) elem_phase(xa[u], rowv, imm, na[u], acc);
        base += step;
        if (base >= nch) break;
        // pong: fetch into a, reduce b
        if (base + step < nch) load_tile(p, roff, base + step, nch, t, xa, na);
#pragma unroll
        for (int u = 0; u < U; ++u) elem_phase(xb[u], rowv, imm, nb[u], acc);
        base += step;
    }
#if STREAM_AR
    PEER_SETTLE(p)
#endif
    STREAM_BLOCK_REDUCE
    if (p.split > 1) {
        float* part = (float*)p.partials + (row * p.split) * NRED;
        if (t == 0) {
#pragma unroll
            for (int r = 0; r < NRED; ++r) part[(u64)sp * NRED + r] = acc[r];
            __threadfence();
            u32 ticket = atomicAdd((u32*)p.counters + row, 1u);
            is_last = ticket == p.split - 1;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        STREAM_INIT
        for (u32 s2 = t; s2 < p.split; s2 += THREADS) {
            STREAM_COMBINE_PARTIAL(part + (u64)s2 * NRED)
        }
        __syncthreads();
        STREAM_BLOCK_REDUCE
        if (t == 0) ((u32*)p.counters)[row] = 0;
    }
    STREAM_POST
}
)CUDA";

// ---------------------------------------------------------------------------------------
// Column-reduce template: the reduced axis K is NOT the innermost one.  Index space
// [O, K, I] with I contiguous in memory.  Threads run along I (C columns each, 16-byte
// loads), the 8 thread rows of a CTA and p.split CTAs share K; per-column accumulators stay
// in registers; partials of split CTAs go to scratch, the last CTA per column tile (ticket)
// combines them in index order.  A reduction over axis 0 of a row-major matrix therefore
// reads whole rows, where the crate walks one column per workgroup (src/reduce.rs:349-373).
// TX threads run along I per CTA (a CTA reads TX * 16 contiguous bytes of every row it
// visits) and TY = 256 / TX thread rows share K.
// Defines expected: NIN NINE NROWL NPRE C U TX TY NRED NIMM; macro COL_LOAD_ELEM(K, X),
// COL_LOAD_ROW(X); functions pre_phase, elem_phase, post_phase; per-reduction macros
// COL_INIT(j) COL_COMB(j, PP, STRIDE) COL_SMEM_ADD(j, w).
// ---------------------------------------------------------------------------------------
static const char* const JIT_COL_KERNEL = R"CUDA(
struct Params {
    u64 O, K, I;
    u64 ptr[NIN + 1];
    i64 so[NIN + 1];
    i64 sk[NIN + 1];
    u64 partials;   // float [NRED][O][split][I]
    u64 counters;   // u32 [O * tiles], zero on entry, zero again on exit
    u32 split;
    u32 kper;       // K rows per split
    float imm[NIMM > 0 ? NIMM : 1];
};

extern "C" __global__ void __launch_bounds__(256, 2) wgf_col_reduce(const __grid_constant__ Params p) {
    __shared__ float red[NRED][TY][TX * C + 1];
    __shared__ u32 is_last;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const u64 o = blockIdx.z;
    const u32 sp = blockIdx.y;
    const u64 col = ((u64)blockIdx.x * TX + tx) * C;
    const bool cv = col < p.I;
    const float* imm = p.imm;
    // values that do not depend on k: per-column operands and arithmetic on them
    float rowl[NROWL > 0 ? NROWL : 1][C];
    float rowv[NPRE > 0 ? NPRE : 1][C];
    if (cv) {
        COL_LOAD_ROW(rowl)
#pragma unroll
        for (int j = 0; j < C; ++j) {
            float rl[NROWL > 0 ? NROWL : 1], rv[NPRE > 0 ? NPRE : 1];
#pragma unroll
            for (int s = 0; s < NROWL; ++s) rl[s] = rowl[s][j];
            pre_phase(rl, imm, rv);
#pragma unroll
            for (int s = 0; s < NPRE; ++s) rowv[s][j] = rv[s];
        }
    }
    float acc[NRED][C];
#pragma unroll
    for (int j = 0; j < C; ++j) { COL_INIT(j) }
    const u64 kbeg = (u64)sp * p.kper;
    const u64 kend = kbeg + p.kper < p.K ? kbeg + p.kper : p.K;
    if (cv) {
        for (u64 k0 = kbeg + ty; k0 < kend; k0 += TY * U) {
            float x[U][NINE > 0 ? NINE : 1][C];
            bool kv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const u64 k = k0 + (u64)u * TY;
                kv[u] = k < kend;
                if (kv[u]) { COL_LOAD_ELEM(k, x[u]) }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!kv[u]) continue;
#pragma unroll
                for (int j = 0; j < C; ++j) {
                    float xe[NINE > 0 ? NINE : 1], rv[NPRE > 0 ? NPRE : 1], a[NRED];
#pragma unroll
                    for (int s = 0; s < NINE; ++s) xe[s] = x[u][s][j];
#pragma unroll
                    for (int s = 0; s < NPRE; ++s) rv[s] = rowv[s][j];
#pragma unroll
                    for (int r = 0; r < NRED; ++r) a[r] = acc[r][j];
                    elem_phase(xe, rv, imm, a);
#pragma unroll
                    for (int r = 0; r < NRED; ++r) acc[r][j] = a[r];
                }
            }
        }
    }
    // combine the 8 thread rows
#pragma unroll
    for (int r = 0; r < NRED; ++r)
#pragma unroll
        for (int j = 0; j < C; ++j) red[r][ty][tx * C + j] = acc[r][j];
    __syncthreads();
    if (ty == 0) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
            COL_INIT(j)
#pragma unroll
            for (int w = 0; w < TY; ++w) { COL_SMEM_ADD(j, w) }
        }
    }
    const u64 tiles = gridDim.x;
    if (p.split > 1) {
        float* part = (float*)p.partials;
        const u64 plane = p.O * p.split * p.I;               // one reduction's partials
        const u64 base = (o * p.split + sp) * p.I + col;
        if (ty == 0 && cv) {
#pragma unroll
            for (int r = 0; r < NRED; ++r)
#pragma unroll
                for (int j = 0; j < C; ++j) part[(u64)r * plane + base + j] = acc[r][j];
        }
        __threadfence();
        __syncthreads();
        if (tx == 0 && ty == 0) {
            u32 ticket = atomicAdd((u32*)p.counters + o * tiles + blockIdx.x, 1u);
            is_last = ticket == p.split - 1;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        if (ty == 0 && cv) {
#pragma unroll
            for (int j = 0; j < C; ++j) { COL_INIT(j) }
            for (u32 s2 = 0; s2 < p.split; ++s2) {
                const float* pp = part + (o * p.split + s2) * p.I + col;
#pragma unroll
                for (int j = 0; j < C; ++j) { COL_COMB(j, pp, plane) }
            }
        }
        if (tx == 0 && ty == 0) ((u32*)p.counters)[o * tiles + blockIdx.x] = 0;
    }
    if (ty == 0 && cv) {
        float y[C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
            float rv[NPRE > 0 ? NPRE : 1], a[NRED];
#pragma unroll
            for (int s = 0; s < NPRE; ++s) rv[s] = rowv[s][j];
#pragma unroll
            for (int r = 0; r < NRED; ++r) a[r] = acc[r][j];
            y[j] = post_phase(a, rv, imm);
        }
        store_chunk<OUT_DT, C, OUT_MODE>((void*)p.ptr[NIN], (i64)(o * p.I + col), C, y);
    }
}
)CUDA";

}  // namespace wgf
