// Fused softmax attention for 16-bit tensors with head dimension 128 on the tcgen05 tensor
// cores (sm_100a):  O = softmax(scale * Q K^T  [causal])  V  per (batch * head).  The [S, S]
// score matrix lives only in tensor memory; nothing but Q, K, V and O touches HBM.  The crate
// has no attention op (its README lists the ops a Llama block needs, README.md:24-38); built
// from its primitives the same result takes a batched matmul, a softmax kernel and a second
// batched matmul with two round trips of the score matrix through memory.
//
// Two kernels.  The default, attention_tc2_kernel (further down), gives a CTA two adjacent query
// tiles at a time and makes one pass over the keys (online softmax); attention_tc_kernel, the
// first version, gives it one query tile and makes two passes.  Both are described where they
// are defined; WGF_ATT_SINGLE=1 selects the first, WGF_ATT_TWO_PASS=1 the two-pass form of the
// default.  What follows describes attention_tc_kernel.
//
// One persistent CTA per SM walks (batch*head, 128-row query tile) work items in the order of
// decode_item (heaviest first when causal, K / V sharing through L2 otherwise).
// Key/value tiles are 128 rows.  Two passes over the keys of an item:
//   pass 1   S = Q K_j^T (tensor cores)            -> row maxima m           (softmax warps)
//   pass 2   S = Q K_j^T again, P = exp2((S - m) * scale * log2 e) as 16-bit -> shared memory,
//            O += P V_j (tensor cores, accumulating in TMEM), l = row sums of P
//   end      O / l -> global memory
// Recomputing S costs a third more tensor work than the single-pass online softmax, but O is
// never rescaled, so nothing has to be read back from and written again to tensor memory per
// tile.  What bounds the kernel is the latency of the per-tile chain S -> softmax -> P -> P V
// (measured: cheaper softmax code, twice the softmax warps and a single-pass variant with a
// third less tensor work all failed to make it faster; the softmax warps and the MMA warp each
// wait for the other about half of the time).
// Warp roles:
//   warp 0     TMA producer (one lane): Q tile, then K / V tiles through a 4-stage ring
//   warp 1     MMA issuer   (one lane): S into one of two TMEM buffers (2 x 128 columns), O in a
//              third (128 columns)
//   warps 2-5  softmax: thread r owns row r of the tile = TMEM lane r
// Synchronisation is by mbarriers only; every wait is bounded and reports through the device
// error word instead of hanging.
#include <algorithm>
#include <cmath>
#include <mutex>
#include <type_traits>

#include "attention.hpp"
#include "tc_common.cuh"

namespace wgf {

using namespace tc;

namespace {

constexpr int AT_STAGES = 4;
constexpr int AT_PANEL = 128 * 128;        // bytes of one 64-column panel: 128 rows x 128 bytes
constexpr int AT_TILE = 2 * AT_PANEL;      // a [128 x 128] 16-bit tile: 32 KiB
constexpr int AT_SMEM = (2 + AT_STAGES) * AT_TILE + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int AT_THREADS = 192;
constexpr unsigned AT_S_COLS = 128, AT_O_COL0 = 256;
constexpr float AT_LAG = 8.f;              // how far (in powers of two) a row maximum may outgrow its reference

struct AtParams {
    int n_q_tiles, n_k_tiles;
    int bh;                  // batch * heads
    int causal;
    int is_bf16;
    float scale_log2e;
    int heads;               // batch*heads index n = batch * heads + head
    // V read in place from a [batch, seq, heads * 128] projection (v_heads > 0): its tensor map is
    // {128, batch * seq, heads}, so item b = batch * v_heads + head finds its rows at
    // (b / v_heads) * v_rows + row and its head at b % v_heads.  v_heads == 0: V is [n, seq, 128].
    int v_heads, v_rows;
    long long o_rs, o_hs, o_bs;   // output row / head / batch stride in elements
    unsigned* error;         // device word: 0 = ok, else code of the wait that gave up
    unsigned long long* prof;   // null, or 26 cycle totals written by CTA 0 of attention_ts_kernel (WGF_ATT_PROFILE=1)
};

// kind::f16 instruction descriptor for M = 128, N = 128 (fields as in matmul_tc.cu)
__device__ __forceinline__ unsigned at_idesc(unsigned bf16, unsigned b_mn_major) {
    return (1u << 4) | (bf16 << 7) | (bf16 << 10) | (b_mn_major << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Work item w -> (batch*head b, query tile qt).  Causal: the heaviest query tiles (most key
// tiles) of all batch*heads first, which balances the CTAs best (measured on [256,2048,128]:
// 648 us; with the order below 748-797 us).  Not causal (all items cost the same): the query
// tiles of one batch*head are consecutive items, so the CTAs that run at the same time read the
// same K / V tiles, which then come from L2 instead of HBM (1228 -> 1095 us).
__device__ __forceinline__ void decode_item(const AtParams& p, long long w, int& b, int& qt) {
    if (p.causal) {
        qt = p.n_q_tiles - 1 - (int)(w / p.bh);
        b = (int)(w % p.bh);
    } else {
        b = (int)(w / p.n_q_tiles);
        qt = (int)(w % p.n_q_tiles);
    }
}

enum {
    Q_FULL = 0, Q_EMPTY, KV_FULL, KV_EMPTY = KV_FULL + AT_STAGES, S_FULL = KV_EMPTY + AT_STAGES, S_EMPTY = S_FULL + 2,
    P_FULL = S_EMPTY + 2, P_EMPTY, O_FULL, O_EMPTY, N_BARS
};

template <typename T>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, T* __restrict__ O, const __grid_constant__ AtParams p) {
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle atoms
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* p_tile = smem + AT_TILE;
    const unsigned q_smem = smem_u32(smem), p_smem = q_smem + AT_TILE, ring = p_smem + AT_TILE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (2 + AT_STAGES) * AT_TILE);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + N_BARS);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (unsigned)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; ++i) {
            const bool four = (i >= S_EMPTY && i < S_EMPTY + 2) || i == P_FULL || i == O_EMPTY;   // one arrival per softmax warp
            mbar_init(bar(i), four ? 4 : 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    const long long items = (long long)p.bh * p.n_q_tiles;
    auto v_row = [&](int row0, int b) { return p.v_heads > 0 ? (b / p.v_heads) * p.v_rows + row0 : row0; };
    auto v_slab = [&](int b) { return p.v_heads > 0 ? b % p.v_heads : b; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 1, q_phase = 1;   // fresh "empty" barriers count as already released
            bool ok = true;
            auto push = [&](const CUtensorMap* map, int row0, int b) -> bool {
                if (!mbar_wait(bar(KV_EMPTY + stage), phase)) {
                    atomicExch(p.error, 11u);
                    return false;
                }
                const unsigned dst = ring + (unsigned)stage * AT_TILE;
                mbar_expect_tx(bar(KV_FULL + stage), AT_TILE);
                tma_load_3d(dst, map, bar(KV_FULL + stage), 0, row0, b);
                tma_load_3d(dst + AT_PANEL, map, bar(KV_FULL + stage), 64, row0, b);
                if (++stage == AT_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
                return true;
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, qt;
                decode_item(p, w, b, qt);
                const int n_kv = p.causal ? qt + 1 : p.n_k_tiles;
                if (!mbar_wait(bar(Q_EMPTY), q_phase)) {
                    atomicExch(p.error, 10u);
                    break;
                }
                q_phase ^= 1;
                mbar_expect_tx(bar(Q_FULL), AT_TILE);
                tma_load_3d(q_smem, &map_q, bar(Q_FULL), 0, qt * 128, b);
                tma_load_3d(q_smem + AT_PANEL, &map_q, bar(Q_FULL), 64, qt * 128, b);
                // the order below is the order in which the MMA warp consumes the ring
                for (int j = 0; j < n_kv && ok; ++j) ok = push(&map_k, j * 128, b);
                for (int j = 0; j < n_kv && ok; ++j) {
                    ok = push(&map_k, j * 128, b);
                    if (ok && j > 0) ok = push(&map_v, v_row((j - 1) * 128, b), v_slab(b));
                }
                if (ok) ok = push(&map_v, v_row((n_kv - 1) * 128, b), v_slab(b));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const unsigned idesc_s = at_idesc((unsigned)p.is_bf16, 0u), idesc_pv = at_idesc((unsigned)p.is_bf16, 1u);
            int stage = 0, sb = 0;
            unsigned phase = 0, q_phase = 0, p_phase = 0, o_phase = 1;
            unsigned s_phase[2] = {1, 1};      // both S buffers start out free
            bool ok = true;
            auto advance = [&]() {
                if (++stage == AT_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            };
            // S[sb] = Q K^T for the K tile at the head of the ring
            auto issue_s = [&]() -> bool {
                if (!mbar_wait(bar(KV_FULL + stage), phase)) {
                    atomicExch(p.error, 21u);
                    return false;
                }
                if (!mbar_wait(bar(S_EMPTY + sb), s_phase[sb])) {
                    atomicExch(p.error, 22u);
                    return false;
                }
                s_phase[sb] ^= 1;
                tc_fence_after();
                const unsigned kt = ring + (unsigned)stage * AT_TILE;
                const unsigned d = tmem_base + (unsigned)sb * AT_S_COLS;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // both K-major: rows of 128 bytes, 8-row groups 1024 bytes apart, 32 bytes per
                    // K step inside a 64-column panel, the second panel 16 KiB further
                    const unsigned off = (unsigned)(kk >> 2) * AT_PANEL + (unsigned)(kk & 3) * 32u;
                    umma_f16(d, smem_desc(q_smem + off, 16, 1024), smem_desc(kt + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
                }
                umma_commit(bar(KV_EMPTY + stage));
                umma_commit(bar(S_FULL + sb));
                advance();
                sb ^= 1;
                return true;
            };
            // O (+)= P V for the V tile at the head of the ring
            auto issue_pv = [&](bool first) -> bool {
                if (first) {
                    if (!mbar_wait(bar(O_EMPTY), o_phase)) {
                        atomicExch(p.error, 23u);
                        return false;
                    }
                    o_phase ^= 1;
                }
                if (!mbar_wait(bar(P_FULL), p_phase)) {
                    atomicExch(p.error, 24u);
                    return false;
                }
                p_phase ^= 1;
                if (!mbar_wait(bar(KV_FULL + stage), phase)) {
                    atomicExch(p.error, 25u);
                    return false;
                }
                tc_fence_after();
                const unsigned vt = ring + (unsigned)stage * AT_TILE;
                const unsigned d = tmem_base + AT_O_COL0;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // A = P, K-major (keys along K).  B = V, N-major: 64-column panels 16 KiB apart
                    // (leading), 8-key groups 1024 bytes apart (stride), 16 keys = 2048 bytes per K step
                    const unsigned long long adesc =
                        smem_desc(p_smem + (unsigned)(kk >> 2) * AT_PANEL + (unsigned)(kk & 3) * 32u, 16, 1024);
                    const unsigned long long bdesc = smem_desc(vt + (unsigned)kk * 2048u, AT_PANEL, 1024);
                    umma_f16(d, adesc, bdesc, idesc_pv, (first && kk == 0) ? 0u : 1u);
                }
                umma_commit(bar(KV_EMPTY + stage));
                umma_commit(bar(P_EMPTY));
                advance();
                return true;
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, qt;
                decode_item(p, w, b, qt);
                const int n_kv = p.causal ? qt + 1 : p.n_k_tiles;
                if (!mbar_wait(bar(Q_FULL), q_phase)) {
                    atomicExch(p.error, 20u);
                    break;
                }
                q_phase ^= 1;
                tc_fence_after();
                for (int j = 0; j < n_kv && ok; ++j) ok = issue_s();          // pass 1
                for (int j = 0; j < n_kv && ok; ++j) {                         // pass 2
                    ok = issue_s();
                    if (ok && j == n_kv - 1) umma_commit(bar(Q_EMPTY));        // Q is free once these MMAs are done
                    if (ok && j > 0) ok = issue_pv(j == 1);
                }
                if (ok) ok = issue_pv(n_kv == 1);
                if (ok) umma_commit(bar(O_FULL));
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax (warps 2..5)
        const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
        const int r = quarter * 32 + lane;                  // row of the query tile
        const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
        unsigned s_phase[2] = {0, 0};
        unsigned pe_phase = 1, o_phase = 0;
        int sb = 0;
        bool ok = true;
        auto wait_all = [&](int which, unsigned parity, unsigned code) -> bool {
            bool got = mbar_wait(bar(which), parity);
            got = __all_sync(0xffffffffu, got);
            if (!got && lane == 0) atomicExch(p.error, code);
            return got;
        };
        for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
            int b, qt;
            decode_item(p, w, b, qt);
            const int n_kv = p.causal ? qt + 1 : p.n_k_tiles;
            // ---- pass 1: row maximum of the raw scores
            // (four independent chains: one warp per scheduler has nothing else to hide the latency
            // of a 128-long dependent chain)
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!(ok = wait_all(S_FULL + sb, s_phase[sb], 31u))) break;
                s_phase[sb] ^= 1;
                tc_fence_after();
                const bool diag = p.causal && j == qt;
#pragma unroll 1
                for (int c = 0; c < 4; c += 2) {
                    unsigned v[64];
                    tmem_ld_32x32(lane_base + (unsigned)sb * AT_S_COLS + (unsigned)c * 32u, v);
                    tmem_ld_32x32(lane_base + (unsigned)sb * AT_S_COLS + (unsigned)(c + 1) * 32u, v + 32);
                    tmem_ld_wait();
                    if (diag) {   // only the key tile on the diagonal carries the mask tests
#pragma unroll
                        for (int i = 0; i < 64; ++i)
                            if (c * 32 + i > r) v[i] = 0xff800000u;   // -inf above the diagonal
                    }
#pragma unroll
                    for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(S_EMPTY + sb));
                sb ^= 1;
            }
            if (!ok) break;
            // ---- pass 2: P = exp2((S - m) * scale * log2 e) -> shared memory, row sums
            const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            const float mc = m * p.scale_log2e;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!(ok = wait_all(S_FULL + sb, s_phase[sb], 32u))) break;
                s_phase[sb] ^= 1;
                if (!(ok = wait_all(P_EMPTY, pe_phase, 33u))) break;     // the previous P V has read the P tile
                pe_phase ^= 1;
                tc_fence_after();
                const bool diag = p.causal && j == qt;
                // 32 score columns at a time; the TMEM load of the next 32 is in flight while the
                // exponentials of the current ones are computed
                auto process = [&](unsigned* v, int c) {
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i > r) v[i] = 0xff800000u;   // -inf above the diagonal: P = 0
                    }
                    float e[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        e[i] = ex2_approx(fmaf(__uint_as_float(v[i]), p.scale_log2e, -mc));
                        l4[i & 3] += e[i];
                    }
                    // A-operand layout (K-major, 128-byte swizzle): row r of panel c/2 is 128 bytes
                    // at r * 128; its 16-byte chunk q sits at position q ^ (r % 8)
                    unsigned char* row = p_tile + (c >> 1) * AT_PANEL + r * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        o.x = pack2<T>(e[8 * q + 0], e[8 * q + 1]);
                        o.y = pack2<T>(e[8 * q + 2], e[8 * q + 3]);
                        o.z = pack2<T>(e[8 * q + 4], e[8 * q + 5]);
                        o.w = pack2<T>(e[8 * q + 6], e[8 * q + 7]);
                        const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
                        *reinterpret_cast<uint4*>(row + chunk * 16) = o;
                    }
                };
                const unsigned s_addr = lane_base + (unsigned)sb * AT_S_COLS;
                unsigned va[32], vb[32];
                tmem_ld_32x32(s_addr, va);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 32u, vb);
                process(va, 0);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 64u, va);
                process(vb, 1);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 96u, vb);
                process(va, 2);
                tmem_ld_wait();
                process(vb, 3);
                tc_fence_before();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor cores
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(P_FULL));
                    mbar_arrive(bar(S_EMPTY + sb));
                }
                sb ^= 1;
            }
            if (!ok) break;
            // ---- O / l -> global memory
            if (!(ok = wait_all(O_FULL, o_phase, 34u))) break;
            o_phase ^= 1;
            tc_fence_after();
            const float inv = 1.0f / ((l4[0] + l4[1]) + (l4[2] + l4[3]));
            T* orow = O + (long long)(b / p.heads) * p.o_bs + (long long)(b % p.heads) * p.o_hs + ((long long)qt * 128 + r) * p.o_rs;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                unsigned v[32];
                tmem_ld_32x32(lane_base + AT_O_COL0 + (unsigned)c * 32u, v);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = pack2<T>(__uint_as_float(v[8 * q + 0]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
                    o.y = pack2<T>(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
                    o.z = pack2<T>(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
                    o.w = pack2<T>(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O_EMPTY));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}


// ---------------------------------------------------------------------------------------
// Two query tiles per CTA.  The kernel above is bound by the latency of its per-tile chain
// S -> softmax -> P -> P V.  Here a CTA works on two adjacent query tiles of one batch*head at
// the same time: each tile has its own Q, S, P and O and its own four softmax warps, the two
// share the K / V ring (every K / V tile is loaded once for both), and the MMA warp alternates
// between them, so one tile's tensor work fills the time the other spends in its softmax.
// Tensor memory: S of tile t in columns 128 t, O in 256 + 128 t.  Shared memory: 2 Q + 2 P tiles
// and a 3-stage ring (224 KiB).  Causal: the first tile of the pair needs one key tile less.
// Measured, f16 causal [256, 2048, 128]: one query tile per CTA, two passes 640 us; two tiles, two
// passes 594 us; two tiles, one pass 535 us (the one pass alone, with one tile per CTA, was slower
// than two passes: 773 us - it lengthens the chain that the second tile is there to hide).
// ---------------------------------------------------------------------------------------
constexpr int A2_STAGES = 3;
constexpr int A2_THREADS = 320;            // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr int A2_SMEM = (4 + A2_STAGES) * AT_TILE + 1024 /*alignment slack*/ + 512 /*barriers*/;
enum {
    Q2_FULL = 0, Q2_EMPTY = 2, KV2_FULL = 4, KV2_EMPTY = KV2_FULL + A2_STAGES, S2_FULL = KV2_EMPTY + A2_STAGES, S2_EMPTY = S2_FULL + 2,
    P2_FULL = S2_EMPTY + 2, P2_EMPTY = P2_FULL + 2, O2_FULL = P2_EMPTY + 2, O2_EMPTY = O2_FULL + 2, N2_BARS = O2_EMPTY + 2
};

// Work item w -> (batch*head b, pair of query tiles pt): same orders as decode_item.
__device__ __forceinline__ void decode_pair(const AtParams& p, int n_pairs, long long w, int& b, int& pt) {
    if (p.causal) {
        pt = n_pairs - 1 - (int)(w / p.bh);
        b = (int)(w % p.bh);
    } else {
        b = (int)(w / n_pairs);
        pt = (int)(w % n_pairs);
    }
}

// ONLINE: one pass over the keys with a lazily updated reference maximum (see below) instead of two.
template <typename T, bool ONLINE>
__global__ void __launch_bounds__(A2_THREADS, 1)
attention_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, T* __restrict__ O, const __grid_constant__ AtParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [Q0][Q1][P0][P1][ring ...]
    const unsigned q_smem0 = smem_u32(smem), p_smem0 = q_smem0 + 2 * AT_TILE, ring = p_smem0 + 2 * AT_TILE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (4 + A2_STAGES) * AT_TILE);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + N2_BARS);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (unsigned)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < N2_BARS; ++i) {
            // one arrival per softmax warp of the tile
            const bool four = (i >= S2_EMPTY && i < S2_EMPTY + 2) || (i >= P2_FULL && i < P2_FULL + 2) || (i >= O2_EMPTY && i < O2_EMPTY + 2);
            mbar_init(bar(i), four ? 4 : 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    const int n_pairs = (p.n_q_tiles + 1) / 2;
    const long long items = (long long)p.bh * n_pairs;
    auto v_row = [&](int row0, int b) { return p.v_heads > 0 ? (b / p.v_heads) * p.v_rows + row0 : row0; };
    auto v_slab = [&](int b) { return p.v_heads > 0 ? b % p.v_heads : b; };
    // key tiles of tile t of pair pt (0: the pair has no second tile)
    auto tiles_of = [&](int pt, int t) -> int {
        const int qt = 2 * pt + t;
        if (qt >= p.n_q_tiles) return 0;
        return p.causal ? qt + 1 : p.n_k_tiles;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 1, q_phase[2] = {1, 1};   // fresh "empty" barriers count as already released
            bool ok = true;
            auto push = [&](const CUtensorMap* map, int row0, int b) -> bool {
                if (!mbar_wait(bar(KV2_EMPTY + stage), phase)) {
                    atomicExch(p.error, 61u);
                    return false;
                }
                const unsigned dst = ring + (unsigned)stage * AT_TILE;
                mbar_expect_tx(bar(KV2_FULL + stage), AT_TILE);
                tma_load_3d(dst, map, bar(KV2_FULL + stage), 0, row0, b);
                tma_load_3d(dst + AT_PANEL, map, bar(KV2_FULL + stage), 64, row0, b);
                if (++stage == A2_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
                return true;
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, pt;
                decode_pair(p, n_pairs, w, b, pt);
                const int n_max = max(tiles_of(pt, 0), tiles_of(pt, 1));
                for (int t = 0; t < 2 && ok; ++t) {
                    if (tiles_of(pt, t) == 0) continue;
                    if (!mbar_wait(bar(Q2_EMPTY + t), q_phase[t])) {
                        atomicExch(p.error, 60u);
                        ok = false;
                        break;
                    }
                    q_phase[t] ^= 1;
                    const unsigned qs = q_smem0 + (unsigned)t * AT_TILE;
                    mbar_expect_tx(bar(Q2_FULL + t), AT_TILE);
                    tma_load_3d(qs, &map_q, bar(Q2_FULL + t), 0, (2 * pt + t) * 128, b);
                    tma_load_3d(qs + AT_PANEL, &map_q, bar(Q2_FULL + t), 64, (2 * pt + t) * 128, b);
                }
                // the order below is the order in which the MMA warp consumes the ring
                if (!ONLINE)
                    for (int j = 0; j < n_max && ok; ++j) ok = push(&map_k, j * 128, b);
                for (int j = 0; j < n_max && ok; ++j) {
                    ok = push(&map_k, j * 128, b);
                    if (ok && j > 0) ok = push(&map_v, v_row((j - 1) * 128, b), v_slab(b));
                }
                if (ok) ok = push(&map_v, v_row((n_max - 1) * 128, b), v_slab(b));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const unsigned idesc_s = at_idesc((unsigned)p.is_bf16, 0u), idesc_pv = at_idesc((unsigned)p.is_bf16, 1u);
            int stage = 0;
            unsigned phase = 0;
            unsigned q_phase[2] = {0, 0}, p_phase[2] = {0, 0}, o_phase[2] = {1, 1}, s_phase[2] = {1, 1};
            bool ok = true;
            int nk[2];
            auto advance = [&]() {
                if (++stage == A2_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            };
            auto wait_or = [&](int which, unsigned ph, unsigned code) -> bool {
                if (mbar_wait(bar(which), ph)) return true;
                atomicExch(p.error, code);
                return false;
            };
            // S_t = Q_t K^T for both tiles that still need key tile j; K is at the head of the ring
            auto issue_s = [&](int j, bool last_pass) -> bool {
                if (!wait_or(KV2_FULL + stage, phase, 71u)) return false;
                const unsigned kt = ring + (unsigned)stage * AT_TILE;
                for (int t = 0; t < 2; ++t) {
                    if (j >= nk[t]) continue;
                    if (!wait_or(S2_EMPTY + t, s_phase[t], 72u)) return false;
                    s_phase[t] ^= 1;
                    tc_fence_after();
                    const unsigned qs = q_smem0 + (unsigned)t * AT_TILE;
                    const unsigned d = tmem_base + (unsigned)t * AT_S_COLS;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const unsigned off = (unsigned)(kk >> 2) * AT_PANEL + (unsigned)(kk & 3) * 32u;
                        umma_f16(d, smem_desc(qs + off, 16, 1024), smem_desc(kt + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
                    }
                    umma_commit(bar(S2_FULL + t));
                    if (last_pass && j == nk[t] - 1) umma_commit(bar(Q2_EMPTY + t));   // Q_t is free once these are done
                }
                umma_commit(bar(KV2_EMPTY + stage));
                advance();
                return true;
            };
            // O_t (+)= P_t V for both tiles that have key tile j; V is at the head of the ring
            auto issue_pv = [&](int j) -> bool {
                if (!wait_or(KV2_FULL + stage, phase, 75u)) return false;
                const unsigned vt = ring + (unsigned)stage * AT_TILE;
                for (int t = 0; t < 2; ++t) {
                    if (j >= nk[t]) continue;
                    if (j == 0) {
                        if (!wait_or(O2_EMPTY + t, o_phase[t], 73u)) return false;
                        o_phase[t] ^= 1;
                    }
                    if (!wait_or(P2_FULL + t, p_phase[t], 74u)) return false;
                    p_phase[t] ^= 1;
                    tc_fence_after();
                    const unsigned ps = p_smem0 + (unsigned)t * AT_TILE;
                    const unsigned d = tmem_base + AT_O_COL0 + (unsigned)t * 128u;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const unsigned long long adesc = smem_desc(ps + (unsigned)(kk >> 2) * AT_PANEL + (unsigned)(kk & 3) * 32u, 16, 1024);
                        const unsigned long long bdesc = smem_desc(vt + (unsigned)kk * 2048u, AT_PANEL, 1024);
                        umma_f16(d, adesc, bdesc, idesc_pv, (j == 0 && kk == 0) ? 0u : 1u);
                    }
                    umma_commit(bar(P2_EMPTY + t));
                    if (j == nk[t] - 1) umma_commit(bar(O2_FULL + t));
                }
                umma_commit(bar(KV2_EMPTY + stage));
                advance();
                return true;
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, pt;
                decode_pair(p, n_pairs, w, b, pt);
                nk[0] = tiles_of(pt, 0);
                nk[1] = tiles_of(pt, 1);
                const int n_max = max(nk[0], nk[1]);
                for (int t = 0; t < 2 && ok; ++t) {
                    if (nk[t] == 0) continue;
                    ok = wait_or(Q2_FULL + t, q_phase[t], 70u);
                    q_phase[t] ^= 1;
                }
                if (!ok) break;
                tc_fence_after();
                if (!ONLINE)
                    for (int j = 0; j < n_max && ok; ++j) ok = issue_s(j, false);   // pass 1
                for (int j = 0; j < n_max && ok; ++j) {                          // pass 2, or the only pass
                    ok = issue_s(j, true);
                    if (ok && j > 0) ok = issue_pv(j - 1);
                }
                if (ok) ok = issue_pv(n_max - 1);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax (warps 2-5: tile 0, warps 6-9: tile 1)
        const int t = (warp - 2) >> 2;
        const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
        const int r = quarter * 32 + lane;                  // row of the query tile
        const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
        const unsigned s_addr = lane_base + (unsigned)t * AT_S_COLS, o_addr = lane_base + AT_O_COL0 + (unsigned)t * 128u;
        unsigned char* p_tile = smem + (2 + t) * AT_TILE;
        unsigned s_phase = 0, pe_phase = 1, o_phase = 0;
        bool ok = true;
        auto wait_all = [&](int which, unsigned parity, unsigned code) -> bool {
            bool got = mbar_wait(bar(which), parity);
            got = __all_sync(0xffffffffu, got);
            if (!got && lane == 0) atomicExch(p.error, code);
            return got;
        };
        for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
            int b, pt;
            decode_pair(p, n_pairs, w, b, pt);
            const int n_kv = tiles_of(pt, t);
            if (n_kv == 0) continue;                         // an odd tile count: the last pair has one tile
            const int qt = 2 * pt + t;
            float l_run = 0.f;
            if constexpr (ONLINE) {
            // Online softmax.  Every row keeps a reference maximum `ref` (scores times scale*log2 e);
            // P = exp2(s*c - ref).  `ref` follows the running maximum only when that has grown by
            // more than AT_LAG since `ref` was set; then O and l of the row are multiplied by
            // exp2(ref_old - ref_new).  In between P simply exceeds 1 (by at most 2^AT_LAG, which
            // 16-bit P and the fp32 accumulators hold easily), so after the first key tile a rescale
            // of O, a round trip of its row through tensor memory, is rare.
            float ref = 0.f;
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!(ok = wait_all(S2_FULL + t, s_phase, 82u))) break;
                s_phase ^= 1;
                tc_fence_after();
                const bool diag = p.causal && j == qt;
                // Both sweeps in two instantiations: only the key tile on the diagonal of a causal item
                // carries the mask tests.
                float alpha = 1.f;
                bool any_grow = false;
                unsigned e[64];
                float l4[4] = {0.f, 0.f, 0.f, 0.f};
                auto sweeps = [&](auto is_diag) {
                    constexpr bool DIAG = decltype(is_diag)::value;
                    // sweep 1: maximum of the row of this tile (four chains)
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
                    for (int c = 0; c < 4; c += 2) {
                        unsigned v[64];
                        tmem_ld_32x32(s_addr + (unsigned)c * 32u, v);
                        tmem_ld_32x32(s_addr + (unsigned)(c + 1) * 32u, v + 32);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 64; ++i) {
                            float sv = __uint_as_float(v[i]);
                            if (DIAG && c * 32 + i > r) sv = -INFINITY;
                            m4[i & 3] = fmaxf(m4[i & 3], sv);
                        }
                    }
                    const float mt = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2e;
                    // (key 0 is visible to every query, so the first tile gives every row a finite maximum)
                    const bool grow = j > 0 && mt > ref + AT_LAG;
                    if (j == 0) ref = mt;
                    if (grow) {
                        alpha = ex2_approx(ref - mt);
                        ref = mt;
                    }
                    any_grow = __any_sync(0xffffffffu, grow);
                    // sweep 2: P, kept in registers until the previous P V has released the P tile
                    auto process = [&](const unsigned* v, int c) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float s0 = __uint_as_float(v[i]), s1 = __uint_as_float(v[i + 1]);
                            if (DIAG && c * 32 + i > r) s0 = -INFINITY;
                            if (DIAG && c * 32 + i + 1 > r) s1 = -INFINITY;
                            const float e0 = ex2_approx(fmaf(s0, p.scale_log2e, -ref));
                            const float e1 = ex2_approx(fmaf(s1, p.scale_log2e, -ref));
                            l4[i & 2] += e0;
                            l4[(i & 2) + 1] += e1;
                            e[c * 16 + (i >> 1)] = pack2<T>(e0, e1);
                        }
                    };
                    {
                        unsigned va[32], vb[32];
                        tmem_ld_32x32(s_addr, va);
                        tmem_ld_wait();
                        tmem_ld_32x32(s_addr + 32u, vb);
                        process(va, 0);
                        tmem_ld_wait();
                        tmem_ld_32x32(s_addr + 64u, va);
                        process(vb, 1);
                        tmem_ld_wait();
                        tmem_ld_32x32(s_addr + 96u, vb);
                        process(va, 2);
                        tmem_ld_wait();
                        process(vb, 3);
                    }
                };
                if (diag) sweeps(std::true_type{});
                else sweeps(std::false_type{});
                l_run = l_run * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
                // the scores are in registers: S can take this tile's next key tile
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(S2_EMPTY + t));
                if (!(ok = wait_all(P2_EMPTY + t, pe_phase, 83u))) break;     // the previous P V is done: O is at rest, P is free
                pe_phase ^= 1;
                if (any_grow) {
                    // rescale this warp's 32 rows of O (lanes whose maximum did not grow multiply by 1)
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        unsigned o[32];
                        tmem_ld_32x32(o_addr + (unsigned)c * 32u, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(o_addr + (unsigned)c * 32u, o);
                    }
                    tmem_st_wait();
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    unsigned char* row = p_tile + (c >> 1) * AT_PANEL + r * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
                        *reinterpret_cast<uint4*>(row + chunk * 16) =
                            make_uint4(e[c * 16 + 4 * q], e[c * 16 + 4 * q + 1], e[c * 16 + 4 * q + 2], e[c * 16 + 4 * q + 3]);
                    }
                }
                tc_fence_before();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor cores
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(P2_FULL + t));
            }
            if (!ok) break;
            } else {
            // ---- pass 1: row maximum of the raw scores (four independent chains)
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!(ok = wait_all(S2_FULL + t, s_phase, 81u))) break;
                s_phase ^= 1;
                tc_fence_after();
                const bool diag = p.causal && j == qt;
#pragma unroll 1
                for (int c = 0; c < 4; c += 2) {
                    unsigned v[64];
                    tmem_ld_32x32(s_addr + (unsigned)c * 32u, v);
                    tmem_ld_32x32(s_addr + (unsigned)(c + 1) * 32u, v + 32);
                    tmem_ld_wait();
                    if (diag) {   // only the key tile on the diagonal carries the mask tests
#pragma unroll
                        for (int i = 0; i < 64; ++i)
                            if (c * 32 + i > r) v[i] = 0xff800000u;   // -inf above the diagonal
                    }
#pragma unroll
                    for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(S2_EMPTY + t));
            }
            if (!ok) break;
            // ---- pass 2: P = exp2((S - m) * scale * log2 e) -> shared memory, row sums
            const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            const float mc = m * p.scale_log2e;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!(ok = wait_all(S2_FULL + t, s_phase, 82u))) break;
                s_phase ^= 1;
                if (!(ok = wait_all(P2_EMPTY + t, pe_phase, 83u))) break;     // the previous P V has read the P tile
                pe_phase ^= 1;
                tc_fence_after();
                const bool diag = p.causal && j == qt;
                auto process = [&](unsigned* v, int c) {
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i > r) v[i] = 0xff800000u;   // -inf above the diagonal: P = 0
                    }
                    float e[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        e[i] = ex2_approx(fmaf(__uint_as_float(v[i]), p.scale_log2e, -mc));
                        l4[i & 3] += e[i];
                    }
                    unsigned char* row = p_tile + (c >> 1) * AT_PANEL + r * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        o.x = pack2<T>(e[8 * q + 0], e[8 * q + 1]);
                        o.y = pack2<T>(e[8 * q + 2], e[8 * q + 3]);
                        o.z = pack2<T>(e[8 * q + 4], e[8 * q + 5]);
                        o.w = pack2<T>(e[8 * q + 6], e[8 * q + 7]);
                        const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
                        *reinterpret_cast<uint4*>(row + chunk * 16) = o;
                    }
                };
                unsigned va[32], vb[32];
                tmem_ld_32x32(s_addr, va);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 32u, vb);
                process(va, 0);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 64u, va);
                process(vb, 1);
                tmem_ld_wait();
                tmem_ld_32x32(s_addr + 96u, vb);
                process(va, 2);
                tmem_ld_wait();
                process(vb, 3);
                tc_fence_before();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor cores
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(P2_FULL + t));
                    mbar_arrive(bar(S2_EMPTY + t));
                }
            }
            if (!ok) break;
            l_run = (l4[0] + l4[1]) + (l4[2] + l4[3]);
            }
            // ---- O / l -> global memory
            if (!(ok = wait_all(O2_FULL + t, o_phase, 84u))) break;
            o_phase ^= 1;
            tc_fence_after();
            const float inv = 1.0f / l_run;
            T* orow = O + (long long)(b / p.heads) * p.o_bs + (long long)(b % p.heads) * p.o_hs + ((long long)qt * 128 + r) * p.o_rs;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                unsigned v[32];
                tmem_ld_32x32(o_addr + (unsigned)c * 32u, v);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = pack2<T>(__uint_as_float(v[8 * q + 0]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
                    o.y = pack2<T>(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
                    o.z = pack2<T>(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
                    o.w = pack2<T>(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O2_EMPTY + t));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

#include "attention_ts.cuh"

}  // namespace

bool attention_supported(DType dt, int64_t seq_q, int64_t seq_k, int64_t head_dim) {
    return (dt == DType::F16 || dt == DType::BF16) && head_dim == 128 && seq_q == seq_k && seq_q >= 128 && seq_q % 128 == 0 &&
           seq_q < (1ll << 24);
}

TensorData run_attention(Device& dev, const TensorData& q_in, const TensorData& k_in, const TensorData& v_in, bool causal,
                         float scale, int merge_heads) {
    // v may also come as the [batch, heads, seq, 128] view of a [batch, seq, heads * 128] projection
    const bool v_view = v_in.layout.rank() == 4;
    WGF_CHECK(q_in.layout.rank() == 3 && k_in.layout.shape == q_in.layout.shape &&
                  (v_view ? v_in.layout.shape[0] * v_in.layout.shape[1] == q_in.layout.shape[0] &&
                                v_in.layout.shape[2] == q_in.layout.shape[1] && v_in.layout.shape[3] == q_in.layout.shape[2]
                          : v_in.layout.shape == q_in.layout.shape),
              WGF_ERR_SHAPE, "attention takes q, k, v of one shape [batch*heads, seq, 128]");
    WGF_CHECK(q_in.dtype == k_in.dtype && q_in.dtype == v_in.dtype, WGF_ERR_DTYPE, "attention operands differ in element type");
    const int64_t BH = q_in.layout.shape[0], S = q_in.layout.shape[1], D = q_in.layout.shape[2];
    WGF_CHECK(attention_supported(q_in.dtype, S, S, D) && BH >= 1 && BH < (1ll << 31), WGF_ERR_UNSUPPORTED,
              "fused attention needs 16-bit elements, head dimension 128 and a sequence length that is a multiple of 128");
    const int64_t heads = merge_heads > 0 ? merge_heads : 1;
    WGF_CHECK(BH % heads == 0, WGF_ERR_SHAPE, "attention: batch*heads is not a multiple of the head count");
    dev.make_current();
    // rows must be contiguous and 16-byte aligned for TMA; anything else is gathered first
    auto usable = [](const TensorData& t) {
        const Layout& l = t.layout;
        return l.strides[2] == 1 && l.strides[1] % 8 == 0 && l.strides[0] % 8 == 0 && ((uintptr_t)t.base_ptr() & 15) == 0 &&
               l.strides[1] >= l.shape[2];
    };
    TensorData q = usable(q_in) ? q_in : run_compact(dev, q_in);
    TensorData k = usable(k_in) ? k_in : run_compact(dev, k_in);
    TensorData v = v_in;
    int v_heads = 0;
    if (v_view) {
        // readable in place if batch folds into the row axis: stride(batch) == seq * stride(row)
        const Layout& l = v_in.layout;
        const bool in_place = l.strides[3] == 1 && l.strides[2] % 8 == 0 && l.strides[1] % 8 == 0 && l.strides[2] >= l.shape[3] &&
                              l.strides[0] == l.shape[2] * l.strides[2] && ((uintptr_t)v_in.base_ptr() & 15) == 0 &&
                              l.shape[0] * l.shape[2] < (1ll << 31);
        if (in_place) {
            v_heads = (int)l.shape[1];
        } else {
            v = run_compact(dev, v_in);
            v.layout = Layout::contiguous({BH, S, D});
            v.layout.offset = 0;
        }
    } else if (!usable(v_in)) {
        v = run_compact(dev, v_in);
    }
    for (const TensorData* t : {&q, &k, &v}) dev.wait_for(*t->buf);
    TensorData out;
    out.dtype = q.dtype;
    // [n, seq, d], or with merged heads [batch, seq, heads * d] (head h of batch b at columns h*d ..)
    out.layout = merge_heads > 0 ? Layout::contiguous({BH / heads, S, heads * D}) : Layout::contiguous({BH, S, D});
    out.buf = dev.alloc((size_t)(BH * S * D) * 2, false);
    if (dev.dry) {
        dev.begin_launch("attention_tc");
        dev.end_launch();
        return out;
    }
    const bool bf16 = q.dtype == DType::BF16;
    CUtensorMap mq, mk, mv;
    const bool maps_ok = encode_3d(&mq, bf16, q.base_ptr(), D, S, BH, q.layout.strides[1], q.layout.strides[0], 64, 128) &&
                         encode_3d(&mk, bf16, k.base_ptr(), D, S, BH, k.layout.strides[1], k.layout.strides[0], 64, 128) &&
                         (v_heads > 0 ? encode_3d(&mv, bf16, v.base_ptr(), D, v.layout.shape[0] * S, v_heads, v.layout.strides[2],
                                                  v.layout.strides[1], 64, 128)
                                      : encode_3d(&mv, bf16, v.base_ptr(), D, S, BH, v.layout.strides[1], v.layout.strides[0], 64, 128));
    WGF_CHECK(maps_ok, WGF_ERR_CUDA, "attention: tensor map creation failed");
    AtParams p{};
    p.n_q_tiles = p.n_k_tiles = (int)(S / 128);
    p.bh = (int)BH;
    p.causal = causal ? 1 : 0;
    p.is_bf16 = bf16 ? 1 : 0;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.heads = (int)heads;
    p.v_heads = v_heads;
    p.v_rows = (int)S;
    p.o_rs = heads * D;
    p.o_hs = D;
    p.o_bs = S * heads * D;
    p.error = dev.error_word();
    // Kernel forms, newest first: P through tensor memory (attention_ts_kernel, the default); P through
    // shared memory with two query tiles per CTA (WGF_ATT_SMEM_P=1: attention_tc2_kernel, one pass, or
    // two with WGF_ATT_TWO_PASS=1); one query tile per CTA (WGF_ATT_SINGLE=1).  These switches are read
    // at every call: the tests go through all the forms in one process.
    const bool single = getenv("WGF_ATT_SINGLE") != nullptr;
    const bool two_pass = getenv("WGF_ATT_TWO_PASS") != nullptr;
    const bool smem_p = single || two_pass || getenv("WGF_ATT_SMEM_P") != nullptr;
    BufferRef prof_buf;
    if (getenv("WGF_ATT_PROFILE") && !smem_p) {
        prof_buf = dev.alloc(26 * sizeof(unsigned long long), true);
        p.prof = (unsigned long long*)prof_buf->ptr;
    }
    const bool pairs = !single;
    const long long items = pairs ? BH * ((S / 128 + 1) / 2) : BH * (S / 128);
    const unsigned grid = (unsigned)std::min<long long>(items, dev.sm_count);
    // the opt-in to more than 48 KiB of dynamic shared memory is a per-device attribute of the kernel
    static std::mutex attr_mu;
    static bool attr_set[64][12] = {};
    auto launch = [&](auto kernel, int slot, int threads, int smem_bytes, auto* optr) {
        {
            std::lock_guard<std::mutex> lk(attr_mu);
            const int ord = dev.ordinal >= 0 && dev.ordinal < 64 ? dev.ordinal : 0;
            if (!attr_set[ord][slot] || dev.ordinal >= 64) {
                WGF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
                attr_set[ord][slot] = true;
            }
        }
        kernel<<<grid, threads, smem_bytes, dev.stream>>>(mq, mk, mv, optr, p);
    };
    dev.begin_launch("attention_tc");
    if (!smem_p) {
        // how the softmax warps go over the scores (see attention_ts.cuh); WGF_ATT_MODE picks another form
        const char* me = getenv("WGF_ATT_MODE");
        const int mode = me ? atoi(me) : 0;
        if (prof_buf) {
            if (bf16) launch(attention_ts_kernel<__nv_bfloat16, 0, true>, 10, TS_THREADS, TS_SMEM, (__nv_bfloat16*)out.base_ptr());
            else launch(attention_ts_kernel<__half, 0, true>, 11, TS_THREADS, TS_SMEM, (__half*)out.base_ptr());
        } else if (bf16) {
            if (mode == 1) launch(attention_ts_kernel<__nv_bfloat16, 1>, 9, TS_THREADS, TS_SMEM, (__nv_bfloat16*)out.base_ptr());
            else launch(attention_ts_kernel<__nv_bfloat16, 0>, 8, TS_THREADS, TS_SMEM, (__nv_bfloat16*)out.base_ptr());
        } else {
            if (mode == 1) launch(attention_ts_kernel<__half, 1>, 7, TS_THREADS, TS_SMEM, (__half*)out.base_ptr());
            else launch(attention_ts_kernel<__half, 0>, 6, TS_THREADS, TS_SMEM, (__half*)out.base_ptr());
        }
    } else if (pairs) {
        const bool online = !getenv("WGF_ATT_TWO_PASS");   // one pass (online softmax) unless switched off
        if (online) {
            if (bf16) launch(attention_tc2_kernel<__nv_bfloat16, true>, 5, A2_THREADS, A2_SMEM, (__nv_bfloat16*)out.base_ptr());
            else launch(attention_tc2_kernel<__half, true>, 4, A2_THREADS, A2_SMEM, (__half*)out.base_ptr());
        } else {
            if (bf16) launch(attention_tc2_kernel<__nv_bfloat16, false>, 3, A2_THREADS, A2_SMEM, (__nv_bfloat16*)out.base_ptr());
            else launch(attention_tc2_kernel<__half, false>, 2, A2_THREADS, A2_SMEM, (__half*)out.base_ptr());
        }
    } else {
        if (bf16) launch(attention_tc_kernel<__nv_bfloat16>, 1, AT_THREADS, AT_SMEM, (__nv_bfloat16*)out.base_ptr());
        else launch(attention_tc_kernel<__half>, 0, AT_THREADS, AT_SMEM, (__half*)out.base_ptr());
    }
    dev.end_launch();
    if (prof_buf) {
        // measurement aid: waits for the kernel and prints where CTA 0's warps spent their cycles
        unsigned long long prof[26];
        WGF_CUDA(cudaStreamSynchronize(dev.stream));
        WGF_CUDA(cudaMemcpy(prof, prof_buf->ptr, sizeof prof, cudaMemcpyDeviceToHost));
        const char* mma[10] = {"other", "wait Q", "wait K0", "wait O empty", "wait P0", "wait P1", "wait V", "wait K", "issue PV", "issue S"};
        const char* sm[8] = {"other", "wait S", "load+max", "rescale", "exp+store", "hand-over", "wait O", "write-out"};
        fprintf(stderr, "[wgf] attention_ts, CTA 0, cycles by role\n  MMA warp:");
        for (int i = 0; i < 10; ++i) fprintf(stderr, " %s %llu,", mma[i], prof[i]);
        for (int t = 0; t < 2; ++t) {
            fprintf(stderr, "\n  softmax warps of tile %d:", t);
            for (int i = 0; i < 8; ++i) fprintf(stderr, " %s %llu,", sm[i], prof[10 + 8 * t + i]);
        }
        fprintf(stderr, "\n");
    }
    return out;
}

}  // namespace wgf
