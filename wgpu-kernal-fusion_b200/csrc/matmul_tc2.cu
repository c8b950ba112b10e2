// f16 / bf16 matmul on CTA PAIRS (tcgen05 cta_group::2): two CTAs of a cluster on neighbouring
// SMs share one 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its own 128
// columns of B (the other half comes from the peer's shared memory inside the tensor cores)
// and accumulates its 128 x 256 half of the tile in its own tensor memory.  Compared with one
// CTA per 128 x 256 tile (matmul_tc.cu) every tcgen05.mma reads 8 KiB instead of 12 KiB of
// operands per SM, so shared-memory bandwidth (128 bytes per clock) no longer caps the tensor
// pipe at about 80 %.  Tiles are walked in bands (tc::banded_tile) so that a wave reuses its
// operand panels through L2, and leftover tiles that would fill at most half of the last wave
// are cut into two 256 x 128 units.
//
// Roles per CTA: warp 0 = TMA producer (both CTAs load their halves; all loads of a stage
// complete on the LEADER's "full" barrier), warp 1 = MMA issuer (leader only; its commits
// arrive on both CTAs' barriers), warps 2-9 = epilogue (each CTA drains its own tensor memory
// and tells the leader when an accumulator is free).  No TMA load uses multicast.  Every wait
// is bounded and reports through the device error word.
//
// Epilogues (MatmulEpilogue, matmul.hpp).  The crate never fuses anything around a MatMul
// (src/compute_graph/resolve.rs:138-154); here the resolver hands two patterns to this kernel:
//   RESIDUAL   C = round(A B) + R for a same-shape R (the residual adds of a decoder block): the
//              epilogue warps read R's rows with 16-byte loads while the accumulator is in registers
//   SILU_MUL   C = silu(A Bg) * (A Bu): the two products share A, so one 256-column tile holds 128
//              columns of the gate product and the same 128 columns of the up product (the leader CTA
//              stages Bg, its peer Bu -- the MMA is unchanged), and the epilogue combines column c
//              with column c + 128 and writes 128 columns.  The gate / up matrices never reach memory.
// Both round exactly where the separate kernels round (the product to the 16-bit type first, then
// every element-wise op on its own), so the results are bit-identical to the unfused graph.
#include <mutex>

#include "matmul.hpp"
#include "tc_common.cuh"

namespace wgf {

using namespace tc;

namespace {

constexpr int P_BM = 128;                 // rows of A per CTA (256 per pair)
constexpr int P_BN = 256;                 // columns of the tile
constexpr int P_BNH = 128;                // columns of B staged per CTA
constexpr int P_BK = 64, P_STAGES = 6, P_UMMA_K = 16;
constexpr int P_A_BYTES = P_BM * P_BK * 2;            // 16 KiB
constexpr int P_B_BYTES = P_BNH * P_BK * 2;           // 16 KiB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;  // per CTA; a stage of the pair is twice that
constexpr int P_EPI_TILE_BYTES = 32 * 128;
constexpr int P_EPI_WARPS = 8;             // per CTA: two per quarter of the accumulator's rows, each half of the columns
constexpr int P_EPI_BYTES = P_EPI_WARPS * P_EPI_TILE_BYTES;   // one staging tile per warp
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + P_EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;
constexpr unsigned PEER_BIT_MASK = 0xFEFFFFFFu;       // clears the CTA-rank bit of a shared-memory address: the even CTA of the pair

struct PairParams {
    long long M, N, K, batch;
    long long c_rs, c_bs;
    int tiles_m, tiles_n;   // tiles of 256 x 256
    int band;               // tile rows per band of the tile order (tc::banded_tile)
    int b_is_kn;
    int is_bf16;
    int use_tma_store;
    // Schedule: every cluster takes `full_waves` whole tiles (tile = wave * clusters + cluster).
    // When the `tail` tiles left over would keep at most half of the clusters busy, each of them
    // is cut along N into `nsplit` = 2 units of 256 x 128, so that the last wave takes half the
    // time of a full one (the tcgen05.mma shape becomes M256 x N128, 64 columns of B per CTA).
    int full_waves, tail, nsplit;
    unsigned* error;
    // epilogue: 0 none, 1 residual add, 2 silu(gate) * up (see the head of this file)
    int epi;
    const void* resid;       // [batch, M, N] like C, element type of C
    long long r_rs, r_bs;
};

// x rounded to T and back: what a value looks like after it has been stored as T
template <typename T> __device__ __forceinline__ float round16(float x);
template <> __device__ __forceinline__ float round16<__half>(float x) { return __half2float(__float2half_rn(x)); }
template <> __device__ __forceinline__ float round16<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <typename T> __device__ __forceinline__ float load16(const T* p);
template <> __device__ __forceinline__ float load16<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float load16<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void unpack2(unsigned u, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__half>(unsigned u, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
    lo = f.x;
    hi = f.y;
}
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(unsigned u, float& lo, float& hi) {
    lo = __uint_as_float(u << 16);
    hi = __uint_as_float(u & 0xffff0000u);
}

// silu(g) * u on values of a 16-bit tensor, op by op as the generated element-wise kernel does it
// (src/composite/silu.rs:4-7: x / (1 + exp(-x)); each op computed in f32 and rounded to the element
// type; exp through ex2.approx of x * log2 e, the form that kernel uses for 16-bit tensors).  The
// result still has to be rounded to T (the store does that).
template <typename T> __device__ __forceinline__ float silu_mul16(float gate_acc, float up_acc) {
    const float g = round16<T>(gate_acc), u = round16<T>(up_acc);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(-g, 1.4426950408889634f)));
    const float d = round16<T>(__fadd_rn(round16<T>(e), 1.0f));
    float q;   // the divisor comes from an exp: that kernel divides with div.full.f32 (Instr::fast_div)
    asm("div.full.f32 %0, %1, %2;" : "=f"(q) : "f"(g), "f"(d));
    q = round16<T>(q);
    return __fmul_rn(q, u);
}

struct Unit {
    long long tile;
    int nw;      // width of the unit in columns: P_BN, or P_BN / nsplit for a tail tile
    int noff;    // first column of the unit inside its tile
};

// The `it`-th unit of work of cluster `cluster` (of `clusters`); false when there is none.
__device__ __forceinline__ bool next_unit(const PairParams& p, long long cluster, long long clusters, int it, Unit& u) {
    u.nw = P_BN;
    u.noff = 0;
    if (it < p.full_waves) {
        u.tile = (long long)it * clusters + cluster;
        return true;
    }
    if (it > p.full_waves) return false;
    if (cluster >= (long long)p.tail * p.nsplit) return false;
    u.tile = (long long)p.full_waves * clusters + cluster / p.nsplit;
    u.nw = P_BN / p.nsplit;
    u.noff = (int)(cluster % p.nsplit) * u.nw;
    return true;
}

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned smem_dst, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' rows] * B[both CTAs' column halves]
__device__ __forceinline__ void umma_pair_f16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                              unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once every
// tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask)
                 : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted on `bar`, which may be the
// peer's barrier (no multicast: one destination)
__device__ __forceinline__ void tma_load_3d_pair(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// arrive on the barrier at the same offset in CTA `cta` of the cluster
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar, unsigned cta) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar), "r"(cta)
        : "memory");
}

__host__ __device__ constexpr unsigned pair_instr_desc(bool b_mn_major, int n) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
}

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
matmul_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c, T* __restrict__ C,
                  const __grid_constant__ PairParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* epi_smem = smem + P_STAGES * P_STAGE_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(epi_smem + P_EPI_BYTES);
    // bars[0..5] full (used in the leader), [6..11] empty, [12..13] accumulator full, [14..15] accumulator empty (leader)
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * P_STAGES + 4);
    const unsigned bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (P_STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * P_STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * P_STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();           // 0: leader of the pair
    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 2 * P_EPI_WARPS);   // one arrival per epilogue warp of either CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before();
    cluster_sync_all();                                 // both CTAs' barriers and tensor memory exist from here on
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
    const long long cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const int k_blocks = (int)((p.K + P_BK - 1) / P_BK);
    const unsigned smem_base = smem_u32(smem);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 1;
            bool ok = true;
            Unit u;
            for (int it = 0; ok && next_unit(p, cluster, clusters, it, u); ++it) {
                const int b = (int)(u.tile / tiles_per_batch);
                const int r = (int)(u.tile % tiles_per_batch);
                int mt, nt;
                tc::banded_tile(r, p.tiles_m, p.tiles_n, p.band, mt, nt);
                const int m0 = mt * 256 + (int)rank * P_BM;
                const int nh = u.nw / 2;                                  // columns of B this CTA stages
                // two B operands: both CTAs stage the same columns, the leader from the first (gate)
                // operand and its peer from the second (up)
                const bool dual = p.epi == 2;
                const CUtensorMap* mb = dual && rank == 1 ? &map_b2 : &map_b;
                const int n0 = dual ? nt * (P_BN / 2) + u.noff / 2 : nt * P_BN + u.noff + (int)rank * nh;
                const unsigned stage_tx = 2u * (unsigned)(P_A_BYTES + nh * P_BK * 2);   // both CTAs' bytes
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase)) {
                        atomicExch(p.error, 41u);
                        ok = false;
                        break;
                    }
                    const unsigned sa = smem_base + stage * P_STAGE_BYTES, sb = sa + P_A_BYTES;
                    const unsigned fb = full_bar(stage) & PEER_BIT_MASK;        // the leader's barrier
                    if (rank == 0) mbar_expect_tx(full_bar(stage), stage_tx);
                    tma_load_3d_pair(sa, &map_a, fb, kb * P_BK, m0, b);
                    // B in boxes of 64 columns (N-major: a [P_BK x 64] panel; K-major: 64 rows of P_BK)
                    for (int j = 0; j < nh / 64; ++j) {
                        if (p.b_is_kn) tma_load_3d_pair(sb + j * (P_BK * 128), mb, fb, n0 + j * 64, kb * P_BK, b);
                        else tma_load_3d_pair(sb + j * (64 * P_BK * 2), mb, fb, kb * P_BK, n0 + j * 64, b);
                    }
                    if (++stage == P_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            const unsigned idesc0 = pair_instr_desc(p.b_is_kn != 0, 0) | ((unsigned)p.is_bf16 << 7) | ((unsigned)p.is_bf16 << 10);
            int stage = 0;
            unsigned phase = 0;
            int acc = 0;
            unsigned acc_phase = 1;
            bool ok = true;
            Unit u;
            for (int it = 0; ok && next_unit(p, cluster, clusters, it, u); ++it) {
                const unsigned idesc = idesc0 | ((unsigned)(u.nw >> 3) << 17);   // N of the instruction = width of the unit
                if (!mbar_wait(acc_empty_bar(acc), acc_phase)) {
                    atomicExch(p.error, 42u);
                    break;
                }
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)acc * P_BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase)) {
                        atomicExch(p.error, 43u);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const unsigned sa = smem_base + stage * P_STAGE_BYTES, sb = sa + P_A_BYTES;
#pragma unroll
                    for (int k = 0; k < P_BK / P_UMMA_K; ++k) {
                        const unsigned long long adesc = smem_desc(sa + k * (P_UMMA_K * 2), 16, 1024);
                        const unsigned long long bdesc = p.b_is_kn ? smem_desc(sb + k * (P_UMMA_K * 128), P_BK * 128, 1024)
                                                                   : smem_desc(sb + k * (P_UMMA_K * 2), 16, 1024);
                        umma_pair_f16(tmem_d, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar(stage));      // frees the stage in both CTAs
                    if (++stage == P_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                umma_commit_pair(acc_full_bar(acc));         // both halves of the accumulator are complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
        // Warps w and w + 4 read the same quarter of the accumulator's rows (tensor-memory lanes
        // 32 (w mod 4) ..) and take one half of its columns each: with short K (two k-blocks per
        // tile, the batched [1024,128] x [128,1024] products) and with the heavier fused epilogues,
        // draining the accumulator sets the pace, and eight warps drain it twice as fast as four.
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        int acc = 0;
        unsigned acc_phase = 0;
        const bool vec_ok = (p.c_rs % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && (p.c_bs % 8 == 0);
        Unit u;
        for (int it = 0; next_unit(p, cluster, clusters, it, u); ++it) {
            const int b = (int)(u.tile / tiles_per_batch);
            const int r = (int)(u.tile % tiles_per_batch);
            int mt, nt;
            tc::banded_tile(r, p.tiles_m, p.tiles_n, p.band, mt, nt);
            // output columns of the unit: all of it, or (two B operands) half of it -- gate in the
            // first half of the accumulator's columns, up in the second
            const bool dual = p.epi == 2;
            const int out_w = dual ? u.nw / 2 : u.nw;
            const long long m0 = (long long)mt * 256 + (long long)rank * P_BM;
            const long long n0 = dual ? (long long)nt * (P_BN / 2) + u.noff / 2 : (long long)nt * P_BN + u.noff;
            bool got = mbar_wait(acc_full_bar(acc), acc_phase);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (lane == 0) atomicExch(p.error, 44u);
                break;
            }
            tc_fence_after();
            const long long m = m0 + quarter * 32 + lane;
            T* crow = C + (long long)b * p.c_bs + m * p.c_rs;
            const T* rrow = p.epi == 1 ? reinterpret_cast<const T*>(p.resid) + (long long)b * p.r_bs + m * p.r_rs : nullptr;
            const bool r_vec = p.epi == 1 && (p.r_rs % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.resid) & 15) == 0) && (p.r_bs % 8 == 0);
            const unsigned acc_addr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * P_BN);
            // 32 finished values of this thread's row, output columns n .. n + 31 (as f32 bit patterns;
            // the store rounds them to T)
            auto finished = [&](int c, unsigned* v) {
                tmem_ld_32x32(acc_addr + (unsigned)c, v);
                if (dual) {
                    unsigned w[32];
                    tmem_ld_32x32(acc_addr + (unsigned)(out_w + c), w);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(silu_mul16<T>(__uint_as_float(v[j]), __uint_as_float(w[j])));
                    return;
                }
                tmem_ld_wait();
                if (p.epi == 1) {
                    const long long n = n0 + c;
                    if (m < p.M && n < p.N) {
                        if (r_vec && n + 31 < p.N) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + n + 8 * q);
                                const unsigned rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                                for (int h = 0; h < 4; ++h) {
                                    float lo, hi;
                                    unpack2<T>(rw[h], lo, hi);
                                    v[8 * q + 2 * h] = __float_as_uint(__fadd_rn(lo, round16<T>(__uint_as_float(v[8 * q + 2 * h]))));
                                    v[8 * q + 2 * h + 1] = __float_as_uint(__fadd_rn(hi, round16<T>(__uint_as_float(v[8 * q + 2 * h + 1]))));
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < p.N) v[j] = __float_as_uint(__fadd_rn(load16<T>(rrow + n + j), round16<T>(__uint_as_float(v[j]))));
                        }
                    }
                }
            };
            // this warp's columns [c_lo, c_hi): half of the unit's, or (a width that does not split
            // into two multiples of 64) all of them for the first warp of the pair and none for the other
            const bool halves = out_w % 128 == 0;
            const int c_lo = halves ? col_half * (out_w / 2) : 0;
            const int c_hi = halves ? c_lo + out_w / 2 : (col_half == 0 ? out_w : 0);
            if (p.use_tma_store) {
#pragma unroll 1
                for (int c = c_lo; c < c_hi; c += 64) {
                    unsigned char* tile_smem = epi_smem + (warp - 2) * P_EPI_TILE_BYTES;
                    if (lane == 0) bulk_wait_read<0>();    // the store before this one has read the staging tile
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        unsigned v[32];
                        finished(c + half * 32, v);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 o;
                            o.x = pack2<T>(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
                            o.y = pack2<T>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
                            o.z = pack2<T>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
                            o.w = pack2<T>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
                            const int chunk = (half * 4 + q) ^ (lane & 7);
                            *reinterpret_cast<uint4*>(tile_smem + lane * 128 + chunk * 16) = o;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    const long long mrow = m0 + quarter * 32, ncol = n0 + c;
                    if (lane == 0 && mrow < p.M && ncol < p.N) {
                        tma_store_3d(&map_c, smem_u32(tile_smem), (int)ncol, (int)mrow, b);
                        bulk_commit();
                    }
                }
            } else {
#pragma unroll 1
                for (int c = c_lo; c < c_hi; c += 32) {
                    unsigned v[32];
                    finished(c, v);
                    const long long n = n0 + c;
                    if (m < p.M && n < p.N) {
                        if (vec_ok && n + 31 < p.N) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 o;
                                o.x = pack2<T>(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
                                o.y = pack2<T>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
                                o.z = pack2<T>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
                                o.w = pack2<T>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
                                *reinterpret_cast<uint4*>(crow + n + 8 * q) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < p.N) {
                                    unsigned pk = pack2<T>(__uint_as_float(v[j]), 0.f);
                                    reinterpret_cast<unsigned short*>(crow)[n + j] = (unsigned short)(pk & 0xffff);
                                }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_bar(acc), 0);    // the leader's barrier counts both CTAs' warps
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (p.use_tma_store && lane == 0) bulk_wait_read<0>();
    }
    tc_fence_before();
    cluster_sync_all();          // nobody signals into a CTA that has left, and both are done with tensor memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace

// Takes the problem if it is big enough for 256 x 256 tiles; `false` hands it to the one-CTA kernel
// (which has no epilogues: a caller that asked for one then runs the separate kernels).
bool matmul_tc_pair_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d,
                         const MatmulEpilogue* epi) {
    static const bool no_pair = getenv("WGF_MATMUL_NO_PAIR") != nullptr;
    static const bool no_tma_store = getenv("WGF_TC_NO_TMA_STORE") != nullptr;
    static const bool no_nsplit = getenv("WGF_MATMUL_NO_NSPLIT") != nullptr;
    static const bool verbose = getenv("WGF_MATMUL_VERBOSE") != nullptr;
    if (no_pair) return false;
    if (dt != DType::F16 && dt != DType::BF16) return false;
    const int kind = epi ? epi->kind : MatmulEpilogue::NONE;
    // a second half tile that is mostly padding wastes the peer CTA
    const long long rem = d.M % 256;
    if (d.M < 256 || d.N < 128 || d.K < 64 || (d.M < 2048 && rem != 0 && rem <= 128)) return false;
    if (d.M >= (1ll << 31) || d.N >= (1ll << 31) || d.K >= (1ll << 31) || d.batch >= (1ll << 31)) return false;
    auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (d.a_cs != 1 || d.a_rs % 8 || !a16(a) || (d.batch > 1 && d.a_bs % 8)) return false;
    const bool b_kn = d.b_cs == 1 && d.b_rs % 8 == 0;
    const bool b_nk = d.b_rs == 1 && d.b_cs % 8 == 0;
    if ((!b_kn && !b_nk) || !a16(b) || (d.batch > 1 && d.b_bs % 8)) return false;
    if (kind == MatmulEpilogue::SILU_MUL && (!epi->b2 || !a16(epi->b2))) return false;
    if (kind == MatmulEpilogue::RESIDUAL && !epi->resid) return false;
    if (dev.sm_count < 2) return false;
    const char* label = kind == MatmulEpilogue::SILU_MUL ? "matmul_tc2_silu_mul" : kind == MatmulEpilogue::RESIDUAL ? "matmul_tc2_residual" : "matmul_tc2";
    if (dev.dry) {
        dev.begin_launch(label);
        dev.end_launch();
        return true;
    }
    const bool bf16 = dt == DType::BF16;
    CUtensorMap map_a, map_b, map_b2;
    if (!encode_3d(&map_a, bf16, a, d.K, d.M, d.batch, d.a_rs, d.a_bs, P_BK, P_BM)) return false;
    auto encode_b = [&](CUtensorMap* m, const void* ptr) {
        return b_kn ? encode_3d(m, bf16, ptr, d.N, d.K, d.batch, d.b_rs, d.b_bs, 64, P_BK)
                    : encode_3d(m, bf16, ptr, d.K, d.N, d.batch, d.b_cs, d.b_bs, P_BK, 64);
    };
    if (!encode_b(&map_b, b)) return false;
    map_b2 = map_b;
    if (kind == MatmulEpilogue::SILU_MUL && !encode_b(&map_b2, epi->b2)) return false;   // same shape and strides as b
    PairParams p{};
    p.M = d.M;
    p.N = d.N;
    p.K = d.K;
    p.batch = d.batch;
    p.c_rs = d.c_rs;
    p.c_bs = d.c_bs;
    p.tiles_m = (int)((d.M + 255) / 256);
    // with two B operands a 256-column tile of the accumulator covers 128 output columns
    const int out_tile_n = kind == MatmulEpilogue::SILU_MUL ? P_BN / 2 : P_BN;
    p.tiles_n = (int)((d.N + out_tile_n - 1) / out_tile_n);
    p.b_is_kn = b_kn ? 1 : 0;
    p.is_bf16 = bf16 ? 1 : 0;
    p.epi = kind;
    if (kind == MatmulEpilogue::RESIDUAL) {
        p.resid = epi->resid;
        p.r_rs = epi->r_rs;
        p.r_bs = epi->r_bs;
    }
    CUtensorMap map_c = map_a;
    p.use_tma_store = 0;
    if (!no_tma_store && d.c_rs % 8 == 0 && (d.batch == 1 || d.c_bs % 8 == 0) && a16(c) &&
        encode_3d(&map_c, bf16, c, d.N, d.M, d.batch, d.c_rs, d.c_bs, 64, 32))
        p.use_tma_store = 1;
    p.error = dev.error_word();
    const long long total = (long long)p.tiles_m * p.tiles_n * d.batch;
    // Schedule (see PairParams).  One cluster per SM pair that the device reports as resident
    // for this kernel; leftover tiles that would keep at most half of the clusters busy are cut
    // in two along N (measured on 4096^3, 34 leftover tiles of 256: 104 us as whole tiles).
    // The opt-in to the kernel's dynamic shared memory and the residency it gives are properties of
    // (device, kernel): looked up once per device.
    static std::mutex state_mu;
    static int resident[64][2];
    static bool known[64][2];
    const int ti = bf16 ? 1 : 0;
    const void* fn = bf16 ? (const void*)matmul_tc2_kernel<__nv_bfloat16> : (const void*)matmul_tc2_kernel<__half>;
    int n_resident = 0;
    {
        std::lock_guard<std::mutex> lk(state_mu);
        const int ord = dev.ordinal >= 0 && dev.ordinal < 64 ? dev.ordinal : -1;
        if (ord < 0 || !known[ord][ti]) {
            WGF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(dev.sm_count & ~1));
            cfg.blockDim = dim3(P_THREADS);
            cfg.dynamicSmemBytes = P_SMEM_BYTES;
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = 2;
            at.val.clusterDim.y = 1;
            at.val.clusterDim.z = 1;
            cfg.attrs = &at;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) {
                cudaGetLastError();
                n = 0;
            }
            n_resident = n;
            if (ord >= 0) {
                resident[ord][ti] = n;
                known[ord][ti] = true;
            }
        } else {
            n_resident = resident[ord][ti];
        }
    }
    if (n_resident < 1) return false;
    long long clusters = std::min<long long>(dev.sm_count / 2, n_resident);
    p.band = band_rows((int)clusters, 256, out_tile_n, p.tiles_m);
    p.full_waves = (int)(total / clusters);
    p.tail = (int)(total % clusters);
    p.nsplit = (p.tail > 0 && 2ll * p.tail <= clusters && !no_nsplit) ? 2 : 1;
    if (p.full_waves == 0) clusters = (long long)p.tail * p.nsplit;   // fewer units than clusters: a smaller grid
    const unsigned grid = 2u * (unsigned)clusters;
    if (verbose)
        fprintf(stderr, "[wgf] matmul_tc2 %lldx%lldx%lld batch %lld epilogue %d: %lld tiles on %lld clusters (%d resident), %d full waves, tail %d cut in %d\n",
                d.M, d.N, d.K, d.batch, kind, total, clusters, n_resident, p.full_waves, p.tail, p.nsplit);
    dev.begin_launch(label);
    if (bf16) matmul_tc2_kernel<__nv_bfloat16><<<grid, P_THREADS, P_SMEM_BYTES, dev.stream>>>(map_a, map_b, map_b2, map_c, (__nv_bfloat16*)c, p);
    else matmul_tc2_kernel<__half><<<grid, P_THREADS, P_SMEM_BYTES, dev.stream>>>(map_a, map_b, map_b2, map_c, (__half*)c, p);
    dev.end_launch();
    return true;
}

}  // namespace wgf
