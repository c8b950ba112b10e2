// attention_ts_kernel: fused softmax attention whose probabilities never leave tensor memory.
// Included by attention_tc.cu (shares AtParams, at_idesc, decode_pair and the tile constants).
//
// What changes against attention_tc2_kernel.  There the softmax warps write P as a 16-bit tile
// into shared memory, from where the P V product reads it back as its A operand: per key tile and
// query tile 32 KiB written and 32 KiB read through the same shared memory that feeds the tensor
// cores their other operands (an M128 x N128 x K16 tcgen05.mma with both operands in shared memory
// reads 8 KiB per 64 cycles of math, all the SM delivers), plus a proxy fence and a hand-over per
// tile.  Here P goes back into TENSOR memory, packed two 16-bit values per 32-bit column over the
// first 64 of the 128 columns that held S (tcgen05.st), and P V takes its A operand from there
// (tcgen05.mma with the A operand in tensor memory): the P V products read only V from shared
// memory, nothing is stored to it by the softmax warps, and the four tiles of shared memory that
// held Q0, Q1, P0, P1 shrink to two, which makes room for a 5-stage K / V ring.
//
// Work and roles (320 threads, one persistent CTA per SM, two adjacent query tiles per item):
//   warp 0     TMA producer (one lane): Q0, Q1, then K(0), V(0), K(1), V(1), ... through the ring
//   warp 1     MMA issuer (one lane), per key tile j and tile t:  P V_t(j), then S_t(j+1) = Q_t K(j+1)^T.
//              The tensor pipe executes one thread's MMAs in issue order, so S_t(j+1) overwrites the
//              columns of P_t(j) only after P V_t(j) has read them, and no barrier guards that.
//   warps 2-5  softmax of tile 0, warps 6-9 of tile 1: thread r owns row r (tensor-memory lane r).
//              One sweep: the 128 scores of the row are loaded into registers once; maximum,
//              exponentials, row sum and the packed P come from the registers.
// Online softmax with a lazily updated reference maximum as in attention_tc2_kernel: P =
// exp2(s * c - ref); ref follows the running maximum only when that has outgrown it by more than
// 2^AT_LAG, and only then O and l of the row are rescaled (O through tcgen05.ld / tcgen05.st).
// When S_t(j) is complete every MMA issued before it is complete too (a commit covers all earlier
// MMAs of the thread), P V_t(j-1) among them: O_t is at rest while the softmax warps of tile t work.
// Tensor memory: S_t / P_t in columns 128 t, O_t in 256 + 128 t.  Every wait is bounded.

// Cycle counters around the waits and phases of each role, CTA 0 only, in the PROF instantiation of
// the kernel (WGF_ATT_PROFILE=1 selects it): 26 totals that run_attention prints after the launch.
// The ordinary instantiation carries none of it.
#define PROF_DECL(n) unsigned long long prof_acc[PROF ? n : 1] = {}; const bool prof_on = PROF && p.prof != nullptr && blockIdx.x == 0; unsigned long long prof_t = prof_on ? clock64() : 0; (void)prof_acc; (void)prof_t
#define PROF_LAP(slot) do { if constexpr (PROF) { if (prof_on) { const unsigned long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; } } } while (0)
#define PROF_FLUSH(base, n) do { if constexpr (PROF) { if (prof_on) for (int i_ = 0; i_ < (n); ++i_) p.prof[(base) + i_] = prof_acc[i_]; } } while (0)

constexpr int TS_STAGES = 5;
constexpr int TS_THREADS = 320;
constexpr int TS_SMEM = (2 + TS_STAGES) * AT_TILE + 1024 /*alignment slack*/ + 512 /*barriers*/;
enum {
    TQ_FULL = 0, TQ_EMPTY = 2, TKV_FULL = 4, TKV_EMPTY = TKV_FULL + TS_STAGES, TS_FULL = TKV_EMPTY + TS_STAGES,
    TP_FULL = TS_FULL + 2, TO_FULL = TP_FULL + 2, TO_EMPTY = TO_FULL + 2, TS_BARS = TO_EMPTY + 2
};

// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (128 rows x 16 K-elements, two per 32-bit
// column) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 registers of every lane -> 16 columns of the warp's 32 tensor-memory lanes.
__device__ __forceinline__ void tmem_st_32x16(unsigned taddr, const unsigned* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
        : "memory");
}

// max(a, b, c) in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// MODE 0: the 128 scores of a row are loaded into registers once (maximum, exponentials and P all come
//         from them); 1: two sweeps over tensor memory, 32 scores at a time (a quarter of the
//         registers, no spills; measured slower: 429 / 732 us against 382 / 592 us causal / full on
//         [256, 2048, 128]).  Also measured and dropped: packed exponentials (ex2.approx.f16x2 keeps the
//         special-function unit as long as two scalar ones: 459 / 801 us), a cubic 2^x on the FMA pipe
//         for half or a quarter of the elements (441 / 721 and 407 / 653 us) and P handed to the MMA
//         warp in two halves (405 / 642 us): per key tile a softmax warp group computes for about 2100
//         cycles and waits for S about as long, the MMA warp waits for P a quarter of its time -- the
//         tiles' softmax phases overlap each other instead of the other tile's MMAs (cycle counters:
//         WGF_ATT_PROFILE=1).
template <typename T, int MODE, bool PROF = false>
__global__ void __launch_bounds__(TS_THREADS, 1)
attention_ts_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, T* __restrict__ O, const __grid_constant__ AtParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [Q0][Q1][ring ...]
    const unsigned q_smem0 = smem_u32(smem), ring = q_smem0 + 2 * AT_TILE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (2 + TS_STAGES) * AT_TILE);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + TS_BARS);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (unsigned)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < TS_BARS; ++i) {
            // one arrival per softmax warp of the tile
            const bool four = (i >= TP_FULL && i < TP_FULL + 2) || (i >= TO_EMPTY && i < TO_EMPTY + 2);
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
            unsigned pos = 0;                          // tiles pushed so far: stage = pos % TS_STAGES
            unsigned q_phase[2] = {1, 1};              // fresh "empty" barriers count as already released
            bool ok = true;
            auto push = [&](const CUtensorMap* map, int row0, int b) -> bool {
                const unsigned stage = pos % TS_STAGES, phase = ((pos / TS_STAGES) & 1u) ^ 1u;
                if (!mbar_wait(bar(TKV_EMPTY + stage), phase)) {
                    atomicExch(p.error, 91u);
                    return false;
                }
                const unsigned dst = ring + stage * AT_TILE;
                mbar_expect_tx(bar(TKV_FULL + stage), AT_TILE);
                tma_load_3d(dst, map, bar(TKV_FULL + stage), 0, row0, b);
                tma_load_3d(dst + AT_PANEL, map, bar(TKV_FULL + stage), 64, row0, b);
                ++pos;
                return true;
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, pt;
                decode_pair(p, n_pairs, w, b, pt);
                const int n_max = max(tiles_of(pt, 0), tiles_of(pt, 1));
                for (int t = 0; t < 2 && ok; ++t) {
                    if (tiles_of(pt, t) == 0) continue;
                    if (!mbar_wait(bar(TQ_EMPTY + t), q_phase[t])) {
                        atomicExch(p.error, 90u);
                        ok = false;
                        break;
                    }
                    q_phase[t] ^= 1;
                    const unsigned qs = q_smem0 + (unsigned)t * AT_TILE;
                    mbar_expect_tx(bar(TQ_FULL + t), AT_TILE);
                    tma_load_3d(qs, &map_q, bar(TQ_FULL + t), 0, (2 * pt + t) * 128, b);
                    tma_load_3d(qs + AT_PANEL, &map_q, bar(TQ_FULL + t), 64, (2 * pt + t) * 128, b);
                }
                // the order in which the MMA warp takes them from the ring
                for (int j = 0; j < n_max && ok; ++j) {
                    ok = push(&map_k, j * 128, b);
                    if (ok) ok = push(&map_v, v_row(j * 128, b), v_slab(b));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const unsigned idesc_s = at_idesc((unsigned)p.is_bf16, 0u), idesc_pv = at_idesc((unsigned)p.is_bf16, 1u);
            unsigned pos = 0;                          // ring position of K(0) of the current item
            unsigned q_phase[2] = {0, 0}, p_phase[2] = {0, 0}, o_phase[2] = {1, 1};
            bool ok = true;
            int nk[2];
            PROF_DECL(10);   // 0 bookkeeping, 1 Q, 2 K(0), 3 O empty, 4 P of tile 0, 5 P of tile 1, 6 V, 7 K(j+1), 8 issue of P V, 9 issue of S
            auto wait_or = [&](int which, unsigned ph, unsigned code) -> bool {
                if (mbar_wait(bar(which), ph)) return true;
                atomicExch(p.error, code);
                return false;
            };
            auto wait_ring = [&](unsigned at, unsigned code) -> bool {
                return wait_or(TKV_FULL + (int)(at % TS_STAGES), (at / TS_STAGES) & 1u, code);
            };
            // S_t = Q_t K^T with K in ring position `at`
            auto issue_s = [&](int t, unsigned at, bool last) {
                const unsigned kt = ring + (at % TS_STAGES) * AT_TILE;
                const unsigned qs = q_smem0 + (unsigned)t * AT_TILE;
                const unsigned d = tmem_base + (unsigned)t * AT_S_COLS;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // both K-major: rows of 128 bytes, 8-row groups 1024 bytes apart, 32 bytes per K
                    // step inside a 64-column panel, the second panel 16 KiB further
                    const unsigned off = (unsigned)(kk >> 2) * AT_PANEL + (unsigned)(kk & 3) * 32u;
                    umma_f16(d, smem_desc(qs + off, 16, 1024), smem_desc(kt + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
                }
                umma_commit(bar(TS_FULL + t));
                if (last) umma_commit(bar(TQ_EMPTY + t));   // Q_t is free once these are done
            };
            // O_t (+)= P_t V with V in ring position `at`; P_t in the first 64 columns of S_t
            auto issue_pv = [&](int t, unsigned at, bool first, bool last) {
                const unsigned vt = ring + (at % TS_STAGES) * AT_TILE;
                const unsigned a = tmem_base + (unsigned)t * AT_S_COLS;
                const unsigned d = tmem_base + AT_O_COL0 + (unsigned)t * 128u;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // A = P from tensor memory: 16 keys = 8 columns per K step.  B = V, N-major: 64-column
                    // panels 16 KiB apart (leading), 8-key groups 1024 bytes apart (stride), 16 keys =
                    // 2048 bytes per K step
                    const unsigned long long bdesc = smem_desc(vt + (unsigned)kk * 2048u, AT_PANEL, 1024);
                    umma_f16_ts(d, a + (unsigned)kk * 8u, bdesc, idesc_pv, (first && kk == 0) ? 0u : 1u);
                }
                if (last) umma_commit(bar(TO_FULL + t));
            };
            for (long long w = blockIdx.x; w < items && ok; w += gridDim.x) {
                int b, pt;
                decode_pair(p, n_pairs, w, b, pt);
                nk[0] = tiles_of(pt, 0);
                nk[1] = tiles_of(pt, 1);
                const int n_max = max(nk[0], nk[1]);
                PROF_LAP(0);
                for (int t = 0; t < 2 && ok; ++t) {
                    if (nk[t] == 0) continue;
                    ok = wait_or(TQ_FULL + t, q_phase[t], 100u);
                    q_phase[t] ^= 1;
                }
                if (!ok) break;
                PROF_LAP(1);
                // S_t(0) for both tiles
                if (!(ok = wait_ring(pos, 101u))) break;
                PROF_LAP(2);
                tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (nk[t] > 0) issue_s(t, pos, nk[t] == 1);
                umma_commit(bar(TKV_EMPTY + (int)(pos % TS_STAGES)));
                for (int j = 0; j < n_max && ok; ++j) {
                    const unsigned at_v = pos + 2u * (unsigned)j + 1u, at_k = at_v + 1u;   // V(j), K(j+1)
                    bool have_v = false, have_k = false;
                    for (int t = 0; t < 2 && ok; ++t) {
                        if (j >= nk[t]) continue;
                        PROF_LAP(0);
                        if (j == 0) {                       // the previous item's O_t has been read out
                            if (!(ok = wait_or(TO_EMPTY + t, o_phase[t], 102u))) break;
                            o_phase[t] ^= 1;
                            PROF_LAP(3);
                        }
                        if (!(ok = wait_or(TP_FULL + t, p_phase[t], 103u))) break;
                        p_phase[t] ^= 1;
                        PROF_LAP(4 + t);
                        if (!have_v) {
                            if (!(ok = wait_ring(at_v, 104u))) break;
                            have_v = true;
                            PROF_LAP(6);
                        }
                        tc_fence_after();
                        PROF_LAP(0);
                        issue_pv(t, at_v, j == 0, j == nk[t] - 1);
                        PROF_LAP(8);
                        if (j + 1 < nk[t]) {
                            if (!have_k) {
                                if (!(ok = wait_ring(at_k, 105u))) break;
                                have_k = true;
                                PROF_LAP(7);
                                tc_fence_after();
                            }
                            PROF_LAP(0);
                            issue_s(t, at_k, j + 1 == nk[t] - 1);
                            PROF_LAP(9);
                        }
                    }
                    if (!ok) break;
                    umma_commit(bar(TKV_EMPTY + (int)(at_v % TS_STAGES)));
                    if (j + 1 < n_max) umma_commit(bar(TKV_EMPTY + (int)(at_k % TS_STAGES)));
                }
                pos += 2u * (unsigned)n_max;
            }
            PROF_LAP(0);
            PROF_FLUSH(0, 10);
        }
    } else {
        // ------------------------------------------------------------------ softmax (warps 2-5: tile 0, warps 6-9: tile 1)
        const int t = (warp - 2) >> 2;
        const int quarter = warp & 3;                       // tensor-memory lanes 32*quarter .. +31 belong to this warp
        const int r = quarter * 32 + lane;                  // row of the query tile
        const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
        const unsigned s_addr = lane_base + (unsigned)t * AT_S_COLS, o_addr = lane_base + AT_O_COL0 + (unsigned)t * 128u;
        unsigned s_phase = 0, o_phase = 0;
        bool ok = true;
        PROF_DECL(8);   // 0 other, 1 wait S, 2 loads + maximum, 3 rescale, 4 exponentials + stores, 5 hand-over, 6 wait O, 7 write-out
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
            float l_run = 0.f, ref = 0.f;
            for (int j = 0; j < n_kv && ok; ++j) {
                PROF_LAP(0);
                if (!(ok = wait_all(TS_FULL + t, s_phase, 110u))) break;
                s_phase ^= 1;
                PROF_LAP(1);
                tc_fence_after();
                float alpha = 1.f;
                float l4[4] = {0.f, 0.f, 0.f, 0.f};
                const bool diag = p.causal && j == qt;   // only the key tile on the diagonal carries the mask
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                unsigned v[MODE == 0 ? 128 : 1];
                auto maxes = [&](const unsigned* x, int c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float sv = __uint_as_float(x[i]);
                        if (diag && c * 32 + i > r) sv = -INFINITY;
                        m4[i & 3] = fmaxf(m4[i & 3], sv);
                    }
                };
                if constexpr (MODE == 0) {
                    tmem_ld_32x32(s_addr, v);
                    tmem_ld_32x32(s_addr + 32u, v + 32);
                    tmem_ld_32x32(s_addr + 64u, v + 64);
                    tmem_ld_32x32(s_addr + 96u, v + 96);
                    tmem_ld_wait();
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 128; ++i)
                            if (i > r) v[i] = 0xff800000u;   // -inf above the diagonal
                    }
#pragma unroll
                    for (int i = 0; i < 128; i += 8) {   // four chains, two scores per instruction
                        m4[0] = fmax3(m4[0], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                        m4[1] = fmax3(m4[1], __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                        m4[2] = fmax3(m4[2], __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                        m4[3] = fmax3(m4[3], __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                    }
                } else {
                    // first sweep: the maximum, 32 scores at a time, the next load in flight meanwhile
                    unsigned va[32], vb[32];
                    tmem_ld_32x32(s_addr, va);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 32u, vb);
                    maxes(va, 0);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 64u, va);
                    maxes(vb, 1);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 96u, vb);
                    maxes(va, 2);
                    tmem_ld_wait();
                    maxes(vb, 3);
                }
                const float mt = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2e;
                // (key 0 is visible to every query, so the first tile gives every row a finite maximum)
                const bool grow = j > 0 && mt > ref + AT_LAG;
                if (j == 0) ref = mt;
                if (grow) {
                    alpha = ex2_approx(ref - mt);
                    ref = mt;
                }
                PROF_LAP(2);
                if (__any_sync(0xffffffffu, grow)) {
                    // S_t(j) is complete, so P V_t(j-1) is too: O_t is at rest.  Rescale this warp's 32
                    // rows (lanes whose maximum did not grow multiply by 1).
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        unsigned o[32];
                        tmem_ld_32x32(o_addr + (unsigned)c * 32u, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(o_addr + (unsigned)c * 32u, o);
                    }
                }
                PROF_LAP(3);
                // P = exp2(s * c - ref), packed two per column over the columns the scores came from
                // (chunk c of 32 scores becomes columns 16 c .. 16 c + 15: always behind the loads)
                const float nref = -ref;
                auto probabilities = [&](const unsigned* x, int c) {
                    unsigned pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float s0 = __uint_as_float(x[i]), s1 = __uint_as_float(x[i + 1]);
                        if (MODE != 0 && diag && c * 32 + i > r) s0 = -INFINITY;
                        if (MODE != 0 && diag && c * 32 + i + 1 > r) s1 = -INFINITY;
                        const float x0 = fmaf(s0, p.scale_log2e, nref), x1 = fmaf(s1, p.scale_log2e, nref);
                        const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                        l4[i & 2] += e0;
                        l4[(i & 2) + 1] += e1;
                        pk[i >> 1] = pack2<T>(e0, e1);
                    }
                    tmem_st_32x16(s_addr + (unsigned)c * 16u, pk);
                };
                if constexpr (MODE == 0) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) probabilities(v + c * 32, c);
                } else {
                    unsigned va[32], vb[32];
                    tmem_ld_32x32(s_addr, va);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 32u, vb);
                    probabilities(va, 0);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 64u, va);
                    probabilities(vb, 1);
                    tmem_ld_wait();
                    tmem_ld_32x32(s_addr + 96u, vb);
                    probabilities(va, 2);
                    tmem_ld_wait();
                    probabilities(vb, 3);
                }
                l_run = l_run * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
                PROF_LAP(4);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(TP_FULL + t));
                PROF_LAP(5);
            }
            if (!ok) break;
            // ---- O / l -> global memory
            if (!(ok = wait_all(TO_FULL + t, o_phase, 111u))) break;
            o_phase ^= 1;
            PROF_LAP(6);
            tc_fence_after();
            const float inv = 1.0f / l_run;
            T* orow = O + (long long)(b / p.heads) * p.o_bs + (long long)(b % p.heads) * p.o_hs + ((long long)qt * 128 + r) * p.o_rs;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                unsigned o[32];
                tmem_ld_32x32(o_addr + (unsigned)c * 32u, o);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 u;
                    u.x = pack2<T>(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
                    u.y = pack2<T>(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
                    u.z = pack2<T>(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
                    u.w = pack2<T>(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = u;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(TO_EMPTY + t));
            PROF_LAP(7);
        }
        if (lane == 0 && quarter == 0) PROF_FLUSH(10 + 8 * t, 8);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}
