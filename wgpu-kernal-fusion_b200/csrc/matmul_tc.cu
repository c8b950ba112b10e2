// f16 / bf16 matmul on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the
// accumulator in tensor memory (TMEM), operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), fp32 accumulation, one rounding.
// Replaces the crate's scalar shared-memory kernel (src/matmul.rs:56-155) for 16-bit types.
//
// One persistent CTA per SM walks output tiles of 128 x 256.  Warp roles:
//   warp 0      TMA producer   (one lane): fills a 4-stage ring of {A 128x64, B 256x64} k-blocks
//   warp 1      MMA issuer     (one lane): 4 x tcgen05.mma (K = 16) per k-block into one of two
//                               TMEM accumulators (2 x 256 columns = all 512 columns of the SM)
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (32 lanes x 32 columns per load),
//                               convert, store to global; overlaps the next tile's main loop
// Synchronisation is by mbarriers only; every wait is bounded and reports through an error
// word instead of hanging.
//
// Layouts: A is [M,K] row-major (K-major).  B is either [N,K] row-major (a transposed view:
// K-major) or [K,N] row-major (N-major); both go straight from global memory through TMA.
// M, N, K need not divide the tile: TMA zero-fills out-of-range reads, stores are guarded.
#include <mutex>

#include "matmul.hpp"
#include "tc_common.cuh"

namespace wgf {

using namespace tc;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;            // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;            // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_TILE_BYTES = 32 * 128;              // one warp's staging tile: 32 rows x 64 f16
constexpr int EPI_BYTES = 4 * 2 * EPI_TILE_BYTES;     // 4 epilogue warps x 2 tiles = 32 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int TC_THREADS = 192;

struct TcParams {
    long long M, N, K, batch;
    long long c_rs, c_bs;
    int tiles_m, tiles_n;
    int band;          // tile rows per band of the tile order (tc::banded_tile)
    int b_is_kn;       // 1: B stored [K,N] (N-major), 0: B stored [N,K] (K-major)
    int is_bf16;
    int use_tma_store; // 1: epilogue stages through shared memory and stores by TMA (needs N % 8 == 0)
    unsigned* error;   // device word: 0 = ok, else code of the wait that gave up
};


// Instruction descriptor for kind::f16: fp32 accumulator (bits 4-5 = 1), A/B format in bits
// 7-9 / 10-12 (0 = f16, 1 = bf16), A/B major in bits 15 / 16 (0 = K-major, 1 = MN-major),
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr unsigned instr_desc(bool bf16, bool b_mn_major) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}


template <typename T>
__global__ void __launch_bounds__(TC_THREADS, 1)
matmul_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, T* __restrict__ C, const __grid_constant__ TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    // stage buffers need 1024-byte alignment for the 128-byte swizzle atoms
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* epi_smem = smem + STAGES * STAGE_BYTES;   // 1024-byte aligned (the stages are 48 KiB each)
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(epi_smem + EPI_BYTES);
    // bars[0..3] full, [4..7] empty, [8..9] accumulator full, [10..11] accumulator empty
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 12);
    const unsigned bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4);   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
    const long long total_tiles = tiles_per_batch * p.batch;
    const int k_blocks = (int)((p.K + BK - 1) / BK);
    const unsigned smem_base = smem_u32(smem);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 1;   // a fresh "empty" barrier counts as already released
            bool ok = true;
            for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int b = (int)(tile / tiles_per_batch);
                const int r = (int)(tile % tiles_per_batch);
                int mt, nt;
                tc::banded_tile(r, p.tiles_m, p.tiles_n, p.band, mt, nt);
                const int m0 = mt * BM, n0 = nt * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase)) {
                        atomicExch(p.error, 1u);
                        ok = false;
                        break;
                    }
                    const unsigned sa = smem_base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    tma_load_3d(sa, &map_a, full_bar(stage), kb * BK, m0, b);
                    if (p.b_is_kn) {
                        // [K,N] storage: four boxes of 64 k-rows x 64 n (one 128-byte swizzle span each)
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_3d(sb + j * (BK * 128), &map_b, full_bar(stage), n0 + j * 64, kb * BK, b);
                    } else {
                        tma_load_3d(sb, &map_b, full_bar(stage), kb * BK, n0, b);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const unsigned idesc = p.b_is_kn ? instr_desc(false, true) | ((unsigned)p.is_bf16 << 7) | ((unsigned)p.is_bf16 << 10)
                                             : instr_desc(false, false) | ((unsigned)p.is_bf16 << 7) | ((unsigned)p.is_bf16 << 10);
            int stage = 0;
            unsigned phase = 0;
            int acc = 0;
            unsigned acc_phase = 1;   // both accumulators start out free
            bool ok = true;
            for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(acc_empty_bar(acc), acc_phase)) {
                    atomicExch(p.error, 2u);
                    break;
                }
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase)) {
                        atomicExch(p.error, 3u);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const unsigned sa = smem_base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // A, K-major: rows of 128 bytes, 8-row groups 1024 bytes apart; 32 bytes per K step
                        const unsigned long long adesc = smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                        // B, K-major: same shape; N-major: 64-column panels 8192 bytes apart (leading),
                        // 8-row k groups 1024 bytes apart (stride); 16 k-rows = 2048 bytes per K step
                        const unsigned long long bdesc = p.b_is_kn ? smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                                                   : smem_desc(sb + k * (UMMA_K * 2), 16, 1024);
                        umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));          // frees the stage when these MMAs are done
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                umma_commit(acc_full_bar(acc));             // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
        int acc = 0;
        unsigned acc_phase = 0;
        int epi_buf = 0;
        const bool vec_ok = (p.c_rs % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && (p.c_bs % 8 == 0);
        for (long long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int b = (int)(tile / tiles_per_batch);
            const int r = (int)(tile % tiles_per_batch);
            int mt, nt;
            tc::banded_tile(r, p.tiles_m, p.tiles_n, p.band, mt, nt);
            const long long m0 = (long long)mt * BM, n0 = (long long)nt * BN;
            if (!mbar_wait(acc_full_bar(acc), acc_phase)) {
                if (lane == 0) atomicExch(p.error, 4u);
                break;
            }
            tc_fence_after();
            const long long m = m0 + quarter * 32 + lane;
            T* crow = C + (long long)b * p.c_bs + m * p.c_rs;
            if (p.use_tma_store) {
                // 64 columns at a time: TMEM -> registers -> this warp's staging tile in shared
                // memory (32 rows x 128 bytes, 128-byte swizzle) -> one TMA store of full 128-byte
                // rows.  Two staging tiles per warp alternate; out-of-range rows/columns are
                // clipped by the tensor map.
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    unsigned char* tile_smem = epi_smem + ((warp - 2) * 2 + epi_buf) * EPI_TILE_BYTES;
                    if (lane == 0) bulk_wait_read<1>();          // the tile used two stores ago has been read
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        unsigned v[32];
                        tmem_ld_32x32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c + half * 32), v);
                        tmem_ld_wait();
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
                    epi_buf ^= 1;
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                unsigned v[32];
                tmem_ld_32x32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c), v);
                tmem_ld_wait();
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (p.use_tma_store && lane == 0) bulk_wait_read<0>();   // shared memory stays valid until the stores have read it
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}


}  // namespace

bool matmul_tc_path(Device& dev, const void* a, const void* b, void* c, DType dt, const MatmulDims& d) {
    static const bool no_tc = getenv("WGF_MATMUL_NO_TC") != nullptr;            // diagnostic switches, read once
    static const bool no_tma_store = getenv("WGF_TC_NO_TMA_STORE") != nullptr;
    if (no_tc) return false;
    if (dt != DType::F16 && dt != DType::BF16) return false;
    // worth it only when a tile is reasonably full
    if (d.M < 64 || d.N < 64 || d.K < 32) return false;
    if (d.M >= (1ll << 31) || d.N >= (1ll << 31) || d.K >= (1ll << 31) || d.batch >= (1ll << 31)) return false;
    auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // A must be K-major with 16-byte aligned rows
    if (d.a_cs != 1 || d.a_rs % 8 || !a16(a) || (d.batch > 1 && d.a_bs % 8)) return false;
    const bool b_kn = d.b_cs == 1 && d.b_rs % 8 == 0;   // [K,N] row-major
    const bool b_nk = d.b_rs == 1 && d.b_cs % 8 == 0;   // [N,K] row-major (transposed view)
    if ((!b_kn && !b_nk) || !a16(b) || (d.batch > 1 && d.b_bs % 8)) return false;
    if (dev.dry) {
        dev.begin_launch("matmul_tc");
        dev.end_launch();
        return true;
    }
    const bool bf16 = dt == DType::BF16;
    CUtensorMap map_a, map_b;
    if (!encode_3d(&map_a, bf16, a, d.K, d.M, d.batch, d.a_rs, d.a_bs, BK, BM)) return false;
    const bool use_kn = b_kn;   // when both descriptions fit (a degenerate extent), either is right
    if (use_kn) {
        if (!encode_3d(&map_b, bf16, b, d.N, d.K, d.batch, d.b_rs, d.b_bs, 64, BK)) return false;
    } else {
        if (!encode_3d(&map_b, bf16, b, d.K, d.N, d.batch, d.b_cs, d.b_bs, BK, BN)) return false;
    }
    TcParams p{};
    p.M = d.M;
    p.N = d.N;
    p.K = d.K;
    p.batch = d.batch;
    p.c_rs = d.c_rs;
    p.c_bs = d.c_bs;
    p.tiles_m = (int)((d.M + BM - 1) / BM);
    p.tiles_n = (int)((d.N + BN - 1) / BN);
    p.b_is_kn = use_kn ? 1 : 0;
    p.is_bf16 = bf16 ? 1 : 0;
    // C through TMA when its rows are 16-byte aligned; otherwise guarded stores from registers
    CUtensorMap map_c = map_a;
    p.use_tma_store = 0;
    if (!no_tma_store && d.c_rs % 8 == 0 && (d.batch == 1 || d.c_bs % 8 == 0) && a16(c) &&
        encode_3d(&map_c, bf16, c, d.N, d.M, d.batch, d.c_rs, d.c_bs, 64, 32))
        p.use_tma_store = 1;
    p.error = dev.error_word();
    const long long total = (long long)p.tiles_m * p.tiles_n * d.batch;
    const unsigned grid = (unsigned)std::min<long long>(total, dev.sm_count);
    p.band = band_rows((int)grid, BM, BN, p.tiles_m);
    // the opt-in to the kernel's dynamic shared memory is a per-device attribute
    static std::mutex attr_mu;
    static bool attr_set[64][2];
    const void* fn = bf16 ? (const void*)matmul_tc_kernel<__nv_bfloat16> : (const void*)matmul_tc_kernel<__half>;
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        const int ord = dev.ordinal >= 0 && dev.ordinal < 64 ? dev.ordinal : -1;
        if (ord < 0 || !attr_set[ord][bf16 ? 1 : 0]) {
            WGF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            if (ord >= 0) attr_set[ord][bf16 ? 1 : 0] = true;
        }
    }
    dev.begin_launch("matmul_tc");
    if (bf16) matmul_tc_kernel<__nv_bfloat16><<<grid, TC_THREADS, SMEM_BYTES, dev.stream>>>(map_a, map_b, map_c, (__nv_bfloat16*)c, p);
    else matmul_tc_kernel<__half><<<grid, TC_THREADS, SMEM_BYTES, dev.stream>>>(map_a, map_b, map_c, (__half*)c, p);
    dev.end_launch();
    return true;
}

}  // namespace wgf
