// Second half of the all-reduce of a few scalars over peer memory (see Comm) as a kernel of its
// own: one CTA waits for the words that every rank posted into this GPU's mailbox, combines them in
// rank order (so every rank ends with the same bits) and writes the results.  Used when a result is
// read before the next posting kernel, which would otherwise do the same in its finishing CTA
// (peer_settle in jit_templates.hpp), has been queued.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "comm.hpp"

namespace wgf {
namespace {

struct CombineParams {
    const unsigned long long* mailbox;   // this GPU's mailbox
    unsigned* err;                       // device error word
    unsigned long long wait_ns;          // limit of the wait for a peer's word
    unsigned world, rank, seq, nvals;
    unsigned index[kMailboxValues];      // word of the slot that holds this value
    unsigned op[kMailboxValues];         // WGF_OP_SUM / MAX / MIN / PRODUCT
    unsigned dtype[kMailboxValues];      // 0 f32, 1 f16, 2 bf16
    void* out[kMailboxValues];
};

__device__ __forceinline__ float combine(unsigned op, float a, float b) {
    switch (op) {
        case WGF_OP_SUM: return a + b;
        case WGF_OP_PRODUCT: return a * b;
        case WGF_OP_MAX: return fmaxf(a, b);
        default: return fminf(a, b);
    }
}

// Warp w serves value w; lane l waits for the words of ranks l, l + 32, ...  A wait that runs
// out sets the error word (51) and leaves this GPU's own value as the result: the kernel always
// returns, and the host sees WGF_ERR_TIMEOUT at its next synchronisation.
__global__ void __launch_bounds__(32 * kMailboxValues) peer_combine_kernel(const CombineParams p) {
    const unsigned v = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (v >= p.nvals) return;
    const unsigned long long* base = p.mailbox + (unsigned long long)((p.seq % kMailboxSlots) * p.world) * kMailboxValues + p.index[v];
    bool all_here = true;
    unsigned long long start = 0;
    for (unsigned r = lane; r < p.world; r += 32) {
        const unsigned long long* slot = base + (unsigned long long)r * kMailboxValues;
        unsigned long long w = 0;
        bool got = false;
        for (unsigned spin = 0; spin < (1u << 30) && !got; ++spin) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(slot) : "memory");
            got = (unsigned)(w >> 32) == p.seq;
            if (!got && (spin & 63u) == 63u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (start == 0) start = now;
                else if (now - start > p.wait_ns) break;
            }
        }
        all_here = all_here && got;
    }
    all_here = __all_sync(0xffffffffu, all_here);
    float acc = 0.f;
    if (lane == 0) {
        // every word is in this GPU's memory now (or the wait ran out): read them in rank order
        const unsigned long long mine = base[(unsigned long long)p.rank * kMailboxValues];
        if (!all_here) {
            atomicExch(p.err, 51u);
            acc = __uint_as_float((unsigned)mine);
        } else {
            for (unsigned r = 0; r < p.world; ++r) {
                unsigned long long w;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(base + (unsigned long long)r * kMailboxValues) : "memory");
                const float x = __uint_as_float((unsigned)w);
                acc = r == 0 ? x : combine(p.op[v], acc, x);
            }
        }
        switch (p.dtype[v]) {
            case 0: *(float*)p.out[v] = acc; break;
            case 1: *(__half*)p.out[v] = __float2half_rn(acc); break;
            default: *(__nv_bfloat16*)p.out[v] = __float2bfloat16_rn(acc); break;
        }
    }
}

}  // namespace

void launch_peer_combine(cudaStream_t stream, const void* mailbox, unsigned* err, uint64_t wait_ns, uint32_t world,
                         uint32_t rank, uint32_t seq, const std::vector<PeerValue>& vals) {
    CombineParams p{};
    p.mailbox = (const unsigned long long*)mailbox;
    p.err = err;
    p.wait_ns = wait_ns;
    p.world = world;
    p.rank = rank;
    p.seq = seq;
    p.nvals = (unsigned)vals.size();
    for (size_t i = 0; i < vals.size(); ++i) {
        p.index[i] = vals[i].index;
        p.op[i] = vals[i].op;
        p.dtype[i] = (unsigned)vals[i].out.dtype;
        p.out[i] = vals[i].out.base_ptr();
    }
    peer_combine_kernel<<<1, 32 * kMailboxValues, 0, stream>>>(p);
}

}  // namespace wgf
