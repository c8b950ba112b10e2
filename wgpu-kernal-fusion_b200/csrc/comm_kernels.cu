// The all-reduce of a few scalars over peer memory (see Comm) as a kernel of its own: one CTA
// does whatever is left of the communicator's open exchanges -- posts this GPU's values of the one
// that is only produced, then waits for the words that every rank posted into this GPU's mailbox,
// combines them in rank order (so every rank ends with the same bits) and writes the results.
// Used when a result is read before the kernels of the following steps, which would otherwise do the
// same work on their way (peer_post / peer_settle in jit_templates.hpp), have been queued.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "comm.hpp"

namespace wgf {
namespace {

struct ExchangeParams {
    unsigned seq, n;                     // n == 0: nothing to do
    unsigned meta[kMailboxValues];       // op code | dtype << 8 | word of the slot << 16 (peer_value_meta)
    void* buf[kMailboxValues];           // the result buffers
};
struct FlushParams {
    const unsigned long long* mailbox;   // this GPU's mailbox
    const unsigned long long* peers;     // device array of every rank's mailbox address
    unsigned* err;                       // device error word
    unsigned long long wait_ns;          // limit of the wait for a peer's word
    unsigned world, rank;
    unsigned n_settle;
    ExchangeParams post, settle[kMailboxLag];
};

__device__ __forceinline__ float combine(unsigned op, float a, float b) {
    return op == 0 ? a + b : op == 1 ? a * b : op == 2 ? fmaxf(a, b) : fminf(a, b);
}
__device__ __forceinline__ float read_as(unsigned dt, const void* p) {
    return dt == 0 ? *(const float*)p : dt == 1 ? __half2float(*(const __half*)p) : __bfloat162float(*(const __nv_bfloat16*)p);
}
__device__ __forceinline__ unsigned long long word_at(unsigned seq, unsigned world, unsigned r, unsigned index) {
    return (unsigned long long)((seq % kMailboxSlots) * world + r) * kMailboxValues + index;
}

// One warp settles value v of exchange e; lane l waits for the words of ranks l, l + 32, ...  A
// wait that runs out sets the error word (51) and leaves this GPU's own value as the result: the
// kernel always returns, and the host sees WGF_ERR_TIMEOUT at its next synchronisation.
__device__ void settle(const FlushParams& p, const ExchangeParams& e, unsigned v) {
    const unsigned lane = threadIdx.x & 31;
    const unsigned op = e.meta[v] & 255u, dt = (e.meta[v] >> 8) & 255u, index = e.meta[v] >> 16;
    bool all_here = true;
    unsigned long long start = 0;
    for (unsigned r = lane; r < p.world; r += 32) {
        const unsigned long long* slot = p.mailbox + word_at(e.seq, p.world, r, index);
        unsigned long long w = 0;
        bool got = false;
        for (unsigned spin = 0; spin < (1u << 30) && !got; ++spin) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(slot) : "memory");
            got = (unsigned)(w >> 32) == e.seq;
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
    if (lane != 0) return;
    if (!all_here) {          // the buffer keeps this GPU's own value
        atomicExch(p.err, 51u);
        return;
    }
    // every word is in this GPU's memory now: read them in rank order
    float acc = 0.f;
    for (unsigned r = 0; r < p.world; ++r) {
        unsigned long long w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p.mailbox + word_at(e.seq, p.world, r, index)) : "memory");
        const float x = __uint_as_float((unsigned)w);
        acc = r == 0 ? x : combine(op, acc, x);
    }
    if (dt == 0) *(float*)e.buf[v] = acc;
    else if (dt == 1) *(__half*)e.buf[v] = __float2half_rn(acc);
    else *(__nv_bfloat16*)e.buf[v] = __float2bfloat16_rn(acc);
}

__global__ void __launch_bounds__(32 * kMailboxValues) peer_flush_kernel(const FlushParams p) {
    if (threadIdx.x < p.post.n) {
        const unsigned m = p.post.meta[threadIdx.x];
        const float mine = read_as((m >> 8) & 255u, p.post.buf[threadIdx.x]);
        const unsigned long long word = ((unsigned long long)p.post.seq << 32) | (unsigned long long)__float_as_uint(mine);
        const unsigned long long at = word_at(p.post.seq, p.world, p.rank, m >> 16);
        for (unsigned r = 0; r < p.world; ++r)
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"((unsigned long long*)p.peers[r] + at), "l"(word) : "memory");
    }
    __syncthreads();   // the values have been read before a settle below overwrites them
    // the (exchange, value) pairs go round the four warps: they are independent of one another
    const unsigned warp = threadIdx.x >> 5;
    unsigned q = 0;
    for (unsigned i = 0; i < p.n_settle; ++i)
        for (unsigned v = 0; v < p.settle[i].n; ++v, ++q)
            if (q % kMailboxValues == warp) settle(p, p.settle[i], v);
}

void fill(ExchangeParams& e, const Comm::Exchange* x) {
    e = ExchangeParams{};
    if (!x) return;
    e.seq = x->seq;
    e.n = (unsigned)x->vals.size();
    for (size_t i = 0; i < x->vals.size(); ++i) {
        e.meta[i] = peer_value_meta(x->vals[i]);
        e.buf[i] = x->vals[i].out.base_ptr();
    }
}

}  // namespace

void launch_peer_flush(cudaStream_t stream, const Comm& c, unsigned* err, const Comm::Exchange* post,
                       const Comm::Exchange* const* settle_list, int n) {
    FlushParams p{};
    p.mailbox = (const unsigned long long*)c.mailbox;
    p.peers = (const unsigned long long*)c.peer_table;
    p.err = err;
    p.wait_ns = c.wait_ns;
    p.world = (unsigned)c.world;
    p.rank = (unsigned)c.rank;
    fill(p.post, post);
    p.n_settle = (unsigned)(n < kMailboxLag ? n : kMailboxLag);   // never more: kMailboxLag - 1 posted + 1 produced
    for (unsigned i = 0; i < p.n_settle; ++i) fill(p.settle[i], settle_list[i]);
    peer_flush_kernel<<<1, 32 * kMailboxValues, 0, stream>>>(p);
}

}  // namespace wgf
