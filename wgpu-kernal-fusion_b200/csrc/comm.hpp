// NCCL communicator for the one exchange the path has: the all-reduce that closes a
// full-tensor reduction whose rows are sharded over GPUs.  libnccl is loaded at run time.
#pragma once
#include <deque>

#include "launch.hpp"
#include "runtime.hpp"

namespace wgf {

// One value of an exchange: how the ranks are combined and where the result goes (a rank-0 tensor).
struct PeerValue {
    uint16_t op;
    uint32_t index;    // which of the kMailboxValues words of a slot the posting kernel used
    TensorData out;
};

struct Comm {
    void* handle = nullptr;  // ncclComm_t
    DeviceRef dev;
    int world = 1, rank = 0;
    // All-reduces of a few scalars WITHOUT a collective launch, over peer memory.  Every rank owns
    // a mailbox of 64-bit words {sequence number << 32 | value bits}, laid out
    // [kMailboxSlots][world source ranks][kMailboxValues], and maps the peers' mailboxes through
    // CUDA IPC.  An exchange goes through three stages, each done by a kernel of this path on the
    // device stream, so that a step of a loop costs one launch and its stream never stops for a peer
    // that is less than kMailboxLag - 1 kernels behind:
    //   produced  kernel k (the one that computes the values) stores this rank's values in the
    //             result buffers, which are marked Buffer::unsettled from then on;
    //   posted    kernel k+1 reads them back first thing and stores one word per value into
    //             slot `k % kMailboxSlots` of every rank's mailbox (NVLink stores for the peers, a
    //             local one for itself); it waits for nothing;
    //   settled   one CTA of kernel k+kMailboxLag waits (bounded: wait_ns) until the own mailbox
    //             holds every rank's word of exchange k, combines them in rank order -- every rank
    //             gets the same bits -- and overwrites the results.  Ranks that run the same
    //             program posted k several kernels earlier, so nothing waits: the CTA asks for the
    //             words when it starts and takes them when it is done with its own rows.  The lag
    //             is what lets ranks drift apart: a rank whose host stalls for a moment holds the
    //             others up only once they are kMailboxLag - 1 kernels ahead of it, so stalls of
    //             different ranks overlap instead of adding up.
    // If a result is read first (Device::wait_for), the device synchronised or a schedule recorded,
    // a one-CTA kernel on the device stream does what is left for the open exchanges (comm_settle).
    //
    // A slot is reused every kMailboxSlots exchanges, with no further gate.  On every rank the
    // stream order is produce(j) < post(j) < settle(j), and settle(j) ends before kernel j+Lag
    // does; settle(j) ends only after every peer's post(j) has arrived.  When rank A posts j, its
    // kernel j has ended, so its settle(j-Lag) is over, so every peer had posted j-Lag, so every
    // peer's kernel j-Lag had ended, and with it the peer's settle(j-2 Lag): the peers have read
    // every exchange up to j-2 Lag, and with kMailboxSlots >= 2 kMailboxLag + 1 the word of
    // exchange j-kMailboxSlots that post j replaces is dead.
    void* mailbox = nullptr;              // this rank's mailbox (device memory)
    std::vector<void*> peer_mailbox;      // [world]; the own entry is `mailbox`
    void* peer_table = nullptr;           // device array of the world mailbox addresses
    uint32_t seq = 0;                     // sequence number of the last exchange
    bool peer_ok = false;                 // every rank mapped every peer
    uint64_t wait_ns = 5000000000ull;     // limit of a settling wait (WGF_PEER_WAIT_MS)
    struct Exchange {
        uint32_t seq = 0;                 // 0: none
        std::vector<PeerValue> vals;      // its results (keeps the buffers alive)
    };
    Exchange produced;                    // values stored, not posted
    std::deque<Exchange> posted;          // posted, not settled, oldest first (at most kMailboxLag - 1)
    ~Comm();
};
constexpr int kMailboxValues = 4;
constexpr int kMailboxSlots = 16;
constexpr int kMailboxLag = 6;
static_assert(kMailboxSlots >= 2 * kMailboxLag + 1, "a slot must have been read before it is posted to again");

// Starts the next exchange: its sequence number, and the two open exchanges that the kernel which
// produces it posts and settles.  Call before launching that kernel.
GrandComm comm_peer_begin(Comm& c, Device& dev);
// After that kernel has been queued: the exchange it settled is closed, the one it posted waits to be
// settled, and `vals` (the kernel's own results, holding this rank's values for now) wait to be posted.
void comm_peer_finish(Comm& c, Device& dev, uint32_t seq, const std::vector<PeerValue>& vals);
// Finishes the open exchanges, if any, with a kernel of its own on the device stream
// (declared in runtime.hpp too: Device::wait_for and Device::sync call it).
void comm_settle(Comm& c, Device& dev);
// The kernel of comm_settle: posts `post` (if not null), then settles the `n` exchanges of `settle` in order.
void launch_peer_flush(cudaStream_t stream, const Comm& c, unsigned* err, const Comm::Exchange* post,
                       const Comm::Exchange* const* settle, int n);
// op | dtype << 8 | value index << 16, as the settling code reads it
uint32_t peer_value_meta(const PeerValue& v);

void comm_unique_id(uint8_t id[WGF_COMM_ID_BYTES]);
std::shared_ptr<Comm> comm_create(const DeviceRef& dev, int world, int rank, const uint8_t id[WGF_COMM_ID_BYTES]);
// In place on `data`, which lies in `out`.  The collective runs on the device's collective stream
// behind everything queued on the device stream so far; `out.pending` is set to its completion event.
void comm_all_reduce(Comm& c, Device& dev, Buffer& out, void* data, int64_t count, DType dt, uint16_t op);

// Contiguous block partition: the first n % world ranks get one unit more.
inline void shard_range(int64_t n, int world, int rank, int64_t& begin, int64_t& end) {
    int64_t base = n / world, extra = n % world;
    begin = rank * base + (rank < extra ? rank : extra);
    end = begin + base + (rank < extra ? 1 : 0);
}

}  // namespace wgf
