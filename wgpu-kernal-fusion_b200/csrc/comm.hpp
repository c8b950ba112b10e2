// NCCL communicator for the one exchange the path has: the all-reduce that closes a
// full-tensor reduction whose rows are sharded over GPUs.  libnccl is loaded at run time.
#pragma once
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
    // CUDA IPC.  The exchange has two halves.  (1) The finishing CTA of the kernel that produces
    // the values POSTS them: one 64-bit store per rank (NVLink stores for the peers, a local one
    // for itself) into slot `sequence % kMailboxSlots`; it waits for nothing.  The result buffers
    // hold this rank's own values from then on and are marked Buffer::unsettled; the exchange is
    // `open`.  (2) SETTLING: wait (bounded: wait_ns) until the own mailbox holds every rank's word
    // with this sequence number, combine them in rank order -- every rank gets the same bits --
    // and overwrite the results.  The next kernel that posts on this communicator does it for the
    // open exchange, in its finishing CTA after its own post: ranks that run the same program have
    // posted the earlier exchange long before, so a step costs one launch and its stream never
    // stops for a peer.  If a result is read first (Device::wait_for), the device synchronised or a
    // schedule recorded, a one-CTA kernel on the device stream settles the open exchange instead.
    //
    // A slot is reused every kMailboxSlots exchanges, with no further gate.  On every rank the
    // stream order is post(j) < settle(j) < post(j+2) (exchange j is settled by the kernel that
    // posts j+1 at the latest), and settle(j) ends only after every peer's post(j) has arrived.
    // When rank A posts k, its settle(k-2) is over, so every peer had posted k-2, so every peer's
    // kernel of exchange k-3 had ended, and with it the peer's settle(k-4): the peers have read
    // every exchange up to k-4, and the word of exchange k-16 that post k replaces is long dead.
    void* mailbox = nullptr;              // this rank's mailbox (device memory)
    std::vector<void*> peer_mailbox;      // [world]; the own entry is `mailbox`
    void* peer_table = nullptr;           // device array of the world mailbox addresses
    uint32_t seq = 0;                     // sequence number of the last exchange
    bool peer_ok = false;                 // every rank mapped every peer
    uint64_t wait_ns = 5000000000ull;     // limit of a settling wait (WGF_PEER_WAIT_MS)
    uint32_t open_seq = 0;                // the posted exchange that is not settled yet (0: none) ...
    std::vector<PeerValue> open_vals;     // ... and its results
    ~Comm();
};
constexpr int kMailboxValues = 4;
constexpr int kMailboxSlots = 16;
static_assert(kMailboxSlots >= 5, "a slot must have been read before it is posted to again");

// Starts the next exchange: the sequence number and mailboxes for the kernel that posts, and the open
// exchange for it to settle.  Call before launching that kernel.
GrandComm comm_peer_begin(Comm& c, Device& dev);
// After the posting kernel has been queued: the exchange it settled is closed, `vals` (its own results,
// holding this rank's values for now) become the open one.
void comm_peer_finish(Comm& c, Device& dev, uint32_t seq, const std::vector<PeerValue>& vals);
// Settles the open exchange, if any, with a kernel of its own on the device stream
// (declared in runtime.hpp too: Device::wait_for and Device::sync call it).
void comm_settle(Comm& c, Device& dev);
void launch_peer_combine(cudaStream_t stream, const void* mailbox, unsigned* err, uint64_t wait_ns, uint32_t world,
                         uint32_t rank, uint32_t seq, const std::vector<PeerValue>& vals);
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
