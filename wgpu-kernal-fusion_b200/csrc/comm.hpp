// NCCL communicator for the one exchange the path has: the all-reduce that closes a
// full-tensor reduction whose rows are sharded over GPUs.  libnccl is loaded at run time.
#pragma once
#include "runtime.hpp"

namespace wgf {

struct Comm {
    void* handle = nullptr;  // ncclComm_t
    DeviceRef dev;
    int world = 1, rank = 0;
    // All-reduces of a few scalars WITHOUT a collective launch, over peer memory.  Every rank owns
    // a mailbox of 64-bit words {sequence number << 32 | value bits}, laid out
    // [kMailboxSlots][world source ranks][kMailboxValues], and maps the peers' mailboxes through
    // CUDA IPC.  The exchange has two halves.  (1) The finishing CTA of the kernel that produces
    // the values POSTS them: one 64-bit store per rank (NVLink stores for the peers, a local one
    // for itself) into slot `sequence % kMailboxSlots`; it waits for nothing, so the kernels
    // queued behind it start at once.  (2) A one-CTA kernel on the device's collective stream
    // waits (bounded: wait_ns) until its own mailbox holds every rank's word with this sequence
    // number, combines them in rank order -- every rank gets the same bits -- and writes the
    // results; the result buffers carry its completion event (Buffer::pending), so only their
    // readers wait for it.
    // A slot is reused every kMailboxSlots exchanges.  A rank's device stream may not run further
    // ahead than kMailboxLag exchanges of its own combine kernels (the stream waits for the
    // event of exchange k - kMailboxLag before the kernel that posts exchange k): when rank A
    // posts k, its combine k - Lag has seen every peer's post k - Lag, so every peer's combine
    // k - 2 Lag is over, and with kMailboxSlots >= 2 kMailboxLag the word that post k replaces
    // has been read.
    void* mailbox = nullptr;              // this rank's mailbox (device memory)
    std::vector<void*> peer_mailbox;      // [world]; the own entry is `mailbox`
    void* peer_table = nullptr;           // device array of the world mailbox addresses
    uint32_t seq = 0;                     // sequence number of the last exchange
    bool peer_ok = false;                 // every rank mapped every peer
    uint64_t wait_ns = 5000000000ull;     // limit of the combine kernel's wait (WGF_PEER_WAIT_MS)
    std::vector<cudaEvent_t> finished;    // [kMailboxSlots] completion events of the combine kernels (also the results' Buffer::pending)
    std::vector<cudaEvent_t> posted;      // [kMailboxSlots] "the posting kernel is queued" events
    ~Comm();
};
constexpr int kMailboxValues = 4;
constexpr int kMailboxSlots = 16;
constexpr int kMailboxLag = 8;
static_assert(kMailboxSlots >= 2 * kMailboxLag, "a slot must have been read before it is posted to again");

// One value of an exchange: how the ranks are combined and where the result goes (a rank-0 tensor).
struct PeerValue {
    uint16_t op;
    uint32_t index;    // which of the kMailboxValues words of a slot the posting kernel used
    TensorData out;
};
// Starts exchange number `seq` (returned): keeps the device stream within kMailboxLag exchanges of
// this rank's combine kernels.  Call before launching the kernel that posts.
uint32_t comm_peer_begin(Comm& c, Device& dev);
// Queues the combine kernel of exchange `seq` on the collective stream, behind everything queued on
// the device stream so far (the posting kernel), and marks the result buffers pending on it.
void comm_peer_finish(Comm& c, Device& dev, uint32_t seq, const std::vector<PeerValue>& vals);
void launch_peer_combine(cudaStream_t stream, const void* mailbox, unsigned* err, uint64_t wait_ns, uint32_t world,
                         uint32_t rank, uint32_t seq, const std::vector<PeerValue>& vals);

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
