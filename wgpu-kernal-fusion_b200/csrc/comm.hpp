// NCCL communicator for the one exchange the path has: the all-reduce that closes a
// full-tensor reduction whose rows are sharded over GPUs.  libnccl is loaded at run time.
#pragma once
#include "runtime.hpp"

namespace wgf {

struct Comm {
    void* handle = nullptr;  // ncclComm_t
    DeviceRef dev;
    int world = 1, rank = 0;
    // All-reduces of a few scalars done INSIDE the kernel that produces them, over peer memory
    // (NVLink stores), instead of a separate NCCL launch.  Every rank owns a mailbox of 64-bit
    // words {sequence number << 32 | value bits}, laid out [2 parities][world source ranks][4
    // values], and maps the peers' mailboxes through CUDA IPC.  The finishing CTA of the kernel
    // stores its value into its slot of every peer's mailbox and reads the others' values from
    // its own, accepting a word once it carries the sequence number of this all-reduce; ranks
    // are combined in rank order, so every rank gets the same bits.  Two parities suffice: a
    // rank cannot finish all-reduce k+1 before every peer has finished k.
    void* mailbox = nullptr;              // this rank's mailbox (device memory)
    std::vector<void*> peer_mailbox;      // [world]; the own entry is `mailbox`
    void* peer_table = nullptr;           // device array of the world mailbox addresses
    uint32_t seq = 0;                     // sequence number of the last in-kernel all-reduce
    bool peer_ok = false;                 // every rank mapped every peer
    ~Comm();
};
constexpr int kMailboxValues = 4;

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
