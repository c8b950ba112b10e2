// NCCL communicator for the one exchange the path has: the all-reduce that closes a
// full-tensor reduction whose rows are sharded over GPUs.  libnccl is loaded at run time.
#pragma once
#include "runtime.hpp"

namespace wgf {

struct Comm {
    void* handle = nullptr;  // ncclComm_t
    DeviceRef dev;
    int world = 1, rank = 0;
    ~Comm();
};

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
