#include "comm.hpp"

#include <dlfcn.h>

#include <cstdlib>

namespace wgf {

namespace {
// The part of the NCCL ABI used here (nccl.h: ncclUniqueId is 128 opaque bytes;
// ncclDataType_t: float32 = 7, float16 = 6, bfloat16 = 9; ncclRedOp_t: sum 0, prod 1, max 2, min 3).
struct NcclId { char internal[128]; };
struct Nccl {
    int (*GetUniqueId)(NcclId*);
    int (*CommInitRank)(void**, int, NcclId, int);
    int (*CommDestroy)(void*);
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t);
    const char* (*GetErrorString)(int);
    static Nccl& get() {
        static Nccl n = [] {
            Nccl v{};
            std::vector<std::string> names;
            if (const char* p = getenv("WGF_NCCL_PATH")) names.push_back(p);
            names.push_back("libnccl.so.2");
            names.push_back("libnccl.so");
            void* h = nullptr;
            for (auto& nm : names)
                if ((h = dlopen(nm.c_str(), RTLD_NOW | RTLD_GLOBAL))) break;
            if (!h) fail(WGF_ERR_NCCL, "cannot load libnccl.so.2 (set WGF_NCCL_PATH)");
            auto sym = [&](const char* s) {
                void* p = dlsym(h, s);
                if (!p) fail(WGF_ERR_NCCL, std::string("NCCL symbol missing: ") + s);
                return p;
            };
            v.GetUniqueId = (decltype(v.GetUniqueId))sym("ncclGetUniqueId");
            v.CommInitRank = (decltype(v.CommInitRank))sym("ncclCommInitRank");
            v.CommDestroy = (decltype(v.CommDestroy))sym("ncclCommDestroy");
            v.AllReduce = (decltype(v.AllReduce))sym("ncclAllReduce");
            v.AllGather = (decltype(v.AllGather))sym("ncclAllGather");
            v.GetErrorString = (decltype(v.GetErrorString))sym("ncclGetErrorString");
            return v;
        }();
        return n;
    }
};
void nccl_check(int r, const char* what) {
    if (r != 0) fail(WGF_ERR_NCCL, std::string(what) + ": " + Nccl::get().GetErrorString(r));
}
}  // namespace

Comm::~Comm() {
    if (dev && !dev->dry) cudaSetDevice(dev->ordinal);
    if (dev && (!posted.empty() || produced.seq)) {
        // results of the last exchanges are still this rank's own values: finish them while the
        // mailboxes exist
        try {
            comm_settle(*this, *dev);
        } catch (...) {
        }
        if (!dev->dry) cudaStreamSynchronize(dev->stream);
    }
    for (int r = 0; r < (int)peer_mailbox.size(); ++r)
        if (r != rank && peer_mailbox[r]) cudaIpcCloseMemHandle(peer_mailbox[r]);
    if (peer_table) cudaFree(peer_table);
    if (mailbox) cudaFree(mailbox);
    if (handle) Nccl::get().CommDestroy(handle);
}

namespace {
// Device scratch that is freed on every way out of setup_mailboxes.
struct DeviceScratch {
    void* p = nullptr;
    ~DeviceScratch() {
        if (p) cudaFree(p);
    }
};

// Maps every peer's mailbox (see Comm).  Anything that does not work leaves peer_ok false on
// EVERY rank (the outcome is agreed through an all-reduce), and all-reduces go through NCCL.
// Between the all-gather and the agreeing all-reduce a local CUDA failure only clears `ok`: a
// rank that threw there would leave the others waiting inside the collective.
void setup_mailboxes(Comm& c) {
    // one warp of the settling code holds the ranks' words, one per lane
    // (a communicator of one rank takes this path only when asked to: a way to time the exchange's
    // code without a second GPU)
    if ((c.world < 2 && !getenv("WGF_PEER_SINGLE_RANK")) || c.world > 32 || getenv("WGF_NO_PEER_ALLREDUCE")) return;
    Device& dev = *c.dev;
    if (const char* ms = getenv("WGF_PEER_WAIT_MS")) {
        const long long v = atoll(ms);
        if (v > 0) c.wait_ns = (uint64_t)v * 1000000ull;
    }
    const size_t box_bytes = (size_t)kMailboxSlots * c.world * kMailboxValues * sizeof(uint64_t);
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    DeviceScratch gather, flag;   // gather: [world + 1] handles, slot `world` is the send buffer
    WGF_CUDA(cudaMalloc(&gather.p, hb * (c.world + 1)));
    WGF_CUDA(cudaMalloc(&flag.p, sizeof(int)));
    int ok = 1;
    cudaIpcMemHandle_t mine{};
    if (cudaMalloc(&c.mailbox, box_bytes) != cudaSuccess || cudaMemset(c.mailbox, 0, box_bytes) != cudaSuccess ||
        cudaIpcGetMemHandle(&mine, c.mailbox) != cudaSuccess)
        ok = 0;
    if (cudaMemcpy((char*)gather.p + hb * c.world, &mine, hb, cudaMemcpyHostToDevice) != cudaSuccess) ok = 0;
    nccl_check(Nccl::get().AllGather((char*)gather.p + hb * c.world, gather.p, hb, /*ncclInt8*/ 0, c.handle, dev.stream),
               "ncclAllGather");
    std::vector<cudaIpcMemHandle_t> all(c.world);
    if (cudaMemcpyAsync(all.data(), gather.p, hb * c.world, cudaMemcpyDeviceToHost, dev.stream) != cudaSuccess ||
        cudaStreamSynchronize(dev.stream) != cudaSuccess)
        ok = 0;
    c.peer_mailbox.assign(c.world, nullptr);
    for (int r = 0; r < c.world && ok; ++r) {
        if (r == c.rank) {
            c.peer_mailbox[r] = c.mailbox;
        } else if (cudaIpcOpenMemHandle(&c.peer_mailbox[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            c.peer_mailbox[r] = nullptr;
            ok = 0;
        }
    }
    if (ok) {
        std::vector<uint64_t> table(c.world);
        for (int r = 0; r < c.world; ++r) table[r] = (uint64_t)(uintptr_t)c.peer_mailbox[r];
        if (cudaMalloc(&c.peer_table, sizeof(uint64_t) * c.world) != cudaSuccess ||
            cudaMemcpy(c.peer_table, table.data(), sizeof(uint64_t) * c.world, cudaMemcpyHostToDevice) != cudaSuccess)
            ok = 0;
    }
    if (cudaMemcpy(flag.p, &ok, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) ok = 0;
    cudaGetLastError();   // a failed mapping is not an error of the library: NCCL takes over
    // every rank must take the same path: minimum of the outcomes (a rank whose copy above failed
    // contributes whatever the word holds, and reads its own `ok` = 0 below)
    nccl_check(Nccl::get().AllReduce(flag.p, flag.p, 1, /*ncclInt32*/ 2, /*ncclMin*/ 3, c.handle, dev.stream), "ncclAllReduce");
    int agreed = 0;
    WGF_CUDA(cudaMemcpyAsync(&agreed, flag.p, sizeof(int), cudaMemcpyDeviceToHost, dev.stream));
    WGF_CUDA(cudaStreamSynchronize(dev.stream));
    c.peer_ok = ok != 0 && agreed != 0;
}
}  // namespace

void comm_unique_id(uint8_t id[WGF_COMM_ID_BYTES]) {
    static_assert(WGF_COMM_ID_BYTES == sizeof(NcclId), "id size");
    NcclId nid;
    nccl_check(Nccl::get().GetUniqueId(&nid), "ncclGetUniqueId");
    std::memcpy(id, &nid, sizeof nid);
}

std::shared_ptr<Comm> comm_create(const DeviceRef& dev, int world, int rank, const uint8_t id[WGF_COMM_ID_BYTES]) {
    WGF_CHECK(world >= 1 && rank >= 0 && rank < world, WGF_ERR_INVALID_ARGUMENT, "bad world size / rank");
    auto c = std::make_shared<Comm>();
    c->dev = dev;
    c->world = world;
    c->rank = rank;
    if (dev->dry) {
        // Compile-only device: no NCCL, no memory.  The communicator takes the peer-memory path, so that
        // the kernels of that path are compiled and its host-side bookkeeping runs without a GPU.
        c->peer_ok = getenv("WGF_NO_PEER_ALLREDUCE") == nullptr;
        return c;
    }
    dev->make_current();
    NcclId nid;
    std::memcpy(&nid, id, sizeof nid);
    nccl_check(Nccl::get().CommInitRank(&c->handle, world, nid, rank), "ncclCommInitRank");
    setup_mailboxes(*c);
    dev->exchange_broken = false;   // fresh mailboxes and sequence numbers
    return c;
}

void comm_all_reduce(Comm& c, Device& dev, Buffer& out, void* data, int64_t count, DType dt, uint16_t op) {
    int ndt = dt == DType::F32 ? 7 : dt == DType::F16 ? 6 : 9;
    int nop = op == WGF_OP_SUM ? 0 : op == WGF_OP_PRODUCT ? 1 : op == WGF_OP_MAX ? 2 : 3;
    void* recv = data;
    if (dev.dry) {
        dev.launches++;
        return;
    }
    dev.make_current();
    dev.wait_for(out);
    cudaStream_t cs = dev.collective_stream();
    dev.begin_launch("all_reduce");
    // The collective runs IN PLACE on the buffer that holds the partial result, on the
    // collective stream, behind everything queued on the device stream so far; the kernels
    // queued after it on the device stream overlap it.  The buffer carries the completion
    // event: its next reader, and the pool when it is returned, wait for it (Buffer::pending).
    cudaEvent_t produced = dev.event();
    WGF_CUDA(cudaEventRecord(produced, dev.stream));
    WGF_CUDA(cudaStreamWaitEvent(cs, produced, 0));
    dev.recycle(produced);
    int r = Nccl::get().AllReduce(recv, recv, (size_t)count, ndt, nop, c.handle, cs);
    dev.end_launch();
    nccl_check(r, "ncclAllReduce");
    out.pending = dev.event();
    WGF_CUDA(cudaEventRecord(out.pending, cs));
}

uint32_t peer_value_meta(const PeerValue& v) {
    const uint32_t op = v.op == WGF_OP_SUM ? 0u : v.op == WGF_OP_PRODUCT ? 1u : v.op == WGF_OP_MAX ? 2u : 3u;
    return op | ((uint32_t)v.out.dtype << 8) | (v.index << 16);
}

namespace {
void unmark(Comm& c, Comm::Exchange& e) {
    for (const PeerValue& v : e.vals)
        if (v.out.buf->unsettled == &c) v.out.buf->unsettled = nullptr;
    e.vals.clear();
    e.seq = 0;
}
}  // namespace

GrandComm comm_peer_begin(Comm& c, Device& dev) {
    // one communicator per device has open exchanges at a time
    if (dev.unsettled_comm && dev.unsettled_comm != &c) comm_settle(*dev.unsettled_comm, dev);
    GrandComm g{};
    g.peer_table = c.peer_table;
    g.world = (uint32_t)c.world;
    g.rank = (uint32_t)c.rank;
    g.seq = ++c.seq;
    g.mailbox = c.mailbox;
    g.wait_ns = c.wait_ns;
    // the oldest posted exchange is settled by this kernel once it is kMailboxLag kernels old
    if ((int)c.posted.size() >= kMailboxLag - 1) {
        const Comm::Exchange& old = c.posted.front();
        g.prev_seq = old.seq;
        g.prev_n = (uint32_t)old.vals.size();
        for (uint32_t i = 0; i < g.prev_n; ++i) {
            g.prev_meta[i] = peer_value_meta(old.vals[i]);
            g.prev_out[i] = old.vals[i].out.base_ptr();
        }
    }
    g.post_seq = c.produced.seq;
    g.post_n = c.produced.seq ? (uint32_t)c.produced.vals.size() : 0u;
    for (uint32_t i = 0; i < g.post_n; ++i) {
        g.post_meta[i] = peer_value_meta(c.produced.vals[i]);
        g.post_src[i] = c.produced.vals[i].out.base_ptr();
    }
    return g;
}

void comm_peer_finish(Comm& c, Device& dev, uint32_t seq, const std::vector<PeerValue>& vals) {
    WGF_CHECK(!vals.empty() && vals.size() <= (size_t)kMailboxValues, WGF_ERR_INVALID_ARGUMENT, "exchange of 1..4 values");
    if ((int)c.posted.size() >= kMailboxLag - 1) {
        unmark(c, c.posted.front());   // the kernel just queued settles it; later work on the device stream sees the results
        c.posted.pop_front();
    }
    if (c.produced.seq) c.posted.push_back(std::move(c.produced));
    c.produced = Comm::Exchange{};
    c.produced.seq = seq;
    c.produced.vals = vals;
    for (const PeerValue& v : vals) v.out.buf->unsettled = &c;
    dev.unsettled_comm = &c;
}

void comm_settle(Comm& c, Device& dev) {
    if (c.posted.empty() && !c.produced.seq) return;
    std::deque<Comm::Exchange> posted;
    Comm::Exchange produced;
    posted.swap(c.posted);
    std::swap(produced, c.produced);
    std::vector<const Comm::Exchange*> todo;
    for (const Comm::Exchange& e : posted) todo.push_back(&e);
    if (produced.seq) todo.push_back(&produced);
    for (const Comm::Exchange* e : todo)
        for (const PeerValue& v : e->vals)
            if (v.out.buf->unsettled == &c) v.out.buf->unsettled = nullptr;
    if (dev.unsettled_comm == &c) dev.unsettled_comm = nullptr;
    dev.launches++;
    if (dev.dry) return;
    dev.make_current();
    launch_peer_flush(dev.stream, c, dev.error_word(), produced.seq ? &produced : nullptr, todo.data(), (int)todo.size());
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(WGF_ERR_CUDA, std::string("peer flush launch failed: ") + cudaGetErrorString(e));
    }
}

}  // namespace wgf
