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
    if (dev) cudaSetDevice(dev->ordinal);
    for (int r = 0; r < (int)peer_mailbox.size(); ++r)
        if (r != rank && peer_mailbox[r]) cudaIpcCloseMemHandle(peer_mailbox[r]);
    if (peer_table) cudaFree(peer_table);
    if (mailbox) cudaFree(mailbox);
    if (handle) Nccl::get().CommDestroy(handle);
}

namespace {
// Maps every peer's mailbox (see Comm).  Anything that does not work leaves peer_ok false on
// EVERY rank (the outcome is agreed through an all-reduce), and all-reduces go through NCCL.
void setup_mailboxes(Comm& c) {
    if (c.world < 2 || c.world > 64 || getenv("WGF_NO_PEER_ALLREDUCE")) return;
    Device& dev = *c.dev;
    const size_t box_bytes = (size_t)2 * c.world * kMailboxValues * sizeof(uint64_t);
    int ok = 1;
    cudaIpcMemHandle_t mine{};
    char* gather = nullptr;     // [world + 1] handles: slot `world` is the send buffer
    int* flag = nullptr;
    if (cudaMalloc(&c.mailbox, box_bytes) != cudaSuccess || cudaMemset(c.mailbox, 0, box_bytes) != cudaSuccess ||
        cudaIpcGetMemHandle(&mine, c.mailbox) != cudaSuccess)
        ok = 0;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    WGF_CUDA(cudaMalloc(&gather, hb * (c.world + 1)));
    WGF_CUDA(cudaMalloc(&flag, sizeof(int)));
    WGF_CUDA(cudaMemcpy(gather + hb * c.world, &mine, hb, cudaMemcpyHostToDevice));
    nccl_check(Nccl::get().AllGather(gather + hb * c.world, gather, hb, /*ncclInt8*/ 0, c.handle, dev.stream), "ncclAllGather");
    std::vector<cudaIpcMemHandle_t> all(c.world);
    WGF_CUDA(cudaMemcpyAsync(all.data(), gather, hb * c.world, cudaMemcpyDeviceToHost, dev.stream));
    WGF_CUDA(cudaStreamSynchronize(dev.stream));
    c.peer_mailbox.assign(c.world, nullptr);
    for (int r = 0; r < c.world && ok; ++r) {
        if (r == c.rank) {
            c.peer_mailbox[r] = c.mailbox;
        } else if (cudaIpcOpenMemHandle(&c.peer_mailbox[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            c.peer_mailbox[r] = nullptr;
            ok = 0;
        }
    }
    cudaGetLastError();   // a failed mapping is not an error of the library: NCCL takes over
    if (ok) {
        std::vector<uint64_t> table(c.world);
        for (int r = 0; r < c.world; ++r) table[r] = (uint64_t)(uintptr_t)c.peer_mailbox[r];
        if (cudaMalloc(&c.peer_table, sizeof(uint64_t) * c.world) != cudaSuccess ||
            cudaMemcpy(c.peer_table, table.data(), sizeof(uint64_t) * c.world, cudaMemcpyHostToDevice) != cudaSuccess)
            ok = 0;
    }
    // every rank must take the same path: minimum of the outcomes
    WGF_CUDA(cudaMemcpy(flag, &ok, sizeof(int), cudaMemcpyHostToDevice));
    nccl_check(Nccl::get().AllReduce(flag, flag, 1, /*ncclInt32*/ 2, /*ncclMin*/ 3, c.handle, dev.stream), "ncclAllReduce");
    WGF_CUDA(cudaMemcpyAsync(&ok, flag, sizeof(int), cudaMemcpyDeviceToHost, dev.stream));
    WGF_CUDA(cudaStreamSynchronize(dev.stream));
    cudaFree(gather);
    cudaFree(flag);
    c.peer_ok = ok != 0;
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
    WGF_CHECK(!dev->dry, WGF_ERR_NCCL, "compile-only device cannot join a communicator");
    dev->make_current();
    NcclId nid;
    std::memcpy(&nid, id, sizeof nid);
    nccl_check(Nccl::get().CommInitRank(&c->handle, world, nid, rank), "ncclCommInitRank");
    setup_mailboxes(*c);
    return c;
}

void comm_all_reduce(Comm& c, Device& dev, Buffer& out, void* data, int64_t count, DType dt, uint16_t op) {
    int ndt = dt == DType::F32 ? 7 : dt == DType::F16 ? 6 : 9;
    int nop = op == WGF_OP_SUM ? 0 : op == WGF_OP_PRODUCT ? 1 : op == WGF_OP_MAX ? 2 : 3;
    void* recv = data;
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

}  // namespace wgf
