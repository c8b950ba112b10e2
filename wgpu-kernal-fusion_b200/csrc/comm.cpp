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
    if (handle) {
        if (dev) cudaSetDevice(dev->ordinal);
        Nccl::get().CommDestroy(handle);
    }
}

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
