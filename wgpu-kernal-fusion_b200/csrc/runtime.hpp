// Device runtime: CUDA context + stream, caching device allocator, CUDA-event timing,
// run-time kernel compilation (NVRTC -> cubin -> module) with a per-device kernel cache.
// Takes the place of src/device.rs, the buffer half of src/tensor.rs, src/query.rs and the
// pipeline/bind-group half of src/kernel.rs in the crate.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <functional>
#include <map>
#include <mutex>
#include <unordered_map>

#include "common.hpp"

namespace wgf {

#define WGF_CUDA(expr)                                                                      \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            ::wgf::fail(_e == cudaErrorMemoryAllocation ? WGF_ERR_OOM : WGF_ERR_CUDA,       \
                        std::string(#expr) + ": " + cudaGetErrorString(_e));                \
    } while (0)

struct Device;
struct Comm;
// Settles the communicator's open exchange over peer memory, if it has one (comm.cpp).
void comm_settle(Comm& c, Device& dev);

// Memory of a recorded schedule (Device::begin_recording).  Blocks handed out while recording
// come back here instead of to the device pool for as long as the schedule lives, so that a
// replay, which writes to the same addresses again, cannot touch memory that the pool has
// given to someone else in the meantime.
struct Arena {
    std::mutex mu;
    bool closed = false;                   // schedule destroyed: blocks go to the device pool again
    std::multimap<size_t, void*> free;     // blocks of the schedule that no live buffer holds
};

struct Buffer {
    std::shared_ptr<Device> dev;
    void* ptr = nullptr;
    size_t bytes = 0;       // requested
    size_t block = 0;       // size of the pool block backing it
    // Set while work on ANOTHER stream (the collective stream) still reads or writes the
    // buffer.  The device stream waits for it before the next use of the buffer and before
    // the block goes back to the pool (Device::wait_for, ~Buffer).
    cudaEvent_t pending = nullptr;
    // `pending` belongs to someone else (a communicator's ring of completion events): waited for like
    // any other, but not returned to the device's event pool afterwards
    bool pending_shared = false;
    // Set while the buffer holds this rank's own value of an all-reduce whose ranks have not been
    // combined yet (see Comm): Device::wait_for settles the exchange before the buffer is read.
    // The communicator keeps the buffer alive for as long as this is set.
    Comm* unsettled = nullptr;
    std::shared_ptr<Arena> arena;   // set for buffers allocated while a schedule was being recorded
    ~Buffer();
};
using BufferRef = std::shared_ptr<Buffer>;

// TensorData of the crate (src/tensor.rs:300-306): buffer + layout + dtype.
struct TensorData {
    BufferRef buf;
    Layout layout;
    DType dtype = DType::F32;
    void* base_ptr() const { return (char*)buf->ptr + layout.offset * (int64_t)dtype_size(dtype); }
    explicit operator bool() const { return (bool)buf; }
};

struct TimingRecord {
    cudaEvent_t start = nullptr, stop = nullptr;
    const char* what = "";
};

struct JitKernel {
    CUmodule module = nullptr;
    CUfunction fn = nullptr;
    int regs = 0;
};

struct Device : std::enable_shared_from_this<Device> {
    int ordinal = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool timing = true;
    // Compile-only device (ordinal -1): builds and compiles every kernel a graph needs but
    // owns no GPU and executes nothing; downloads fail.  Lets the resolver and the generated
    // CUDA source be checked on a machine without a GPU.
    bool dry = false;
    std::atomic<uint64_t> launches{0}, compiles{0};

    static std::shared_ptr<Device> create(int ordinal);
    ~Device();

    void make_current() const;
    void sync();

    // ---- memory ----
    BufferRef alloc(size_t bytes, bool zero);
    void upload(const Buffer& b, size_t off, const void* src, size_t n);
    // src must be page-locked; with `rec`, an event pair around the copy (on the upload stream) is stored there
    void upload_async(Buffer& b, size_t off, const void* src, size_t n, TimingRecord* rec = nullptr);
    void download(const Buffer& b, size_t off, void* dst, size_t n);
    // 65536 zero-initialised u32 tickets for kernels that elect a last-arriving CTA; every
    // such kernel leaves them zero again.
    void* counters();
    static constexpr int kCounters = 65536;
    // A device word that kernels with bounded waits set when a wait gives up (0 = fine).
    // sync() and download() read it after the stream has drained and raise WGF_ERR_TIMEOUT.
    unsigned* error_word();
    // Checked build (environment WGF_CHECKED=1, read when the device is created): generated kernels
    // test every tensor access against the extents bound here (see CHK_FAILS in jit_templates.hpp).
    // A launcher of a generated kernel names the buffers of its launch with chk_bind before
    // Device::launch, which uploads the table on the device stream.  Schedules cannot be recorded.
    bool checked = false;
    void chk_bind(const Buffer* b);
    void check_error_word();
    // Set once a combine kernel of an all-reduce over peer memory gave up waiting for a peer (error
    // code 51): the ranks are out of step from then on, and further all-reduces on this device are
    // refused with WGF_ERR_TIMEOUT until its communicators have been released and made anew.
    std::atomic<bool> exchange_broken{false};
    // The communicator whose last exchange over peer memory is posted but not settled (see Comm), if any.
    Comm* unsettled_comm = nullptr;
    // Second stream for collectives, so that an all-reduce overlaps the kernels queued behind it.
    cudaStream_t collective_stream();
    // Orders the device stream behind any collective still using `b` (no-op otherwise).
    void wait_for(Buffer& b);
    uint64_t reserved_bytes() const { return reserved_; }
    uint64_t in_use_bytes() const { return in_use_; }
    void release_block(void* p, size_t block);
    // Same, but only once `ev` (recorded on the collective stream) has completed.
    void release_block_after(void* p, size_t block, cudaEvent_t ev, bool shared_event = false);
    void trim();

    // ---- kernels ----
    // Looks `key` up in the cache; on a miss calls `source()` and compiles it.  The kernel
    // `entry` names the `extern "C" __global__` function in that source.
    const JitKernel& kernel(const std::string& key, const char* entry, const std::function<std::string()>& source);
    // Launch a run-time compiled kernel taking ONE by-value struct parameter.
    void launch(const JitKernel& k, dim3 grid, dim3 block, size_t smem, const void* params,
                const char* what);
    // Resident CTAs per SM for this kernel at the given block size (no dynamic shared memory).
    int max_blocks_per_sm(const JitKernel& k, int threads);
    // Book-keeping for kernels launched with <<<>>> from this library's own .cu files.
    void begin_launch(const char* what);
    void end_launch();

    // ---- recorded schedules (CUDA graph capture of everything queued on `stream`) ----
    // While recording, kernels are captured instead of run; calls that wait for the device,
    // copy between host and device, or involve another stream fail with WGF_ERR_UNSUPPORTED.
    struct Recorded {
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        std::shared_ptr<Arena> arena;
        uint64_t kernels = 0;
        // Buffers from BEFORE the recording that its kernels read (inputs, weights): every replay
        // reads their addresses again, so the schedule holds them until it is destroyed -- a
        // caller that drops its handle does not send the block back to the pool under the graph.
        std::vector<BufferRef> inputs;
    };
    bool recording() const { return (bool)arena_; }
    void begin_recording();
    // Ends the capture, instantiates the graph and runs it once, so that every tensor
    // materialised while recording holds its value as after an ordinary materialisation.
    Recorded end_recording();
    void replay(const Recorded& r);
    void destroy_recorded(Recorded& r);
    void refuse_while_recording(const char* what) const;
    // Called for every buffer a kernel of the recording is about to read or write; keeps the ones
    // that do not belong to the recording's own arena (see Recorded::inputs).  No-op otherwise.
    void note_recorded_buffer(const BufferRef& b);
    const std::shared_ptr<Arena>& arena() const { return arena_; }

    // Timing sink: while set, every launch appends an event pair to it.
    std::vector<TimingRecord>* sink = nullptr;
    cudaEvent_t event();
    void recycle(cudaEvent_t e);

   private:
    std::mutex mu_;
    std::multimap<size_t, void*> free_;
    uint64_t reserved_ = 0, in_use_ = 0;
    std::unordered_map<std::string, JitKernel> kernels_;
    std::vector<cudaEvent_t> event_pool_;
    TimingRecord pending_;
    void* counters_ = nullptr;
    unsigned* error_word_ = nullptr;
    bool nvtx_open_ = false;                                  // a range of begin_launch waits for its end_launch
    void* chk_table_ = nullptr;                               // device copy of the extents of the current launch
    std::vector<std::pair<uint64_t, uint64_t>> chk_bound_;    // [lo, hi) of the buffers named since the last launch
    cudaStream_t collective_stream_ = nullptr;
    cudaStream_t upload_stream_ = nullptr;
    struct Deferred {
        void* ptr;
        size_t block;
        cudaEvent_t ev;
        bool shared_event;   // not ours to recycle
    };
    std::vector<Deferred> deferred_;
    std::shared_ptr<Arena> arena_;     // non-null while recording
    std::vector<BufferRef> recorded_inputs_;
    uint64_t recording_from_ = 0;      // value of `launches` when recording began
    void drain_deferred_locked();
    void* raw_alloc(size_t block);
};
using DeviceRef = std::shared_ptr<Device>;

// Compile CUDA C++ to an sm_100a cubin with NVRTC (no GPU needed).  Throws WGF_ERR_COMPILE
// with the compiler log on failure.
std::vector<char> compile_to_cubin(const std::string& source, const std::string& name);

// Driver entry points fetched through the runtime (the library does not link libcuda).
struct DriverApi {
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t) = nullptr;
    void* TensorMapEncodeTiled = nullptr;
    static const DriverApi& get();
};

}  // namespace wgf
