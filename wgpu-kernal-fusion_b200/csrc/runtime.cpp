#include <nvtx3/nvToolsExt.h>   // header-only: ranges cost nothing unless a profiler is attached
#include "runtime.hpp"

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <fstream>

namespace wgf {

// ---------------------------------------------------------------------------------------
// Driver entry points
// ---------------------------------------------------------------------------------------
static void* driver_symbol(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        fail(WGF_ERR_CUDA, std::string("driver entry point not found: ") + name + " (" +
                               cudaGetErrorString(e) + ")");
    return fn;
}

const DriverApi& DriverApi::get() {
    static DriverApi api = [] {
        DriverApi a;
        a.ModuleLoadData = (decltype(a.ModuleLoadData))driver_symbol("cuModuleLoadData");
        a.ModuleUnload = (decltype(a.ModuleUnload))driver_symbol("cuModuleUnload");
        a.ModuleGetFunction = (decltype(a.ModuleGetFunction))driver_symbol("cuModuleGetFunction");
        a.LaunchKernel = (decltype(a.LaunchKernel))driver_symbol("cuLaunchKernel");
        a.FuncSetAttribute = (decltype(a.FuncSetAttribute))driver_symbol("cuFuncSetAttribute");
        a.FuncGetAttribute = (decltype(a.FuncGetAttribute))driver_symbol("cuFuncGetAttribute");
        a.GetErrorString = (decltype(a.GetErrorString))driver_symbol("cuGetErrorString");
        a.OccupancyMaxActiveBlocksPerMultiprocessor = (decltype(a.OccupancyMaxActiveBlocksPerMultiprocessor))driver_symbol(
            "cuOccupancyMaxActiveBlocksPerMultiprocessor");
        a.TensorMapEncodeTiled = driver_symbol("cuTensorMapEncodeTiled");
        return a;
    }();
    return api;
}

static void cu_check(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return;
    const char* s = nullptr;
    DriverApi::get().GetErrorString(r, &s);
    fail(WGF_ERR_CUDA, std::string(what) + ": " + (s ? s : "unknown driver error"));
}

// ---------------------------------------------------------------------------------------
// NVRTC, loaded at run time so the library itself loads on machines without it
// ---------------------------------------------------------------------------------------
namespace {
struct Nvrtc {
    typedef void* Program;
    int (*CreateProgram)(Program*, const char*, const char*, int, const char* const*, const char* const*);
    int (*CompileProgram)(Program, int, const char* const*);
    int (*GetProgramLogSize)(Program, size_t*);
    int (*GetProgramLog)(Program, char*);
    int (*GetCUBINSize)(Program, size_t*);
    int (*GetCUBIN)(Program, char*);
    int (*DestroyProgram)(Program*);
    const char* (*GetErrorString)(int);
    std::string include_dir;

    static Nvrtc& get() {
        static Nvrtc n = [] {
            Nvrtc v{};
            std::vector<std::string> names;
            if (const char* p = getenv("WGF_NVRTC_PATH")) names.push_back(p);
            names.push_back("libnvrtc.so.12");
            names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
            names.push_back("libnvrtc.so");
            void* h = nullptr;
            std::string tried;
            for (auto& nm : names) {
                h = dlopen(nm.c_str(), RTLD_NOW | RTLD_LOCAL);
                if (h) break;
                tried += nm + " ";
            }
            if (!h) fail(WGF_ERR_COMPILE, "cannot load NVRTC (tried: " + tried + ")");
            auto sym = [&](const char* s) {
                void* p = dlsym(h, s);
                if (!p) fail(WGF_ERR_COMPILE, std::string("NVRTC symbol missing: ") + s);
                return p;
            };
            v.CreateProgram = (decltype(v.CreateProgram))sym("nvrtcCreateProgram");
            v.CompileProgram = (decltype(v.CompileProgram))sym("nvrtcCompileProgram");
            v.GetProgramLogSize = (decltype(v.GetProgramLogSize))sym("nvrtcGetProgramLogSize");
            v.GetProgramLog = (decltype(v.GetProgramLog))sym("nvrtcGetProgramLog");
            v.GetCUBINSize = (decltype(v.GetCUBINSize))sym("nvrtcGetCUBINSize");
            v.GetCUBIN = (decltype(v.GetCUBIN))sym("nvrtcGetCUBIN");
            v.DestroyProgram = (decltype(v.DestroyProgram))sym("nvrtcDestroyProgram");
            v.GetErrorString = (decltype(v.GetErrorString))sym("nvrtcGetErrorString");
            return v;
        }();
        return n;
    }
};

uint64_t fnv1a(const std::string& s) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : s) {
        h ^= c;
        h *= 1099511628211ull;
    }
    return h;
}

std::string cache_dir() {
    const char* d = getenv("WGF_KERNEL_CACHE");
    return d ? std::string(d) : std::string();
}
}  // namespace

std::vector<char> compile_to_cubin(const std::string& source, const std::string& name) {
    // On-disk cache of compiled kernels, keyed by a hash of the complete source text.
    std::string dir = cache_dir(), path;
    if (!dir.empty()) {
        char buf[64];
        snprintf(buf, sizeof buf, "/%016llx_%zu.cubin", (unsigned long long)fnv1a(source), source.size());
        path = dir + buf;
        std::ifstream f(path, std::ios::binary);
        if (f) {
            std::vector<char> data((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
            if (!data.empty()) return data;
        }
    }
    Nvrtc& n = Nvrtc::get();
    Nvrtc::Program prog = nullptr;
    int r = n.CreateProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
    if (r != 0) fail(WGF_ERR_COMPILE, std::string("nvrtcCreateProgram: ") + n.GetErrorString(r));
    // --fmad=false: every op of a fused chain rounds on its own, as separate shader functions do.
    const bool verbose = getenv("WGF_JIT_VERBOSE") != nullptr;  // print registers / spills per kernel
    const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17",
                          "-default-device", "--extra-device-vectorization", "--ptxas-options=-v"};
    r = n.CompileProgram(prog, verbose ? 6 : 5, opts);
    if (verbose && r == 0) {
        if (getenv("WGF_DUMP_SOURCE")) fprintf(stderr, "---- %s ----\n%s\n", name.c_str(), source.c_str());
        size_t ls = 0;
        n.GetProgramLogSize(prog, &ls);
        std::string log(ls, '\0');
        if (ls) n.GetProgramLog(prog, &log[0]);
        fprintf(stderr, "[wgf jit] %s", log.c_str());
    }
    if (r != 0) {
        size_t ls = 0;
        n.GetProgramLogSize(prog, &ls);
        std::string log(ls, '\0');
        if (ls) n.GetProgramLog(prog, &log[0]);
        n.DestroyProgram(&prog);
        if (getenv("WGF_DUMP_SOURCE")) fprintf(stderr, "---- %s ----\n%s\n", name.c_str(), source.c_str());
        fail(WGF_ERR_COMPILE, "kernel '" + name + "' failed to compile:\n" + log);
    }
    size_t cs = 0;
    n.GetCUBINSize(prog, &cs);
    std::vector<char> cubin(cs);
    n.GetCUBIN(prog, cubin.data());
    n.DestroyProgram(&prog);
    if (!path.empty()) {
        mkdir(dir.c_str(), 0755);
        std::string tmp = path + ".tmp" + std::to_string((long)getpid());
        std::ofstream f(tmp, std::ios::binary);
        if (f) {
            f.write(cubin.data(), (std::streamsize)cubin.size());
            f.close();
            rename(tmp.c_str(), path.c_str());
        }
    }
    return cubin;
}

// ---------------------------------------------------------------------------------------
// Buffer / Device
// ---------------------------------------------------------------------------------------
Buffer::~Buffer() {
    if (ptr && dev) {
        if (arena) {
            // a block of a recorded schedule stays with the schedule while that one lives
            std::lock_guard<std::mutex> g(arena->mu);
            if (!arena->closed) {
                if (pending && !pending_shared) dev->recycle(pending);
                arena->free.emplace(block, ptr);
                return;
            }
        }
        // a collective may still touch the block: it goes back to the pool once that is over
        if (pending) dev->release_block_after(ptr, block, pending, pending_shared);
        else dev->release_block(ptr, block);
    }
}

void Device::release_block_after(void* p, size_t block, cudaEvent_t ev, bool shared_event) {
    std::lock_guard<std::mutex> g(mu_);
    deferred_.push_back({p, block, ev, shared_event});
}

// Moves blocks whose collective has finished from the deferred list to the pool.  mu_ held.
void Device::drain_deferred_locked() {
    for (size_t i = 0; i < deferred_.size();) {
        if (cudaEventQuery(deferred_[i].ev) == cudaSuccess) {
            free_.emplace(deferred_[i].block, deferred_[i].ptr);
            in_use_ -= deferred_[i].block;
            if (!deferred_[i].shared_event) event_pool_.push_back(deferred_[i].ev);
            deferred_[i] = deferred_.back();
            deferred_.pop_back();
        } else {
            cudaGetLastError();   // cudaErrorNotReady is not an error
            ++i;
        }
    }
}

cudaStream_t Device::collective_stream() {
    if (!collective_stream_ && !dry) {
        make_current();
        WGF_CUDA(cudaStreamCreateWithFlags(&collective_stream_, cudaStreamNonBlocking));
    }
    return collective_stream_;
}

void Device::wait_for(Buffer& b) {
    if (b.unsettled) comm_settle(*b.unsettled, *this);   // the ranks' values are combined before anyone reads the result
    if (!b.pending) return;
    cudaSetDevice(ordinal);
    // an event recorded outside a capture cannot become a dependency inside it: wait on the host
    if (recording()) cudaEventSynchronize(b.pending);
    else cudaStreamWaitEvent(stream, b.pending, 0);
    if (!b.pending_shared) recycle(b.pending);
    b.pending = nullptr;
    b.pending_shared = false;
}

std::shared_ptr<Device> Device::create(int ordinal) {
    if (ordinal == -1) {
        auto d = std::make_shared<Device>();
        d->ordinal = -1;
        d->dry = true;
        d->timing = false;
        d->sm_count = 148;
        d->checked = getenv("WGF_CHECKED") != nullptr;   // compiles the checked kernels (nothing runs)
        return d;
    }
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess)
        fail(WGF_ERR_CUDA, std::string("no CUDA device available: ") + cudaGetErrorString(e));
    WGF_CHECK(ordinal >= 0 && ordinal < count, WGF_ERR_INVALID_ARGUMENT,
              "device ordinal " + std::to_string(ordinal) + " out of range (" + std::to_string(count) + " devices)");
    auto d = std::make_shared<Device>();
    d->ordinal = ordinal;
    WGF_CUDA(cudaSetDevice(ordinal));
    WGF_CUDA(cudaFree(nullptr));  // establish the primary context
    cudaDeviceProp prop;
    WGF_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    WGF_CHECK(prop.major == 10, WGF_ERR_UNSUPPORTED,
              std::string("this library is built for sm_100a only; device is sm_") +
                  std::to_string(prop.major) + std::to_string(prop.minor));
    d->sm_count = prop.multiProcessorCount;
    WGF_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
    DriverApi::get();
    d->checked = getenv("WGF_CHECKED") != nullptr;
    return d;
}

Device::~Device() {
    if (arena_ && !dry && stream) {
        // destroyed in the middle of a recording: close the capture and drop what it holds
        cudaSetDevice(ordinal);
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(stream, &g);
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
    }
    if (dry) {
        for (auto& kv : free_) free(kv.second);
        return;
    }
    cudaSetDevice(ordinal);
    if (stream) cudaStreamSynchronize(stream);
    for (auto& kv : kernels_)
        if (kv.second.module) DriverApi::get().ModuleUnload(kv.second.module);
    for (auto& kv : free_) cudaFree(kv.second);
    for (auto e : event_pool_) cudaEventDestroy(e);
    if (counters_) cudaFree(counters_);
    if (error_word_) cudaFree(error_word_);
    if (chk_table_) cudaFree(chk_table_);
    if (collective_stream_) {
        cudaStreamSynchronize(collective_stream_);
        cudaStreamDestroy(collective_stream_);
    }
    if (upload_stream_) {
        cudaStreamSynchronize(upload_stream_);
        cudaStreamDestroy(upload_stream_);
    }
    for (auto& d : deferred_) {
        cudaFree(d.ptr);
        cudaEventDestroy(d.ev);
    }
    if (stream) cudaStreamDestroy(stream);
}

void Device::make_current() const {
    if (!dry) WGF_CUDA(cudaSetDevice(ordinal));
}

void Device::sync() {
    refuse_while_recording("wgf_device_sync");
    if (unsettled_comm) comm_settle(*unsettled_comm, *this);   // after a synchronisation every result is final
    if (dry) return;
    make_current();
    WGF_CUDA(cudaStreamSynchronize(stream));
    if (collective_stream_) WGF_CUDA(cudaStreamSynchronize(collective_stream_));
    if (upload_stream_) WGF_CUDA(cudaStreamSynchronize(upload_stream_));
    {
        std::lock_guard<std::mutex> g(mu_);
        if (!deferred_.empty()) drain_deferred_locked();
    }
    check_error_word();
}

void Device::chk_bind(const Buffer* b) {
    if (checked && b && b->ptr) chk_bound_.emplace_back((uint64_t)(uintptr_t)b->ptr, (uint64_t)(uintptr_t)b->ptr + b->bytes);
}

unsigned* Device::error_word() {
    if (dry) return nullptr;
    if (!error_word_) {
        make_current();
        WGF_CUDA(cudaMalloc(&error_word_, 256));
        WGF_CUDA(cudaMemsetAsync(error_word_, 0, 256, stream));
    }
    return error_word_;
}

// Called with the stream drained.
void Device::check_error_word() {
    if (!error_word_) return;
    unsigned v = 0;
    WGF_CUDA(cudaMemcpy(&v, error_word_, sizeof v, cudaMemcpyDeviceToHost));
    if (v == 61) {
        uint64_t detail[3] = {0, 0, 0};
        cudaMemcpy(detail, error_word_, sizeof detail, cudaMemcpyDeviceToHost);
        cudaMemset(error_word_, 0, sizeof detail);
        char msg[224];
        snprintf(msg, sizeof msg, "checked build: a generated kernel asked for %llu bytes at device address 0x%llx, outside every "
                 "buffer bound to its launch; the access was not made", (unsigned long long)detail[2], (unsigned long long)detail[1]);
        fail(WGF_ERR_CUDA, msg);
    }
    if (v) {
        cudaMemset(error_word_, 0, sizeof v);
        if (v == 51) exchange_broken = true;
        fail(WGF_ERR_TIMEOUT, "a kernel gave up on a bounded wait (code " + std::to_string(v) +
                                  "); its result is not valid");
    }
}

static size_t round_block(size_t bytes) {
    if (bytes < 512) return 512;
    if (bytes < (1u << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + ((1u << 20) - 1)) & ~size_t((1u << 20) - 1);
}

void* Device::raw_alloc(size_t block) {
    if (dry) {
        void* h = aligned_alloc(512, block);
        if (!h) fail(WGF_ERR_OOM, "host allocation failed");
        reserved_ += block;
        return h;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, block);
    if (e == cudaErrorMemoryAllocation && !recording()) {
        cudaGetLastError();
        // give cached blocks back to the driver and retry once
        WGF_CUDA(cudaStreamSynchronize(stream));
        for (auto& kv : free_) {
            cudaFree(kv.second);
            reserved_ -= kv.first;
        }
        free_.clear();
        e = cudaMalloc(&p, block);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(e == cudaErrorMemoryAllocation ? WGF_ERR_OOM : WGF_ERR_CUDA,
             "device allocation of " + std::to_string(block) + " bytes failed: " + cudaGetErrorString(e));
    }
    reserved_ += block;
    return p;
}

BufferRef Device::alloc(size_t bytes, bool zero) {
    make_current();
    size_t block = round_block(bytes);
    void* p = nullptr;
    if (arena_) {
        // blocks that this recording has already used and released come first
        std::lock_guard<std::mutex> g(arena_->mu);
        auto it = arena_->free.lower_bound(block);
        if (it != arena_->free.end() && it->first <= block + block / 4 + 4096) {
            p = it->second;
            block = it->first;
            arena_->free.erase(it);
        }
    }
    if (!p) {
        std::lock_guard<std::mutex> g(mu_);
        // Blocks that wait for a collective are looked at only when the pool has nothing that fits (or
        // when many have piled up): asking the driver about every one of them on every allocation cost
        // the host several microseconds per step.
        if (deferred_.size() > 64) drain_deferred_locked();
        auto fits = [&] {
            auto it = free_.lower_bound(block);
            // reuse a cached block unless it would waste more than a quarter of itself
            return it != free_.end() && it->first <= block + block / 4 + 4096 ? it : free_.end();
        };
        auto it = fits();
        if (it == free_.end() && !deferred_.empty()) {
            drain_deferred_locked();
            it = fits();
        }
        if (it != free_.end()) {
            p = it->second;
            block = it->first;
            free_.erase(it);
        } else {
            p = raw_alloc(block);
        }
        in_use_ += block;
    }
    auto b = std::make_shared<Buffer>();
    b->dev = shared_from_this();
    b->arena = arena_;
    b->ptr = p;
    b->bytes = bytes;
    b->block = block;
    if (zero && bytes && !dry) WGF_CUDA(cudaMemsetAsync(p, 0, bytes, stream));
    return b;
}

void Device::release_block(void* p, size_t block) {
    // All work that touches the block was queued on `stream`; any later user of the block
    // queues on the same stream, so handing it out again needs no wait.
    std::lock_guard<std::mutex> g(mu_);
    free_.emplace(block, p);
    in_use_ -= block;
}

void Device::trim() {
    refuse_while_recording("trimming the pool");
    if (dry) return;
    make_current();
    WGF_CUDA(cudaStreamSynchronize(stream));
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : free_) {
        cudaFree(kv.second);
        reserved_ -= kv.first;
    }
    free_.clear();
}

void Device::upload(const Buffer& b, size_t off, const void* src, size_t n) {
    WGF_CHECK(off + n <= b.bytes, WGF_ERR_INVALID_ARGUMENT, "upload past the end of the buffer");
    refuse_while_recording("an upload");
    if (!n || dry) return;
    make_current();
    WGF_CUDA(cudaMemcpyAsync((char*)b.ptr + off, src, n, cudaMemcpyHostToDevice, stream));
    // The source may be pageable and reused by the caller right away.
    WGF_CUDA(cudaStreamSynchronize(stream));
}

// Upload from PAGE-LOCKED host memory on the upload stream: returns at once, overlaps whatever the
// device stream is doing (kernels, a download in the other PCIe direction).  The copy is ordered
// behind everything queued on the device stream so far, because the pool may have handed out a block
// that earlier kernels still use; the buffer carries the completion event (Buffer::pending).
void Device::upload_async(Buffer& b, size_t off, const void* src, size_t n, TimingRecord* rec) {
    WGF_CHECK(off + n <= b.bytes, WGF_ERR_INVALID_ARGUMENT, "upload past the end of the buffer");
    refuse_while_recording("an upload");
    if (!n || dry) return;
    make_current();
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, src);
    if (e != cudaSuccess || attr.type != cudaMemoryTypeHost) {
        cudaGetLastError();
        fail(WGF_ERR_INVALID_ARGUMENT, "asynchronous upload needs page-locked host memory (wgf_host_alloc)");
    }
    if (!upload_stream_) WGF_CUDA(cudaStreamCreateWithFlags(&upload_stream_, cudaStreamNonBlocking));
    wait_for(b);
    cudaEvent_t before = event();
    WGF_CUDA(cudaEventRecord(before, stream));
    WGF_CUDA(cudaStreamWaitEvent(upload_stream_, before, 0));
    recycle(before);
    if (rec) {
        rec->start = event();
        rec->stop = event();
        rec->what = "upload";
        WGF_CUDA(cudaEventRecord(rec->start, upload_stream_));
    }
    WGF_CUDA(cudaMemcpyAsync((char*)b.ptr + off, src, n, cudaMemcpyHostToDevice, upload_stream_));
    if (rec) WGF_CUDA(cudaEventRecord(rec->stop, upload_stream_));
    b.pending = event();
    WGF_CUDA(cudaEventRecord(b.pending, upload_stream_));
}

void Device::download(const Buffer& b, size_t off, void* dst, size_t n) {
    WGF_CHECK(off + n <= b.bytes, WGF_ERR_INVALID_ARGUMENT, "download past the end of the buffer");
    refuse_while_recording("a download");
    WGF_CHECK(!dry, WGF_ERR_CUDA, "compile-only device: nothing was executed, there is nothing to download");
    make_current();
    wait_for(const_cast<Buffer&>(b));
    if (n) WGF_CUDA(cudaMemcpyAsync(dst, (const char*)b.ptr + off, n, cudaMemcpyDeviceToHost, stream));
    WGF_CUDA(cudaStreamSynchronize(stream));
    check_error_word();
}

void* Device::counters() {
    if (dry) return nullptr;
    if (!counters_) {
        make_current();
        WGF_CUDA(cudaMalloc(&counters_, kCounters * sizeof(uint32_t)));
        WGF_CUDA(cudaMemsetAsync(counters_, 0, kCounters * sizeof(uint32_t), stream));
    }
    return counters_;
}

cudaEvent_t Device::event() {
    {
        std::lock_guard<std::mutex> g(mu_);
        if (!event_pool_.empty()) {
            cudaEvent_t e = event_pool_.back();
            event_pool_.pop_back();
            return e;
        }
    }
    cudaEvent_t e;
    WGF_CUDA(cudaEventCreate(&e));
    return e;
}

void Device::recycle(cudaEvent_t e) {
    std::lock_guard<std::mutex> g(mu_);
    event_pool_.push_back(e);
}

const JitKernel& Device::kernel(const std::string& key, const char* entry, const std::function<std::string()>& source) {
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = kernels_.find(key);
        if (it != kernels_.end()) return it->second;
    }
    make_current();
    std::string src = source();
    if (checked) {
        char defs[192];
        if (!dry && !chk_table_) {
            WGF_CUDA(cudaMalloc(&chk_table_, 512));
            WGF_CUDA(cudaMemset(chk_table_, 0, 512));
        }
        snprintf(defs, sizeof defs, "#define WGF_CHECKED 1\n#define WGF_CHK_TABLE 0x%llxull\n#define WGF_CHK_ERR 0x%llxull\n",
                 (unsigned long long)(uintptr_t)chk_table_, (unsigned long long)(uintptr_t)error_word());
        src = defs + src;
    }
    std::vector<char> cubin = compile_to_cubin(src, entry);
    compiles++;
    if (dry) {
        std::lock_guard<std::mutex> g(mu_);
        return kernels_.emplace(key, JitKernel{}).first->second;
    }
    const DriverApi& api = DriverApi::get();
    JitKernel k;
    cu_check(api.ModuleLoadData(&k.module, cubin.data()), "cuModuleLoadData");
    cu_check(api.ModuleGetFunction(&k.fn, k.module, entry), "cuModuleGetFunction");
    api.FuncGetAttribute(&k.regs, CU_FUNC_ATTRIBUTE_NUM_REGS, k.fn);
    std::lock_guard<std::mutex> g(mu_);
    auto ins = kernels_.emplace(key, k);
    if (!ins.second) api.ModuleUnload(k.module);  // another thread won the race
    return ins.first->second;
}

int Device::max_blocks_per_sm(const JitKernel& k, int threads) {
    if (dry || !k.fn) return std::max(1, 2048 / threads);
    int n = 0;
    CUresult r = DriverApi::get().OccupancyMaxActiveBlocksPerMultiprocessor(&n, k.fn, threads, 0);
    if (r != CUDA_SUCCESS || n < 1) n = 1;
    return n;
}

void Device::begin_launch(const char* what) {
    static const bool trace = getenv("WGF_TRACE_LAUNCHES") != nullptr;   // diagnostic: one line per kernel queued
    if (trace) fprintf(stderr, "[wgf] launch %s\n", what);
    // WGF_NVTX=1: every kernel the library queues sits in a named range on the host time line (a
    // profiler that follows NVTX shows which part of a materialisation each launch belongs to)
    static const bool nvtx = getenv("WGF_NVTX") != nullptr;
    if (nvtx) {
        nvtxRangePushA(what);
        nvtx_open_ = true;
    }
    launches++;
    if (timing && sink && !dry && !recording()) {
        pending_.start = event();
        pending_.stop = event();
        pending_.what = what;
        WGF_CUDA(cudaEventRecord(pending_.start, stream));
    }
}

void Device::end_launch() {
    if (nvtx_open_) {
        nvtxRangePop();
        nvtx_open_ = false;
    }
    if (pending_.start) {
        WGF_CUDA(cudaEventRecord(pending_.stop, stream));
        if (sink) sink->push_back(pending_);
        pending_ = TimingRecord{};
    }
    if (dry) return;
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(WGF_ERR_CUDA, std::string("kernel launch failed: ") + cudaGetErrorString(e));
    }
}

void Device::launch(const JitKernel& k, dim3 grid, dim3 block, size_t smem, const void* params,
                    const char* what) {
    make_current();
    begin_launch(what);
    if (dry) {
        end_launch();
        return;
    }
    if (checked) {
        // the extents of this launch's buffers, stream-ordered between the previous kernel and this one
        struct {
            uint64_t n, lo[24], hi[24];
        } t{};
        WGF_CHECK(chk_bound_.size() <= 24, WGF_ERR_UNSUPPORTED, "checked build: more than 24 buffers in one launch");
        t.n = chk_bound_.size();
        for (size_t i = 0; i < chk_bound_.size(); ++i) {
            t.lo[i] = chk_bound_[i].first;
            t.hi[i] = chk_bound_[i].second;
        }
        static const long shrink = getenv("WGF_CHECKED_SHRINK") ? atol(getenv("WGF_CHECKED_SHRINK")) : 0;   // test hook:
        // the last buffer bound (the result) is declared this many bytes shorter than it is, so that
        // accesses that are in fact valid are refused and reported
        if (shrink > 0 && t.n) t.hi[t.n - 1] -= std::min<uint64_t>((uint64_t)shrink, t.hi[t.n - 1] - t.lo[t.n - 1]);
        chk_bound_.clear();
        WGF_CUDA(cudaMemcpyAsync(chk_table_, &t, sizeof t, cudaMemcpyHostToDevice, stream));
    }
    void* args[] = {const_cast<void*>(params)};
    CUresult r = DriverApi::get().LaunchKernel(k.fn, grid.x, grid.y, grid.z, block.x, block.y, block.z,
                                               (unsigned)smem, (CUstream)stream, args, nullptr);
    cu_check(r, what);
    end_launch();
}

// ---------------------------------------------------------------------------------------
// recorded schedules
// ---------------------------------------------------------------------------------------
void Device::refuse_while_recording(const char* what) const {
    if (recording())
        fail(WGF_ERR_UNSUPPORTED, std::string(what) + " is not possible while a schedule is being recorded "
                                                       "(finish it with wgf_schedule_end first)");
}

void Device::begin_recording() {
    WGF_CHECK(!recording(), WGF_ERR_INVALID_ARGUMENT, "a schedule is already being recorded on this device");
    WGF_CHECK(!checked, WGF_ERR_UNSUPPORTED, "the checked build (WGF_CHECKED) uploads a table before every launch and cannot record schedules");
    if (!dry) {
        make_current();
        // everything the capture must not contain happens now: the one-time set-up of the
        // ticket counters and the error word, and the end of all work on the other streams
        counters();
        error_word();
        sync();
        WGF_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeRelaxed));
    }
    arena_ = std::make_shared<Arena>();
    recorded_inputs_.clear();
    recording_from_ = launches.load();
}

void Device::note_recorded_buffer(const BufferRef& b) {
    if (!recording() || !b || b->arena == arena_) return;
    for (const BufferRef& have : recorded_inputs_)
        if (have.get() == b.get()) return;
    recorded_inputs_.push_back(b);
}

Device::Recorded Device::end_recording() {
    WGF_CHECK(recording(), WGF_ERR_INVALID_ARGUMENT, "no schedule is being recorded on this device");
    Recorded r;
    r.arena = arena_;
    r.kernels = launches.load() - recording_from_;
    r.inputs.swap(recorded_inputs_);
    arena_.reset();
    if (dry) return r;
    make_current();
    cudaError_t e = cudaStreamEndCapture(stream, &r.graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&r.exec, r.graph, 0);
    if (e == cudaSuccess) e = cudaGraphLaunch(r.exec, stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        destroy_recorded(r);
        fail(WGF_ERR_CUDA, std::string("recording the schedule failed: ") + cudaGetErrorString(e));
    }
    return r;
}

void Device::replay(const Recorded& r) {
    refuse_while_recording("replaying a schedule");
    launches += r.kernels;
    if (dry) return;
    make_current();
    WGF_CUDA(cudaGraphLaunch(r.exec, stream));
}

void Device::destroy_recorded(Recorded& r) {
    if (!dry) {
        cudaSetDevice(ordinal);
        // a replay may still be running: its memory must not reach the pool before it ends
        if (r.exec) cudaStreamSynchronize(stream);
        if (r.exec) cudaGraphExecDestroy(r.exec);
        if (r.graph) cudaGraphDestroy(r.graph);
    }
    r.exec = nullptr;
    r.graph = nullptr;
    r.inputs.clear();   // no replay can read them any more
    if (r.arena) {
        std::multimap<size_t, void*> blocks;
        {
            std::lock_guard<std::mutex> g(r.arena->mu);
            r.arena->closed = true;
            blocks.swap(r.arena->free);
        }
        for (auto& kv : blocks) release_block(kv.second, kv.first);
        r.arena.reset();
    }
}

}  // namespace wgf
