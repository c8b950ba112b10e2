// Turns a fused Program into CUDA source around the hand-written templates, compiles it on
// first use (cached per device) and launches it.  Replaces the WGSL text generation of
// src/element_wise.rs:64-130, src/pair_wise.rs:112-159, src/reduce.rs:83-281 and the launch
// arithmetic of src/visit_tiled.rs:149-193 / src/reduce.rs:321-386.
#include <map>
#include <mutex>
#include <algorithm>
#include <sstream>

#include "jit_templates.hpp"
#include "launch.hpp"

namespace wgf {

namespace {

// ---------------------------------------------------------------------------------------
// expression text
// ---------------------------------------------------------------------------------------
const char* unary_fn(uint16_t op) {
    switch (op) {
        case WGF_OP_EXP: return "op_exp";
        case WGF_OP_EXP2: return "op_exp2";
        case WGF_OP_LOG: return "op_log";
        case WGF_OP_LOG2: return "op_log2";
        case WGF_OP_SQRT: return "op_sqrt";
        case WGF_OP_SIN: return "op_sin";
        case WGF_OP_COS: return "op_cos";
        case WGF_OP_TAN: return "op_tan";
        case WGF_OP_ASIN: return "op_asin";
        case WGF_OP_ACOS: return "op_acos";
        case WGF_OP_ATAN: return "op_atan";
        case WGF_OP_SINH: return "op_sinh";
        case WGF_OP_COSH: return "op_cosh";
        case WGF_OP_TANH: return "op_tanh";
        case WGF_OP_ASINH: return "op_asinh";
        case WGF_OP_ACOSH: return "op_acosh";
        case WGF_OP_ATANH: return "op_atanh";
        case WGF_OP_ABS: return "fabsf";
        default: return nullptr;
    }
}

std::string rounded(DType dt, const std::string& e) {
    if (dt == DType::F16) return "rh(" + e + ")";
    if (dt == DType::BF16) return "rb(" + e + ")";
    return e;
}

// Text of instruction `in` given the text of its operands.
std::string instr_expr(const Instr& in, const std::string& a, const std::string& b) {
    switch (in.kind) {
        case IKind::Unary:
            if (in.op == WGF_OP_SQR) return rounded(in.dtype, "(" + a + " * " + a + ")");
            if (in.op == WGF_OP_NEG) return "(-" + a + ")";
            if (in.op == WGF_OP_ABS) return "fabsf(" + a + ")";
            // exp of a 16-bit tensor: its result is rounded to 11 (8) bits anyway, so the two-instruction
            // form (error about 1e-6 relative) gives the same 16-bit value as expf except where the
            // exact result lies within that distance of a rounding boundary
            if (in.op == WGF_OP_EXP && (in.dtype != DType::F32 || in.approx)) return rounded(in.dtype, "op_exp_sfu(" + a + ")");
            // an argument known to lie in [-1, 1] needs no range reduction
            if (in.arg_unit && in.op == WGF_OP_SIN) return rounded(in.dtype, "op_sin_unit(" + a + ")");
            if (in.arg_unit && in.op == WGF_OP_COS) return rounded(in.dtype, "op_cos_unit(" + a + ")");
            return rounded(in.dtype, std::string(unary_fn(in.op)) + "(" + a + ")");
        case IKind::Scalar: {
            std::string c = "imm[" + std::to_string(in.slot) + "]";
            switch (in.op) {
                case WGF_OP_ADD_C: return rounded(in.dtype, "(" + a + " + " + c + ")");
                case WGF_OP_SUB_C: return rounded(in.dtype, "(" + a + " - " + c + ")");
                case WGF_OP_RSUB_C: return rounded(in.dtype, "(" + c + " - " + a + ")");
                case WGF_OP_MUL_C: return rounded(in.dtype, "(" + a + " * " + c + ")");
                case WGF_OP_DIV_C: return rounded(in.dtype, "(" + a + " / " + c + ")");
                default: return rounded(in.dtype, in.fast_div ? "op_div_full(" + c + ", " + a + ")" : "(" + c + " / " + a + ")");
            }
        }
        case IKind::Cast: return rounded(in.dtype, a);
        case IKind::Binary:
            switch (in.op) {
                case WGF_OP_ADD: return rounded(in.dtype, "(" + a + " + " + b + ")");
                case WGF_OP_SUB: return rounded(in.dtype, "(" + a + " - " + b + ")");
                case WGF_OP_MUL: return rounded(in.dtype, "(" + a + " * " + b + ")");
                case WGF_OP_DIV: return rounded(in.dtype, in.fast_div ? "op_div_full(" + a + ", " + b + ")" : "(" + a + " / " + b + ")");
                default: return rounded(in.dtype, "op_pow(" + a + ", " + b + ")");
            }
        default: return "";
    }
}

const char* red_name(uint16_t op) {
    switch (op) {
        case WGF_OP_SUM: return "RED_SUM";
        case WGF_OP_MAX: return "RED_MAX";
        case WGF_OP_MIN: return "RED_MIN";
        default: return "RED_PROD";
    }
}

std::string vn(int i) { return "v" + std::to_string(i); }

// ---------------------------------------------------------------------------------------
// host-side parameter block, laid out like the `Params` struct of the templates
// ---------------------------------------------------------------------------------------
struct ParamWriter {
    std::vector<unsigned char> bytes;
    template <typename T> void put(T v) {
        size_t at = bytes.size();
        bytes.resize(at + sizeof(T));
        std::memcpy(bytes.data() + at, &v, sizeof(T));
    }
    void finish() {
        while (bytes.size() % 8) bytes.push_back(0);
    }
};

// PEER_SETTLE_PARAMS of the templates: the earlier exchanges that a kernel of the all-reduce path posts and settles.
void put_settle(ParamWriter& w, const GrandComm* gc) {
    w.put<uint64_t>(gc ? (uint64_t)(uintptr_t)gc->mailbox : 0);
    w.put<uint64_t>(gc ? gc->wait_ns : 0);
    for (int i = 0; i < 4; ++i) w.put<uint64_t>(gc ? (uint64_t)(uintptr_t)gc->prev_out[i] : 0);
    for (int i = 0; i < 4; ++i) w.put<uint64_t>(gc ? (uint64_t)(uintptr_t)gc->post_src[i] : 0);
    for (int i = 0; i < 4; ++i) w.put<uint32_t>(gc ? gc->prev_meta[i] : 0);
    for (int i = 0; i < 4; ++i) w.put<uint32_t>(gc ? gc->post_meta[i] : 0);
    w.put<uint32_t>(gc ? gc->prev_seq : 0);
    w.put<uint32_t>(gc ? gc->prev_n : 0);
    w.put<uint32_t>(gc ? gc->post_seq : 0);
    w.put<uint32_t>(gc ? gc->post_n : 0);
}

void magic_for(uint32_t d, uint32_t& m, uint32_t& s) {
    if (d <= 1) {
        m = 0;
        s = 0;
        return;
    }
    uint32_t lg = 0;
    while ((1ull << lg) < d) lg++;  // ceil(log2 d)
    uint32_t p = 31 + lg;
    m = (uint32_t)(((1ull << p) + d - 1) / d);
    s = p - 32;
}

// Tuning overrides read from the environment (WGF_TUNE_<NAME>=int); absent = `dflt`.  Each name is
// looked up once per process (a launch asks for half a dozen of them, and a scan of the environment
// costs about as much as everything else the launcher does for a small kernel).
int tune(const char* name, int dflt) {
    struct Entry {
        bool set;
        int value;
    };
    static std::mutex mu;
    static std::map<std::string, Entry> seen;
    std::lock_guard<std::mutex> g(mu);
    auto it = seen.find(name);
    if (it == seen.end()) {
        const std::string key = std::string("WGF_TUNE_") + name;
        const char* v = getenv(key.c_str());
        it = seen.emplace(name, Entry{v != nullptr, v ? atoi(v) : 0}).first;
    }
    return it->second.set ? it->second.value : dflt;
}

// Checked build: names the buffers of the launch that follows (Device::chk_bind); the result last.
static void bind_checked(Device& dev, const std::vector<TensorData>& in, const TensorData& out,
                         const std::vector<TensorData>* more = nullptr) {
    if (!dev.checked) return;
    for (const TensorData& t : in) dev.chk_bind(t.buf.get());
    if (more)
        for (const TensorData& t : *more) dev.chk_bind(t.buf.get());
    dev.chk_bind(out.buf.get());
}

// The helpers every generated kernel starts with.
std::string prelude() {
    // warp-wide max / min through redux.sync (f32 form of sm_100a)
    static const std::string text =
        std::string("#define WGF_REDUX ") + (tune("REDUX", 1) ? "1\n" : "0\n") + JIT_PRELUDE;
    return text;
}

int pow2_at_least(int64_t v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Canonical index space: extent-1 axes dropped, adjacent axes merged where every tensor
// allows it.  `strides[t]` are the strides of tensor t over `shape`.
void collapse(std::vector<int64_t>& shape, std::vector<std::vector<int64_t>>& strides) {
    std::vector<int64_t> ns;
    std::vector<std::vector<int64_t>> nst(strides.size());
    for (size_t d = 0; d < shape.size(); ++d) {
        if (shape[d] == 1) continue;
        if (!ns.empty()) {
            bool merge = true;
            for (size_t t = 0; t < strides.size(); ++t)
                if (nst[t].back() != strides[t][d] * shape[d]) merge = false;
            if (merge) {
                ns.back() *= shape[d];
                for (size_t t = 0; t < strides.size(); ++t) nst[t].back() = strides[t][d];
                continue;
            }
        }
        ns.push_back(shape[d]);
        for (size_t t = 0; t < strides.size(); ++t) nst[t].push_back(strides[t][d]);
    }
    if (ns.empty()) {
        ns.push_back(1);
        for (auto& s : nst) s.push_back(0);
    }
    shape = ns;
    strides = nst;
}

bool aligned_to(const TensorData& td, int64_t bytes) {
    return ((uintptr_t)td.base_ptr() % (uintptr_t)bytes) == 0;
}

bool can_alias(const TensorData& td, const std::vector<int64_t>& shape, DType out_dt) {
    if (dtype_size(td.dtype) != dtype_size(out_dt)) return false;
    if (td.layout.shape != shape) return false;
    if (!td.layout.is_dense() || td.layout.allocation_overlaps()) return false;
    return td.buf.use_count() <= 1;  // 0: a non-owning alias whose owner allowed the overwrite
}

// ---------------------------------------------------------------------------------------
// element-wise kernel
// ---------------------------------------------------------------------------------------
std::string ew_prog_text(const Program& prog) {
    std::ostringstream s;
    s << "DEV float prog(const float (&x)[NIN][C], int j, const float* imm) {\n";
    for (int i = 0; i < (int)prog.ins.size(); ++i) {
        const Instr& in = prog.ins[i];
        if (in.kind == IKind::Load)
            s << "    float " << vn(i) << " = x[" << in.slot << "][j];\n";
        else
            s << "    float " << vn(i) << " = "
              << instr_expr(in, vn(in.a), in.b >= 0 ? vn(in.b) : std::string()) << ";\n";
    }
    s << "    return " << vn(prog.result) << ";\n}\n";
    return s.str();
}

struct EwConfig {
    int R, C, U, idx64, out_mode;
    std::vector<int> mode;  // per input slot
    int minb = 1;
};

std::string ew_source(const Program& prog, const EwConfig& c) {
    std::ostringstream s;
    s << prelude();
    s << "#define R " << c.R << "\n#define NIN " << prog.n_slots() << "\n#define C " << c.C
      << "\n#define U " << c.U << "\n#define MINB " << c.minb << "\n#define IDX64 " << c.idx64 << "\n#define NIMM "
      << prog.imms.size() << "\n#define OUT_DT " << (int)prog.out_dtype() << "\n#define OUT_MODE "
      << c.out_mode << "\n";
    s << ew_prog_text(prog);
    s << "#define LOAD_INPUTS(off, nvalid, X) \\\n";
    for (int t = 0; t < prog.n_slots(); ++t)
        s << "    load_chunk<" << (int)prog.slot_dtype[t] << ", C, " << c.mode[t]
          << ">((const void*)p.ptr[" << t << "], off[" << t << "], p.stride[" << t
          << " * R + R - 1], nvalid, X[" << t << "]); \\\n";
    s << "\n";
    s << JIT_EW_KERNEL;
    return s.str();
}

}  // namespace

std::string debug_ew_source(const Program& prog, int rank, int chunk) {
    EwConfig c{rank, chunk, 2, 0, chunk > 1 ? 0 : 1, std::vector<int>(prog.n_slots(), chunk > 1 ? 0 : 1)};
    return ew_source(prog, c);
}

// With `try_tiled` only the shared-memory-staged variant is attempted: an empty result means
// that it does not apply.
static TensorData run_elementwise_impl(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                                       const std::vector<int64_t>& shape, int inplace_slot, bool try_tiled = false);

// Operands whose innermost axis is strided (a transposed view) would be read with adjacent
// threads far apart.  When such operands are contiguous along another axis, the kernel stages
// their tiles through shared memory (JIT_EW_TILE_KERNEL); where that variant does not apply
// (operands contiguous along different axes, too many of them) each is first brought into the
// kernel's index order by the tiled-transpose copy, and the private copy may then serve as
// the output buffer.
TensorData run_elementwise(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                           const std::vector<int64_t>& shape, int inplace_slot) {
    int64_t n = 1;
    for (auto v : shape) n *= v;
    if (n < 65536 || shape.empty() || !tune("EW_PRETRANSPOSE", 1)) return run_elementwise_impl(dev, prog, in, shape, inplace_slot);
    if (tune("EW_TILED", 1)) {
        bool transposed = false;
        for (size_t t = 0; t < in.size(); ++t) {
            const Layout& l = in[t].layout;
            const int r = l.rank();
            if (r < 2 || l.shape != shape || l.shape[r - 1] <= 1 || l.strides[r - 1] == 0 || l.strides[r - 1] == 1) continue;
            for (int d = 0; d < r - 1; ++d) transposed |= l.strides[d] == 1 && l.shape[d] >= 8;
        }
        if (transposed) {
            TensorData out = run_elementwise_impl(dev, prog, in, shape, inplace_slot, true);
            if (out.buf) return out;
        }
    }
    std::vector<TensorData> ins;
    for (size_t t = 0; t < in.size(); ++t) {
        const Layout& l = in[t].layout;
        const int r = l.rank();
        bool strided_inner = r >= 2 && l.shape == shape && l.shape[r - 1] > 1 && l.strides[r - 1] != 0 && l.strides[r - 1] != 1;
        bool other_contig = false;
        for (int d = 0; strided_inner && d < r - 1; ++d) other_contig |= l.strides[d] == 1 && l.shape[d] >= 8;
        if (strided_inner && other_contig) {
            if (ins.empty()) ins = in;
            // only the distinct elements are moved: axes of stride 0 stay broadcast
            TensorData core = in[t];
            for (int d = 0; d < r; ++d)
                if (l.strides[d] == 0) core.layout.shape[d] = 1;
            ins[t] = run_compact(dev, core);
            bool broadcast = false;
            for (int d = 0; d < r; ++d)
                if (l.strides[d] == 0 && l.shape[d] > 1) {
                    ins[t].layout.shape[d] = l.shape[d];
                    ins[t].layout.strides[d] = 0;
                    broadcast = true;
                }
            if (inplace_slot < 0 && !broadcast) inplace_slot = (int)t;
        }
    }
    return run_elementwise_impl(dev, prog, ins.empty() ? in : ins, shape, inplace_slot);
}

static TensorData run_elementwise_impl(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                                       const std::vector<int64_t>& shape, int inplace_slot, bool try_tiled) {
    const int nin = prog.n_slots();
    WGF_CHECK((int)in.size() == nin, WGF_ERR_INVALID_ARGUMENT, "input count does not match the program");
    WGF_CHECK(nin >= 1 && nin <= 16, WGF_ERR_UNSUPPORTED, "fused kernel takes 1..16 inputs");
    for (auto& t : in) dev.wait_for(*t.buf);   // inputs still owned by a collective
    const DType out_dt = prog.out_dtype();
    int64_t n = 1;
    for (auto v : shape) n *= v;

    // output: reuse an input's buffer when allowed, else a fresh contiguous buffer
    TensorData out;
    if (inplace_slot >= 0 && can_alias(in[inplace_slot], shape, out_dt)) {
        out = in[inplace_slot];
        out.dtype = out_dt;
    } else {
        out.buf = dev.alloc((size_t)std::max<int64_t>(n, 1) * dtype_size(out_dt), false);
        out.layout = Layout::contiguous(shape);
        out.dtype = out_dt;
    }
    if (n == 0) return out;

    std::vector<int64_t> cshape = shape;
    std::vector<std::vector<int64_t>> st(nin + 1);
    for (int t = 0; t < nin; ++t) {
        WGF_CHECK(in[t].layout.shape == shape, WGF_ERR_SHAPE, "fused input shape differs from the index space");
        st[t] = in[t].layout.strides;
    }
    st[nin] = Layout::contiguous_strides(shape);  // dense output (also when aliased)
    collapse(cshape, st);
    const int R = (int)cshape.size();
    WGF_CHECK(R <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");

    bool any16 = dtype_size(out_dt) == 2;
    for (int t = 0; t < nin; ++t) any16 |= dtype_size(in[t].dtype) == 2;
    EwConfig cfg;
    cfg.R = R;
    cfg.C = any16 ? 8 : 4;
    if (R > 1 && cshape[R - 1] % cfg.C != 0) cfg.C = (any16 && cshape[R - 1] % 4 == 0) ? 4 : 1;
    cfg.idx64 = n >= (1ll << 31);
    auto classify = [&](const TensorData& td, const std::vector<int64_t>& s) {
        int64_t inner = s[R - 1];
        if (inner == 0) return 2;
        if (inner != 1) return 3;
        if (cfg.C == 1) return 1;
        int64_t need = std::min<int64_t>(16, cfg.C * (int64_t)dtype_size(td.dtype));
        if (!aligned_to(td, need)) return 1;
        for (int d = 0; d < R - 1; ++d)
            if ((s[d] * (int64_t)dtype_size(td.dtype)) % need) return 1;
        return 0;
    };
    cfg.mode.resize(nin);
    for (int t = 0; t < nin; ++t) cfg.mode[t] = classify(in[t], st[t]);
    cfg.out_mode = classify(out, st[nin]);

    if (try_tiled) {
        // Operands that are contiguous along another axis than the output (transposed views) are
        // staged through shared memory tile by tile; see JIT_EW_TILE_KERNEL.  All of them must
        // share that axis and allow 16-byte loads along it; 4-byte elements and chunks of 4 only;
        // shared memory holds up to two staged 64 x 64 tiles.
        int pax = -1, nstaged = 0;
        bool ok = R >= 2 && !any16 && cfg.C == 4;
        std::vector<int> sidx(nin, -1);
        for (int t = 0; t < nin && ok; ++t) {
            if (cfg.mode[t] != 3) continue;
            int dc = -1;
            for (int d = 0; d < R - 1; ++d)
                if (st[t][d] == 1 && cshape[d] >= 8) dc = d;
            if (dc < 0) continue;   // stays a strided operand
            if (pax >= 0 && pax != dc) ok = false;
            pax = dc;
            sidx[t] = nstaged++;
            ok = ok && cshape[dc] % 4 == 0 && aligned_to(in[t], 16);
            for (int d = 0; d < R && ok; ++d)
                if (d != dc) ok = st[t][d] % 4 == 0;
        }
        ok = ok && nstaged >= 1 && nstaged <= 2;
        int64_t tiles = 0;
        if (ok) {
            const int64_t tiles_p = (cshape[pax] + 63) / 64, tiles_l = (cshape[R - 1] + 63) / 64;
            tiles = tiles_p * tiles_l;
            for (int d = 0; d < R - 1; ++d) {
                ok = ok && cshape[d] < (1ll << 31);
                if (d != pax) tiles *= cshape[d];
            }
            ok = ok && cshape[R - 1] < (1ll << 31) && tiles < (1ll << 31);
        }
        if (!ok) return TensorData();   // the caller falls back to a transposing copy
        std::ostringstream key;
        key << "ewt|" << R << "|" << cfg.C << "|" << pax << "|" << cfg.out_mode << "|";
        for (int t = 0; t < nin; ++t) key << (sidx[t] >= 0 ? 4 : cfg.mode[t]);
        key << "|" << prog.signature();
        const JitKernel& k = dev.kernel(key.str(), "wgf_elementwise_tiled", [&] {
            std::ostringstream s;
            s << prelude();
            s << "#define R " << R << "\n#define NIN " << nin << "\n#define C " << cfg.C << "\n#define NIMM " << prog.imms.size()
              << "\n#define OUT_DT " << (int)out_dt << "\n#define OUT_MODE " << cfg.out_mode << "\n#define PAX " << pax
              << "\n#define NSTAGED " << nstaged << "\n";
            s << ew_prog_text(prog);
            s << "#define TILE_STAGE \\\n";
            for (int t = 0; t < nin; ++t)
                if (sidx[t] >= 0)
                    s << "    { float4 v_[4]; \\\n"
                      << "      for (int i = 0; i < 4; ++i) { const u32 ll = l0 + r16 + 16 * i; \\\n"
                      << "        v_[i] = (pp < P && ll < L) ? load_f4((const void*)p.ptr[" << t << "], base[" << t
                      << "] + (i64)pp + (i64)ll * p.stride[" << t << " * R + R - 1]) : make_float4(0.f, 0.f, 0.f, 0.f); } \\\n"
                      << "      for (int i = 0; i < 4; ++i) { const int li = r16 + 16 * i; \\\n"
                      << "        stage[" << sidx[t] << "][4 * c16 + 0][li] = v_[i].x; stage[" << sidx[t] << "][4 * c16 + 1][li] = v_[i].y; \\\n"
                      << "        stage[" << sidx[t] << "][4 * c16 + 2][li] = v_[i].z; stage[" << sidx[t] << "][4 * c16 + 3][li] = v_[i].w; } } \\\n";
            s << "\n#define TILE_INPUTS(X) \\\n";
            for (int t = 0; t < nin; ++t) {
                if (sidx[t] >= 0)
                    s << "    for (int j = 0; j < C; ++j) X[" << t << "][j] = stage[" << sidx[t] << "][pi][tx * C + j]; \\\n";
                else
                    s << "    load_chunk<" << (int)prog.slot_dtype[t] << ", C, " << cfg.mode[t] << ">((const void*)p.ptr[" << t
                      << "], base[" << t << "] + (i64)pp * p.stride[" << t << " * R + PAX] + (i64)l * p.stride[" << t
                      << " * R + R - 1], p.stride[" << t << " * R + R - 1], nvalid, X[" << t << "]); \\\n";
            }
            s << "\n";
            s << JIT_EW_TILE_KERNEL;
            return s.str();
        });
        ParamWriter w;
        for (int t = 0; t < nin; ++t) w.put<uint64_t>((uint64_t)(uintptr_t)in[t].base_ptr());
        w.put<uint64_t>((uint64_t)(uintptr_t)out.base_ptr());
        for (int t = 0; t <= nin; ++t)
            for (int d = 0; d < R; ++d) w.put<int64_t>(st[t][d]);
        for (int d = 0; d < R; ++d) w.put<uint32_t>((uint32_t)cshape[d]);
        w.put<uint32_t>((uint32_t)((cshape[pax] + 63) / 64));
        w.put<uint32_t>((uint32_t)((cshape[R - 1] + 63) / 64));
        for (float f : prog.imms) w.put<float>(f);
        if (prog.imms.empty()) w.put<float>(0.f);
        w.finish();
        bind_checked(dev, in, out);
        dev.launch(k, dim3((unsigned)tiles), dim3(256), 0, w.bytes.data(), "elementwise_tiled");
        return out;
    }
    const int64_t nchunks = (n + cfg.C - 1) / cfg.C;
    // U chunks per thread are loaded before the first is used, at most EW_BUDGET input values
    // held as floats.  Measured on B200: 16 beats 32 and 64 on every chain with two or more
    // inputs or 16-bit elements (f16 a+b 142 -> 83 us, f16 silu(a)*b 277 -> 120 us on
    // [8192,11008]): residency of more CTAs hides latency better than deeper unrolling.
    int umax = std::max(1, std::min(4, tune("EW_BUDGET", 16) / (nin * cfg.C)));
    int64_t want = nchunks / (256ll * 4 * dev.sm_count);
    cfg.U = (int)std::max<int64_t>(1, std::min<int64_t>(umax, want));
    cfg.minb = tune("EW_MINB", 1);

    std::ostringstream key;
    key << "ew|" << R << "|" << cfg.C << "|" << cfg.U << "|" << cfg.minb << "|" << cfg.idx64 << "|" << cfg.out_mode << "|";
    for (int m : cfg.mode) key << m;
    key << "|" << prog.signature();
    const JitKernel& k = dev.kernel(key.str(), "wgf_elementwise", [&] { return ew_source(prog, cfg); });

    ParamWriter w;
    w.put<uint64_t>((uint64_t)n);
    for (int t = 0; t < nin; ++t) w.put<uint64_t>((uint64_t)(uintptr_t)in[t].base_ptr());
    w.put<uint64_t>((uint64_t)(uintptr_t)out.base_ptr());
    for (int t = 0; t < nin; ++t)
        for (int d = 0; d < R; ++d) w.put<int64_t>(st[t][d]);
    for (int d = 0; d < R; ++d) w.put<uint32_t>((uint32_t)cshape[d]);
    std::vector<uint32_t> mm(R), ms(R);
    for (int d = 0; d < R; ++d) magic_for((uint32_t)std::min<int64_t>(cshape[d], 0x7fffffff), mm[d], ms[d]);
    for (int d = 0; d < R; ++d) w.put<uint32_t>(mm[d]);
    for (int d = 0; d < R; ++d) w.put<uint32_t>(ms[d]);
    for (float f : prog.imms) w.put<float>(f);
    if (prog.imms.empty()) w.put<float>(0.f);
    w.finish();

    int64_t blocks = (nchunks + 256ll * cfg.U - 1) / (256ll * cfg.U);
    WGF_CHECK(blocks < (1ll << 31), WGF_ERR_UNSUPPORTED, "tensor too large for one launch");
    bind_checked(dev, in, out);
    dev.launch(k, dim3((unsigned)blocks), dim3(256), 0, w.bytes.data(), "elementwise");
    return out;
}

// ---------------------------------------------------------------------------------------
// row kernels
// ---------------------------------------------------------------------------------------
namespace {

struct RowConfig {
    int RO, C, NCH, GROUP, RPC, out_mode, minb;
    bool out_has_h, prefetch;
    std::vector<int> mode;       // per slot: 0 vec, 1 scalar, 3 strided; 2 = row value (cstride 0)
    std::vector<char> invariant; // per slot: does not depend on the row (all outer strides 0)
};

void replace_all(std::string& text, const std::string& marker, const std::string& with) {
    size_t at = 0;
    while ((at = text.find(marker, at)) != std::string::npos) {
        text.replace(at, marker.size(), with);
        at += with.size();
    }
}

std::string row_source(const Program& prog_in, const RowConfig& c) {
    Program prog = prog_in;
    prog.mark_sum_only();   // exps that only feed sums
    std::ostringstream s;
    s << prelude();
    s << "#define RO " << c.RO << "\n#define NIN " << prog.n_slots() << "\n#define C " << c.C
      << "\n#define NCH " << c.NCH << "\n#define GROUP " << c.GROUP << "\n#define RPC " << c.RPC
      << "\n#define NRED " << prog.n_reduces() << "\n#define NIMM " << prog.imms.size()
      << "\n#define MINB " << c.minb << "\n#define NGRAND " << prog.grands.size() << "\n";
    // inv: loaded once per CTA; decl/pre/take: double-buffered per-row loads; b: per-row body
    std::ostringstream inv, decl, pre, take, b;
    int red_idx = 0;
    auto operand = [&](int i, const char* idx) {
        return prog.ins[i].vk == VKind::Row ? vn(i) : vn(i) + "[" + idx + "]";
    };
    // text of a whole-row load of slot t into array `dst`, guarded by `valid[k]`, row offset `off`
    auto row_load = [&](std::ostringstream& o, int t, const std::string& dst, const char* valid, const std::string& off) {
        o << "\n#pragma unroll\n for (int k = 0; k < NCH; ++k) {\n"
          << "  if (" << valid << "[k]) load_chunk<" << (int)prog.slot_dtype[t] << ", C, " << c.mode[t]
          << ">((const void*)p.ptr[" << t << "], " << off << " + (i64)((k * GROUP + t) * C) * "
          << (c.mode[t] == 3 ? "p.cstride[" + std::to_string(t) + "]" : std::string("1"))
          << ", p.cstride[" << t << "], C, &" << dst << "[k * C]);\n"
          << "  else { \n#pragma unroll\n for (int j = 0; j < C; ++j) " << dst << "[k * C + j] = 0.f; }\n}\n";
    };
    for (int i = 0; i < (int)prog.ins.size(); ++i) {
        const Instr& in = prog.ins[i];
        if (in.kind == IKind::Load) {
            int t = in.slot;
            std::string dt = std::to_string((int)prog.slot_dtype[t]);
            if (in.vk == VKind::Row) {
                if (c.invariant[t])
                    inv << "const float " << vn(i) << " = load1<" << dt << ">((const void*)p.ptr[" << t << "], 0);\n";
                else
                    b << "float " << vn(i) << " = crv ? load1<" << dt << ">((const void*)p.ptr[" << t << "], coff["
                      << t << "]) : 0.f;\n";
            } else if (c.invariant[t]) {
                inv << "float " << vn(i) << "[EPT];\n";
                row_load(inv, t, vn(i), "cv", "(i64)0");
            } else if (!c.prefetch) {
                take << "float " << vn(i) << "[EPT];\n";
                row_load(take, t, vn(i), "kv", "coff[" + std::to_string(t) + "]");
            } else {
                // next-row buffer n<i>, filled ahead of the reductions of the current row
                decl << "float n" << i << "[EPT];\n";
                pre << "if (rv) {";
                row_load(pre, t, "n" + std::to_string(i), "cv", "roff[" + std::to_string(t) + "]");
                pre << "}\n";
                take << "float " << vn(i) << "[EPT];\n#pragma unroll\n for (int e = 0; e < EPT; ++e) " << vn(i)
                     << "[e] = n" << i << "[e];\n";
            }
        } else if (in.kind == IKind::RowReduce) {
            const char* op = red_name(in.op);
            b << "float " << vn(i) << ";\n{ float a_ = red_ident<" << op << ">();\n"
              << "\n#pragma unroll\n for (int k = 0; k < NCH; ++k) if (kv[k]) {\n"
              << "  \n#pragma unroll\n for (int j = 0; j < C; ++j) a_ = red_comb<" << op << ">(a_, "
              << operand(in.a, "k * C + j") << "); }\n";
            if (c.GROUP > 32)
                b << vn(i) << " = group_reduce<" << op << ", GROUP>(a_, red_smem[" << red_idx << "][g], t); }\n";
            else
                b << vn(i) << " = group_reduce<" << op << ", GROUP>(a_, (float*)0, t); }\n";
            if (in.dtype != DType::F32) b << vn(i) << " = " << rounded(in.dtype, vn(i)) << ";\n";
            red_idx++;
        } else if (in.vk == VKind::Row) {
            b << "float " << vn(i) << " = " << instr_expr(in, vn(in.a), in.b >= 0 ? vn(in.b) : std::string())
              << ";\n";
        } else if (in.kind == IKind::Binary && in.op == WGF_OP_DIV && prog.ins[in.b].vk == VKind::Row) {
            // a row of values divided by one per-row value: one correctly rounded reciprocal per
            // row and a multiply per element (<= 2 ulp from the quotient) instead of an IEEE
            // division per element, which would make the kernel instruction-bound
            b << "const float q" << i << " = 1.0f / " << vn(in.b) << ";\nfloat " << vn(i)
              << "[EPT];\n\n#pragma unroll\n for (int e = 0; e < EPT; ++e) " << vn(i) << "[e] = "
              << rounded(in.dtype, "(" + operand(in.a, "e") + " * q" + std::to_string(i) + ")") << ";\n";
        } else {
            b << "float " << vn(i) << "[EPT];\n\n#pragma unroll\n for (int e = 0; e < EPT; ++e) " << vn(i)
              << "[e] = " << instr_expr(in, operand(in.a, "e"), in.b >= 0 ? operand(in.b, "e") : std::string())
              << ";\n";
        }
    }
    const int res = prog.result;
    const int odt = (int)prog.out_dtype();
    if (c.out_has_h) {
        b << "\n#pragma unroll\n for (int k = 0; k < NCH; ++k) if (kv[k]) {\n";
        if (prog.ins[res].vk == VKind::Row) {
            b << "  float y_[C]; \n#pragma unroll\n for (int j = 0; j < C; ++j) y_[j] = " << vn(res) << ";\n"
              << "  store_chunk<" << odt << ", C, " << c.out_mode << ">((void*)p.ptr[NIN], coff[NIN] + (i64)((k * GROUP + t) * C), C, y_);\n";
        } else {
            b << "  store_chunk<" << odt << ", C, " << c.out_mode
              << ">((void*)p.ptr[NIN], coff[NIN] + (i64)((k * GROUP + t) * C), C, &" << vn(res) << "[k * C]);\n";
        }
        b << "}\n";
    } else {
        b << "if (crv && t == 0) store1<" << odt << ">((void*)p.ptr[NIN], coff[NIN], " << vn(res) << ");\n";
    }
    // companion whole-tensor reductions: accumulated per thread over all its rows
    std::ostringstream gblock, gput, gfinish;
    for (int gi = 0; gi < (int)prog.grands.size(); ++gi) {
        const Grand& gr = prog.grands[gi];
        const char* op = red_name(gr.op);
        const std::string id = std::to_string(gi);
        inv << "float ga" << id << " = red_ident<" << op << ">();\n";
        b << "\n#pragma unroll\n for (int k = 0; k < NCH; ++k) if (kv[k]) {\n"
          << "  \n#pragma unroll\n for (int j = 0; j < C; ++j) ga" << id << " = red_comb<" << op << ">(ga" << id << ", "
          << operand(gr.a, "k * C + j") << "); }\n";
        gblock << "const float gp" << id << " = group_reduce<" << op << ", THREADS>(ga" << id << ", g_smem[" << id
               << "], (int)threadIdx.x);\n";
        gput << "gpart[(u64)blockIdx.x * NGRAND + " << id << "] = gp" << id << ";\n";
        gfinish << "{ float a_ = red_ident<" << op << ">();\n"
                << "  for (u32 b_ = threadIdx.x; b_ < gridDim.x; b_ += THREADS) a_ = red_comb<" << op
                << ">(a_, __ldcg(gpart + (u64)b_ * NGRAND + " << id << "));\n"
                << "  __syncthreads();\n  a_ = group_reduce<" << op << ", THREADS>(a_, g_smem[" << id
                << "], (int)threadIdx.x);\n  if (threadIdx.x == 0) {\n";
        gfinish << "    store1<" << (int)gr.dtype << ">((void*)p.gout[" << id << "], 0, a_); } }\n";
    }
    // A group_reduce reuses its shared-memory slot in the next iteration: all reads of this
    // iteration must be done before the next row writes.
    // (with two or more reductions the barrier of the second one already orders that)
    if (c.GROUP > 32 && prog.n_reduces() == 1) b << "__syncthreads();\n";
    std::string tmpl = JIT_ROW_KERNEL;
    replace_all(tmpl, "ROW_GRAND_BLOCK", gblock.str());
    replace_all(tmpl, "ROW_GRAND_PUT", gput.str());
    replace_all(tmpl, "ROW_GRAND_FINISH", gfinish.str());
    bool posts = false;
    for (const Grand& gr : prog.grands) posts = posts || gr.all_reduce;
    // A kernel whose values are all-reduced stores this GPU's values like any other; it posts the
    // values of the exchange before its own first thing, and its last CTA settles the oldest open
    // exchange around its share of the rows (see Comm).
    replace_all(tmpl, "ROW_GRAND_POST", posts ? "PEER_POST(p) PEER_PEEK(p)" : "");
    replace_all(tmpl, "ROW_GRAND_SETTLE", posts ? "PEER_SETTLE(p)" : "");
    replace_all(tmpl, "ROW_INVARIANT", inv.str());
    replace_all(tmpl, "ROW_NEXT_DECL", decl.str());
    replace_all(tmpl, "ROW_PREFETCH", pre.str());
    replace_all(tmpl, "ROW_TAKE", take.str());
    replace_all(tmpl, "ROW_BODY", b.str());
    s << tmpl;
    return s.str();
}

struct StreamConfig {
    int RO, C, U, minb;
    std::vector<int> mode;
};

std::string stream_source(const Program& prog_in, const StreamConfig& c) {
    Program prog = prog_in;
    prog.mark_sum_only();   // exps that only feed sums
    const int n = (int)prog.ins.size();
    std::vector<char> dep(n, 0);
    for (int i = 0; i < n; ++i) {
        const Instr& in = prog.ins[i];
        char d = in.kind == IKind::RowReduce;
        if (in.a >= 0) d |= dep[in.a];
        if (in.b >= 0) d |= dep[in.b];
        dep[i] = d;
    }
    // slots read per element, in slot order
    std::vector<int> eslot(prog.n_slots(), -1);
    int nine = 0;
    for (auto& in : prog.ins)
        if (in.kind == IKind::Load && in.vk == VKind::Elem) eslot[in.slot] = 0;
    for (int t = 0; t < prog.n_slots(); ++t)
        if (eslot[t] == 0) eslot[t] = nine++;
    std::vector<int> rowv_index(n, -1);
    int nrowv = 0;
    std::ostringstream pre, elem, post, init, comb, blk, load;
    int red_idx = 0;
    std::vector<int> red_of(n, -1);
    for (int i = 0; i < n; ++i) {
        const Instr& in = prog.ins[i];
        std::string a = in.a >= 0 ? vn(in.a) : "", bb = in.b >= 0 ? vn(in.b) : "";
        if (in.kind == IKind::RowReduce) {
            const char* op = red_name(in.op);
            red_of[i] = red_idx;
            // accumulate inside the element loop
            std::string src = prog.ins[in.a].vk == VKind::Row && !dep[in.a]
                                  ? "rowv[" + std::to_string(rowv_index[in.a]) + "]" : vn(in.a);
            elem << "        acc[" << red_idx << "] = red_comb<" << op << ">(acc[" << red_idx << "], " << src << ");\n";
            init << "acc[" << red_idx << "] = red_ident<" << op << ">(); ";
            comb << "acc[" << red_idx << "] = red_comb<" << op << ">(acc[" << red_idx << "], __ldcg((PP) + "
                 << red_idx << ")); ";
            blk << "acc[" << red_idx << "] = group_reduce<" << op << ", THREADS>(acc[" << red_idx << "], red_smem["
                << red_idx << "], t); ";
            post << "float " << vn(i) << " = " << rounded(in.dtype, "acc[" + std::to_string(red_idx) + "]") << "; ";
            red_idx++;
        } else if (in.vk == VKind::Row && !dep[i]) {
            if (in.kind == IKind::Load)
                pre << "float " << vn(i) << " = load1<" << (int)prog.slot_dtype[in.slot] << ">((const void*)p.ptr["
                    << in.slot << "], roff[" << in.slot << "]); ";
            else
                pre << "float " << vn(i) << " = " << instr_expr(in, a, bb) << "; ";
            rowv_index[i] = nrowv++;
        } else if (in.vk == VKind::Row) {
            post << "float " << vn(i) << " = " << instr_expr(in, a, bb) << "; ";
        } else {
            auto opnd = [&](int j) {
                if (prog.ins[j].vk == VKind::Row) return "rowv[" + std::to_string(rowv_index[j]) + "]";
                return vn(j);
            };
            if (in.kind == IKind::Load)
                elem << "        float " << vn(i) << " = x[" << eslot[in.slot] << "][j];\n";
            else
                elem << "        float " << vn(i) << " = "
                     << instr_expr(in, opnd(in.a), in.b >= 0 ? opnd(in.b) : std::string()) << ";\n";
        }
    }
    for (int t = 0; t < prog.n_slots(); ++t)
        if (eslot[t] >= 0)
            load << "load_chunk<" << (int)prog.slot_dtype[t] << ", C, " << c.mode[t] << ">((const void*)p.ptr[" << t
                 << "], roff[" << t << "] + (i64)(COL) * " << (c.mode[t] == 3 ? "p.cstride[" + std::to_string(t) + "]" : std::string("1"))
                 << ", p.cstride[" << t << "], NV, X[" << eslot[t] << "]); ";

    std::ostringstream s;
    s << prelude();
    s << "#define RO " << c.RO << "\n#define NIN " << prog.n_slots() << "\n#define NINE " << nine
      << "\n#define C " << c.C << "\n#define U " << c.U << "\n#define NRED " << prog.n_reduces()
      << "\n#define NIMM " << prog.imms.size() << "\n#define MINB " << c.minb << "\n";
    s << "DEV void elem_phase(const float (&x)[NINE > 0 ? NINE : 1][C], const float* rowv, const float* imm, int nvalid, float* acc) {\n"
      // full chunks (all but the ragged end of a row) take a path without per-element predicates
      << "  if (nvalid == C) {\n#pragma unroll\n    for (int j = 0; j < C; ++j) {\n" << elem.str() << "    }\n  } else {\n"
      << "#pragma unroll\n    for (int j = 0; j < C; ++j) {\n      if (j < nvalid) {\n"
      << elem.str() << "      }\n    }\n  }\n}\n";
    s << "#define STREAM_PRE " << pre.str() << " float rowv[" << std::max(nrowv, 1) << "]; ";
    if (nrowv == 0) s << "rowv[0] = 0.f; ";
    for (int i = 0; i < n; ++i)
        if (rowv_index[i] >= 0) s << "rowv[" << rowv_index[i] << "] = " << vn(i) << "; ";
    s << "\n#define STREAM_INIT " << init.str() << "\n";
    s << "#define STREAM_COMBINE_PARTIAL(PP) " << comb.str() << "\n";
    s << "#define STREAM_BLOCK_REDUCE " << blk.str() << "\n";
    s << "#define STREAM_LOAD(COL, NV, X) " << load.str() << "\n";
    s << "#define STREAM_AR " << (prog.result_all_reduce ? 1 : 0) << "\n";
    s << "#define STREAM_POST " << post.str() << " if (t == 0) { float r_ = " << vn(prog.result) << "; ";
    s << "store1<" << (int)prog.out_dtype() << ">((void*)p.ptr[NIN], roff[NIN], r_); }\n";
    s << JIT_STREAM_KERNEL;
    return s.str();
}

// ---- column reduce: reduced axis is not the innermost one --------------------------------
struct ColConfig {
    int C, U, out_mode;
    int TX = 32;                // threads along the contiguous axis per CTA (256 / TX thread rows share K)
    std::vector<int> mode;      // per slot: 0 vector, 1 scalar, 2 one value for all columns
    std::vector<char> is_row;   // per slot: does not vary along the reduced axis
};

std::string col_source(const Program& prog_in, const ColConfig& c) {
    Program prog = prog_in;
    prog.mark_sum_only();   // exps that only feed sums
    const int n = (int)prog.ins.size();
    std::vector<char> dep(n, 0);
    for (int i = 0; i < n; ++i) {
        const Instr& in = prog.ins[i];
        char d = in.kind == IKind::RowReduce;
        if (in.a >= 0) d |= dep[in.a];
        if (in.b >= 0) d |= dep[in.b];
        dep[i] = d;
    }
    std::vector<int> eslot(prog.n_slots(), -1), rslot(prog.n_slots(), -1);
    int nine = 0, nrowl = 0;
    for (int t = 0; t < prog.n_slots(); ++t) {
        if (c.is_row[t]) rslot[t] = nrowl++;
        else eslot[t] = nine++;
    }
    std::vector<int> pre_index(n, -1);
    int npre = 0, red_idx = 0;
    std::ostringstream pre, elem, post, init, comb, sadd;
    auto opnd_elem = [&](int j) {
        return prog.ins[j].vk == VKind::Row ? "rv[" + std::to_string(pre_index[j]) + "]" : vn(j);
    };
    auto opnd_post = [&](int j) { return pre_index[j] >= 0 ? "rv[" + std::to_string(pre_index[j]) + "]" : vn(j); };
    for (int i = 0; i < n; ++i) {
        const Instr& in = prog.ins[i];
        if (in.kind == IKind::RowReduce) {
            const char* op = red_name(in.op);
            elem << "    a[" << red_idx << "] = red_comb<" << op << ">(a[" << red_idx << "], " << opnd_elem(in.a) << ");\n";
            init << "acc[" << red_idx << "][J] = red_ident<" << op << ">(); ";
            comb << "acc[" << red_idx << "][J] = red_comb<" << op << ">(acc[" << red_idx << "][J], __ldcg((PP) + "
                 << red_idx << " * (STRIDE) + J)); ";
            sadd << "acc[" << red_idx << "][J] = red_comb<" << op << ">(acc[" << red_idx << "][J], red[" << red_idx
                 << "][W][tx * C + J]); ";
            post << "    float " << vn(i) << " = " << rounded(in.dtype, "a[" + std::to_string(red_idx) + "]") << ";\n";
            red_idx++;
        } else if (in.vk == VKind::Row && !dep[i]) {
            if (in.kind == IKind::Load)
                pre << "    float " << vn(i) << " = rl[" << rslot[in.slot] << "];\n";
            else
                pre << "    float " << vn(i) << " = " << instr_expr(in, vn(in.a), in.b >= 0 ? vn(in.b) : std::string()) << ";\n";
            pre_index[i] = npre++;
            pre << "    rv[" << pre_index[i] << "] = " << vn(i) << ";\n";
        } else if (in.vk == VKind::Row) {
            post << "    float " << vn(i) << " = "
                 << instr_expr(in, opnd_post(in.a), in.b >= 0 ? opnd_post(in.b) : std::string()) << ";\n";
        } else if (in.kind == IKind::Load) {
            elem << "    float " << vn(i) << " = xe[" << eslot[in.slot] << "];\n";
        } else {
            elem << "    float " << vn(i) << " = "
                 << instr_expr(in, opnd_elem(in.a), in.b >= 0 ? opnd_elem(in.b) : std::string()) << ";\n";
        }
    }
    std::ostringstream le, lr;
    for (int t = 0; t < prog.n_slots(); ++t) {
        std::ostringstream& o = c.is_row[t] ? lr : le;
        o << "load_chunk<" << (int)prog.slot_dtype[t] << ", C, " << c.mode[t] << ">((const void*)p.ptr[" << t
          << "], (i64)o * p.so[" << t << "] + " << (c.is_row[t] ? std::string("0") : "(i64)(KK) * p.sk[" + std::to_string(t) + "]")
          << " + " << (c.mode[t] == 2 ? "0" : "(i64)col") << ", 1, C, X[" << (c.is_row[t] ? rslot[t] : eslot[t]) << "]); ";
    }
    std::ostringstream s;
    s << prelude();
    s << "#define NIN " << prog.n_slots() << "\n#define NINE " << nine << "\n#define NROWL " << nrowl << "\n#define NPRE "
      << npre << "\n#define C " << c.C << "\n#define U " << c.U << "\n#define TX " << c.TX << "\n#define TY " << 256 / c.TX
      << "\n#define NRED " << prog.n_reduces() << "\n#define NIMM "
      << prog.imms.size() << "\n#define OUT_DT " << (int)prog.out_dtype() << "\n#define OUT_MODE " << c.out_mode << "\n";
    s << "DEV void pre_phase(const float* rl, const float* imm, float* rv) {\n" << pre.str() << "}\n";
    s << "DEV void elem_phase(const float* xe, const float* rv, const float* imm, float* a) {\n" << elem.str() << "}\n";
    s << "DEV float post_phase(const float* a, const float* rv, const float* imm) {\n" << post.str() << "    return "
      << opnd_post(prog.result) << ";\n}\n";
    s << "#define COL_INIT(J) " << init.str() << "\n";
    s << "#define COL_COMB(J, PP, STRIDE) " << comb.str() << "\n";
    s << "#define COL_SMEM_ADD(J, W) " << sadd.str() << "\n";
    s << "#define COL_LOAD_ELEM(KK, X) " << le.str() << "\n";
    s << "#define COL_LOAD_ROW(X) " << lr.str() << "\n";
    s << JIT_COL_KERNEL;
    return s.str();
}

}  // namespace

int64_t max_resident_row(bool) { return 32768; }

TensorData run_rows(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                    const std::vector<int64_t>& shape, bool out_has_h, int inplace_slot,
                    std::vector<TensorData>* grand_out, const GrandComm* gc) {
    const int nin = prog.n_slots();
    WGF_CHECK((int)in.size() == nin, WGF_ERR_INVALID_ARGUMENT, "input count does not match the program");
    WGF_CHECK(nin >= 1 && nin <= 16, WGF_ERR_UNSUPPORTED, "fused kernel takes 1..16 inputs");
    for (auto& t : in) dev.wait_for(*t.buf);   // inputs still owned by a collective
    WGF_CHECK(!shape.empty(), WGF_ERR_RANK, "row kernel needs rank >= 1");
    WGF_CHECK(prog.grands.empty() || (out_has_h && grand_out && prog.grands.size() <= 4), WGF_ERR_INVALID_ARGUMENT,
              "companion reductions need a per-element result");
    WGF_CHECK(out_has_h || prog.out_kind() == VKind::Row, WGF_ERR_INVALID_ARGUMENT,
              "a per-element result needs an output with the row axis");
    const DType out_dt = prog.out_dtype();
    const int rank = (int)shape.size();
    const int64_t H = shape[rank - 1];
    std::vector<int64_t> oshape(shape.begin(), shape.end() - 1);
    int64_t rows = 1;
    for (auto v : oshape) rows *= v;
    const std::vector<int64_t>& out_shape = out_has_h ? shape : oshape;
    int64_t n_out = out_has_h ? rows * H : rows;

    TensorData out;
    if (out_has_h && inplace_slot >= 0 && can_alias(in[inplace_slot], shape, out_dt)) {
        out = in[inplace_slot];
        out.dtype = out_dt;
    } else {
        out.buf = dev.alloc((size_t)std::max<int64_t>(n_out, 1) * dtype_size(out_dt), false);
        out.layout = Layout::contiguous(out_shape);
        out.dtype = out_dt;
    }
    WGF_CHECK(prog.grands.empty() || n_out > 0, WGF_ERR_INVALID_ARGUMENT, "companion reductions over an empty index space");
    if (n_out == 0) return out;
    WGF_CHECK(rows < (1ll << 31), WGF_ERR_UNSUPPORTED, "too many rows for one launch");

    // outer strides per tensor (+ output), collapsed; column strides kept apart
    std::vector<std::vector<int64_t>> st(nin + 1);
    std::vector<int64_t> cs(nin + 1);
    for (int t = 0; t < nin; ++t) {
        WGF_CHECK(in[t].layout.shape == shape, WGF_ERR_SHAPE, "fused input shape differs from the index space");
        st[t].assign(in[t].layout.strides.begin(), in[t].layout.strides.end() - 1);
        cs[t] = H == 1 ? 0 : in[t].layout.strides[rank - 1];
    }
    {
        std::vector<int64_t> os = Layout::contiguous_strides(out_shape);
        st[nin].assign(os.begin(), os.begin() + (rank - 1));
        cs[nin] = out_has_h ? 1 : 0;
    }
    std::vector<int64_t> coshape = oshape;
    collapse(coshape, st);
    const int RO = (int)coshape.size();

    // which slots are per-row values
    std::vector<char> slot_row(nin, 0);
    for (auto& i : prog.ins)
        if (i.kind == IKind::Load) slot_row[i.slot] = i.vk == VKind::Row;
    for (int t = 0; t < nin; ++t)
        WGF_CHECK(!slot_row[t] || cs[t] == 0 || H == 1, WGF_ERR_INVALID_ARGUMENT, "row-kind slot varies along the row");

    bool any16 = dtype_size(out_dt) == 2;
    for (int t = 0; t < nin; ++t) any16 |= dtype_size(in[t].dtype) == 2;
    auto vec_ok = [&](const void* base, DType dt, const std::vector<int64_t>& s, int C) {
        int64_t need = std::min<int64_t>(16, C * (int64_t)dtype_size(dt));
        if ((uintptr_t)base % (uintptr_t)need) return false;
        for (int d = 0; d < RO; ++d)
            if (coshape[d] > 1 && (s[d] * (int64_t)dtype_size(dt)) % need) return false;
        return true;
    };
    auto pick_modes = [&](int C, std::vector<int>& mode, int& out_mode, bool need_divisible) {
        bool all_vec = C > 1 && (!need_divisible || H % C == 0);
        mode.assign(nin, 1);
        for (int t = 0; t < nin; ++t) {
            if (slot_row[t] || cs[t] == 0) mode[t] = 2;
            else if (cs[t] != 1) mode[t] = 3;
            else if (all_vec && vec_ok(in[t].base_ptr(), in[t].dtype, st[t], C)) mode[t] = 0;
            else { mode[t] = 1; all_vec = false; }
        }
        out_mode = 1;
        if (out_has_h) {
            if (all_vec && vec_ok(out.base_ptr(), out_dt, st[nin], C)) out_mode = 0;
            else all_vec = false;
        }
        return all_vec;
    };

    const bool single_phase = !prog.multi_phase() && !out_has_h;

    // ---- column reduce: the reduced axis is strided and the last kept axis is the contiguous one
    if (single_phase && (RO == 1 || RO == 2) && H >= 1 && tune("COL_REDUCE", 1)) {
        const int64_t I = coshape[RO - 1], O = RO == 2 ? coshape[0] : 1;
        bool ok = I >= 32 && O <= 65535, any_contig = false;
        for (int t = 0; t < nin && ok; ++t) {
            const int64_t si = st[t][RO - 1];
            if (si != 0 && si != 1) ok = false;
            if (!slot_row[t] && si == 1 && cs[t] != 1) any_contig = true;
            if (!slot_row[t] && cs[t] == 1 && H > 1) ok = false;   // contiguous along the reduced axis: row kernels
        }
        if (ok && any_contig) {
            ColConfig cfg;
            cfg.is_row.assign(slot_row.begin(), slot_row.end());
            cfg.C = any16 ? 8 : 4;
            auto col_vec_ok = [&](const void* base, DType dt, int64_t so, int64_t sk, int C) {
                const int64_t need = std::min<int64_t>(16, C * (int64_t)dtype_size(dt));
                if ((uintptr_t)base % (uintptr_t)need) return false;
                const int64_t es = (int64_t)dtype_size(dt);
                return (O == 1 || (so * es) % need == 0) && (H == 1 || (sk * es) % need == 0);
            };
            auto pick = [&](int C) {
                bool all_vec = C > 1 && I % C == 0;
                cfg.mode.assign(nin, 1);
                for (int t = 0; t < nin; ++t) {
                    const int64_t si = st[t][RO - 1], so = RO == 2 ? st[t][0] : 0;
                    if (si == 0) cfg.mode[t] = 2;
                    else if (all_vec && col_vec_ok(in[t].base_ptr(), in[t].dtype, so, slot_row[t] ? 0 : cs[t], C)) cfg.mode[t] = 0;
                    else all_vec = false;
                }
                cfg.out_mode = 1;
                if (all_vec && col_vec_ok(out.base_ptr(), out_dt, I, 0, C)) cfg.out_mode = 0;
                else all_vec = false;
                return all_vec;
            };
            if (!pick(cfg.C)) {
                cfg.C = 1;
                pick(1);
            }
            int nine = 0;
            for (int t = 0; t < nin; ++t) nine += !slot_row[t];
            cfg.U = std::max(1, std::min(tune("COL_U", 4), tune("COL_BUDGET", 32) / (std::max(nine, 1) * cfg.C)));
            // measured on f32 [8192,4096].sum(0): 64 threads along the row and 4 thread rows
            // 32.2 us; 32 x 8: 38.0; 128 x 2: 37.0; 256 x 1: 44.1
            cfg.TX = tune("COL_TX", I >= 64ll * cfg.C ? 64 : 32);
            std::ostringstream key;
            key << "col|" << cfg.C << "|" << cfg.U << "|" << cfg.TX << "|" << cfg.out_mode << "|";
            for (int m : cfg.mode) key << m;
            key << "|";
            for (int v : cfg.is_row) key << v;
            key << "|" << prog.signature();
            const JitKernel& k = dev.kernel(key.str(), "wgf_col_reduce", [&] { return col_source(prog, cfg); });
            const int64_t tiles = (I + (int64_t)cfg.TX * cfg.C - 1) / ((int64_t)cfg.TX * cfg.C);
            int64_t split = std::max<int64_t>(1, ((int64_t)dev.sm_count * 4 + tiles * O - 1) / (tiles * O));
            split = std::min<int64_t>(split, std::max<int64_t>(1, H / 64));
            if (tiles * O > Device::kCounters || tiles > 65535 * 32768ll) split = 1;
            split = std::min<int64_t>(split, 65535);
            int64_t kper = (H + split - 1) / split;
            kper = (kper + 7) / 8 * 8;
            split = (H + kper - 1) / kper;
            BufferRef partials;
            if (split > 1)
                partials = dev.alloc((size_t)(prog.n_reduces() * O * split * I) * sizeof(float), false);
            ParamWriter w;
            w.put<uint64_t>((uint64_t)O);
            w.put<uint64_t>((uint64_t)H);
            w.put<uint64_t>((uint64_t)I);
            for (int t = 0; t < nin; ++t) w.put<uint64_t>((uint64_t)(uintptr_t)in[t].base_ptr());
            w.put<uint64_t>((uint64_t)(uintptr_t)out.base_ptr());
            for (int t = 0; t <= nin; ++t) w.put<int64_t>(RO == 2 ? st[t][0] : 0);
            for (int t = 0; t <= nin; ++t) w.put<int64_t>(cs[t]);
            w.put<uint64_t>(partials ? (uint64_t)(uintptr_t)partials->ptr : 0);
            w.put<uint64_t>((uint64_t)(uintptr_t)dev.counters());
            w.put<uint32_t>((uint32_t)split);
            w.put<uint32_t>((uint32_t)kper);
            for (float f : prog.imms) w.put<float>(f);
            if (prog.imms.empty()) w.put<float>(0.f);
            w.finish();
            bind_checked(dev, in, out);
            dev.launch(k, dim3((unsigned)tiles, (unsigned)split, (unsigned)O), dim3(cfg.TX, 256 / cfg.TX), 0, w.bytes.data(), "col_reduce");
            return out;
        }
    }

    bool use_stream = false;
    if (single_phase) {
        // enough rows to fill the machine and a row short enough for registers -> resident
        bool resident_ok = H >= 1 && H <= 8192 && rows >= 4ll * dev.sm_count;
        use_stream = !resident_ok;
    } else {
        WGF_CHECK(H <= max_resident_row(any16), WGF_ERR_UNSUPPORTED, "row too long for a row-fused kernel");
    }

    WGF_CHECK(!prog.result_all_reduce || use_stream, WGF_ERR_UNSUPPORTED, "in-kernel all-reduce is part of the streaming reduction only");

    auto put_common = [&](ParamWriter& w) {
        w.put<uint64_t>((uint64_t)rows);
        for (int t = 0; t < nin; ++t) w.put<uint64_t>((uint64_t)(uintptr_t)in[t].base_ptr());
        w.put<uint64_t>((uint64_t)(uintptr_t)out.base_ptr());
        for (int t = 0; t <= nin; ++t)
            for (int d = 0; d < RO; ++d) w.put<int64_t>(st[t][d]);
        for (int t = 0; t <= nin; ++t) w.put<int64_t>(cs[t]);
    };
    auto put_tail = [&](ParamWriter& w) {
        for (int d = 0; d < RO; ++d) w.put<uint32_t>((uint32_t)coshape[d]);
        for (int d = 0; d < RO; ++d) {
            uint32_t m, s;
            magic_for((uint32_t)coshape[d], m, s);
            w.put<uint32_t>(m);
        }
        for (int d = 0; d < RO; ++d) {
            uint32_t m, s;
            magic_for((uint32_t)coshape[d], m, s);
            w.put<uint32_t>(s);
        }
        for (float f : prog.imms) w.put<float>(f);
        if (prog.imms.empty()) w.put<float>(0.f);
        w.finish();
    };

    if (!use_stream) {
        RowConfig cfg;
        cfg.RO = RO;
        cfg.out_has_h = out_has_h;
        cfg.C = any16 ? 8 : 4;
        if (!pick_modes(cfg.C, cfg.mode, cfg.out_mode, true)) {
            // some tensor cannot be vectorised: fall back to one element per access so that
            // consecutive threads still touch consecutive addresses
            cfg.C = 1;
            pick_modes(1, cfg.mode, cfg.out_mode, true);
        }
        const int64_t chunks = (H + cfg.C - 1) / cfg.C;
        // elements of the row per thread: 16 floats, or 32 values of a 16-bit type (the same 64
        // bytes in flight per thread and row)
        const int target = std::max(1, tune("ROW_EPT", any16 ? 32 : 16) / cfg.C);
        cfg.GROUP = std::min(1024, std::max(32, pow2_at_least((chunks + target - 1) / target)));
        cfg.NCH = (int)((chunks + cfg.GROUP - 1) / cfg.GROUP);
        WGF_CHECK(cfg.NCH * cfg.C <= 64, WGF_ERR_UNSUPPORTED, "row too long for a row-fused kernel");
        int threads = std::max(cfg.GROUP, 128);
        cfg.RPC = threads / cfg.GROUP;
        cfg.minb = tune("ROW_MINB", std::max(1, std::min(4, 768 / threads)));
        // the next row is loaded ahead in f32 kernels; with 16-bit rows the converted copy costs
        // too many registers (measured: f16 softmax rows 333 us with, 245 us without)
        cfg.prefetch = tune("ROW_PREFETCH", any16 ? 0 : 1) != 0;
        cfg.invariant.assign(nin, 0);
        for (int t = 0; t < nin; ++t) {
            bool inv = true;
            for (int d = 0; d < RO; ++d) inv = inv && (st[t][d] == 0 || coshape[d] == 1);
            cfg.invariant[t] = inv;
        }
        std::ostringstream key;
        key << "row|" << RO << "|" << cfg.C << "|" << cfg.NCH << "|" << cfg.GROUP << "|" << cfg.RPC << "|"
            << cfg.out_mode << "|" << out_has_h << "|" << cfg.minb << cfg.prefetch << "|";
        for (int m : cfg.mode) key << m;
        key << "|";
        for (int v : cfg.invariant) key << v;
        key << "|" << prog.signature();
        const JitKernel& k = dev.kernel(key.str(), "wgf_rows", [&] { return row_source(prog, cfg); });
        // persistent CTAs: as many as fit on the machine at once, each walking several rows
        int64_t blocks = (rows + cfg.RPC - 1) / cfg.RPC;
        if (tune("ROW_PERSIST", 1)) {
            const int64_t slots = (int64_t)dev.sm_count * dev.max_blocks_per_sm(k, cfg.GROUP * cfg.RPC);
            blocks = std::min<int64_t>(blocks, slots);
        }
        ParamWriter w;
        put_common(w);
        w.put<uint32_t>((uint32_t)H);
        w.put<uint32_t>(0);
        BufferRef gpartials;
        if (!prog.grands.empty()) {
            const size_t ng = prog.grands.size();
            gpartials = dev.alloc((size_t)blocks * ng * sizeof(float), false);
            w.put<uint64_t>((uint64_t)(uintptr_t)gpartials->ptr);
            w.put<uint64_t>((uint64_t)(uintptr_t)dev.counters());
            grand_out->clear();
            for (const Grand& gr : prog.grands) {
                TensorData g;
                g.buf = dev.alloc(dtype_size(gr.dtype), false);
                g.layout = Layout::contiguous({});
                g.dtype = gr.dtype;
                w.put<uint64_t>((uint64_t)(uintptr_t)g.base_ptr());
                grand_out->push_back(g);
                WGF_CHECK(!gr.all_reduce || gc, WGF_ERR_INVALID_ARGUMENT, "in-kernel all-reduce without a communicator");
            }
            w.put<uint64_t>(gc ? (uint64_t)(uintptr_t)gc->peer_table : 0);
            w.put<uint64_t>((uint64_t)(uintptr_t)dev.error_word());
            w.put<uint32_t>(gc ? gc->world : 1);
            w.put<uint32_t>(gc ? gc->rank : 0);
            w.put<uint32_t>(gc ? gc->seq : 0);
            w.put<uint32_t>(0);
            put_settle(w, gc);
        }
        put_tail(w);
        bind_checked(dev, in, out, grand_out);
        dev.launch(k, dim3((unsigned)blocks), dim3(cfg.GROUP * cfg.RPC), 0, w.bytes.data(), "rows");
        return out;
    }

    // streaming reduce
    StreamConfig cfg;
    cfg.RO = RO;
    cfg.C = any16 ? 8 : 4;
    int dummy;
    if (!pick_modes(cfg.C, cfg.mode, dummy, false)) {
        cfg.C = 1;
        pick_modes(1, cfg.mode, dummy, false);
    }
    int nine = 0;
    for (int t = 0; t < nin; ++t) nine += !(slot_row[t] || cs[t] == 0);
    // a slot with column stride 0 that the program loads per element is read as broadcast
    cfg.U = std::max(1, std::min(tune("STREAM_U", 2), 64 / (std::max(nine, 1) * cfg.C)));
    cfg.minb = tune("STREAM_MINB", 4);
    std::ostringstream key;
    key << "stream|" << RO << "|" << cfg.C << "|" << cfg.U << "|" << cfg.minb << "|";
    for (int m : cfg.mode) key << m;
    key << "|" << prog.signature();
    const JitKernel& k = dev.kernel(key.str(), "wgf_stream_reduce", [&] { return stream_source(prog, cfg); });
    // one wave of CTAs: every resident slot of the machine gets one share of the rows
    const int64_t nch = (H + cfg.C - 1) / cfg.C;
    const int64_t per_cta = 256ll * cfg.U;
    const int64_t slots = (int64_t)dev.sm_count * dev.max_blocks_per_sm(k, 256);
    int64_t max_split = std::max<int64_t>(1, (nch + per_cta - 1) / per_cta);
    int64_t split = std::max<int64_t>(1, slots * tune("STREAM_WAVES", 1) / rows);
    split = std::min<int64_t>({split, max_split, 2048});
    if (rows > Device::kCounters) split = 1;
    BufferRef partials;
    if (split > 1)
        partials = dev.alloc((size_t)(rows * split * std::max(prog.n_reduces(), 1)) * sizeof(float), false);
    ParamWriter w;
    put_common(w);
    w.put<uint64_t>(partials ? (uint64_t)(uintptr_t)partials->ptr : 0);
    w.put<uint64_t>((uint64_t)(uintptr_t)dev.counters());
    w.put<uint64_t>((uint64_t)H);
    w.put<uint32_t>((uint32_t)split);
    w.put<uint32_t>(0);
    if (prog.result_all_reduce) {
        WGF_CHECK(gc && rows == 1, WGF_ERR_INVALID_ARGUMENT, "in-kernel all-reduce needs a communicator and a single result");
        w.put<uint64_t>((uint64_t)(uintptr_t)gc->peer_table);
        w.put<uint64_t>((uint64_t)(uintptr_t)dev.error_word());
        w.put<uint32_t>(gc->world);
        w.put<uint32_t>(gc->rank);
        w.put<uint32_t>(gc->seq);
        w.put<uint32_t>(0);
        put_settle(w, gc);
    }
    put_tail(w);
    bind_checked(dev, in, out);
    dev.launch(k, dim3((unsigned)(rows * split)), dim3(256), 0, w.bytes.data(), "stream_reduce");
    return out;
}

}  // namespace wgf
