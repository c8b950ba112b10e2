// Fused-kernel IR.  A Program is a straight-line SSA list over two kinds of values:
//   Elem - one value per element of the kernel's index space [outer..., H]
//   Row  - one value per row (uniform along the last axis H): results of reductions over H,
//          operands broadcast along H, and arithmetic between such values.
// The resolver lowers a region of the lazy graph (chains of the crate's ElementWise /
// PairWise / Reduce nodes, src/compute_graph/resolve.rs:49-196) to one Program; codegen.cpp
// turns a Program into CUDA source built around hand-written kernel templates.
#pragma once
#include <sstream>

#include "common.hpp"

namespace wgf {

enum class VKind : uint8_t { Elem = 0, Row = 1 };
enum class IKind : uint8_t { Load = 0, Unary, Scalar, Cast, Binary, RowReduce };

struct Instr {
    IKind kind;
    uint16_t op = 0;   // WGF_OP_*
    int a = -1, b = -1;
    int slot = -1;     // Load: input slot; Scalar: index into imms
    DType dtype = DType::F32;
    VKind vk = VKind::Elem;
    // Set by Program::mark_sum_only for an f32 exp whose value nothing can observe except through
    // sums: it may be computed as 2^(x * log2 e) by the special-function unit (about 1e-6
    // relative, |x| * 6e-8 more for large |x|), well inside the 1e-5 bound of a reduction.
    bool approx = false;
    // `inexact`: the value carries the error of an approximated function (a transcendental, pow, a
    // reduction whose order is free) -- the oracle's value for it is only known to 2 ulp anyway.
    // `fast_div`: a division whose DIVISOR is inexact (silu's x / (1 + exp(-x)), a softmax written
    // out by hand): computed with div.full.f32 (<= 2 ulp over the full range, a third of the
    // instructions of the IEEE sequence) -- an exactly rounded quotient of an approximate divisor
    // buys nothing.  Quotients of exact values (t / 3.0, a / b) stay IEEE and bit-exact.  Both flags
    // follow from the instructions, so they need no place in the signature.
    bool inexact = false;
    bool fast_div = false;
    // `unit`: the value lies in [-1, 1] (or is NaN) whatever the inputs are -- a sine, cosine or tanh,
    // and what abs / neg / sqr / products / casts make of such values.  `arg_unit`: operand `a` is such
    // a value: a sine or cosine of it needs no range reduction (op_sin_unit / op_cos_unit).
    bool unit = false;
    bool arg_unit = false;
};

inline bool op_is_exact_unary(uint16_t op) { return op == WGF_OP_SQR || op == WGF_OP_SQRT || op == WGF_OP_ABS || op == WGF_OP_NEG; }

// A companion output of a row kernel: Elem value `a` reduced with `op` over the WHOLE index
// space (all rows, all columns) to one scalar, computed while the rows pass through registers.
// With `all_reduce` the scalar is further combined (with `ar_op`) across the GPUs of a
// communicator by the same kernel, over peer memory.
struct Grand {
    uint16_t op;
    int a;
    DType dtype;
    bool all_reduce = false;
    uint16_t ar_op = 0;
};

struct Program {
    std::vector<Instr> ins;
    std::vector<DType> slot_dtype;  // element type of each input slot
    std::vector<float> imms;
    std::vector<Grand> grands;
    int result = -1;
    // The single (rank-0) result of a streaming reduction is combined with `result_ar_op` across
    // the GPUs of a communicator by the kernel itself.
    bool result_all_reduce = false;
    uint16_t result_ar_op = 0;

    int n_slots() const { return (int)slot_dtype.size(); }
    // Marks every f32 exp that is used only as the operand of sum reductions (Instr::approx).
    // The marks follow from the instructions, so they need no place in the signature.
    void mark_sum_only() {
        for (int i = 0; i < (int)ins.size(); ++i) {
            Instr& e = ins[i];
            e.approx = false;
            if (e.kind != IKind::Unary || e.op != WGF_OP_EXP || e.dtype != DType::F32 || i == result) continue;
            int uses = 0;
            bool only_sums = true;
            for (const Instr& u : ins) {
                if (u.kind == IKind::Load || (u.a != i && u.b != i)) continue;
                uses++;
                only_sums = only_sums && u.kind == IKind::RowReduce && u.op == WGF_OP_SUM;
            }
            for (const Grand& g : grands)
                if (g.a == i) {
                    uses++;
                    only_sums = only_sums && g.op == WGF_OP_SUM;
                }
            e.approx = uses > 0 && only_sums;
        }
    }
    DType out_dtype() const { return ins[result].dtype; }
    VKind out_kind() const { return ins[result].vk; }
    int n_reduces() const {
        int n = 0;
        for (auto& i : ins) n += i.kind == IKind::RowReduce;
        return n;
    }

    int load(int slot, DType dt, VKind vk) {
        for (int i = 0; i < (int)ins.size(); ++i)
            if (ins[i].kind == IKind::Load && ins[i].slot == slot) return i;
        Instr in{IKind::Load};
        in.slot = slot;
        in.dtype = dt;
        in.vk = vk;
        ins.push_back(in);
        return (int)ins.size() - 1;
    }
    int new_slot(DType dt) {
        slot_dtype.push_back(dt);
        return (int)slot_dtype.size() - 1;
    }
    int unary(uint16_t op, int a) {
        Instr in{IKind::Unary};
        in.op = op;
        in.a = a;
        in.dtype = ins[a].dtype;
        in.vk = ins[a].vk;
        in.inexact = ins[a].inexact || !op_is_exact_unary(op);
        in.arg_unit = ins[a].unit;
        in.unit = op == WGF_OP_SIN || op == WGF_OP_COS || op == WGF_OP_TANH ||
                  (ins[a].unit && (op == WGF_OP_ABS || op == WGF_OP_NEG || op == WGF_OP_SQR));
        ins.push_back(in);
        return (int)ins.size() - 1;
    }
    int scalar(uint16_t op, int a, float c) {
        Instr in{IKind::Scalar};
        in.op = op;
        in.a = a;
        in.slot = (int)imms.size();
        imms.push_back(c);
        in.dtype = ins[a].dtype;
        in.vk = ins[a].vk;
        in.inexact = ins[a].inexact;
        in.fast_div = op == WGF_OP_RDIV_C && ins[a].inexact;
        ins.push_back(in);
        return (int)ins.size() - 1;
    }
    int cast(int a, DType to) {
        Instr in{IKind::Cast};
        in.op = WGF_OP_CAST;
        in.a = a;
        in.dtype = to;
        in.vk = ins[a].vk;
        in.inexact = ins[a].inexact;
        in.unit = ins[a].unit;   // rounding to a narrower type keeps |v| <= 1
        ins.push_back(in);
        return (int)ins.size() - 1;
    }
    int binary(uint16_t op, int a, int b) {
        Instr in{IKind::Binary};
        in.op = op;
        in.a = a;
        in.b = b;
        in.dtype = ins[a].dtype;
        in.vk = (ins[a].vk == VKind::Row && ins[b].vk == VKind::Row) ? VKind::Row : VKind::Elem;
        in.inexact = ins[a].inexact || ins[b].inexact || op == WGF_OP_POW;
        in.fast_div = op == WGF_OP_DIV && ins[b].inexact;
        in.unit = op == WGF_OP_MUL && ins[a].unit && ins[b].unit;
        ins.push_back(in);
        return (int)ins.size() - 1;
    }
    int row_reduce(uint16_t op, int a) {
        Instr in{IKind::RowReduce};
        in.op = op;
        in.a = a;
        in.dtype = ins[a].dtype;
        in.vk = VKind::Row;
        in.inexact = ins[a].inexact || op == WGF_OP_SUM || op == WGF_OP_PRODUCT;   // max / min of exact values are exact
        ins.push_back(in);
        return (int)ins.size() - 1;
    }

    // True if some Elem value depends on the result of a RowReduce, i.e. the row has to be
    // kept (in registers) across a reduction.
    bool multi_phase() const {
        std::vector<char> dep(ins.size(), 0);
        for (size_t i = 0; i < ins.size(); ++i) {
            const Instr& in = ins[i];
            char d = 0;
            if (in.a >= 0) d |= dep[in.a];
            if (in.b >= 0) d |= dep[in.b];
            if (in.kind == IKind::RowReduce) {
                if (d) return true;  // a reduction of something that depends on a reduction
                d = 1;
            } else if (d && in.vk == VKind::Elem) {
                return true;
            }
            dep[i] = d;
        }
        return false;
    }

    // Text form; immediates are kernel parameters, so their values are not part of it.
    std::string signature() const {
        std::string s;
        s.reserve(16 + 24 * ins.size());
        auto num = [&s](int v) {   // decimal, no stream machinery: this runs for every launch
            char buf[12];
            int n = 0;
            unsigned u = v < 0 ? (unsigned)(-(long long)v) : (unsigned)v;
            do {
                buf[n++] = (char)('0' + u % 10);
                u /= 10;
            } while (u);
            if (v < 0) s.push_back('-');
            while (n) s.push_back(buf[--n]);
        };
        for (auto d : slot_dtype) {
            s.push_back('s');
            num((int)d);
        }
        s.push_back('|');
        for (auto& in : ins) {
            num((int)in.kind);
            s.push_back('.');
            num(in.op);
            s.push_back('.');
            num(in.a);
            s.push_back('.');
            num(in.b);
            s.push_back('.');
            num(in.slot);
            s.push_back('.');
            num((int)in.dtype);
            s.push_back('.');
            num((int)in.vk);
            s.push_back(';');
        }
        s += "->";
        num(result);
        if (result_all_reduce) {
            s.push_back('A');
            num(result_ar_op);
        }
        for (auto& g : grands) {
            s += "|g";
            num(g.op);
            s.push_back('.');
            num(g.a);
            s.push_back('.');
            num((int)g.dtype);
            if (g.all_reduce) {
                s.push_back('a');
                num(g.ar_op);
            }
        }
        return s;
    }
};

}  // namespace wgf
