// Launchers of the fused kernel family (run-time compiled) and of the precompiled kernels.
#pragma once
#include "ir.hpp"
#include "runtime.hpp"

namespace wgf {

// Every input's layout must have the rank of `shape` (stride 0 where it is broadcast).
// `inplace_slot` >= 0 names an input whose buffer the caller allows to be overwritten; it
// is used only if its layout is dense, non-overlapping, covers the index space one-to-one
// and its element width equals the result's.  Otherwise a new contiguous buffer is made.
TensorData run_elementwise(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                           const std::vector<int64_t>& shape, int inplace_slot);

// Index space `shape` = [outer..., H]; reductions run over the last axis.  An Elem result
// has shape `shape`, a Row result has shape `shape` without its last axis.
// `out_has_h` says whether the result keeps the last axis (a Row-kind result is then written
// to every column of its row).  A program with companion reductions (`prog.grands`) needs
// `out_has_h` and a non-empty index space; their rank-0 results are returned in `grand_out`.
// Companion reductions marked `all_reduce` are exchanged through the mailboxes of a communicator
// (see Comm): the kernel stores this GPU's values of exchange `seq`, posts the values of the
// exchange before it (post_*) and settles the oldest open one once that is kMailboxLag kernels old (prev_*).
struct GrandComm {
    const void* peer_table;   // device array of the ranks' mailbox addresses
    uint32_t world, rank, seq;
    const void* mailbox;      // this rank's own mailbox: where the settled exchange is read
    uint64_t wait_ns;         // limit of the wait for a peer's word
    uint32_t prev_seq, prev_n;   // prev_n == 0: nothing to settle
    uint32_t prev_meta[4];    // op code (0 sum, 1 product, 2 max, 3 min) | dtype << 8 | value index << 16
    void* prev_out[4];
    uint32_t post_seq, post_n;   // post_n == 0: nothing to post
    uint32_t post_meta[4];    // same encoding
    void* post_src[4];        // result buffers that hold this GPU's values of exchange post_seq
};
TensorData run_rows(Device& dev, const Program& prog, const std::vector<TensorData>& in,
                    const std::vector<int64_t>& shape, bool out_has_h, int inplace_slot,
                    std::vector<TensorData>* grand_out = nullptr, const GrandComm* gc = nullptr);

// Longest row the register-resident row kernel accepts, for the given element width mix.
int64_t max_resident_row(bool any_16bit);

// Source text of the kernel `run_*` would compile (for tests and inspection without a GPU).
std::string debug_ew_source(const Program& prog, int rank, int chunk);

// ---- precompiled kernels (move_kernels.cu, matmul*.cu) ----
// dst[idx] = src[idx] for every index of the common shape; element bits are moved unchanged.
void run_copy(Device& dev, const TensorData& dst, const TensorData& src);
// A dense row-major copy of `src` (a new buffer).
TensorData run_compact(Device& dev, const TensorData& src);
TensorData run_matmul(Device& dev, const TensorData& a, const TensorData& b);
// The product with an element-wise step done in the kernel's epilogue (tcgen05 CTA-pair kernel, 16-bit
// types): `out = round(a b) + resid`, and `out = silu(a bg) * (a bu)`.  Bit-identical to the separate
// kernels.  Return false, having launched nothing, when that kernel does not take the problem.
bool run_matmul_residual(Device& dev, const TensorData& a, const TensorData& b, const TensorData& resid, TensorData& out);
bool run_matmul_silu_mul(Device& dev, const TensorData& a, const TensorData& bg, const TensorData& bu, TensorData& out);
// Rotary embedding of x [.., seq, embed] (rank 3 or 4, last axis contiguous or gathered first)
// with cos / sin [>= seq, embed / 2]; bit-identical to the chain of separate ops (rope.cu).
TensorData run_rope(Device& dev, const TensorData& x, const TensorData& cos, const TensorData& sin);

}  // namespace wgf
