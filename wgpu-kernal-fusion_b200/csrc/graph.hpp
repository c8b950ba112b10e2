// Lazy compute graph and fusion resolver.
//
// Node kinds mirror the crate's eight node maps (src/compute_graph/mod.rs:265-276).  A graph
// object carries the crate's `merge` semantics (src/compute_graph/mod.rs:168-185): the graphs
// of the two operands of a binary op are united, and handles made from either keep working.
// Unlike the crate, nodes own their inputs, results are memoised per node, and a node that
// has been materialised lets go of its inputs, so intermediate device buffers are returned
// as soon as nothing can read them again.
#pragma once
#include <unordered_map>
#include <unordered_set>

#include "launch.hpp"

namespace wgf {

struct Comm;

enum class NodeKind : uint8_t {
    Tensor, ElementWise, PairWise, Reduce, MatMul, MapLayout, Resize, SliceAssign, AllReduce,
    Attention,  // fused causal softmax attention (no counterpart in the crate); imm = scale
    Rope        // rotary embedding as one kernel; inputs x, cos, sin
};

struct ViewOp {
    enum Kind : uint8_t { Slice, Transpose, BroadcastAxis, Expand } kind = Slice;
    std::vector<int64_t> starts, ends;  // Slice
    int a = 0, b = 0;                   // Transpose
    int axis = 0;                       // BroadcastAxis: position of the new stride-0 axis
    int64_t size = 0;                   //                and its extent
    std::vector<int64_t> shape;         // Expand: target shape
    Layout apply(const Layout& in) const;
};

struct GraphInner;
struct GraphCell {
    std::shared_ptr<GraphInner> inner;
};

struct Node {
    uint64_t id = 0;
    NodeKind kind = NodeKind::Tensor;
    DeviceRef dev;
    std::vector<int64_t> shape;
    DType dtype = DType::F32;
    std::vector<std::shared_ptr<Node>> inputs;
    // payload
    uint16_t op = 0;
    float imm = 0.f;
    int axis = 0;
    ViewOp view;
    std::vector<int64_t> new_shape, fill_shape, starts, ends;
    std::shared_ptr<Comm> comm;
    // Scratch of the resolver, used instead of hash containers keyed by node: a "set" is an epoch
    // number, and the node belongs to it while the slot of that kind carries the epoch.
    struct Scratch {
        uint64_t epoch = 0;
        int value = 0;
    };
    enum { S_FUSED = 0, S_LEAF, S_HAS_REDUCE, S_SEEN, S_VALUE, S_DIES, S_COUNT };
    Scratch scratch[S_COUNT];
    // state
    TensorData cached;
    int handles = 0;
    std::vector<Node*> consumers;
    std::shared_ptr<GraphCell> graph;

    ~Node();
    void drop_inputs();
    int rank() const { return (int)shape.size(); }
    int64_t numel() const {
        int64_t n = 1;
        for (auto v : shape) n *= v;
        return n;
    }
};
using NodeRef = std::shared_ptr<Node>;

struct GraphInner {
    std::shared_ptr<GraphInner> forwarded;          // set once this graph has been merged away
    uint64_t live_nodes = 0;                        // nodes alive in this graph (the crate keeps node maps)
    std::vector<TimingRecord> timings;              // src/compute_graph/mod.rs:275
    DeviceRef dev;
    ~GraphInner();
};

std::shared_ptr<GraphInner> graph_of(const NodeRef& n);
void merge_graphs(const NodeRef& a, const NodeRef& b);

// ---- node constructors (validate like the crate's front-ends, but return errors) ----
NodeRef make_tensor(const DeviceRef& dev, TensorData td);
NodeRef make_unary(const NodeRef& x, uint16_t op);
NodeRef make_scalar(const NodeRef& x, uint16_t op, float c);
NodeRef make_cast(const NodeRef& x, DType to);
NodeRef make_binary(const NodeRef& a, const NodeRef& b, uint16_t op);
NodeRef make_reduce(const NodeRef& x, uint16_t op, int axis);
NodeRef make_matmul(const NodeRef& a, const NodeRef& b);
NodeRef make_view(const NodeRef& x, const ViewOp& v);
NodeRef make_resize(const NodeRef& x, const std::vector<int64_t>& new_shape,
                    const std::vector<int64_t>& fill_shape);
NodeRef make_slice_assign(const NodeRef& target, const std::vector<int64_t>& starts,
                          const std::vector<int64_t>& ends, const NodeRef& value);
NodeRef make_all_reduce(const NodeRef& x, const std::shared_ptr<Comm>& comm, uint16_t op);

// ---- views / composites (src/map_layout.rs, src/composite/) ----
NodeRef view_slice(const NodeRef& x, const std::vector<int64_t>& starts, const std::vector<int64_t>& ends);
NodeRef view_transpose(const NodeRef& x, int a, int b);
NodeRef view_broadcast(const NodeRef& x, const std::vector<int64_t>& out_shape);
NodeRef view_broadcast_axis(const NodeRef& x, int axis, int64_t size);
NodeRef view_expand(const NodeRef& x, const std::vector<int64_t>& out_shape);
NodeRef op_reshape(const NodeRef& x, const std::vector<int64_t>& new_shape);
NodeRef op_cat(const std::vector<NodeRef>& parts, int dim);
NodeRef op_narrow(const NodeRef& x, int axis, int64_t start, int64_t len);
NodeRef op_unsqueeze(const NodeRef& x, int axis);
NodeRef op_silu(const NodeRef& x);
NodeRef op_layer_norm(const NodeRef& x, const NodeRef& weight, float eps);
NodeRef op_softmax(const NodeRef& x);
NodeRef op_softmax_last_dim(const NodeRef& x);
NodeRef op_rope(const NodeRef& x, const NodeRef& cos, const NodeRef& sin);
// softmax(scale * q k^T + mask) v over [batch*heads, seq, head_dim] tensors.  `mask` is an
// additive [seq, seq] tensor or null; with a null mask `causal` masks the keys after each
// query and, where the shapes allow (16-bit, head_dim 128, seq a multiple of 128), one fused
// tensor-core kernel runs instead of matmul / softmax / matmul.
NodeRef op_attention(const NodeRef& q, const NodeRef& k, const NodeRef& v, const NodeRef& mask, bool causal, float scale);
NodeRef op_llama_block(const NodeRef& x, const NodeRef& wq, const NodeRef& wk, const NodeRef& wv, const NodeRef& wo,
                       const NodeRef& wg, const NodeRef& wu, const NodeRef& wd, const NodeRef& norm1,
                       const NodeRef& norm2, const NodeRef& cos, const NodeRef& sin, const NodeRef& mask,
                       int n_heads, float eps);

// The resolver: returns the materialised result of `n` (cached in the node afterwards).
// Kernels are queued on the device stream; nothing waits.
TensorData resolve(const NodeRef& n);

// Resolves all of `nodes` as one request: a whole-tensor reduction among them is computed
// inside the row kernel of another requested tensor when both cover the same index space.
void resolve_many(const std::vector<NodeRef>& nodes);

std::string graphviz(const NodeRef& n);

}  // namespace wgf
