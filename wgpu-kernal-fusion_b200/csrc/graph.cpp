#include "graph.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <functional>
#include <sstream>

#include "attention.hpp"
#include "comm.hpp"
#include "half.hpp"
#include "matmul.hpp"

namespace wgf {

// ---------------------------------------------------------------------------------------
// graph store (src/compute_graph/mod.rs:152-276)
// ---------------------------------------------------------------------------------------
static std::atomic<uint64_t> g_next_id{1};

static std::shared_ptr<GraphInner> find_graph(const std::shared_ptr<GraphCell>& cell) {
    std::shared_ptr<GraphInner> g = cell->inner;
    while (g->forwarded) g = g->forwarded;
    cell->inner = g;
    return g;
}

std::shared_ptr<GraphInner> graph_of(const NodeRef& n) { return find_graph(n->graph); }

GraphInner::~GraphInner() {
    if (dev)
        for (auto& t : timings) {
            if (t.start) dev->recycle(t.start);
            if (t.stop) dev->recycle(t.stop);
        }
}

void merge_graphs(const NodeRef& a, const NodeRef& b) {
    auto ga = find_graph(a->graph), gb = find_graph(b->graph);
    if (ga == gb) return;
    ga->live_nodes += gb->live_nodes;
    gb->live_nodes = 0;
    ga->timings.insert(ga->timings.end(), gb->timings.begin(), gb->timings.end());
    gb->timings.clear();
    gb->forwarded = ga;
    b->graph->inner = ga;
}

Node::~Node() {
    drop_inputs();
    if (graph) find_graph(graph)->live_nodes--;
}

void Node::drop_inputs() {
    for (auto& in : inputs) {
        auto& c = in->consumers;
        auto it = std::find(c.begin(), c.end(), this);
        if (it != c.end()) c.erase(it);
    }
    inputs.clear();
}

static NodeRef new_node(NodeKind kind, const DeviceRef& dev, std::vector<int64_t> shape, DType dt,
                        std::vector<NodeRef> inputs) {
    auto n = std::make_shared<Node>();
    n->id = g_next_id++;
    n->kind = kind;
    n->dev = dev;
    n->shape = std::move(shape);
    n->dtype = dt;
    for (auto& in : inputs) {
        WGF_CHECK(in->dev == dev, WGF_ERR_INVALID_ARGUMENT, "operands live on different devices");
        in->consumers.push_back(n.get());
    }
    if (inputs.empty()) {
        n->graph = std::make_shared<GraphCell>();
        n->graph->inner = std::make_shared<GraphInner>();
        n->graph->inner->dev = dev;
    } else {
        n->graph = inputs[0]->graph;
        for (size_t i = 1; i < inputs.size(); ++i) merge_graphs(inputs[0], inputs[i]);
    }
    n->inputs = std::move(inputs);
    find_graph(n->graph)->live_nodes++;
    return n;
}

// ---------------------------------------------------------------------------------------
// views (src/map_layout.rs:26-98, src/layout.rs:17-31)
// ---------------------------------------------------------------------------------------
Layout ViewOp::apply(const Layout& in) const {
    Layout out = in;
    switch (kind) {
        case Slice:
            for (int i = 0; i < in.rank(); ++i) {
                out.offset += starts[i] * in.strides[i];
                out.shape[i] = ends[i] - starts[i];
            }
            break;
        case Transpose:
            std::swap(out.shape[a], out.shape[b]);
            std::swap(out.strides[a], out.strides[b]);
            break;
        case BroadcastAxis:
            out.shape.insert(out.shape.begin() + axis, size);
            out.strides.insert(out.strides.begin() + axis, 0);
            break;
        case Expand:
            for (int i = 0; i < in.rank(); ++i)
                if (in.shape[i] == 1 && shape[i] != 1) {
                    out.shape[i] = shape[i];
                    out.strides[i] = 0;
                }
            break;
    }
    return out;
}

// ---------------------------------------------------------------------------------------
// node constructors
// ---------------------------------------------------------------------------------------
static bool is_unary(uint16_t op) { return op <= WGF_OP_NEG; }
static bool is_scalar(uint16_t op) { return op >= WGF_OP_ADD_C && op <= WGF_OP_RDIV_C; }
static bool is_binary(uint16_t op) { return op >= WGF_OP_ADD && op <= WGF_OP_POW; }
static bool is_reduce(uint16_t op) { return op >= WGF_OP_SUM && op <= WGF_OP_PRODUCT; }

NodeRef make_tensor(const DeviceRef& dev, TensorData td) {
    auto n = new_node(NodeKind::Tensor, dev, td.layout.shape, td.dtype, {});
    n->cached = std::move(td);
    return n;
}

NodeRef make_unary(const NodeRef& x, uint16_t op) {
    WGF_CHECK(is_unary(op), WGF_ERR_INVALID_ARGUMENT, "not a unary opcode");
    auto n = new_node(NodeKind::ElementWise, x->dev, x->shape, x->dtype, {x});
    n->op = op;
    return n;
}

NodeRef make_scalar(const NodeRef& x, uint16_t op, float c) {
    WGF_CHECK(is_scalar(op), WGF_ERR_INVALID_ARGUMENT, "not a scalar opcode");
    auto n = new_node(NodeKind::ElementWise, x->dev, x->shape, x->dtype, {x});
    n->op = op;
    n->imm = c;
    return n;
}

NodeRef make_cast(const NodeRef& x, DType to) {
    auto n = new_node(NodeKind::ElementWise, x->dev, x->shape, to, {x});
    n->op = WGF_OP_CAST;
    return n;
}

NodeRef make_binary(const NodeRef& a, const NodeRef& b, uint16_t op) {
    WGF_CHECK(is_binary(op), WGF_ERR_INVALID_ARGUMENT, "not a binary opcode");
    WGF_CHECK(a->shape == b->shape, WGF_ERR_SHAPE, "pairwise operands must have equal shapes");  // src/pair_wise.rs:92
    WGF_CHECK(a->dtype == b->dtype, WGF_ERR_DTYPE, "pairwise operands must have equal element types");
    auto n = new_node(NodeKind::PairWise, a->dev, a->shape, a->dtype, {a, b});
    n->op = op;
    return n;
}

NodeRef make_reduce(const NodeRef& x, uint16_t op, int axis) {
    WGF_CHECK(is_reduce(op), WGF_ERR_INVALID_ARGUMENT, "not a reduce opcode");
    WGF_CHECK(axis >= 0 && axis < x->rank(), WGF_ERR_INVALID_ARGUMENT, "reduce axis out of range");
    std::vector<int64_t> s = x->shape;
    s.erase(s.begin() + axis);  // src/tensor.rs:221-242
    auto n = new_node(NodeKind::Reduce, x->dev, s, x->dtype, {x});
    n->op = op;
    n->axis = axis;
    return n;
}

NodeRef make_matmul(const NodeRef& a, const NodeRef& b) {
    WGF_CHECK(a->dtype == b->dtype, WGF_ERR_DTYPE, "matmul operands must have equal element types");
    WGF_CHECK(a->rank() == b->rank() && (a->rank() == 2 || a->rank() == 3), WGF_ERR_RANK,
              "matmul takes two rank-2 tensors, or two rank-3 tensors (batched)");
    const int r = a->rank();
    WGF_CHECK(a->shape[r - 1] == b->shape[r - 2], WGF_ERR_SHAPE, "matmul inner dimensions differ");  // src/matmul.rs:194
    if (r == 3) WGF_CHECK(a->shape[0] == b->shape[0], WGF_ERR_SHAPE, "matmul batch sizes differ");
    std::vector<int64_t> s = a->shape;
    s[r - 1] = b->shape[r - 1];
    return new_node(NodeKind::MatMul, a->dev, s, a->dtype, {a, b});
}

NodeRef make_view(const NodeRef& x, const ViewOp& v) {
    Layout l = v.apply(Layout::contiguous(x->shape));
    auto n = new_node(NodeKind::MapLayout, x->dev, l.shape, x->dtype, {x});
    n->view = v;
    return n;
}

NodeRef make_resize(const NodeRef& x, const std::vector<int64_t>& new_shape,
                    const std::vector<int64_t>& fill_shape) {
    auto n = new_node(NodeKind::Resize, x->dev, new_shape, x->dtype, {x});
    n->new_shape = new_shape;
    n->fill_shape = fill_shape;
    return n;
}

NodeRef make_slice_assign(const NodeRef& target, const std::vector<int64_t>& starts,
                          const std::vector<int64_t>& ends, const NodeRef& value) {
    WGF_CHECK(target->dtype == value->dtype, WGF_ERR_DTYPE, "slice_assign element types differ");
    WGF_CHECK(target->rank() == value->rank(), WGF_ERR_RANK, "slice_assign ranks differ");
    for (int i = 0; i < target->rank(); ++i) {
        WGF_CHECK(starts[i] >= 0 && starts[i] <= ends[i] && ends[i] <= target->shape[i], WGF_ERR_SHAPE,
                  "slice_assign range outside the target");
        WGF_CHECK(ends[i] - starts[i] == value->shape[i], WGF_ERR_SHAPE,
                  "slice_assign value shape differs from the range");
    }
    auto n = new_node(NodeKind::SliceAssign, target->dev, target->shape, target->dtype, {target, value});
    n->starts = starts;
    n->ends = ends;
    return n;
}

NodeRef make_all_reduce(const NodeRef& x, const std::shared_ptr<Comm>& comm, uint16_t op) {
    WGF_CHECK(is_reduce(op), WGF_ERR_INVALID_ARGUMENT, "not a reduce opcode");
    auto n = new_node(NodeKind::AllReduce, x->dev, x->shape, x->dtype, {x});
    n->op = op;
    n->comm = comm;
    return n;
}

NodeRef view_slice(const NodeRef& x, const std::vector<int64_t>& starts, const std::vector<int64_t>& ends) {
    for (int i = 0; i < x->rank(); ++i)
        WGF_CHECK(starts[i] >= 0 && starts[i] <= ends[i] && ends[i] <= x->shape[i], WGF_ERR_SHAPE,
                  "slice range outside the tensor");
    ViewOp v;
    v.kind = ViewOp::Slice;
    v.starts = starts;
    v.ends = ends;
    return make_view(x, v);
}

NodeRef view_transpose(const NodeRef& x, int a, int b) {
    WGF_CHECK(a >= 0 && b >= 0 && a < x->rank() && b < x->rank(), WGF_ERR_INVALID_ARGUMENT,
              "transpose axis out of range");
    ViewOp v;
    v.kind = ViewOp::Transpose;
    v.a = a;
    v.b = b;
    return make_view(x, v);
}

NodeRef view_broadcast_axis(const NodeRef& x, int axis, int64_t size) {
    WGF_CHECK(axis >= 0 && axis <= x->rank(), WGF_ERR_INVALID_ARGUMENT, "broadcast axis out of range");
    WGF_CHECK(x->rank() + 1 <= WGF_MAX_RANK, WGF_ERR_RANK, "rank above 8");
    WGF_CHECK(size >= 0, WGF_ERR_SHAPE, "negative extent");
    ViewOp v;
    v.kind = ViewOp::BroadcastAxis;
    v.axis = axis;
    v.size = size;
    return make_view(x, v);
}

// src/map_layout.rs:69-98: the new axis goes where the common prefix of the shapes ends.
NodeRef view_broadcast(const NodeRef& x, const std::vector<int64_t>& out_shape) {
    WGF_CHECK((int)out_shape.size() == x->rank() + 1, WGF_ERR_RANK, "broadcast adds exactly one axis");
    int new_dim = 0;
    while (new_dim < x->rank() && x->shape[new_dim] == out_shape[new_dim]) new_dim++;
    for (int i = new_dim; i < x->rank(); ++i)
        WGF_CHECK(x->shape[i] == out_shape[i + 1], WGF_ERR_SHAPE, "broadcast shapes do not line up");
    return view_broadcast_axis(x, new_dim, out_shape[new_dim]);
}

NodeRef view_expand(const NodeRef& x, const std::vector<int64_t>& out_shape) {
    WGF_CHECK((int)out_shape.size() == x->rank(), WGF_ERR_RANK, "expand keeps the rank");
    for (int i = 0; i < x->rank(); ++i)
        WGF_CHECK(x->shape[i] == out_shape[i] || x->shape[i] == 1, WGF_ERR_SHAPE,
                  "expand only stretches axes of extent 1");
    ViewOp v;
    v.kind = ViewOp::Expand;
    v.shape = out_shape;
    return make_view(x, v);
}

// ---------------------------------------------------------------------------------------
// composites (src/composite/)
// ---------------------------------------------------------------------------------------
NodeRef op_reshape(const NodeRef& x, const std::vector<int64_t>& new_shape) {
    int64_t a = 1, b = 1;
    for (auto v : x->shape) a *= v;
    for (auto v : new_shape) b *= v;
    WGF_CHECK(a == b, WGF_ERR_SHAPE, "reshape changes the number of elements");  // src/resize.rs:133-136
    return make_resize(x, new_shape, new_shape);
}

NodeRef op_narrow(const NodeRef& x, int axis, int64_t start, int64_t len) {
    WGF_CHECK(axis >= 0 && axis < x->rank(), WGF_ERR_INVALID_ARGUMENT, "narrow axis out of range");
    WGF_CHECK(start >= 0 && len >= 0 && start + len <= x->shape[axis], WGF_ERR_SHAPE, "narrow range outside the axis");
    std::vector<int64_t> s(x->rank(), 0), e = x->shape;
    s[axis] = start;
    e[axis] = start + len;
    return view_slice(x, s, e);
}

NodeRef op_unsqueeze(const NodeRef& x, int axis) {
    WGF_CHECK(axis >= 0 && axis <= x->rank(), WGF_ERR_INVALID_ARGUMENT, "unsqueeze axis out of range");
    std::vector<int64_t> s = x->shape;
    s.insert(s.begin() + axis, 1);
    return op_reshape(x, s);  // src/composite/unsqueeze.rs:5-14
}

// src/composite/cat.rs:4-40: resize the first part to the full shape, slice_assign the rest.
NodeRef op_cat(const std::vector<NodeRef>& parts, int dim) {
    WGF_CHECK(!parts.empty(), WGF_ERR_INVALID_ARGUMENT, "cat of nothing");
    const int r = parts[0]->rank();
    WGF_CHECK(dim >= 0 && dim < r, WGF_ERR_INVALID_ARGUMENT, "cat axis out of range");
    std::vector<int64_t> shape = parts[0]->shape;
    shape[dim] = 0;
    for (auto& p : parts) {
        WGF_CHECK(p->rank() == r, WGF_ERR_RANK, "cat ranks differ");
        for (int i = 0; i < r; ++i)
            if (i == dim) shape[i] += p->shape[i];
            else WGF_CHECK(shape[i] == p->shape[i], WGF_ERR_SHAPE, "cat shapes differ off the joined axis");
    }
    NodeRef larger = make_resize(parts[0], shape, parts[0]->shape);
    int64_t index = parts[0]->shape[dim];
    for (size_t k = 1; k < parts.size(); ++k) {
        std::vector<int64_t> s(r, 0), e = shape;
        s[dim] = index;
        e[dim] = index + parts[k]->shape[dim];
        larger = make_slice_assign(larger, s, e, parts[k]);
        index = e[dim];
    }
    return larger;
}

// src/composite/silu.rs:4-7: x / (1 + exp(-x))
NodeRef op_silu(const NodeRef& x) {
    NodeRef d = make_scalar(make_unary(make_unary(x, WGF_OP_NEG), WGF_OP_EXP), WGF_OP_ADD_C, 1.f);
    return make_binary(x, d, WGF_OP_DIV);
}

// src/composite/rms_norm.rs:8-15, for any rank >= 1 over the last axis.  The broadcasts name
// their axis (the crate's prefix rule puts the weight on the wrong axis for square inputs).
NodeRef op_layer_norm(const NodeRef& x, const NodeRef& weight, float eps) {
    WGF_CHECK(x->rank() >= 1, WGF_ERR_RANK, "layer_norm needs rank >= 1");
    const int last = x->rank() - 1;
    const int64_t hidden = x->shape[last];
    WGF_CHECK(weight->rank() == 1 && weight->shape[0] == hidden, WGF_ERR_SHAPE,
              "layer_norm weight must have the length of the last axis");
    WGF_CHECK(weight->dtype == x->dtype, WGF_ERR_DTYPE, "layer_norm weight element type differs");
    NodeRef f = make_cast(x, DType::F32);
    NodeRef norm = make_scalar(make_reduce(make_unary(f, WGF_OP_SQR), WGF_OP_SUM, last), WGF_OP_DIV_C, (float)hidden);
    NodeRef denom = make_unary(make_scalar(norm, WGF_OP_ADD_C, eps), WGF_OP_SQRT);
    NodeRef normed = make_binary(f, view_broadcast_axis(denom, last, hidden), WGF_OP_DIV);
    NodeRef w = weight;
    for (int i = 0; i < last; ++i) w = view_broadcast_axis(w, i, x->shape[i]);
    return make_binary(make_cast(normed, x->dtype), w, WGF_OP_MUL);
}

// src/composite/softmax.rs:4-10 (rank 1, no max-subtraction)
NodeRef op_softmax(const NodeRef& x) {
    WGF_CHECK(x->rank() == 1, WGF_ERR_RANK, "softmax takes a rank-1 tensor; see softmax_last_dim");
    NodeRef e = make_unary(x, WGF_OP_EXP);
    NodeRef s = view_broadcast_axis(make_reduce(e, WGF_OP_SUM, 0), 0, x->shape[0]);
    return make_binary(e, s, WGF_OP_DIV);
}

NodeRef op_softmax_last_dim(const NodeRef& x) {
    WGF_CHECK(x->rank() >= 1, WGF_ERR_RANK, "softmax needs rank >= 1");
    const int last = x->rank() - 1;
    const int64_t h = x->shape[last];
    NodeRef m = view_broadcast_axis(make_reduce(x, WGF_OP_MAX, last), last, h);
    NodeRef e = make_unary(make_binary(x, m, WGF_OP_SUB), WGF_OP_EXP);
    NodeRef s = view_broadcast_axis(make_reduce(e, WGF_OP_SUM, last), last, h);
    return make_binary(e, s, WGF_OP_DIV);
}

// src/composite/rope.rs:5-22 with its evident intent: cos/sin are [seq_max, D/2], doubled
// along the last axis, cut to the sequence length and broadcast over the leading axis.
NodeRef op_rope(const NodeRef& x, const NodeRef& cos, const NodeRef& sin) {
    WGF_CHECK(x->rank() == 3, WGF_ERR_RANK, "rope takes [heads, sequence, embed]");
    WGF_CHECK(cos->rank() == 2 && sin->rank() == 2 && cos->shape == sin->shape, WGF_ERR_SHAPE,
              "rope cos/sin must be equal rank-2 tensors");
    const int64_t heads = x->shape[0], seq = x->shape[1], d = x->shape[2];
    WGF_CHECK(cos->shape[1] * 2 == d && cos->shape[0] >= seq, WGF_ERR_SHAPE,
              "rope cos/sin must be [>= sequence, embed / 2]");
    WGF_CHECK(cos->dtype == x->dtype && sin->dtype == x->dtype, WGF_ERR_DTYPE, "rope element types differ");
    // One kernel with the roundings of the composed form below (kept for odd embed sizes)
    if (d % 2 == 0 && d >= 2) return new_node(NodeKind::Rope, x->dev, x->shape, x->dtype, {x, cos, sin});
    NodeRef c = view_broadcast_axis(op_narrow(op_cat({cos, cos}, 1), 0, 0, seq), 0, heads);
    NodeRef s = view_broadcast_axis(op_narrow(op_cat({sin, sin}, 1), 0, 0, seq), 0, heads);
    NodeRef x1 = op_narrow(x, 2, 0, d / 2), x2 = op_narrow(x, 2, d / 2, d - d / 2);
    NodeRef rot = op_cat({make_unary(x2, WGF_OP_NEG), x1}, 2);
    return make_binary(make_binary(x, c, WGF_OP_MUL), make_binary(rot, s, WGF_OP_MUL), WGF_OP_ADD);
}

NodeRef op_attention(const NodeRef& q, const NodeRef& k, const NodeRef& v, const NodeRef& mask, bool causal, float scale) {
    WGF_CHECK(q->rank() == 3 && k->rank() == 3 && v->rank() == 3, WGF_ERR_RANK, "attention takes [batch*heads, seq, head_dim] tensors");
    WGF_CHECK(q->shape[0] == k->shape[0] && q->shape[2] == k->shape[2] && k->shape == v->shape, WGF_ERR_SHAPE,
              "attention: q is [n, seq_q, d], k and v are [n, seq_k, d]");
    WGF_CHECK(q->dtype == k->dtype && q->dtype == v->dtype, WGF_ERR_DTYPE, "attention operands differ in element type");
    const int64_t n = q->shape[0], sq = q->shape[1], sk = k->shape[1], d = q->shape[2];
    if (mask) {
        WGF_CHECK(mask->rank() == 2 && mask->shape[0] == sq && mask->shape[1] == sk, WGF_ERR_SHAPE,
                  "attention mask must be [seq_q, seq_k]");
        WGF_CHECK(mask->dtype == q->dtype, WGF_ERR_DTYPE, "attention mask differs in element type");
    }
    if (!mask && attention_supported(q->dtype, sq, sk, d)) {
        auto node = new_node(NodeKind::Attention, q->dev, q->shape, q->dtype, {q, k, v});
        node->imm = scale;
        node->axis = causal ? 1 : 0;
        return node;
    }
    WGF_CHECK(mask || !causal, WGF_ERR_UNSUPPORTED,
              "causal attention without a mask needs 16-bit elements, head_dim 128 and seq a multiple of 128; pass an additive mask");
    NodeRef scores = make_matmul(q, view_transpose(k, 1, 2));                       // [n, seq_q, seq_k]
    NodeRef scaled = make_scalar(scores, WGF_OP_MUL_C, scale);
    NodeRef masked = mask ? make_binary(scaled, view_broadcast_axis(mask, 0, n), WGF_OP_ADD) : scaled;
    NodeRef probs = op_softmax_last_dim(masked);                                    // one fused row kernel
    return make_matmul(probs, v);
}

// Llama-style decoder block forward (no counterpart in the crate, whose README only lists the
// ops such a block needs, README.md:24-38); a composition of the primitives above:
//   h   = x + Wo . attention(rope(Wq . n1), rope(Wk . n1), Wv . n1),   n1 = rms_norm(x, norm1)
//   out = h + Wd . (silu(Wg . n2) * (Wu . n2)),                        n2 = rms_norm(h, norm2)
// x is [batch, seq, hidden]; weights are stored [out_features, in_features]; cos/sin are
// [>= seq, head_dim / 2]; `mask` is the additive attention mask [seq, seq] (0 / -inf for causal),
// or null for causal attention through the fused tensor-core kernel.
NodeRef op_llama_block(const NodeRef& x, const NodeRef& wq, const NodeRef& wk, const NodeRef& wv, const NodeRef& wo,
                       const NodeRef& wg, const NodeRef& wu, const NodeRef& wd, const NodeRef& norm1,
                       const NodeRef& norm2, const NodeRef& cos, const NodeRef& sin, const NodeRef& mask,
                       int n_heads, float eps) {
    WGF_CHECK(x->rank() == 3, WGF_ERR_RANK, "llama block input is [batch, seq, hidden]");
    const int64_t B = x->shape[0], S = x->shape[1], Hd = x->shape[2];
    WGF_CHECK(n_heads > 0 && Hd % n_heads == 0, WGF_ERR_SHAPE, "hidden size must divide into the heads");
    const int64_t D = Hd / n_heads;
    auto is2 = [](const NodeRef& w, int64_t o, int64_t i) { return w->rank() == 2 && w->shape[0] == o && w->shape[1] == i; };
    WGF_CHECK(is2(wq, Hd, Hd) && is2(wk, Hd, Hd) && is2(wv, Hd, Hd) && is2(wo, Hd, Hd), WGF_ERR_SHAPE,
              "attention weights must be [hidden, hidden]");
    WGF_CHECK(wg->rank() == 2 && wg->shape[1] == Hd && wu->shape == wg->shape && is2(wd, Hd, wg->shape[0]), WGF_ERR_SHAPE,
              "MLP weights must be [inter, hidden], [inter, hidden], [hidden, inter]");
    WGF_CHECK(!mask || is2(mask, S, S), WGF_ERR_SHAPE, "attention mask must be [seq, seq]");
    auto linear = [](const NodeRef& a, const NodeRef& w) { return make_matmul(a, view_transpose(w, 0, 1)); };
    // [B*S, Hd] -> [B*heads, S, D]
    auto split_heads = [&](const NodeRef& t) {
        NodeRef r = op_reshape(t, {B, S, (int64_t)n_heads, D});
        return op_reshape(view_transpose(r, 1, 2), {B * n_heads, S, D});
    };
    NodeRef x2 = op_reshape(x, {B * S, Hd});
    NodeRef n1 = op_layer_norm(x2, norm1, eps);
    WGF_CHECK(cos->rank() == 2 && sin->rank() == 2 && cos->shape == sin->shape && cos->shape[1] * 2 == D && cos->shape[0] >= S,
              WGF_ERR_SHAPE, "rope cos/sin must be [>= sequence, head_dim / 2]");
    WGF_CHECK(cos->dtype == x->dtype && sin->dtype == x->dtype, WGF_ERR_DTYPE, "rope element types differ");
    // rotary embedding read straight from the projection's [B, S, heads, D] layout (a transposed
    // view) and written as [B*heads, S, D]: splitting the heads costs no copy of its own
    auto rope_heads = [&](const NodeRef& t) {
        NodeRef t4 = view_transpose(op_reshape(t, {B, S, (int64_t)n_heads, D}), 1, 2);       // [B, heads, S, D]
        NodeRef r = new_node(NodeKind::Rope, t->dev, {B, (int64_t)n_heads, S, D}, t->dtype, {t4, cos, sin});
        return op_reshape(r, {B * n_heads, S, D});
    };
    NodeRef q = rope_heads(linear(n1, wq));
    NodeRef k = rope_heads(linear(n1, wk));
    NodeRef v_proj = linear(n1, wv);
    const float scale = 1.0f / std::sqrt((float)D);
    NodeRef merged;
    if (!mask && attention_supported(x->dtype, S, S, D)) {
        // The fused kernel reads V in place through the [B, heads, S, D] view of the projection (no
        // head-splitting copy) and writes the heads side by side: [B, S, heads * D] (no merging copy).
        NodeRef v4 = view_transpose(op_reshape(v_proj, {B, S, (int64_t)n_heads, D}), 1, 2);
        NodeRef att = new_node(NodeKind::Attention, x->dev, {B, S, Hd}, x->dtype, {q, k, v4});
        att->imm = scale;
        att->axis = 1;
        att->new_shape = {(int64_t)n_heads};
        merged = op_reshape(att, {B * S, Hd});
    } else {
        NodeRef ctx = op_attention(q, k, split_heads(v_proj), mask, true, scale);  // [B*heads, S, D]
        merged = op_reshape(view_transpose(op_reshape(ctx, {B, (int64_t)n_heads, S, D}), 1, 2), {B * S, Hd});
    }
    NodeRef h = make_binary(x2, linear(merged, wo), WGF_OP_ADD);
    NodeRef n2 = op_layer_norm(h, norm2, eps);
    NodeRef act = make_binary(op_silu(linear(n2, wg)), linear(n2, wu), WGF_OP_MUL);  // one fused kernel
    NodeRef out = make_binary(h, linear(act, wd), WGF_OP_ADD);
    return op_reshape(out, {B, S, Hd});
}

// ---------------------------------------------------------------------------------------
// resolver (src/compute_graph/resolve.rs:16-248, extended)
// ---------------------------------------------------------------------------------------
namespace {

bool is_ew(const Node* n) { return n->kind == NodeKind::ElementWise || n->kind == NodeKind::PairWise; }

// A set of nodes (or a map node -> int) kept in the nodes' own scratch slots: membership means
// "slot `kind` carries this set's epoch".  Sets of one kind used at the same time overwrite each
// other's entries, so a caller that runs nested resolutions re-inserts what it still needs.
static uint64_t g_mark_epoch = 0;
struct MarkSet {
    uint64_t epoch;
    int kind;
    explicit MarkSet(int k) : epoch(++g_mark_epoch), kind(k) {}
    bool contains(const Node* n) const { return n->scratch[kind].epoch == epoch; }
    bool insert(Node* n, int value = 0) {
        if (contains(n)) return false;
        n->scratch[kind].epoch = epoch;
        n->scratch[kind].value = value;
        return true;
    }
    int get(const Node* n) const { return n->scratch[kind].value; }
    void erase(Node* n) const {
        if (contains(n)) n->scratch[kind].epoch = 0;
    }
};

// Will `x` be unreachable once `root` has been materialised and has let go of its inputs?
// While a schedule is being recorded, a buffer may be overwritten in place only if it was
// produced inside the recording: a replay runs its producer again.  Overwriting a buffer from
// outside (an input of the schedule) would make the second run read what the first one wrote.
// After the recording the same holds the other way round: a buffer that belongs to a schedule
// that still exists is written by every replay, so nothing outside may move into it in place
// (a tensor computed in place from a recorded result would change under its holder at the next
// replay).
bool replay_may_overwrite(const Device& dev, const TensorData& td) {
    if (dev.recording()) return td.buf && td.buf->arena == dev.arena();
    if (td.buf && td.buf->arena) {
        std::lock_guard<std::mutex> g(td.buf->arena->mu);
        return td.buf->arena->closed;
    }
    return true;
}

bool dies_with(Node* x, Node* root, MarkSet& memo) {
    if (x == root) return true;
    if (memo.contains(x)) return memo.get(x) != 0;
    bool dead = x->handles == 0;
    if (dead)
        for (Node* c : x->consumers)
            if (!dies_with(c, root, memo)) {
                dead = false;
                break;
            }
    memo.insert(x, dead ? 1 : 0);
    return dead;
}

TensorData resolve_node(Node* n);

// ---- element-wise steps that move into the epilogue of the matmul that feeds them ----------------
// The crate never fuses anything around a MatMul (src/compute_graph/resolve.rs:138-154).  Two
// patterns are handed to the tensor-core kernel's epilogue here, when the product is a 16-bit
// tensor that nothing else can read: `product + t` (either order) for a tensor t of the same shape,
// and `silu(a . bg) * (a . bu)` with silu as the composite spells it, x / (1 + exp(-x)).  The
// kernel rounds where the separate kernels would, so the result has the same bits either way; when
// it does not take the problem (small or unaligned shapes, f32), the ordinary path runs.
bool is16(DType d) { return d == DType::F16 || d == DType::BF16; }

// true if `x` is an unmaterialised node without handles whose consumers are exactly `users`
bool private_to(const Node* x, std::initializer_list<const Node*> users) {
    if (x->cached || x->handles != 0 || x->consumers.size() != users.size()) return false;
    for (const Node* u : users)
        if (std::find(x->consumers.begin(), x->consumers.end(), u) == x->consumers.end()) return false;
    return true;
}

// big enough for the CTA-pair kernel (its own test is on the materialised operands; this one keeps
// small products out of the way of the ordinary fusion)
bool pair_kernel_shape(const Node* m) {
    const int r = m->rank();
    if (r != 2 && r != 3) return false;
    const int64_t M = m->shape[r - 2], N = m->shape[r - 1], K = m->inputs[0]->shape[r - 1];
    const int64_t rem = M % 256;
    return M >= 256 && N >= 128 && K >= 64 && !(M < 2048 && rem != 0 && rem <= 128);   // as matmul_tc_pair_path decides
}

struct EpilogueMatch {
    int kind = MatmulEpilogue::NONE;
    Node* m1 = nullptr;   // the product (RESIDUAL), or the gate product (SILU_MUL)
    Node* m2 = nullptr;   // the up product (SILU_MUL)
    Node* resid = nullptr;
};

// Does `n` together with the matmul(s) below it form one of the two patterns?  Looks at the graph only.
EpilogueMatch match_matmul_epilogue(const Node* n) {
    EpilogueMatch none;
    if (n->cached || n->kind != NodeKind::PairWise || !is16(n->dtype) || n->numel() == 0) return none;
    if (n->op == WGF_OP_ADD) {
        for (int side = 0; side < 2; ++side) {
            Node* m = n->inputs[side].get();
            Node* r = n->inputs[1 - side].get();
            if (m == r || m->kind != NodeKind::MatMul || !private_to(m, {n}) || !pair_kernel_shape(m)) continue;
            EpilogueMatch e;
            e.kind = MatmulEpilogue::RESIDUAL;
            e.m1 = m;
            e.resid = r;
            return e;
        }
        return none;
    }
    if (n->op != WGF_OP_MUL) return none;
    for (int side = 0; side < 2; ++side) {
        Node* s = n->inputs[side].get();        // silu(m1) = m1 / (1 + exp(-m1))
        Node* m2 = n->inputs[1 - side].get();
        if (s == m2 || m2->kind != NodeKind::MatMul || !private_to(m2, {n}) || !pair_kernel_shape(m2)) continue;
        if (s->kind != NodeKind::PairWise || s->op != WGF_OP_DIV || !private_to(s, {n})) continue;
        Node* m1 = s->inputs[0].get();
        Node* d1 = s->inputs[1].get();          // 1 + exp(-m1)
        if (m1->kind != NodeKind::MatMul || d1->kind != NodeKind::ElementWise || d1->op != WGF_OP_ADD_C || d1->imm != 1.0f ||
            !private_to(d1, {s}))
            continue;
        Node* e1 = d1->inputs[0].get();
        if (e1->kind != NodeKind::ElementWise || e1->op != WGF_OP_EXP || !private_to(e1, {d1})) continue;
        Node* n1 = e1->inputs[0].get();
        if (n1->kind != NodeKind::ElementWise || n1->op != WGF_OP_NEG || !private_to(n1, {e1}) || n1->inputs[0].get() != m1) continue;
        if (!private_to(m1, {s, n1}) || m1 == m2 || m1->inputs[0].get() != m2->inputs[0].get()) continue;
        EpilogueMatch e;
        e.kind = MatmulEpilogue::SILU_MUL;
        e.m1 = m1;
        e.m2 = m2;
        return e;
    }
    return none;
}

bool epilogue_fusion_on() { return getenv("WGF_NO_MATMUL_EPILOGUE") == nullptr; }   // read per call: tests compare both ways in one process

// One fused kernel: a region of element-wise / pair-wise nodes, optionally with reductions
// over one axis and their broadcasts back ("row mode").
struct Region {
    Node* root;
    bool row_mode = false;
    bool out_has_h = true;
    std::vector<int64_t> E;       // shape of the per-element domain (graph order)
    std::vector<int64_t> Rw;      // shape of the per-row domain
    std::vector<int> axes;        // reduced axes of E (one, or a trailing block when folded)
    Node* fold_top = nullptr;     // outermost node of a folded reduce chain
    Node* fold_x = nullptr;       // its per-element input
    MarkSet has_reduce_memo{Node::S_HAS_REDUCE};
    std::vector<Node*> leaves, fused_nodes;
    MarkSet leaf_set{Node::S_LEAF};
    MarkSet visited{Node::S_FUSED};
    int n_fused = 0;

    enum Dom { Elem, Row };

    // Marks again what nested resolutions (of the leaves) may have overwritten.
    void restamp() {
        for (Node* n : fused_nodes) visited.insert(n);
        for (Node* n : leaves) leaf_set.insert(n);
    }
    bool reduce_matches(const Node* n) const {
        if (n == fold_top) return true;
        return n->kind == NodeKind::Reduce && !n->cached && axes.size() == 1 && n->axis == axes[0] &&
               n->inputs[0]->shape == E;
    }
    bool row_chain_has_reduce(Node* n) {
        if (n->cached || n->shape != Rw) return false;
        if (has_reduce_memo.contains(n)) return has_reduce_memo.get(n) != 0;
        bool r = false;
        if (n->kind == NodeKind::Reduce) r = reduce_matches(n);
        else if (is_ew(n))
            for (auto& in : n->inputs) r = r || row_chain_has_reduce(in.get());
        has_reduce_memo.insert(n, r ? 1 : 0);
        return r;
    }
    bool bcast_of_row(const Node* n) const {
        return n->kind == NodeKind::MapLayout && n->view.kind == ViewOp::BroadcastAxis && axes.size() == 1 &&
               n->view.axis == axes[0] && n->view.size == E[axes[0]] && n->inputs[0]->shape == Rw;
    }
    bool fused(Node* n, Dom d) {
        if (n->cached) return false;
        if (n != root && (n_fused >= 200 || leaves.size() >= 12)) return false;
        if (d == Elem) {
            if (n->shape != E) return false;
            // a step that the matmul below it can do in its epilogue is left to that kernel
            if (n != root && n->kind == NodeKind::PairWise && epilogue_fusion_on() &&
                match_matmul_epilogue(n).kind != MatmulEpilogue::NONE)
                return false;
            if (is_ew(n)) return true;
            if (row_mode && bcast_of_row(n)) return row_chain_has_reduce(n->inputs[0].get());
            return false;
        }
        if (!row_mode || n->shape != Rw) return false;
        if (n->kind == NodeKind::Reduce) return reduce_matches(n);
        if (is_ew(n)) return row_chain_has_reduce(n);
        return false;
    }
    void collect(Node* n, Dom d) {
        if (!fused(n, d)) {
            if (leaf_set.insert(n)) leaves.push_back(n);
            return;
        }
        if (!visited.insert(n)) return;
        fused_nodes.push_back(n);
        n_fused++;
        if (n == fold_top) {
            collect(fold_x, Elem);
        } else if (n->kind == NodeKind::Reduce) {
            collect(n->inputs[0].get(), Elem);
        } else if (n->kind == NodeKind::MapLayout) {
            collect(n->inputs[0].get(), Row);
        } else {
            for (auto& in : n->inputs) collect(in.get(), d);
        }
    }
};

// Finds, below an element-shaped root, a broadcast-along-the-last-axis of a reduction over
// that axis (RmsNorm, softmax, ...).
bool find_row_pattern(Node* n, const std::vector<int64_t>& E, MarkSet& seen, Region& probe) {
    if (n->cached || n->shape != E || !seen.insert(n)) return false;
    if (n->kind == NodeKind::MapLayout) return probe.bcast_of_row(n) && probe.row_chain_has_reduce(n->inputs[0].get());
    if (!is_ew(n)) return false;
    for (auto& in : n->inputs)
        if (find_row_pattern(in.get(), E, seen, probe)) return true;
    return false;
}

// Finds the first reduction below a row-shaped root, walking element-wise nodes of equal shape.
Node* find_reduce_below(Node* n, const std::vector<int64_t>& shape, MarkSet& seen) {
    if (n->cached || n->shape != shape || !seen.insert(n)) return nullptr;
    if (n->kind == NodeKind::Reduce) return n;
    if (!is_ew(n)) return nullptr;
    for (auto& in : n->inputs)
        if (Node* r = find_reduce_below(in.get(), shape, seen)) return r;
    return nullptr;
}

// Moves the axes in `axes` to the end (keeping their order) and merges them into one axis.
// Returns false if the layout does not allow the merge.
bool to_index_layout(const Layout& in, const std::vector<int>& axes, Layout& out) {
    out = Layout();
    out.offset = in.offset;
    std::vector<char> red(in.rank(), 0);
    for (int a : axes) red[a] = 1;
    for (int i = 0; i < in.rank(); ++i)
        if (!red[i]) {
            out.shape.push_back(in.shape[i]);
            out.strides.push_back(in.strides[i]);
        }
    int64_t h = 1, hs = 0;
    bool first = true;
    for (int k = (int)axes.size() - 1; k >= 0; --k) {
        int a = axes[k];
        if (in.shape[a] == 1) continue;
        if (first) {
            hs = in.strides[a];
            first = false;
        } else if (in.strides[a] != hs * h) {
            return false;
        }
        h *= in.shape[a];
    }
    out.shape.push_back(h);
    out.strides.push_back(first ? 0 : hs);
    return true;
}

float round_imm(float c, DType dt) {
    if (dt == DType::F16) return f16_to_f32(f32_to_f16(c));
    if (dt == DType::BF16) return bf16_to_f32(f32_to_bf16(c));
    return c;
}

struct Emitter {
    Region& rg;
    Program prog;
    std::vector<TensorData> slots;
    std::vector<Node*> slot_leaf;
    MarkSet value{Node::S_VALUE};
    bool ok = true;

    explicit Emitter(Region& r) : rg(r) {}

    int leaf(Node* n, Region::Dom d) {
        const TensorData& td = n->cached;
        Layout L;
        if (!rg.row_mode) {
            L = td.layout;
        } else if (d == Region::Row) {
            L = td.layout;
            L.shape.push_back(1);
            L.strides.push_back(0);
            // extent of the row axis is filled in by the caller's index shape
        } else if (!to_index_layout(td.layout, rg.axes, L)) {
            ok = false;
            return prog.load(0, td.dtype, VKind::Elem);
        }
        int slot = -1;
        for (int s = 0; s < (int)slots.size(); ++s)
            if (slots[s].buf == td.buf && slots[s].dtype == td.dtype && slots[s].layout.offset == L.offset &&
                slots[s].layout.strides == L.strides)
                slot = s;
        if (slot < 0) {
            slot = prog.new_slot(td.dtype);
            TensorData sd;
            sd.buf = td.buf;
            sd.dtype = td.dtype;
            sd.layout = L;
            slots.push_back(sd);
            slot_leaf.push_back(n);
        } else if (slot_leaf[slot] != n) {
            slot_leaf[slot] = nullptr;  // two leaves share the view: never overwrite it
        }
        VKind k = VKind::Elem;
        if (rg.row_mode && (d == Region::Row || (L.strides.back() == 0 && L.shape.back() > 1))) k = VKind::Row;
        return prog.load(slot, td.dtype, k);
    }

    int emit(Node* n, Region::Dom d) {
        if (value.contains(n)) return value.get(n);
        int v;
        if (rg.leaf_set.contains(n)) {
            v = leaf(n, d);
        } else if (n == rg.fold_top) {
            v = prog.row_reduce(n->op, emit(rg.fold_x, Region::Elem));
        } else if (n->kind == NodeKind::Reduce) {
            v = prog.row_reduce(n->op, emit(n->inputs[0].get(), Region::Elem));
        } else if (n->kind == NodeKind::MapLayout) {
            v = emit(n->inputs[0].get(), Region::Row);
        } else if (n->kind == NodeKind::PairWise) {
            int a = emit(n->inputs[0].get(), d);
            int b = emit(n->inputs[1].get(), d);
            v = prog.binary(n->op, a, b);
        } else {
            int a = emit(n->inputs[0].get(), d);
            if (n->op == WGF_OP_CAST) v = prog.cast(a, n->dtype);
            else if (n->op >= WGF_OP_ADD_C) v = prog.scalar(n->op, a, round_imm(n->imm, prog.ins[a].dtype));
            else v = prog.unary(n->op, a);
        }
        value.insert(n, v);
        return v;
    }
};

// Sets up the region for `root`; returns false if `root` has to run as plain element-wise
// or (for a Reduce root) cannot be folded with the reductions below it.
void plan_region(Region& rg, bool allow_fold) {
    Node* root = rg.root;
    rg.row_mode = false;
    if (is_ew(root)) {
        // (1) element-shaped result with reductions over the last axis inside
        if (root->rank() >= 1 && root->shape.back() >= 1 && root->shape.back() <= max_resident_row(false)) {
            Region probe;
            probe.root = root;
            probe.row_mode = true;
            probe.E = root->shape;
            probe.Rw.assign(root->shape.begin(), root->shape.end() - 1);
            probe.axes = {root->rank() - 1};
            MarkSet seen(Node::S_SEEN);
            if (find_row_pattern(root, root->shape, seen, probe)) {
                rg.row_mode = true;
                rg.out_has_h = true;
                rg.E = probe.E;
                rg.Rw = probe.Rw;
                rg.axes = probe.axes;
                return;
            }
        }
        // (2) row-shaped result: element-wise epilogue on top of a reduction
        MarkSet seen(Node::S_SEEN);
        if (Node* r = find_reduce_below(root, root->shape, seen)) {
            rg.row_mode = true;
            rg.out_has_h = false;
            rg.E = r->inputs[0]->shape;
            rg.Rw = root->shape;
            rg.axes = {r->axis};
            return;
        }
        rg.E = root->shape;
        return;
    }
    // root is a Reduce
    rg.row_mode = true;
    rg.out_has_h = false;
    rg.Rw = root->shape;
    rg.E = root->inputs[0]->shape;
    rg.axes = {root->axis};
    if (!allow_fold) return;
    // fold reduce-of-reduce with the same op when the reduced axes form a trailing block
    // (this makes `t.sum(0).sum(0)` on a matrix one full-tensor reduction)
    Node* x = root;
    std::vector<Node*> chain;
    while (true) {
        chain.push_back(x);
        Node* in = x->inputs[0].get();
        if (in->kind != NodeKind::Reduce || in->op != root->op || in->cached || in->handles != 0 ||
            in->consumers.size() != 1)
            break;
        x = in;
    }
    if (chain.size() < 2) return;
    Node* base = chain.back()->inputs[0].get();
    std::vector<int> idx(base->rank());
    for (int i = 0; i < base->rank(); ++i) idx[i] = i;
    std::vector<int> reduced;
    for (int k = (int)chain.size() - 1; k >= 0; --k) {
        reduced.push_back(idx[chain[k]->axis]);
        idx.erase(idx.begin() + chain[k]->axis);
    }
    std::sort(reduced.begin(), reduced.end());
    const int first = base->rank() - (int)reduced.size();
    for (int i = 0; i < (int)reduced.size(); ++i)
        if (reduced[i] != first + i) return;  // not a trailing block
    rg.E = base->shape;
    rg.axes = reduced;
    rg.fold_top = root;
    rg.fold_x = base;
}

// Nodes requested together with `g_companion_host` (resolve_many): whole-tensor reductions
// that may ride along in the host's row kernel, which already has every element in registers.
// Each candidate comes with the all-reduce node requested on top of it, if any.
struct Candidate {
    Node* reduce;
    Node* all_reduce;
};
thread_local Node* g_companion_host = nullptr;
thread_local std::vector<Candidate>* g_companions = nullptr;

// The per-element expression under a reduction (or folded chain of reductions) of a whole
// tensor of shape `E` to a scalar; nullptr if `c` is not of that form.
Node* companion_expr(Node* c, const std::vector<int64_t>& E) {
    if (c->cached || c->kind != NodeKind::Reduce || c->rank() != 0) return nullptr;
    Region cr;
    cr.root = c;
    plan_region(cr, true);
    if (!cr.Rw.empty() || cr.E != E) return nullptr;
    return cr.fold_top ? cr.fold_x : c->inputs[0].get();
}

// Adds the element-wise nodes under `n` to the host region `rg` (same index space); anything
// else becomes an input of the kernel.
void gather_companion(Node* n, Region& rg) {
    if (rg.visited.contains(n)) return;   // already computed by the host
    if (!n->cached && is_ew(n) && n->shape == rg.E) {
        rg.visited.insert(n);
        rg.fused_nodes.push_back(n);
        rg.n_fused++;
        for (auto& in : n->inputs) gather_companion(in.get(), rg);
    } else if (rg.leaf_set.insert(n)) {
        rg.leaves.push_back(n);
    }
}

// An all-reduce node asks the kernel that computes its (rank-0) input to do the exchange too.
struct ArRequest {
    Node* root;
    Comm* comm;
    uint16_t op;
    bool done;
};
thread_local ArRequest* g_ar_request = nullptr;

TensorData run_region(Node* root, bool allow_fold = true) {
    std::vector<Candidate> candidates;
    if (g_companions && root == g_companion_host) {
        candidates = *g_companions;
        g_companions = nullptr;   // leaves resolved below must not pick them up again
    }
    ArRequest* arq = g_ar_request && g_ar_request->root == root ? g_ar_request : nullptr;
    g_ar_request = nullptr;       // likewise
    Region rg;
    rg.root = root;
    plan_region(rg, allow_fold);
    rg.collect(root, rg.row_mode && !rg.out_has_h ? Region::Row : Region::Elem);
    for (Node* l : rg.leaves) resolve_node(l);   // a candidate the host depends on is computed here
    rg.restamp();
    struct Companion {
        Node* reduce;       // the reduction node
        Node* expr;         // its per-element expression
        Node* all_reduce;   // the all-reduce node on top of it that the kernel performs too, or null
    };
    std::vector<Companion> companions;
    Comm* kernel_comm = nullptr;   // one communicator per kernel
    if (rg.row_mode && rg.out_has_h && root->numel() > 0) {
        for (const Candidate& cand : candidates) {
            Node* c = cand.reduce;
            if (c->dev != root->dev || companions.size() >= (size_t)kMailboxValues) continue;
            Node* expr = companion_expr(c, rg.E);
            if (!expr) continue;
            const size_t nf = rg.fused_nodes.size(), nl = rg.leaves.size();
            const int fused_before = rg.n_fused;
            gather_companion(expr, rg);
            if (rg.leaves.size() > 12 || rg.n_fused > 200) {   // too big: take its nodes out again
                for (size_t i = nf; i < rg.fused_nodes.size(); ++i) rg.visited.erase(rg.fused_nodes[i]);
                for (size_t i = nl; i < rg.leaves.size(); ++i) rg.leaf_set.erase(rg.leaves[i]);
                rg.fused_nodes.resize(nf);
                rg.leaves.resize(nl);
                rg.n_fused = fused_before;
                continue;
            }
            // The all-reduce on top of it is done by the same kernel over peer memory when the
            // partial result of this GPU is not observable on its own.
            Node* ar = cand.all_reduce;
            const bool fuse_ar = ar && !ar->cached && ar->comm && ar->comm->peer_ok && !root->dev->exchange_broken && c->handles == 0 &&
                                 c->consumers.size() == 1 && c->consumers[0] == ar &&
                                 (!kernel_comm || kernel_comm == ar->comm.get());
            if (fuse_ar) kernel_comm = ar->comm.get();
            companions.push_back(Companion{c, expr, fuse_ar ? ar : nullptr});
        }
        if (!companions.empty()) {
            for (Node* l : rg.leaves) resolve_node(l);
            rg.restamp();
        }
    }

    Emitter em(rg);
    int res = em.emit(root, rg.row_mode && !rg.out_has_h ? Region::Row : Region::Elem);
    em.prog.result = res;
    for (auto& ce : companions) {
        int v = em.emit(ce.expr, Region::Elem);
        Grand g{ce.reduce->op, v, ce.reduce->dtype};
        if (ce.all_reduce) {
            g.all_reduce = true;
            g.ar_op = ce.all_reduce->op;
        }
        em.prog.grands.push_back(g);
    }
    if (!em.ok) {
        WGF_CHECK(rg.fold_top != nullptr, WGF_ERR_UNSUPPORTED, "internal: unmergeable index space");
        g_ar_request = arq;
        return run_region(root, false);  // some input cannot be flattened: reduce axis by axis
    }
    // A streaming reduction to one scalar that feeds only an all-reduce does the exchange itself.
    bool result_ar = false;
    if (arq && rg.row_mode && !rg.out_has_h && root->rank() == 0 && !em.prog.multi_phase() && companions.empty()) {
        int64_t elements = 1;
        for (auto v : rg.E) elements *= v;
        if (elements > 0) {
            em.prog.result_all_reduce = true;
            em.prog.result_ar_op = arq->op;
            kernel_comm = arq->comm;
            result_ar = true;
        }
    }

    // index space
    std::vector<int64_t> index_shape;
    if (rg.row_mode) {
        index_shape = rg.Rw;
        int64_t h = 1;
        for (int a : rg.axes) h *= rg.E[a];
        index_shape.push_back(h);
        for (auto& s : em.slots) s.layout.shape = index_shape;  // row-domain leaves get the row axis, stride 0
    } else {
        index_shape = rg.E;
    }

    // in-place candidate: an input that nothing can read after this kernel
    int inplace = -1;
    Node* donor = nullptr;
    TensorData saved;
    if (!rg.row_mode || rg.out_has_h) {
        MarkSet memo(Node::S_DIES);
        const DType odt = em.prog.out_dtype();
        for (int s = 0; s < (int)em.slots.size() && inplace < 0; ++s) {
            Node* l = em.slot_leaf[s];
            if (!l || !dies_with(l, root, memo)) continue;
            const TensorData& sd = em.slots[s];
            if (!replay_may_overwrite(*root->dev, sd)) continue;
            if (dtype_size(sd.dtype) != dtype_size(odt) || !sd.layout.is_dense() || sd.layout.allocation_overlaps())
                continue;
            long shared = 0;
            for (auto& o : em.slots) shared += o.buf == sd.buf;
            if (shared != 1 || sd.buf.use_count() != 2) continue;  // the leaf's cache + this slot
            inplace = s;
            donor = l;
        }
    }
    if (donor) {
        // The donor's cache lets go of the buffer, so that the slot holds the only reference
        // (what the launcher checks).  Its layout is kept to put the cache back on failure.
        saved.layout = donor->cached.layout;
        saved.dtype = donor->cached.dtype;
        donor->cached = TensorData();
    }
    TensorData out;
    std::vector<TensorData> grand_out;
    try {
        Device& dev = *root->dev;
        GrandComm gc{};
        // the exchange carries a sequence number that the host advances per launch
        if (kernel_comm) dev.refuse_while_recording("an all-reduce");
        if (kernel_comm) {
            // an input that is a result of the open exchange is settled first: the kernel then has no
            // exchange to settle, instead of rewriting a value it also reads
            for (auto& t : em.slots) dev.wait_for(*t.buf);
            gc = comm_peer_begin(*kernel_comm, dev);
        }
        if (rg.row_mode) out = run_rows(dev, em.prog, em.slots, index_shape, rg.out_has_h, inplace, &grand_out, kernel_comm ? &gc : nullptr);
        else out = run_elementwise(dev, em.prog, em.slots, index_shape, inplace);
        if (kernel_comm) {
            // The kernel posts this GPU's values to every rank's mailbox (and settles the exchange
            // before this one).  The other half of this exchange -- wait for the peers' values, combine
            // in rank order, overwrite the results -- rides in the next kernel that posts, or runs as
            // a kernel of its own when a result is read first.
            std::vector<PeerValue> vals;
            if (result_ar) vals.push_back(PeerValue{arq->op, 0u, out});
            for (size_t i = 0; i < companions.size(); ++i)
                if (companions[i].all_reduce) vals.push_back(PeerValue{companions[i].all_reduce->op, (uint32_t)i, grand_out[i]});
            comm_peer_finish(*kernel_comm, dev, gc.seq, vals);
        }
    } catch (...) {
        if (donor) {
            saved.buf = em.slots[inplace].buf;
            donor->cached = std::move(saved);
        }
        throw;
    }
    if (result_ar) arq->done = true;
    for (size_t i = 0; i < companions.size(); ++i) {
        // the value belongs to the all-reduce node when the kernel did that too (the reduction
        // node below it is never materialised and goes away with the all-reduce's inputs)
        Node* c = companions[i].all_reduce ? companions[i].all_reduce : companions[i].reduce;
        c->cached = grand_out[i];
        c->drop_inputs();
    }
    out.layout.shape = root->shape;  // same element count and order; restores extent-1 axes
    if ((int)out.layout.strides.size() != root->rank()) out.layout.strides = Layout::contiguous_strides(root->shape);
    return out;
}

bool try_matmul_epilogue(Node* n, TensorData& out) {
    const EpilogueMatch e = match_matmul_epilogue(n);
    if (e.kind == MatmulEpilogue::NONE || !epilogue_fusion_on()) return false;
    Device& dev = *n->dev;
    if (e.kind == MatmulEpilogue::RESIDUAL) {
        TensorData a = resolve_node(e.m1->inputs[0].get());
        TensorData b = resolve_node(e.m1->inputs[1].get());
        TensorData res = resolve_node(e.resid);
        return run_matmul_residual(dev, a, b, res, out);
    }
    TensorData a = resolve_node(e.m1->inputs[0].get());
    TensorData bg = resolve_node(e.m1->inputs[1].get());
    TensorData bu = resolve_node(e.m2->inputs[1].get());
    return run_matmul_silu_mul(dev, a, bg, bu, out);
}

TensorData resolve_node(Node* n) {
    if (n->cached) {
        // every read of already materialised data passes here: a recording keeps what it reads
        n->dev->note_recorded_buffer(n->cached.buf);
        return n->cached;
    }
    Device& dev = *n->dev;
    TensorData out;
    switch (n->kind) {
        case NodeKind::Tensor:
            fail(WGF_ERR_INVALID_HANDLE, "tensor node without data");
        case NodeKind::MapLayout: {  // src/compute_graph/resolve.rs:198-208
            TensorData in = resolve_node(n->inputs[0].get());
            out.buf = in.buf;
            out.dtype = in.dtype;
            out.layout = n->view.apply(in.layout);
            break;
        }
        case NodeKind::ElementWise:
        case NodeKind::PairWise:
        case NodeKind::Reduce:
            if (!try_matmul_epilogue(n, out)) out = run_region(n);
            break;
        case NodeKind::MatMul: {  // src/compute_graph/resolve.rs:138-154
            TensorData a = resolve_node(n->inputs[0].get());
            TensorData b = resolve_node(n->inputs[1].get());
            out = run_matmul(dev, a, b);
            break;
        }
        case NodeKind::Rope: {
            TensorData x = resolve_node(n->inputs[0].get());
            TensorData c = resolve_node(n->inputs[1].get());
            TensorData s = resolve_node(n->inputs[2].get());
            out = run_rope(dev, x, c, s);
            break;
        }
        case NodeKind::Attention: {
            TensorData q = resolve_node(n->inputs[0].get());
            TensorData k = resolve_node(n->inputs[1].get());
            TensorData v = resolve_node(n->inputs[2].get());
            out = run_attention(dev, q, k, v, n->axis != 0, n->imm, n->new_shape.empty() ? 0 : (int)n->new_shape[0]);
            break;
        }
        case NodeKind::Resize: {  // src/compute_graph/resolve.rs:210-226
            TensorData in = resolve_node(n->inputs[0].get());
            const bool reshape = n->new_shape == n->fill_shape;
            if (reshape) {
                // a reshape of row-major data is a view; anything else is gathered first
                TensorData dense = in.layout.is_dense() && !in.layout.allocation_overlaps() ? in : run_compact(dev, in);
                out.buf = dense.buf;
                out.dtype = dense.dtype;
                out.layout = Layout::contiguous(n->new_shape);
                out.layout.offset = dense.layout.offset;
            } else {
                Layout full = Layout::contiguous(n->new_shape);
                out.buf = dev.alloc((size_t)std::max<int64_t>(full.numel(), 1) * dtype_size(n->dtype), true);
                out.dtype = n->dtype;
                out.layout = full;
                TensorData box = out;
                for (int i = 0; i < full.rank(); ++i) {
                    WGF_CHECK(n->fill_shape[i] <= n->new_shape[i], WGF_ERR_SHAPE, "resize cannot shrink an axis");
                    box.layout.shape[i] = n->fill_shape[i];
                }
                run_copy(dev, box, in);
            }
            break;
        }
        case NodeKind::SliceAssign: {  // src/compute_graph/resolve.rs:228-244
            Node* tn = n->inputs[0].get();
            TensorData target = resolve_node(tn);
            TensorData value = resolve_node(n->inputs[1].get());
            // The crate writes into the target's buffer.  That is kept only when nothing else
            // can still read the old contents; otherwise the target is copied first.
            MarkSet memo(Node::S_DIES);
            bool own = dies_with(tn, n, memo) && !target.layout.allocation_overlaps() &&
                       replay_may_overwrite(dev, target);
            if (own) {
                tn->cached = TensorData();           // `target` now holds the only reference if unshared
                own = target.buf.use_count() == 1;
                if (!own) tn->cached = target;
            }
            if (!own) target = run_compact(dev, target);
            ViewOp v;
            v.kind = ViewOp::Slice;
            v.starts = n->starts;
            v.ends = n->ends;
            TensorData window = target;
            window.layout = v.apply(target.layout);
            run_copy(dev, window, value);
            out = target;
            break;
        }
        case NodeKind::AllReduce: {
            dev.refuse_while_recording("an all-reduce");
            WGF_CHECK(!dev.exchange_broken, WGF_ERR_TIMEOUT,
                      "an earlier all-reduce gave up waiting for a peer: the ranks are out of step; release the communicator");
            Node* src = n->inputs[0].get();
            // A scalar that only this all-reduce can see is exchanged by the kernel that computes
            // it (over peer memory) where that kernel is a streaming reduction; see ArRequest.
            ArRequest arq{src, n->comm.get(), n->op, false};
            if (!src->cached && n->comm && n->comm->peer_ok && src->rank() == 0 && src->handles == 0 &&
                src->consumers.size() == 1 && (src->kind == NodeKind::Reduce || is_ew(src)))
                g_ar_request = &arq;
            TensorData in;
            try {
                in = resolve_node(src);
            } catch (...) {
                g_ar_request = nullptr;
                throw;
            }
            g_ar_request = nullptr;
            if (arq.done) {
                out = in;
                break;
            }
            const bool dense_in = in.layout.is_dense() && !in.layout.allocation_overlaps();
            // The collective runs in place.  If nothing else can read the partial result any
            // more, its own buffer is used (no copy); otherwise a dense copy is reduced.
            MarkSet memo(Node::S_DIES);
            bool own = dense_in && dies_with(src, n, memo);
            if (own) {
                src->cached = TensorData();
                own = in.buf.use_count() == 1;
                if (!own) src->cached = in;
            }
            out = own ? in : run_compact(dev, in);
            out.layout.shape = n->shape;
            if ((int)out.layout.strides.size() != n->rank()) out.layout.strides = Layout::contiguous_strides(n->shape);
            dev.wait_for(*out.buf);
            comm_all_reduce(*n->comm, dev, *out.buf, out.base_ptr(), out.layout.numel(), n->dtype, n->op);
            break;
        }
    }
    n->cached = out;
    n->drop_inputs();
    return out;
}

}  // namespace

TensorData resolve(const NodeRef& n) {
    if (n->cached) return n->cached;
    Device& dev = *n->dev;
    dev.make_current();
    auto g = graph_of(n);
    dev.sink = dev.timing ? &g->timings : nullptr;
    try {
        TensorData out = resolve_node(n.get());
        dev.sink = nullptr;
        return out;
    } catch (...) {
        dev.sink = nullptr;
        throw;
    }
}

// Resolves several tensors as one request.  Whole-tensor reductions among them (also below a
// requested all-reduce) are offered to the row kernels of the other requested tensors: where
// both read the same index space, the reduction is computed by that kernel and costs no
// second pass over memory.  The crate resolves one tensor per call (src/tensor.rs:551-554)
// and lists fusing sibling reductions as future work (README.md:19-22).
void resolve_many(const std::vector<NodeRef>& nodes) {
    std::vector<NodeRef> keep;   // the candidates stay alive whatever the hosts resolve
    std::vector<Candidate> comps;
    for (auto& n : nodes) {
        NodeRef c = n;
        Node* ar = nullptr;
        if (!c->cached && c->kind == NodeKind::AllReduce) {
            ar = c.get();
            c = c->inputs[0];
        }
        if (!c->cached && c->kind == NodeKind::Reduce && c->rank() == 0) {
            keep.push_back(c);
            comps.push_back(Candidate{c.get(), ar});
        }
    }
    for (auto& n : nodes) {
        if (n->cached || !is_ew(n.get()) || comps.empty()) continue;
        g_companion_host = n.get();
        g_companions = &comps;
        try {
            resolve(n);
        } catch (...) {
            g_companions = nullptr;
            g_companion_host = nullptr;
            throw;
        }
        g_companions = nullptr;
        g_companion_host = nullptr;
        comps.erase(std::remove_if(comps.begin(), comps.end(),
                                   [](const Candidate& c) {
                                       return (bool)c.reduce->cached || (c.all_reduce && (bool)c.all_reduce->cached);
                                   }),
                    comps.end());
    }
    for (auto& n : nodes) resolve(n);
}

// ---------------------------------------------------------------------------------------
// Graphviz dump (src/compute_graph/visualize.rs)
// ---------------------------------------------------------------------------------------
std::string graphviz(const NodeRef& root) {
    static const char* kinds[] = {"tensor", "element_wise", "pair_wise", "reduce", "mat_mul",
                                  "map_layout", "resize", "slice_assign", "all_reduce", "attention", "rope"};
    std::ostringstream s;
    s << "digraph compute_graph {\n";
    std::unordered_set<Node*> seen;
    std::function<void(Node*)> walk = [&](Node* n) {
        if (!seen.insert(n).second) return;
        s << "  n" << n->id << " [label=\"" << kinds[(int)n->kind];
        if (n->kind != NodeKind::Tensor && n->kind != NodeKind::MapLayout && n->kind != NodeKind::Resize &&
            n->kind != NodeKind::SliceAssign && n->kind != NodeKind::MatMul)
            s << " op=" << n->op;
        s << " " << dtype_name(n->dtype) << " [";
        for (size_t i = 0; i < n->shape.size(); ++i) s << (i ? "," : "") << n->shape[i];
        s << "]" << (n->cached ? " *" : "") << "\"];\n";
        for (auto& in : n->inputs) {
            walk(in.get());
            s << "  n" << in->id << " -> n" << n->id << ";\n";
        }
    };
    walk(root.get());
    s << "}\n";
    return s.str();
}

}  // namespace wgf
