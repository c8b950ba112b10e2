// Fused softmax attention on the tcgen05 tensor cores (attention_tc.cu).
#pragma once
#include "launch.hpp"

namespace wgf {

// True if run_attention can take tensors [batch*heads, seq_q, head_dim] x [batch*heads, seq_k, head_dim].
bool attention_supported(DType dt, int64_t seq_q, int64_t seq_k, int64_t head_dim);

// softmax(scale * q k^T, keys after the query masked out when `causal`) v  for every batch*head.
// q, k, v: [batch*heads, seq, 128] of one 16-bit type; views that are not row-contiguous are
// gathered first.  Returns a new contiguous tensor of the same shape and type; with
// `merge_heads` = h > 0 the leading axis is read as batch * h + head and the result is written
// as [batch, seq, h * 128] (the heads side by side in each row), which saves the transposing
// copy that merging heads otherwise needs.
TensorData run_attention(Device& dev, const TensorData& q, const TensorData& k, const TensorData& v, bool causal, float scale,
                         int merge_heads = 0);

}  // namespace wgf
