// Shared reference math for com.microsoft operators (used by the generic
// kernels, the collective kernels and as the oracle for the GPU kernels).
#pragma once
#include <ATen/ATen.h>

#include <string>
#include <vector>

#include "graph.h"

namespace ortb {
namespace contrib {

std::vector<int64_t> ToVec(const at::Tensor& t);

struct MoeAttrs {
  int64_t k = 1;
  std::string activation = "relu";
  bool normalize = false;
  int64_t swiglu_fusion = 0;
  bool has_limit = false;
  float swiglu_limit = 0.f;
  float alpha = 1.f, beta = 0.f;
};
MoeAttrs ParseMoeAttrs(const Node& n);

// x [T,H], logits [T,E]; fc1 [E_local, F*I, H], fc2 [E_local, H, I], optional fc3 [E_local, I, H].
// Only experts in [expert_begin, expert_end) contribute (expert_end < 0 = all); the
// weight stacks are indexed relative to expert_begin.
at::Tensor MoeForward(const at::Tensor& x, const at::Tensor& logits, const at::Tensor& fc1, const at::Tensor& fc1_b,
                      const at::Tensor& fc2, const at::Tensor& fc2_b, const at::Tensor& fc3, const at::Tensor& fc3_b,
                      const MoeAttrs& a, int64_t expert_begin, int64_t expert_end);

at::Tensor DequantizeNBits(const at::Tensor& B, const at::Tensor& scales, const at::Tensor& zero_points, int64_t N,
                           int64_t K, int64_t bits, int64_t block_size, at::ScalarType out_type);

at::Tensor DequantizeQMoeWeights(const at::Tensor& w, const at::Tensor& scales, int64_t bits, int64_t block);

at::Tensor RotaryBSNH(const at::Tensor& x, const at::Tensor& pos, const at::Tensor& cos_cache,
                      const at::Tensor& sin_cache, bool interleaved, int64_t rot_dim, float scale);

// additive mask [B, 1, 1 or S, T] from the mask_index forms of the BERT Attention operator (lengths, end / start
// positions, 2-D / 3-D / 4-D 0-1 masks); masked positions get `filter`
at::Tensor AttentionMaskBias(const at::Tensor& mask_index, int64_t B, int64_t S, int64_t T, float filter, at::Device dev);

// LongformerAttention on projected inputs (kernels_contrib4.cc): qkv / gqkv [B, S, 3 * hidden] float -> [B, S, hidden]
at::Tensor LongformerCore(const at::Tensor& qkv, const at::Tensor& gqkv, const at::Tensor& mask, const at::Tensor& global, int64_t N, int64_t w);

struct GqaInputs {
  at::Tensor query, key, value, past_key, past_value, seqlens_k, cos_cache, sin_cache, position_ids, attention_bias,
      head_sink;
  int64_t total_sequence_length = 0;
  bool share_buffer = false;
};
struct GqaAttrs {
  int64_t num_heads = 0, kv_num_heads = 0, local_window_size = -1;
  bool do_rotary = false, rotary_interleaved = false, smooth_softmax = false;
  float scale = 0.f, softcap = 0.f;
};
struct GqaResult {
  at::Tensor output, present_key, present_value;
};
GqaResult GqaForward(const GqaInputs& in, const GqaAttrs& a);

}  // namespace contrib
}  // namespace ortb
