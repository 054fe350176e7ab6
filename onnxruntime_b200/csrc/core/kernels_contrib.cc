// com.microsoft contrib operators written against ATen.  These are the CPU
// execution provider's implementations and the numerical oracle for the
// hand-written sm_100a kernels.  The math restates the reference's CPU contrib
// kernels (onnxruntime/contrib_ops/cpu/bert/{attention_cpu_base.h,
// gqa_attention_base.h,rotary_embedding.cc}, skip_layer_norm.cc,
// quantization/matmul_nbits_impl.cc, moe/moe_cpu.cc) in tensor form.
#include <ATen/ATen.h>

#include <cmath>
#include <limits>

#include "collective.h"
#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace contrib {

std::vector<int64_t> ToVec(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

at::Tensor FastGeluRef(const at::Tensor& x) { return at::gelu(x, "tanh"); }

at::Tensor ApplyRotary(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin, bool interleaved) {
  // x [..., rot]; cos/sin broadcastable to [..., rot/2]
  if (interleaved) {
    at::Tensor x1 = x.slice(-1, 0, c10::nullopt, 2), x2 = x.slice(-1, 1, c10::nullopt, 2);
    return at::stack({x1 * cos - x2 * sin, x2 * cos + x1 * sin}, -1).flatten(-2);
  }
  const int64_t half = x.size(-1) / 2;
  at::Tensor x1 = x.narrow(-1, 0, half), x2 = x.narrow(-1, half, half);
  return at::cat({x1 * cos - x2 * sin, x2 * cos + x1 * sin}, -1);
}

// x: [B, S, N, H]; pos: [B, S] int64; caches [max, rot/2].
at::Tensor RotaryBSNH(const at::Tensor& x, const at::Tensor& pos, const at::Tensor& cos_cache,
                      const at::Tensor& sin_cache, bool interleaved, int64_t rot_dim, float scale) {
  const int64_t H = x.size(3);
  if (rot_dim == 0) rot_dim = cos_cache.size(1) * 2;
  at::Tensor p = pos.to(cos_cache.device());
  at::Tensor cos = cos_cache.index({p}).unsqueeze(2).to(at::kFloat);  // B,S,1,rot/2
  at::Tensor sin = sin_cache.index({p}).unsqueeze(2).to(at::kFloat);
  at::Tensor xf = x.to(at::kFloat);
  at::Tensor y = ApplyRotary(xf.narrow(-1, 0, rot_dim), cos, sin, interleaved);
  if (rot_dim < H) y = at::cat({y, xf.narrow(-1, rot_dim, H - rot_dim)}, -1);
  if (scale != 1.0f) y = y * scale;
  return y.to(x.scalar_type());
}

at::Tensor DequantizeNBits(const at::Tensor& B, const at::Tensor& scales, const at::Tensor& zero_points, int64_t N,
                           int64_t K, int64_t bits, int64_t block_size, at::ScalarType out_type) {
  ORTB_ENFORCE_ARG(bits == 4 || bits == 8, "MatMulNBits supports bits = 4 or 8");
  const int64_t n_blocks = (K + block_size - 1) / block_size;
  at::Tensor q;
  if (bits == 4) {
    at::Tensor b = B.reshape({N, n_blocks, block_size / 2}).to(at::kInt);
    at::Tensor lo = at::bitwise_and(b, 0xF), hi = at::bitwise_and(at::bitwise_right_shift(b, 4), 0xF);
    q = at::stack({lo, hi}, -1).reshape({N, n_blocks, block_size}).to(at::kFloat);
  } else {
    q = B.reshape({N, n_blocks, block_size}).to(at::kFloat);
  }
  at::Tensor s = scales.reshape({N, n_blocks, 1}).to(at::kFloat);
  at::Tensor zp;
  if (zero_points.defined()) {
    if (zero_points.scalar_type() == at::kByte) {
      if (bits == 4) {
        at::Tensor z = zero_points.reshape({N, -1}).to(at::kInt);
        at::Tensor lo = at::bitwise_and(z, 0xF), hi = at::bitwise_and(at::bitwise_right_shift(z, 4), 0xF);
        zp = at::stack({lo, hi}, -1).reshape({N, -1}).narrow(1, 0, n_blocks).to(at::kFloat).unsqueeze(-1);
      } else {
        zp = zero_points.reshape({N, n_blocks, 1}).to(at::kFloat);
      }
    } else {
      zp = zero_points.reshape({N, n_blocks, 1}).to(at::kFloat);
    }
  } else {
    zp = at::full({1}, static_cast<double>(1 << (bits - 1)), q.options());
  }
  at::Tensor w = ((q - zp) * s).reshape({N, n_blocks * block_size}).narrow(1, 0, K);
  return w.to(out_type);
}

at::Tensor ActivationByName(const at::Tensor& x, const std::string& name) {
  if (name == "relu") return at::relu(x);
  if (name == "gelu") return at::gelu(x);
  if (name == "silu") return at::silu(x);
  if (name == "identity") return x;
  ORTB_THROW(INVALID_ARGUMENT, "unknown activation_type ", name);
}

// Mixture of experts on one device.  x [T,H], logits [T,E]; fc1 [E, F*I, H], fc2 [E, H, I], optional fc3 [E, I, H].
at::Tensor MoeForward(const at::Tensor& x_in, const at::Tensor& logits, const at::Tensor& fc1, const at::Tensor& fc1_b,
                      const at::Tensor& fc2, const at::Tensor& fc2_b, const at::Tensor& fc3, const at::Tensor& fc3_b,
                      const MoeAttrs& a, int64_t expert_begin, int64_t expert_end) {
  const int64_t T = x_in.size(0), E = logits.size(1);
  at::Tensor xf = x_in.to(at::kFloat);
  at::Tensor probs = at::softmax(logits.to(at::kFloat), -1);
  at::Tensor topv, topi;
  std::tie(topv, topi) = at::topk(probs, a.k, -1, true, true);
  if (a.normalize) topv = topv / topv.sum(-1, true);
  at::Tensor out = at::zeros({T, fc2.size(1)}, xf.options());
  if (expert_end < 0) expert_end = E;
  for (int64_t e = expert_begin; e < expert_end; ++e) {
    const int64_t le = e - expert_begin;  // index into the (possibly local) weight stacks
    at::Tensor hit = topi.eq(e);                      // [T,k]
    at::Tensor rows = at::nonzero(hit.any(-1)).reshape({-1});
    if (rows.numel() == 0) continue;
    at::Tensor w = (topv * hit.to(at::kFloat)).sum(-1).index_select(0, rows);  // [R]
    at::Tensor xe = xf.index_select(0, rows);                                    // [R,H]
    at::Tensor h = at::matmul(xe, fc1[le].to(at::kFloat).t());
    if (fc1_b.defined()) h = h + fc1_b[le].to(at::kFloat);
    at::Tensor act;
    if (a.activation == "swiglu") {
      at::Tensor g, l;
      if (a.swiglu_fusion == 1) {
        g = h.slice(-1, 0, c10::nullopt, 2);
        l = h.slice(-1, 1, c10::nullopt, 2);
      } else if (a.swiglu_fusion == 2) {
        const int64_t I = h.size(-1) / 2;
        g = h.narrow(-1, 0, I);
        l = h.narrow(-1, I, I);
      } else {
        ORTB_ENFORCE_ARG(fc3.defined(), "MoE swiglu with swiglu_fusion=0 needs fc3 weights");
        g = h;
        l = at::matmul(xe, fc3[le].to(at::kFloat).t());
        if (fc3_b.defined()) l = l + fc3_b[le].to(at::kFloat);
      }
      if (a.has_limit) {
        g = at::clamp_max(g, a.swiglu_limit);
        l = at::clamp(l, -a.swiglu_limit, a.swiglu_limit);
      }
      act = g * at::sigmoid(g * a.alpha) * (l + a.beta);
    } else {
      act = ActivationByName(h, a.activation);
      if (fc3.defined()) {
        at::Tensor l = at::matmul(xe, fc3[le].to(at::kFloat).t());
        if (fc3_b.defined()) l = l + fc3_b[le].to(at::kFloat);
        act = act * l;
      }
    }
    at::Tensor y = at::matmul(act, fc2[le].to(at::kFloat).t());
    if (fc2_b.defined()) y = y + fc2_b[le].to(at::kFloat);
    out.index_add_(0, rows, y * w.unsqueeze(-1));
  }
  return out.to(x_in.scalar_type());
}

MoeAttrs ParseMoeAttrs(const Node& n) {
  MoeAttrs a;
  a.k = n.attr_i("k", 1);
  a.activation = n.attr_s("activation_type", "relu");
  a.normalize = n.attr_i("normalize_routing_weights", 0) != 0;
  a.swiglu_fusion = n.attr_i("swiglu_fusion", 0);
  a.has_limit = n.has_attr("swiglu_limit");
  a.swiglu_limit = n.attr_f("swiglu_limit", 0.f);
  a.alpha = n.attr_f("activation_alpha", 1.f);
  a.beta = n.attr_f("activation_beta", 0.f);
  ORTB_ENFORCE_ARG(n.attr_i("use_sparse_mixer", 0) == 0, "use_sparse_mixer is not supported");
  return a;
}

// GroupQueryAttention reference (fp32 math).  See the op contract in
// docs/ContribOperators.md (GroupQueryAttention) of the reference.
GqaResult GqaForward(const GqaInputs& in, const GqaAttrs& a) {
  const int64_t B = in.query.size(0), S = in.query.size(1);
  const int64_t N = a.num_heads, Nk = a.kv_num_heads;
  at::Tensor q, k, v;
  int64_t H;
  if (!in.key.defined()) {
    H = in.query.size(2) / (N + 2 * Nk);
    q = in.query.narrow(2, 0, N * H);
    k = in.query.narrow(2, N * H, Nk * H);
    v = in.query.narrow(2, (N + Nk) * H, Nk * H);
  } else {
    H = in.query.size(2) / N;
    q = in.query;
    k = in.key;
    v = in.value;
  }
  q = q.reshape({B, S, N, H});
  k = k.reshape({B, S, Nk, H});
  v = v.reshape({B, S, Nk, H});
  at::Tensor seqlens = in.seqlens_k.to(at::kCPU, at::kLong).reshape({-1});
  const int64_t total = in.total_sequence_length;
  const bool first_prompt = (S == total);
  std::vector<int64_t> past_len(B), tot_len(B);
  for (int64_t b = 0; b < B; ++b) {
    tot_len[b] = seqlens[b].item<int64_t>() + 1;
    past_len[b] = first_prompt ? 0 : tot_len[b] - S;
    ORTB_ENFORCE_ARG(past_len[b] >= 0, "GroupQueryAttention: seqlens_k is smaller than the sequence length");
  }
  // positions of the new tokens
  at::Tensor pos;
  if (in.position_ids.defined()) {
    pos = in.position_ids.to(at::kLong).reshape({B, S});
  } else {
    pos = at::arange(S, at::TensorOptions().dtype(at::kLong)).unsqueeze(0).repeat({B, 1});
    for (int64_t b = 0; b < B; ++b) pos[b] += past_len[b];
    pos = pos.to(q.device());
  }
  if (a.do_rotary) {
    ORTB_ENFORCE_ARG(in.cos_cache.defined() && in.sin_cache.defined(), "do_rotary needs cos_cache and sin_cache");
    q = RotaryBSNH(q, pos, in.cos_cache, in.sin_cache, a.rotary_interleaved, 0, 1.0f);
    k = RotaryBSNH(k, pos, in.cos_cache, in.sin_cache, a.rotary_interleaved, 0, 1.0f);
  }
  // present buffers
  at::Tensor pk, pv;
  int64_t cap = total;
  if (in.past_key.defined()) cap = std::max<int64_t>(cap, in.past_key.size(2));
  if (in.past_key.defined() && in.share_buffer) {
    pk = in.past_key;
    pv = in.past_value;
  } else {
    pk = at::zeros({B, Nk, cap, H}, k.options());
    pv = at::zeros({B, Nk, cap, H}, v.options());
    if (in.past_key.defined() && !first_prompt) {
      const int64_t ps = in.past_key.size(2);
      pk.narrow(2, 0, ps).copy_(in.past_key);
      pv.narrow(2, 0, ps).copy_(in.past_value);
    }
  }
  const double scale = a.scale != 0.f ? a.scale : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor out = at::zeros({B, S, N, H}, q.options());
  const int64_t group = N / Nk;
  for (int64_t b = 0; b < B; ++b) {
    const int64_t pl = past_len[b];
    const int64_t n_new = first_prompt ? std::min<int64_t>(S, tot_len[b]) : S;
    pk[b].narrow(1, pl, n_new).copy_(k[b].narrow(0, 0, n_new).transpose(0, 1));
    pv[b].narrow(1, pl, n_new).copy_(v[b].narrow(0, 0, n_new).transpose(0, 1));
    const int64_t T = pl + n_new;
    at::Tensor kb = pk[b].narrow(1, 0, T).to(at::kFloat).repeat_interleave(group, 0);  // N,T,H
    at::Tensor vb = pv[b].narrow(1, 0, T).to(at::kFloat).repeat_interleave(group, 0);
    at::Tensor qb = q[b].transpose(0, 1).to(at::kFloat);                                // N,S,H
    at::Tensor s = at::matmul(qb, kb.transpose(1, 2)) * scale;                           // N,S,T
    if (a.softcap > 0.f) s = at::tanh(s / a.softcap) * a.softcap;
    if (in.attention_bias.defined()) {
      at::Tensor bias = in.attention_bias;
      at::Tensor bb = bias.size(0) == 1 ? bias[0] : bias[b];  // [N or 1, S, T_total]
      s = s + bb.narrow(-1, 0, T).to(at::kFloat);
    }
    // causal + local window mask on absolute positions
    at::Tensor qpos = (at::arange(S, s.options().dtype(at::kLong)) + pl).unsqueeze(1);  // S,1
    at::Tensor kpos = at::arange(T, s.options().dtype(at::kLong)).unsqueeze(0);         // 1,T
    at::Tensor allowed = kpos.le(qpos);
    if (a.local_window_size > 0) allowed = allowed.logical_and(kpos.gt(qpos - a.local_window_size));
    s = s.masked_fill(allowed.logical_not().unsqueeze(0), -std::numeric_limits<float>::infinity());
    at::Tensor p;
    if (in.head_sink.defined() || a.smooth_softmax) {
      at::Tensor sink = in.head_sink.defined() ? in.head_sink.to(at::kFloat).reshape({N, 1, 1}).expand({N, S, 1})
                                               : at::zeros({N, S, 1}, s.options());
      p = at::softmax(at::cat({s, sink}, -1), -1).narrow(-1, 0, T);
    } else {
      p = at::softmax(s, -1);
    }
    at::Tensor ob = at::matmul(p, vb);  // N,S,H
    out[b].copy_(ob.transpose(0, 1).to(out.scalar_type()));
  }
  GqaResult r;
  r.output = out.reshape({B, S, N * H});
  r.present_key = pk;
  r.present_value = pv;
  return r;
}

}  // namespace contrib

namespace {

using Ctx = OpKernelContext;
using namespace contrib;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

void SkipLayerNormImpl(Ctx& ctx, bool simplified) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& skip = ctx.RequiredInput(1);
  const at::Tensor& gamma = ctx.RequiredInput(2);
  const int beta_idx = simplified ? -1 : 3, bias_idx = simplified ? 3 : 4;
  const double eps = ctx.node().attr_f("epsilon", 1e-5f);
  at::Tensor sum = x.to(at::kFloat) + skip.to(at::kFloat);
  if (ctx.HasInput(bias_idx)) sum = sum + ctx.Input(bias_idx).to(at::kFloat);
  // the residual stream is stored in the activation dtype and the statistics use the stored value's fp32 image
  at::Tensor sum_t = sum.to(x.scalar_type());
  at::Tensor y, mean, inv;
  if (simplified) {
    inv = at::rsqrt(at::mean(sum * sum, {-1}, true) + eps);
    y = sum * inv * gamma.to(at::kFloat);
  } else {
    mean = at::mean(sum, {-1}, true);
    at::Tensor c = sum - mean;
    inv = at::rsqrt(at::mean(c * c, {-1}, true) + eps);
    y = c * inv * gamma.to(at::kFloat);
    if (beta_idx >= 0 && ctx.HasInput(beta_idx)) y = y + ctx.Input(beta_idx).to(at::kFloat);
  }
  ctx.SetOutput(0, y.to(x.scalar_type()));
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1) && mean.defined()) ctx.SetOutput(1, mean);
  if (ctx.OutputCount() > 2 && ctx.OutputNeeded(2)) ctx.SetOutput(2, inv);
  if (ctx.OutputCount() > 3 && ctx.OutputNeeded(3)) ctx.SetOutput(3, sum_t);
}

void EmbedLayerNormImpl(Ctx& ctx) {
  at::Tensor ids = ctx.RequiredInput(0).to(at::kLong);
  const at::Tensor& word = ctx.RequiredInput(2);
  const at::Tensor& pos_emb = ctx.RequiredInput(3);
  const int64_t B = ids.size(0), S = ids.size(1);
  at::Tensor emb = word.index({ids.to(word.device())});
  at::Tensor pos_ids;
  if (ctx.HasInput(8)) pos_ids = ctx.Input(8).to(at::kLong).to(word.device());
  else pos_ids = at::arange(S, at::TensorOptions().dtype(at::kLong).device(word.device())).unsqueeze(0).expand({B, S});
  emb = emb + pos_emb.index({pos_ids});
  if (ctx.HasInput(1) && ctx.HasInput(4)) emb = emb + ctx.Input(4).index({ctx.Input(1).to(at::kLong).to(word.device())});
  const double eps = ctx.node().attr_f("epsilon", 1e-12f);
  at::Tensor ef = emb.to(at::kFloat);
  at::Tensor mean = at::mean(ef, {-1}, true);
  at::Tensor c = ef - mean;
  at::Tensor y = c * at::rsqrt(at::mean(c * c, {-1}, true) + eps) * ctx.RequiredInput(5).to(at::kFloat) +
                 ctx.RequiredInput(6).to(at::kFloat);
  ctx.SetOutput(0, y.to(word.scalar_type()));
  if (ctx.OutputCount() > 1) {
    if (ctx.HasInput(7)) ctx.SetOutput(1, ctx.Input(7).to(at::kInt).sum(-1).to(at::kInt));
    else ctx.SetOutput(1, at::zeros({B}, at::TensorOptions().dtype(at::kInt).device(word.device())));
  }
  if (ctx.OutputCount() > 2 && ctx.OutputNeeded(2)) ctx.SetOutput(2, emb);
}

// additive mask [B,1,1 or S,T] from the BERT Attention mask_index forms
at::Tensor BertMask(const at::Tensor& mask_index, int64_t B, int64_t S, int64_t T, float filter, at::Device dev) {
  at::Tensor m = mask_index.to(dev);
  at::Tensor valid;
  if (m.dim() == 1 && m.size(0) == B) {
    valid = at::arange(T, at::TensorOptions().dtype(at::kLong).device(dev)).unsqueeze(0).lt(m.to(at::kLong).unsqueeze(1));  // B,T
    valid = valid.reshape({B, 1, 1, T});
  } else if (m.dim() == 1 && m.size(0) == 2 * B) {
    at::Tensor ar = at::arange(T, at::TensorOptions().dtype(at::kLong).device(dev)).unsqueeze(0);
    at::Tensor end = m.narrow(0, 0, B).to(at::kLong).unsqueeze(1), start = m.narrow(0, B, B).to(at::kLong).unsqueeze(1);
    valid = ar.ge(start).logical_and(ar.lt(end)).reshape({B, 1, 1, T});
  } else if (m.dim() == 2) {
    valid = m.ne(0).reshape({B, 1, 1, T});
  } else if (m.dim() == 3) {
    valid = m.ne(0).reshape({B, 1, S, T});
  } else if (m.dim() == 4) {
    valid = m.ne(0);
  } else {
    ORTB_THROW(INVALID_ARGUMENT, "Attention: unsupported mask_index shape");
  }
  return at::where(valid, at::zeros({1}, at::TensorOptions().dtype(at::kFloat).device(dev)),
                   at::full({1}, filter, at::TensorOptions().dtype(at::kFloat).device(dev)));
}

void BertAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& w = ctx.RequiredInput(1);
  const int64_t B = x.size(0), S = x.size(1);
  const int64_t N = n.attr_i("num_heads", 1);
  std::vector<int64_t> sizes = n.attr_ints("qkv_hidden_sizes");
  at::Tensor qkv = at::matmul(x, w);
  if (ctx.HasInput(2)) qkv = qkv + ctx.Input(2);
  int64_t qs, ks, vs;
  if (sizes.size() == 3) { qs = sizes[0]; ks = sizes[1]; vs = sizes[2]; }
  else { qs = ks = vs = qkv.size(-1) / 3; }
  at::Tensor q = qkv.narrow(-1, 0, qs).reshape({B, S, N, qs / N}).transpose(1, 2);
  at::Tensor k = qkv.narrow(-1, qs, ks).reshape({B, S, N, ks / N}).transpose(1, 2);
  at::Tensor v = qkv.narrow(-1, qs + ks, vs).reshape({B, S, N, vs / N}).transpose(1, 2);
  int64_t past_len = 0;
  if (ctx.HasInput(4)) {
    const at::Tensor& past = ctx.Input(4);  // [2,B,N,P,H]
    past_len = past.size(3);
    if (ctx.HasInput(6)) past_len = ctx.Input(6).cpu().item<int64_t>();
    k = at::cat({past[0].narrow(2, 0, past_len), k}, 2);
    v = at::cat({past[1].narrow(2, 0, past_len), v}, 2);
  }
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, at::stack({k, v}, 0).contiguous());
  const int64_t T = k.size(2), H = q.size(3);
  const double scale = n.has_attr("scale") && n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor s = at::matmul(q.to(at::kFloat), k.to(at::kFloat).transpose(-1, -2)) * scale;
  if (ctx.HasInput(5)) s = s + ctx.Input(5).to(at::kFloat);
  const float filter = n.attr_f("mask_filter_value", -10000.f);
  if (ctx.HasInput(3)) s = s + BertMask(ctx.Input(3), B, S, T, filter, s.device());
  if (n.attr_i("unidirectional", 0)) {
    at::Tensor causal = at::ones({S, T}, s.options().dtype(at::kBool)).tril(T - S);
    s = s.masked_fill(causal.logical_not(), filter);
  }
  at::Tensor y = at::matmul(at::softmax(s, -1), v.to(at::kFloat)).to(x.scalar_type());
  ctx.SetOutput(0, y.transpose(1, 2).reshape({B, S, vs}).contiguous());
}

void MultiHeadAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const int64_t N = n.attr_i("num_heads", 1);
  at::Tensor q = ctx.RequiredInput(0);
  const int64_t B = q.size(0), S = q.size(1);
  at::Tensor k, v;
  if (q.dim() == 5) {
    // packed QKV [B,S,N,3,H]
    k = q.select(3, 1);
    v = q.select(3, 2);
    q = q.select(3, 0);
    q = q.transpose(1, 2);
    k = k.transpose(1, 2);
    v = v.transpose(1, 2);
  } else {
    ORTB_ENFORCE_ARG(ctx.HasInput(1), "MultiHeadAttention needs key");
    k = ctx.Input(1);
    if (k.dim() == 5) {
      // packed KV [B,L,N,2,H]
      v = k.select(3, 1).transpose(1, 2);
      k = k.select(3, 0).transpose(1, 2);
    } else if (k.dim() == 4) {
      v = ctx.RequiredInput(2);  // already BNSH
    } else {
      v = ctx.RequiredInput(2);
      k = k.reshape({B, k.size(1), N, -1}).transpose(1, 2);
      v = v.reshape({B, v.size(1), N, -1}).transpose(1, 2);
    }
    q = q.reshape({B, S, N, -1}).transpose(1, 2);
  }
  if (ctx.HasInput(3)) {
    const at::Tensor& bias = ctx.Input(3);
    const int64_t qh = q.size(1) * q.size(3), kh = k.size(1) * k.size(3), vh = v.size(1) * v.size(3);
    q = q + bias.narrow(0, 0, qh).reshape({1, N, 1, -1});
    k = k + bias.narrow(0, qh, kh).reshape({1, N, 1, -1});
    v = v + bias.narrow(0, qh + kh, vh).reshape({1, N, 1, -1});
  }
  if (ctx.HasInput(6)) k = at::cat({ctx.Input(6), k}, 2);
  if (ctx.HasInput(7)) v = at::cat({ctx.Input(7), v}, 2);
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, k.contiguous());
  if (ctx.OutputCount() > 2 && ctx.OutputNeeded(2)) ctx.SetOutput(2, v.contiguous());
  const int64_t T = k.size(2), H = q.size(3);
  const double scale = n.has_attr("scale") && n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor s = at::matmul(q.to(at::kFloat), k.to(at::kFloat).transpose(-1, -2)) * scale;
  if (ctx.HasInput(5)) s = s + ctx.Input(5).to(at::kFloat);
  const float filter = n.attr_f("mask_filter_value", -10000.f);
  if (ctx.HasInput(4)) s = s + BertMask(ctx.Input(4), B, S, T, filter, s.device());
  if (n.attr_i("unidirectional", 0)) {
    at::Tensor causal = at::ones({S, T}, s.options().dtype(at::kBool)).tril(T - S);
    s = s.masked_fill(causal.logical_not(), filter);
  }
  at::Tensor y = at::matmul(at::softmax(s, -1), v.to(at::kFloat)).to(ctx.RequiredInput(0).scalar_type());
  ctx.SetOutput(0, y.transpose(1, 2).reshape({B, S, -1}).contiguous());
}

void ContribRotaryImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor pos = ctx.RequiredInput(1).to(at::kLong);
  const at::Tensor& cos = ctx.RequiredInput(2);
  const at::Tensor& sin = ctx.RequiredInput(3);
  const bool interleaved = n.attr_i("interleaved", 0) != 0;
  int64_t N = n.attr_i("num_heads", 0);
  const int64_t rot = n.attr_i("rotary_embedding_dim", 0);
  at::Tensor x = x_in;
  const bool bnsh = x.dim() == 4;
  int64_t B = x.size(0), S;
  if (bnsh) {
    S = x.size(2);
    x = x.transpose(1, 2);
  } else {
    S = x.size(1);
    const int64_t H = rot > 0 && N > 0 ? x.size(2) / N : cos.size(1) * 2;
    if (N == 0) N = x.size(2) / H;
    x = x.reshape({B, S, N, x.size(2) / N});
  }
  if (pos.numel() == 1) {
    pos = at::arange(S, pos.options()).unsqueeze(0).expand({B, S}) + pos.reshape({1, 1}).to(at::kCPU);
  }
  at::Tensor y = RotaryBSNH(x, pos.reshape({B, S}), cos, sin, interleaved, rot, n.attr_f("scale", 1.f));
  if (bnsh) ctx.SetOutput(0, y.transpose(1, 2).contiguous());
  else ctx.SetOutput(0, y.reshape(x_in.sizes()));
}

void GqaImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  GqaInputs in;
  in.query = ctx.RequiredInput(0);
  if (ctx.HasInput(1)) in.key = ctx.Input(1);
  if (ctx.HasInput(2)) in.value = ctx.Input(2);
  if (ctx.HasInput(3)) in.past_key = ctx.Input(3);
  if (ctx.HasInput(4)) in.past_value = ctx.Input(4);
  in.seqlens_k = ctx.RequiredInput(5);
  in.total_sequence_length = ctx.RequiredInput(6).cpu().to(at::kLong).reshape({-1})[0].item<int64_t>();
  if (ctx.HasInput(7)) in.cos_cache = ctx.Input(7);
  if (ctx.HasInput(8)) in.sin_cache = ctx.Input(8);
  if (ctx.HasInput(9)) in.position_ids = ctx.Input(9);
  if (ctx.HasInput(10)) in.attention_bias = ctx.Input(10);
  if (ctx.HasInput(11)) in.head_sink = ctx.Input(11);
  // Per-head RMS norm of Q and K before the rotary embedding (q_norm_weight / k_norm_weight, Qwen3-style models):
  // a packed QKV input is split so that the normalised parts travel as separate query / key / value.
  if (ctx.HasInput(14) || ctx.HasInput(15)) {
    ORTB_ENFORCE_ARG(ctx.HasInput(14) && ctx.HasInput(15), "q_norm_weight and k_norm_weight must be given together");
    const int64_t N = n.attr_i("num_heads", 0), Nk = n.attr_i("kv_num_heads", 0);
    const float eps = n.attr_f("qk_norm_epsilon", 1e-6f);
    const int64_t B = in.query.size(0), S = in.query.size(1);
    if (!in.key.defined()) {
      const int64_t H = in.query.size(2) / (N + 2 * Nk);
      at::Tensor packed = in.query;
      in.query = packed.narrow(2, 0, N * H);
      in.key = packed.narrow(2, N * H, Nk * H);
      in.value = packed.narrow(2, (N + Nk) * H, Nk * H);
    }
    auto head_norm = [&](const at::Tensor& x, int64_t heads, const at::Tensor& w) {
      at::Tensor xf = x.reshape({B, S, heads, -1}).to(at::kFloat);
      at::Tensor y = xf * at::rsqrt(xf.pow(2).mean(-1, true) + eps) * w.to(at::kFloat);
      return y.reshape({B, S, -1}).to(x.scalar_type());
    };
    in.query = head_norm(in.query, N, ctx.Input(14));
    in.key = head_norm(in.key, Nk, ctx.Input(15));
  }
  // Quantised KV cache (k_scale / v_scale; int8 or float8 e4m3 caches, per tensor or per channel): the past is
  // expanded to the compute type, attention runs as usual, and the present is quantised back - into the past
  // buffer itself when it has room, as the float path does.
  const bool quant_cache = ctx.HasInput(12) || ctx.HasInput(13);
  at::Tensor q_past_k, q_past_v, k_scale, v_scale;
  if (quant_cache) {
    ORTB_ENFORCE_ARG(ctx.HasInput(12) && ctx.HasInput(13), "k_scale and v_scale must be given together");
    ORTB_ENFORCE_ARG(n.attr_i("kv_cache_bit_width", 8) == 8, "4-bit KV caches are not supported by this kernel");
    k_scale = ctx.Input(12).to(at::kFloat);
    v_scale = ctx.Input(13).to(at::kFloat);
    q_past_k = in.past_key;
    q_past_v = in.past_value;
    if (q_past_k.defined()) {
      const at::ScalarType ct = q_past_k.scalar_type();
      ORTB_ENFORCE_ARG(ct == at::kChar || ct == at::kFloat8_e4m3fn, "quantised KV cache must be int8 or float8e4m3fn");
      in.past_key = (q_past_k.to(at::kFloat) * k_scale).to(in.query.scalar_type());
      in.past_value = (q_past_v.to(at::kFloat) * v_scale).to(in.query.scalar_type());
    }
  }
  // A past buffer with room for the new tokens is updated in place and returned as present
  // (the reference's past_present_share_buffer mode); otherwise present is a new tensor.
  in.share_buffer = in.past_key.defined() && in.past_key.size(2) >= in.total_sequence_length;
  GqaAttrs a;
  a.num_heads = n.attr_i("num_heads", 0);
  a.kv_num_heads = n.attr_i("kv_num_heads", 0);
  a.do_rotary = n.attr_i("do_rotary", 0) != 0;
  a.rotary_interleaved = n.attr_i("rotary_interleaved", 0) != 0;
  a.local_window_size = n.attr_i("local_window_size", -1);
  a.scale = n.attr_f("scale", 0.f);
  a.softcap = n.attr_f("softcap", 0.f);
  a.smooth_softmax = n.attr_i("smooth_softmax", 0) != 0;
  GqaResult r = GqaForward(in, a);
  ctx.SetOutput(0, r.output);
  if (quant_cache) {
    const at::ScalarType ct = q_past_k.defined() ? q_past_k.scalar_type()
                                                 : (n.attr_s("k_quant_type", "PER_TENSOR") == "NONE" ? in.query.scalar_type() : at::kChar);
    auto quantise = [&](const at::Tensor& x, const at::Tensor& scale, const at::Tensor& into) {
      at::Tensor y = x.to(at::kFloat) / scale;
      at::Tensor q = ct == at::kChar ? at::clamp(at::round(y), -128, 127).to(at::kChar) : at::clamp(y, -448.f, 448.f).to(ct);
      if (into.defined() && into.sizes() == q.sizes()) {
        into.copy_(q);
        return into;
      }
      return q;
    };
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, quantise(r.present_key, k_scale, q_past_k));
    if (ctx.OutputCount() > 2) ctx.SetOutput(2, quantise(r.present_value, v_scale, q_past_v));
    return;
  }
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, r.present_key);
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, r.present_value);
}

void MatMulNBitsImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& a = ctx.RequiredInput(0);
  const int64_t K = n.attr_i("K", 0), N = n.attr_i("N", 0), bits = n.attr_i("bits", 4), bs = n.attr_i("block_size", 32);
  at::Tensor zp = ctx.HasInput(3) ? ctx.Input(3) : at::Tensor();
  ORTB_ENFORCE_ARG(!ctx.HasInput(4), "MatMulNBits g_idx is not supported");
  at::Tensor w = DequantizeNBits(ctx.RequiredInput(1), ctx.RequiredInput(2), zp, N, K, bits, bs, at::kFloat);
  at::Tensor y = at::matmul(a.to(at::kFloat), w.t());
  if (ctx.HasInput(5)) y = y + ctx.Input(5).to(at::kFloat);
  // extensions written by the GPU lowering passes: sum over the ranks first, then a residual (input 6)
  if (n.attr_i("all_reduce", 0)) y = AllReduceSum(ctx.session(), y);
  if (ctx.HasInput(6)) y = y + ctx.Input(6).to(at::kFloat);
  ctx.SetOutput(0, y.to(a.scalar_type()));
}

void MoeImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  MoeAttrs a = ParseMoeAttrs(ctx.node());
  at::Tensor x2 = x.reshape({-1, x.size(-1)});
  auto opt = [&](int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); };
  at::Tensor y = MoeForward(x2, ctx.RequiredInput(1).reshape({x2.size(0), -1}), ctx.RequiredInput(2), opt(3),
                            ctx.RequiredInput(4), opt(5), opt(6), opt(7), a, 0, -1);
  ctx.SetOutput(0, y.reshape(x.sizes()));
}

}  // namespace

namespace contrib {
at::Tensor AttentionMaskBias(const at::Tensor& mask_index, int64_t B, int64_t S, int64_t T, float filter, at::Device dev) {
  return BertMask(mask_index, B, S, T, filter, dev);
}

// QMoE expert weights [E, rows, K * bits / 8] with symmetric scales per output row ([E, rows]) or per block along K
// ([E, rows, K / block]) -> float [E, rows, K]
at::Tensor DequantizeQMoeWeights(const at::Tensor& w, const at::Tensor& scales, int64_t bits, int64_t block) {
  if (!w.defined()) return at::Tensor();
  const int64_t E = w.size(0), rows = w.size(1);
  const int64_t K = bits == 4 ? w.size(2) * 2 : w.size(2);
  at::Tensor q;
  if (bits == 4) {
    at::Tensor b = w.to(at::kInt);
    q = at::stack({at::bitwise_and(b, 0xF), at::bitwise_and(at::bitwise_right_shift(b, 4), 0xF)}, -1).reshape({E, rows, K}).to(at::kFloat) - 8.0;
  } else {
    q = w.to(at::kFloat) - 128.0;
  }
  at::Tensor s = scales.to(at::kFloat);
  if (s.dim() == 2) s = s.unsqueeze(-1);                       // per output row
  else if (block > 0) s = s.repeat_interleave(block, 2).narrow(2, 0, K);  // per block along K
  return q * s;
}
}  // namespace contrib

namespace {

// QMoE: block- or column-quantised expert weights; dequantise, then run the dense MoE.
void QMoeImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  MoeAttrs a = ParseMoeAttrs(n);
  const int64_t bits = n.attr_i("expert_weight_bits", 4);
  const int64_t block = n.attr_i("block_size", 0);
  at::Tensor x2 = x.reshape({-1, x.size(-1)});
  auto opt = [&](int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); };
  // inputs: 0 input, 1 router_probs, 2 fc1_w, 3 fc1_scales, 4 fc1_bias, 5 fc2_w, 6 fc2_scales, 7 fc2_bias, 8 fc3_w, 9 fc3_scales, 10 fc3_bias
  auto dequant = [&](const at::Tensor& w, const at::Tensor& scales) { return contrib::DequantizeQMoeWeights(w, scales, bits, block); };
  at::Tensor fc1 = dequant(ctx.RequiredInput(2), ctx.RequiredInput(3));
  at::Tensor fc2 = dequant(ctx.RequiredInput(5), ctx.RequiredInput(6));
  at::Tensor fc3 = dequant(opt(8), opt(9));
  at::Tensor y = MoeForward(x2, ctx.RequiredInput(1).reshape({x2.size(0), -1}), fc1, opt(4), fc2, opt(7), fc3, opt(10), a, 0, -1);
  ctx.SetOutput(0, y.reshape(x.sizes()));
}

void GemmFloat8Impl(Ctx& ctx) {
  const Node& n = ctx.node();
  at::Tensor a = ctx.RequiredInput(0).to(at::kFloat), b = ctx.RequiredInput(1).to(at::kFloat);
  if (n.attr_i("transA", 0)) a = a.t();
  if (n.attr_i("transB", 0)) b = b.t();
  // inputs: A, B, C, scaleA, scaleB, scaleY
  if (ctx.HasInput(3)) a = a * ctx.Input(3).to(at::kFloat);
  if (ctx.HasInput(4)) b = b * ctx.Input(4).to(at::kFloat);
  at::Tensor y = at::matmul(a, b) * n.attr_f("alpha", 1.f);
  if (ctx.HasInput(2)) y = y + ctx.Input(2).to(at::kFloat) * n.attr_f("beta", 0.f);
  const std::string act = n.attr_s("activation", "NONE");
  if (act == "RELU") y = at::relu(y);
  else if (act == "GELU") y = at::gelu(y);
  if (ctx.HasInput(5)) y = y / ctx.Input(5).to(at::kFloat);
  const int64_t dt = n.attr_i("dtype", 1);
  ctx.SetOutput(0, y.to(ToTorchType(static_cast<int32_t>(dt))));
}

// PagedAttention reference: packed tokens, block-table addressed KV cache updated in place.
void PagedAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const int64_t N = n.attr_i("num_heads", 0), Nk = n.attr_i("kv_num_heads", 0);
  at::Tensor q = ctx.RequiredInput(0);
  at::Tensor k, v;
  at::Tensor kc = ctx.RequiredInput(3), vc = ctx.RequiredInput(4);  // [num_blocks, block_size, Nk, H]
  const int64_t H = kc.size(3), block_size = kc.size(1);
  const int64_t T = q.size(0);
  if (ctx.HasInput(1)) {
    k = ctx.Input(1);
    v = ctx.RequiredInput(2);
  } else {
    k = q.narrow(1, N * H, Nk * H);
    v = q.narrow(1, (N + Nk) * H, Nk * H);
    q = q.narrow(1, 0, N * H);
  }
  q = q.reshape({T, N, H});
  k = k.reshape({T, Nk, H});
  v = v.reshape({T, Nk, H});
  std::vector<int64_t> cum = ToVec(ctx.RequiredInput(5));   // [B+1]
  std::vector<int64_t> past = ToVec(ctx.RequiredInput(6));  // [B]
  at::Tensor block_table = ctx.RequiredInput(7).to(at::kCPU, at::kLong);
  const int64_t B = static_cast<int64_t>(past.size());
  const bool do_rotary = n.attr_i("do_rotary", 0) != 0;
  const double scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 0.f) : 1.0 / std::sqrt(static_cast<double>(H));
  const int64_t window = n.attr_i("local_window_size", -1);
  const float softcap = n.attr_f("softcap", 0.f);
  at::Tensor out = at::zeros({T, N, H}, q.options());
  const int64_t group = N / Nk;
  for (int64_t b = 0; b < B; ++b) {
    const int64_t t0 = cum[b], S = cum[b + 1] - cum[b], pl = past[b];
    if (S == 0) continue;
    at::Tensor qb = q.narrow(0, t0, S), kb = k.narrow(0, t0, S), vb = v.narrow(0, t0, S);
    if (do_rotary) {
      at::Tensor pos = (at::arange(S, at::TensorOptions().dtype(at::kLong)) + pl).unsqueeze(0);
      qb = RotaryBSNH(qb.unsqueeze(0), pos, ctx.RequiredInput(8), ctx.RequiredInput(9), n.attr_i("rotary_interleaved", 0) != 0, 0, 1.f)[0];
      kb = RotaryBSNH(kb.unsqueeze(0), pos, ctx.RequiredInput(8), ctx.RequiredInput(9), n.attr_i("rotary_interleaved", 0) != 0, 0, 1.f)[0];
    }
    // write the new tokens into their blocks
    for (int64_t s = 0; s < S; ++s) {
      const int64_t p = pl + s;
      const int64_t blk = block_table[b][p / block_size].item<int64_t>();
      kc[blk][p % block_size].copy_(kb[s]);
      vc[blk][p % block_size].copy_(vb[s]);
    }
    const int64_t L = pl + S;
    const int64_t nblk = (L + block_size - 1) / block_size;
    at::Tensor blocks = block_table[b].narrow(0, 0, nblk).to(kc.device());
    at::Tensor kk = kc.index_select(0, blocks).reshape({nblk * block_size, Nk, H}).narrow(0, 0, L);
    at::Tensor vv = vc.index_select(0, blocks).reshape({nblk * block_size, Nk, H}).narrow(0, 0, L);
    at::Tensor kf = kk.to(at::kFloat).permute({1, 0, 2}).repeat_interleave(group, 0);  // N,L,H
    at::Tensor vf = vv.to(at::kFloat).permute({1, 0, 2}).repeat_interleave(group, 0);
    at::Tensor qf = qb.to(at::kFloat).permute({1, 0, 2});                               // N,S,H
    at::Tensor s = at::matmul(qf, kf.transpose(1, 2)) * scale;
    if (softcap > 0.f) s = at::tanh(s / softcap) * softcap;
    at::Tensor qpos = (at::arange(S, s.options().dtype(at::kLong)) + pl).unsqueeze(1);
    at::Tensor kpos = at::arange(L, s.options().dtype(at::kLong)).unsqueeze(0);
    at::Tensor allowed = kpos.le(qpos);
    if (window > 0) allowed = allowed.logical_and(kpos.gt(qpos - window));
    s = s.masked_fill(allowed.logical_not().unsqueeze(0), -std::numeric_limits<float>::infinity());
    out.narrow(0, t0, S).copy_(at::matmul(at::softmax(s, -1), vf).permute({1, 0, 2}).to(out.scalar_type()));
  }
  ctx.SetOutput(0, out.reshape({T, N * H}));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, kc);
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, vc);
}

}  // namespace

void RegisterContribKernels(KernelRegistry& r) {
  r.RegisterFn(MS, "SkipLayerNormalization", 1, kMax, [](Ctx& ctx) { SkipLayerNormImpl(ctx, false); });
  r.RegisterFn(MS, "SkipSimplifiedLayerNormalization", 1, kMax, [](Ctx& ctx) { SkipLayerNormImpl(ctx, true); });
  r.RegisterFn(MS, "EmbedLayerNormalization", 1, kMax, EmbedLayerNormImpl);
  r.RegisterFn(MS, "FastGelu", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0);
    if (ctx.HasInput(1)) x = x + ctx.Input(1);
    ctx.SetOutput(0, FastGeluRef(x));
  });
  r.RegisterFn(MS, "BiasGelu", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, at::gelu(ctx.RequiredInput(0) + ctx.RequiredInput(1))); });
  r.RegisterFn(MS, "Gelu", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, at::gelu(ctx.RequiredInput(0))); });
  r.RegisterFn(MS, "QuickGelu", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x * at::sigmoid(x * ctx.node().attr_f("alpha", 1.702f)));
  });
  r.RegisterFn(MS, "BiasAdd", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, ctx.RequiredInput(0) + ctx.RequiredInput(1) + ctx.RequiredInput(2));
  });
  r.RegisterFn(MS, "BiasSplitGelu", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0) + ctx.RequiredInput(1);
    const int64_t h = x.size(-1) / 2;
    ctx.SetOutput(0, x.narrow(-1, 0, h) * at::gelu(x.narrow(-1, h, h)));
  });
  r.RegisterFn(MS, "BiasSoftmax", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t axis = ctx.node().attr_i("axis", 1);
    if (axis < 0) axis += x.dim();
    at::Tensor s = x + ctx.RequiredInput(1);
    int64_t outer = 1;
    for (int64_t i = 0; i < axis; ++i) outer *= s.size(i);
    ctx.SetOutput(0, at::softmax(s.reshape({outer, -1}), 1).reshape(s.sizes()));
  });
  auto fused_matmul = [](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor a = ctx.RequiredInput(0), b = ctx.RequiredInput(1);
    if (n.attr_i("transBatchA", 0)) a = a.movedim(0, -2);
    if (n.attr_i("transBatchB", 0)) b = b.movedim(0, -2);
    if (n.attr_i("transA", 0) && a.dim() >= 2) a = a.transpose(-1, -2);
    if (n.attr_i("transB", 0) && b.dim() >= 2) b = b.transpose(-1, -2);
    at::Tensor y = at::matmul(a, b);
    const float alpha = n.attr_f("alpha", 1.f);
    ctx.SetOutput(0, alpha == 1.f ? y : y * alpha);
  };
  r.RegisterFn(MS, "FusedMatMul", 1, kMax, fused_matmul);
  r.RegisterFn(MS, "TransposeMatMul", 1, kMax, fused_matmul);
  r.RegisterFn(MS, "Attention", 1, kMax, BertAttentionImpl, {6});
  r.RegisterFn(MS, "MultiHeadAttention", 1, kMax, MultiHeadAttentionImpl);
  r.RegisterFn(MS, "RotaryEmbedding", 1, kMax, ContribRotaryImpl);
  r.RegisterFn(MS, "GroupQueryAttention", 1, kMax, GqaImpl, {6});
  r.RegisterFn(MS, "PagedAttention", 1, kMax, PagedAttentionImpl, {5, 6});
  r.RegisterFn(MS, "MatMulNBits", 1, kMax, MatMulNBitsImpl);
  r.RegisterFn(MS, "MoE", 1, kMax, MoeImpl);
  r.RegisterFn(MS, "QMoE", 1, kMax, QMoeImpl);
  r.RegisterFn(MS, "GemmFloat8", 1, kMax, GemmFloat8Impl);
  r.RegisterFn(MS, "Inverse", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, at::linalg_inv(ctx.RequiredInput(0))); });
  r.RegisterFn(MS, "Trilu", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t k = ctx.HasInput(1) ? ctx.Input(1).cpu().item<int64_t>() : 0;
    ctx.SetOutput(0, ctx.node().attr_i("upper", 1) ? at::triu(x, k) : at::tril(x, k));
  }, {1});
  r.RegisterFn(MS, "QuantizeLinear", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor scale = ctx.RequiredInput(1).to(at::kFloat);
    at::ScalarType out_t = ctx.HasInput(2) ? ctx.Input(2).scalar_type() : at::kByte;
    at::Tensor q = at::round(x.to(at::kFloat) / scale);
    if (ctx.HasInput(2)) q = q + ctx.Input(2).to(at::kFloat);
    const double lo = out_t == at::kChar ? -128 : 0, hi = out_t == at::kChar ? 127 : 255;
    ctx.SetOutput(0, at::clamp(q, lo, hi).to(out_t));
  });
  r.RegisterFn(MS, "DequantizeLinear", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0).to(at::kFloat);
    if (ctx.HasInput(2)) x = x - ctx.Input(2).to(at::kFloat);
    ctx.SetOutput(0, (x * ctx.RequiredInput(1).to(at::kFloat)).to(ctx.RequiredInput(1).scalar_type()));
  });
  r.RegisterFn(MS, "GroupNorm", 1, kMax, [](Ctx& ctx) {
    // NHWC input, optional Swish
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor nchw = x.permute({0, 3, 1, 2});
    at::Tensor y = at::group_norm(nchw.to(at::kFloat), ctx.node().attr_i("groups", 32), ctx.RequiredInput(1).to(at::kFloat),
                                  ctx.RequiredInput(2).to(at::kFloat), ctx.node().attr_f("epsilon", 1e-5f), false);
    if (ctx.node().attr_i("activation", 0) == 1) y = y * at::sigmoid(y);
    ctx.SetOutput(0, y.permute({0, 2, 3, 1}).contiguous().to(x.scalar_type()));
  });
  // com.ortb200: ops the GPU lowering passes create; these ATen versions keep an optimized model loadable anywhere
  // an RMS normalisation folded into the GEMM in front of it: rms_eps attribute + gamma input
  auto normed_input = [](Ctx& ctx, int gamma_index) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const float eps = ctx.node().attr_f("rms_eps", 0.f);
    if (eps <= 0.f) return x;
    at::Tensor xf = x.to(at::kFloat);
    at::Tensor y = xf * at::rsqrt(xf.pow(2).mean(-1, true) + eps);
    return (y.to(x.scalar_type()) * ctx.RequiredInput(gamma_index)).to(x.scalar_type());
  };
  r.RegisterFn("com.ortb200", "FusedGemm", 1, kMax, [normed_input](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor y = at::matmul(normed_input(ctx, 4), ctx.RequiredInput(1));
    if (ctx.HasInput(2)) y = y + ctx.Input(2);
    const std::string act = n.attr_s("activation", "none");
    if (act == "gelu") y = at::gelu(y);
    else if (act == "fastgelu") y = at::gelu(y, "tanh");
    else if (act == "relu") y = at::relu(y);
    else if (act == "silu") y = at::silu(y);
    else if (act == "quickgelu") y = y * at::sigmoid(y * 1.702);
    else if (act != "none") ORTB_THROW(INVALID_ARGUMENT, "FusedGemm: unknown activation ", act);
    if (n.attr_i("all_reduce", 0)) y = AllReduceSum(ctx.session(), y);
    if (ctx.HasInput(3)) y = y + ctx.Input(3);
    ctx.SetOutput(0, y);
  });
  r.RegisterFn("com.ortb200", "SwiGLU", 1, kMax, [](Ctx& ctx) {
    // [..., 2 I] -> silu(x[..., :I]) * x[..., I:]
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t I = x.size(-1) / 2;
    ctx.SetOutput(0, at::silu(x.narrow(-1, 0, I)) * x.narrow(-1, I, I));
  });
  r.RegisterFn("com.ortb200", "GemmSwiGLU", 1, kMax, [normed_input](Ctx& ctx) {
    at::Tensor x = normed_input(ctx, 3);
    ctx.SetOutput(0, at::silu(at::matmul(x, ctx.RequiredInput(1))) * at::matmul(x, ctx.RequiredInput(2)));
  });
}

}  // namespace ortb
