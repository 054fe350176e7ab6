// com.microsoft: the linear-attention family (CausalConvWithState, LinearAttention, LinearAttentionGate) and
// SparseAttention.  The recurrences are written token by token with batched tensor operations per step, which is the
// operator's stated semantics ("equivalent to running the recurrent update sequentially for each token").
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
#include <limits>

#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

at::Tensor OptT(Ctx& ctx, int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); }

// CausalConvWithState, ndim = 1: input [B, C, L], weight [C, 1, k], past_state [B, C, k - 1] (or [W, B, C, k - 1]).
void CausalConvImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  ORTB_ENFORCE(n.attr_i("ndim", 1) == 1, "CausalConvWithState: only ndim = 1 is implemented");
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& w = ctx.RequiredInput(1);
  const int64_t B = x.size(0), C = x.size(1), L = x.size(2), k = w.size(2), W = n.attr_i("state_window", 0);
  ORTB_ENFORCE_ARG(W >= 0 && W <= 8, "CausalConvWithState: state_window must be in [0, 8]");
  at::Tensor past = OptT(ctx, 3);
  if (past.defined() && past.dim() == 4) past = past[past.size(0) - 1];
  if (!past.defined()) past = at::zeros({B, C, k - 1}, x.options());
  at::Tensor virt = at::cat({past.to(x.scalar_type()), x}, 2);              // [B, C, k - 1 + L]
  c10::optional<at::Tensor> bias;
  if (ctx.HasInput(2)) bias = ctx.Input(2);
  at::Tensor y = at::conv1d(virt, w, bias, at::IntArrayRef{1}, at::IntArrayRef{0}, at::IntArrayRef{1}, C);  // depthwise, valid -> [B, C, L]
  const std::string act = n.attr_s("activation", "none");
  if (act == "silu" || act == "swish") y = at::silu(y);
  else ORTB_ENFORCE_ARG(act == "none" || act.empty(), "CausalConvWithState: unknown activation '", act, "'");
  ctx.SetOutput(0, y);
  if (ctx.OutputCount() > 1) {
    // state after input position p = virtual positions [p + 1, p + k - 1]
    auto state_after = [&](int64_t p) { return virt.narrow(2, p + 1, k - 1); };
    if (W == 0) {
      ctx.SetOutput(1, state_after(L - 1).contiguous());
    } else {
      at::Tensor st = at::zeros({W, B, C, k - 1}, x.options());
      for (int64_t j = 0; j < W; ++j) {
        const int64_t p = L - W + j;
        if (p >= 0) st[j].copy_(state_after(p));
      }
      ctx.SetOutput(1, st);
    }
  }
}

// LinearAttention: state S [B, Hkv, dk, dv] in float32.
void LinearAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& q_in = ctx.RequiredInput(0);
  const at::Tensor& k_in = ctx.RequiredInput(1);
  const at::Tensor& v_in = ctx.RequiredInput(2);
  const int64_t Hq = n.attr_i("q_num_heads", 0), Hkv = n.attr_i("kv_num_heads", 0), W = n.attr_i("state_window", 0);
  ORTB_ENFORCE_ARG(Hq > 0 && Hkv > 0, "LinearAttention: q_num_heads and kv_num_heads are required");
  const std::string rule = n.attr_s("update_rule", "gated_delta");
  const bool gated = rule == "gated" || rule == "gated_delta", delta = rule == "delta" || rule == "gated_delta";
  ORTB_ENFORCE_ARG(gated || delta || rule == "linear", "LinearAttention: unknown update_rule '", rule, "'");
  const int64_t B = q_in.size(0), T = q_in.size(1), dk = q_in.size(2) / Hq, dv = v_in.size(2) / Hkv;
  ORTB_ENFORCE_ARG(k_in.size(2) == Hkv * dk, "LinearAttention: key width does not match kv_num_heads * d_k");
  const double scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(dk));
  at::Tensor q = q_in.to(at::kFloat).reshape({B, T, Hq, dk});
  at::Tensor k = k_in.to(at::kFloat).reshape({B, T, Hkv, dk});
  at::Tensor v = v_in.to(at::kFloat).reshape({B, T, Hkv, dv});
  at::Tensor decay = OptT(ctx, 4), beta = OptT(ctx, 5);
  ORTB_ENFORCE_ARG(!gated || decay.defined(), "LinearAttention: update_rule '", rule, "' needs decay");
  ORTB_ENFORCE_ARG(!delta || beta.defined(), "LinearAttention: update_rule '", rule, "' needs beta");
  if (decay.defined()) {
    decay = decay.to(at::kFloat);
    decay = decay.size(2) == Hkv ? decay.reshape({B, T, Hkv, 1}) : decay.reshape({B, T, Hkv, dk});
  }
  if (beta.defined()) beta = beta.to(at::kFloat).expand({B, T, Hkv}).reshape({B, T, Hkv, 1, 1});
  at::Tensor past = OptT(ctx, 3);
  at::ScalarType state_type = past.defined() ? past.scalar_type() : q_in.scalar_type();
  if (past.defined() && past.dim() == 5) past = past[past.size(0) - 1];
  at::Tensor S = past.defined() ? past.to(at::kFloat).clone() : at::zeros({B, Hkv, dk, dv}, q.options());
  const int64_t Hout = std::max(Hq, Hkv);
  at::Tensor out = at::empty({B, T, Hout, dv}, q.options());
  at::Tensor window;
  if (W > 0) window = at::zeros({W, B, Hkv, dk, dv}, q.options());
  for (int64_t t = 0; t < T; ++t) {
    at::Tensor kt = k.select(1, t), vt = v.select(1, t);                    // [B, Hkv, dk], [B, Hkv, dv]
    if (gated) S = S * at::exp(decay.select(1, t)).unsqueeze(-1);            // per head or per key dimension
    if (delta) {
      at::Tensor pred = at::einsum("bhkv,bhk->bhv", {S, kt});               // S^T k
      S = S + beta.select(1, t) * kt.unsqueeze(-1) * (vt - pred).unsqueeze(-2);
    } else {
      S = S + kt.unsqueeze(-1) * vt.unsqueeze(-2);
    }
    at::Tensor qt = q.select(1, t);                                          // [B, Hq, dk]
    at::Tensor o;
    if (Hq >= Hkv) {
      at::Tensor Sx = S.repeat_interleave(Hq / Hkv, 1);                      // query head h reads kv head h / group
      o = at::einsum("bhk,bhkv->bhv", {qt, Sx});
    } else {
      o = at::einsum("bhk,bhkv->bhv", {qt.repeat_interleave(Hkv / Hq, 1), S});
    }
    out.select(1, t).copy_(o * scale);
    if (W > 0 && t >= T - W) window[t - (T - W)].copy_(S);
  }
  ctx.SetOutput(0, out.reshape({B, T, Hout * dv}).to(q_in.scalar_type()));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, (W > 0 ? window : S).to(state_type));
}

// SparseAttention (contrib_ops/cuda/sparse/sparse_attention.cc) restated as GroupQueryAttention with an additive
// mask: query position i may see key j when j <= i and block (i / bs, j / bs) is listed in the CSR layout of the
// head's layout (head % num_layout).
void SparseAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  contrib::GqaInputs in;
  in.query = ctx.RequiredInput(0);
  in.key = OptT(ctx, 1);
  in.value = OptT(ctx, 2);
  in.past_key = ctx.RequiredInput(3);
  in.past_value = ctx.RequiredInput(4);
  in.share_buffer = true;
  in.cos_cache = OptT(ctx, 9);
  in.sin_cache = OptT(ctx, 10);
  at::Tensor key_lens = ctx.RequiredInput(8).to(at::kCPU, at::kLong).reshape({-1});
  in.seqlens_k = key_lens - 1;
  in.total_sequence_length = ctx.RequiredInput(7).to(at::kCPU, at::kLong).reshape({-1})[0].item<int64_t>();
  contrib::GqaAttrs a;
  a.num_heads = n.attr_i("num_heads", 0);
  a.kv_num_heads = n.attr_i("kv_num_heads", 0);
  a.do_rotary = n.attr_i("do_rotary", 0) != 0;
  a.rotary_interleaved = n.attr_i("rotary_interleaved", 0) != 0;
  a.scale = n.attr_f("scale", 0.f);
  const int64_t bs = n.attr_i("sparse_block_size", 64);
  const int64_t B = in.query.size(0), S = in.query.size(1), total = in.total_sequence_length;
  // dense block mask [layouts, blocks, blocks] from the CSR arrays
  at::Tensor rows = ctx.RequiredInput(5).to(at::kCPU, at::kLong), cols = ctx.RequiredInput(6).to(at::kCPU, at::kLong);
  const int64_t layouts = rows.size(0), blocks = rows.size(1) - 1;
  at::Tensor block_mask = at::zeros({layouts, blocks, blocks}, at::TensorOptions().dtype(at::kBool));
  auto bm = block_mask.accessor<bool, 3>();
  auto ra = rows.accessor<int64_t, 2>();
  auto ca = cols.accessor<int64_t, 2>();
  for (int64_t l = 0; l < layouts; ++l) {
    for (int64_t r = 0; r < blocks; ++r) {
      for (int64_t e = ra[l][r]; e < ra[l][r + 1]; ++e) {
        const int64_t c = ca[l][e];
        if (c >= 0 && c < blocks) bm[l][r][c] = true;
      }
    }
  }
  ORTB_ENFORCE_ARG(total <= blocks * bs, "SparseAttention: total_sequence_length exceeds the block layout");
  const bool first_prompt = S == total;
  const float neg = -std::numeric_limits<float>::infinity();
  at::Tensor bias = at::full({B, a.num_heads, S, total}, neg, at::TensorOptions().dtype(at::kFloat));
  at::Tensor key_block = at::arange(total, at::TensorOptions().dtype(at::kLong)).floor_divide(bs);     // [T]
  for (int64_t b = 0; b < B; ++b) {
    const int64_t past = first_prompt ? 0 : key_lens[b].item<int64_t>() - S;
    at::Tensor qpos = at::arange(S, at::TensorOptions().dtype(at::kLong)) + past;                      // absolute rows
    at::Tensor causal = at::arange(total, at::TensorOptions().dtype(at::kLong)).unsqueeze(0).le(qpos.unsqueeze(1));  // [S, T]
    at::Tensor qblock = qpos.floor_divide(bs).clamp_max(blocks - 1);
    for (int64_t h = 0; h < a.num_heads; ++h) {
      at::Tensor m = block_mask[h % layouts].index_select(0, qblock).index_select(1, key_block);       // [S, T]
      bias[b][h].masked_fill_(m.logical_and(causal), 0.f);
    }
  }
  in.attention_bias = bias.to(in.query.device());
  contrib::GqaResult res = contrib::GqaForward(in, a);
  ctx.SetOutput(0, res.output);
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, res.present_key);
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, res.present_value);
}

}  // namespace

void RegisterContribKernels4Linear(KernelRegistry& r) {
  r.RegisterFn(MS, "CausalConvWithState", 1, kMax, CausalConvImpl);
  r.RegisterFn(MS, "LinearAttention", 1, kMax, LinearAttentionImpl);
  r.RegisterFn(MS, "LinearAttentionGate", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    at::Tensor z = a.to(at::kFloat) + ctx.RequiredInput(1).to(at::kFloat);
    ctx.SetOutput(0, (ctx.RequiredInput(2).to(at::kFloat) * at::softplus(z)).to(a.scalar_type()));
    if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) {
      ORTB_ENFORCE_ARG(ctx.HasInput(3), "LinearAttentionGate: the beta output needs input b");
      ctx.SetOutput(1, at::sigmoid(ctx.Input(3).to(at::kFloat)).to(ctx.Input(3).scalar_type()));
    }
  });
  r.RegisterFn(MS, "SparseAttention", 1, kMax, SparseAttentionImpl, {5, 6, 7, 8});
}

}  // namespace ortb
