// com.microsoft contrib operators, fourth group: the decoder-masked attentions (single-token decoding with a beam
// cache indirection), LongformerAttention, SparseAttention, GatedRelativePositionBias, multimodal rotary embedding and
// the linear-attention family.  Generic ATen implementations (CPU provider and CUDA tensors alike); the dense-mask
// restatements are the oracle form of what the reference computes with specialised kernels.
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

int64_t HostInt(const at::Tensor& t) { return t.to(at::kCPU, at::kLong).reshape({-1})[0].item<int64_t>(); }

at::Tensor OptT(Ctx& ctx, int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); }

// Shared tail of the two decoder-masked operators (contrib_ops/cpu/bert/decoder_masked_multihead_attention.cc,
// contrib_ops/cuda/decoder/decoder_masked_self_attention.cc).  q, k, v: [B, N, 1, H] for the new token.  Caches are
// plain [B, N, capacity, H] buffers.  With a beam cache indirection [batch, beam, max_len], the key / value of past
// step t for row (b, j) is read from row (b, indirection[b, j, t]).
struct DecoderStep {
  at::Tensor q, k, v;                 // new token
  at::Tensor past_k, past_v;          // may be undefined
  at::Tensor mask, bias, indirection;  // optional
  int64_t past_len = 0, beam = 1;
  bool share_buffer = false;
  double scale = 0;
  float filter = -10000.f;
};

void RunDecoderStep(Ctx& ctx, const DecoderStep& d, int out_key_index, at::Tensor* qk_out) {
  const int64_t B = d.q.size(0), N = d.q.size(1), H = d.q.size(3), Hv = d.v.size(3);
  const int64_t T = d.past_len + 1;
  at::Tensor pk, pv;
  if (d.share_buffer) {
    ORTB_ENFORCE_ARG(d.past_k.defined() && d.past_k.size(2) >= T, "past buffer is too small for past_sequence_length + 1");
    pk = d.past_k;
    pv = d.past_v;
  } else {
    pk = at::empty({B, N, T, H}, d.k.options());
    pv = at::empty({B, N, T, Hv}, d.v.options());
    if (d.past_len > 0) {
      pk.narrow(2, 0, d.past_len).copy_(d.past_k.narrow(2, 0, d.past_len));
      pv.narrow(2, 0, d.past_len).copy_(d.past_v.narrow(2, 0, d.past_len));
    }
  }
  pk.narrow(2, d.past_len, 1).copy_(d.k);
  pv.narrow(2, d.past_len, 1).copy_(d.v);
  at::Tensor keys = pk.narrow(2, 0, T), vals = pv.narrow(2, 0, T);
  if (d.indirection.defined() && d.beam > 1 && d.past_len > 0) {
    const int64_t batch = B / d.beam;
    at::Tensor ind = d.indirection.to(at::kLong).to(keys.device()).narrow(2, 0, d.past_len);   // [batch, beam, past]
    at::Tensor rows = ind + (at::arange(batch, ind.options()) * d.beam).reshape({batch, 1, 1});  // absolute row
    rows = rows.reshape({B, 1, d.past_len, 1});
    auto regather = [&](const at::Tensor& cache, int64_t width) {
      // out[r, n, t, :] = cache[rows[r, t], n, t, :]
      at::Tensor idx = rows.expand({B, N, d.past_len, width});
      at::Tensor past = cache.narrow(2, 0, d.past_len).gather(0, idx);
      return at::cat({past, cache.narrow(2, d.past_len, 1)}, 2);
    };
    keys = regather(pk, H);
    vals = regather(pv, Hv);
  }
  at::Tensor s = at::matmul(d.q.to(at::kFloat), keys.to(at::kFloat).transpose(-1, -2)) * d.scale;   // [B, N, 1, T]
  if (qk_out != nullptr) *qk_out = s;
  if (d.bias.defined()) s = s + d.bias.to(at::kFloat).narrow(-1, 0, T);
  if (d.mask.defined()) {
    at::Tensor valid = d.mask.to(s.device()).narrow(1, 0, T).ne(0).reshape({B, 1, 1, T});
    s = s + at::where(valid, at::zeros({1}, s.options()), at::full({1}, d.filter, s.options()));
  }
  at::Tensor y = at::matmul(at::softmax(s, -1), vals.to(at::kFloat)).to(d.q.scalar_type());       // [B, N, 1, Hv]
  ctx.SetOutput(0, y.transpose(1, 2).reshape({B, 1, N * Hv}).contiguous());
  if (out_key_index >= 0) {
    if (ctx.OutputCount() > out_key_index) ctx.SetOutput(out_key_index, pk);
    if (ctx.OutputCount() > out_key_index + 1) ctx.SetOutput(out_key_index + 1, pv);
  }
}

void DecoderMaskedMhaImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const int64_t N = n.attr_i("num_heads", 1);
  at::Tensor query = ctx.RequiredInput(0);
  const int64_t B = query.size(0);
  ORTB_ENFORCE_ARG(query.dim() == 3 && query.size(1) == 1, "DecoderMaskedMultiHeadAttention: sequence length must be 1");
  at::Tensor bias = OptT(ctx, 10);
  at::Tensor key = OptT(ctx, 1), value = OptT(ctx, 2);
  DecoderStep d;
  d.filter = n.attr_f("mask_filter_value", -10000.f);
  d.mask = OptT(ctx, 3);
  d.bias = OptT(ctx, 4);
  const bool cross = key.defined() && key.dim() == 4;
  if (cross) {
    // cross attention: key / value are the encoder's projected states [B, N, L, H]; nothing is appended
    at::Tensor q = query;
    if (bias.defined()) q = q + bias.narrow(0, 0, q.size(2));
    const int64_t H = q.size(2) / N, L = key.size(2);
    q = q.reshape({B, 1, N, H}).transpose(1, 2);
    const double scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
    at::Tensor s = at::matmul(q.to(at::kFloat), key.to(at::kFloat).transpose(-1, -2)) * scale;
    if (ctx.OutputCount() > 3 && ctx.OutputNeeded(3)) ctx.SetOutput(3, s);
    if (d.bias.defined()) s = s + d.bias.to(at::kFloat);
    if (d.mask.defined()) {
      at::Tensor valid = d.mask.to(s.device()).narrow(1, 0, L).ne(0).reshape({B, 1, 1, L});
      s = s + at::where(valid, at::zeros({1}, s.options()), at::full({1}, d.filter, s.options()));
    }
    at::Tensor y = at::matmul(at::softmax(s, -1), value.to(at::kFloat)).to(query.scalar_type());
    ctx.SetOutput(0, y.transpose(1, 2).reshape({B, 1, N * value.size(3)}).contiguous());
    return;
  }
  at::Tensor q, k, v;
  if (!key.defined()) {  // packed QKV [B, 1, 2 * hidden + v_hidden] with hidden == v_hidden
    const int64_t hidden = query.size(2) / 3;
    if (bias.defined()) query = query + bias;
    q = query.narrow(2, 0, hidden);
    k = query.narrow(2, hidden, hidden);
    v = query.narrow(2, 2 * hidden, hidden);
  } else {
    q = query;
    k = key;
    v = value;
    if (bias.defined()) {
      q = q + bias.narrow(0, 0, q.size(2));
      k = k + bias.narrow(0, q.size(2), k.size(2));
      v = v + bias.narrow(0, q.size(2) + k.size(2), v.size(2));
    }
  }
  const int64_t H = q.size(2) / N, Hv = v.size(2) / N;
  d.q = q.reshape({B, 1, N, H}).transpose(1, 2);
  d.k = k.reshape({B, 1, N, H}).transpose(1, 2);
  d.v = v.reshape({B, 1, N, Hv}).transpose(1, 2);
  d.past_k = OptT(ctx, 5);
  d.past_v = OptT(ctx, 6);
  d.share_buffer = n.attr_i("past_present_share_buffer", 0) != 0 && d.past_k.defined();
  d.past_len = ctx.HasInput(7) ? HostInt(ctx.Input(7)) : (d.past_k.defined() ? d.past_k.size(2) : 0);
  d.beam = ctx.HasInput(8) ? HostInt(ctx.Input(8)) : 1;
  d.indirection = OptT(ctx, 9);
  d.scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor qk;
  const bool want_qk = ctx.OutputCount() > 3 && ctx.OutputNeeded(3);
  RunDecoderStep(ctx, d, 1, want_qk ? &qk : nullptr);
  if (want_qk) ctx.SetOutput(3, qk);
}

// DecoderMaskedSelfAttention: input [B, 1, hidden] x weights [hidden, 3 * hidden] + bias, past [2, B, N, cap, H].
void DecoderMaskedSelfImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const int64_t N = n.attr_i("num_heads", 1);
  const at::Tensor& x = ctx.RequiredInput(0);
  const int64_t B = x.size(0);
  ORTB_ENFORCE_ARG(x.dim() == 3 && x.size(1) == 1, "DecoderMaskedSelfAttention: sequence length must be 1");
  at::Tensor qkv = at::matmul(x, ctx.RequiredInput(1));
  if (ctx.HasInput(2)) qkv = qkv + ctx.Input(2);
  const int64_t hidden = qkv.size(2) / 3, H = hidden / N;
  DecoderStep d;
  d.q = qkv.narrow(2, 0, hidden).reshape({B, 1, N, H}).transpose(1, 2);
  d.k = qkv.narrow(2, hidden, hidden).reshape({B, 1, N, H}).transpose(1, 2);
  d.v = qkv.narrow(2, 2 * hidden, hidden).reshape({B, 1, N, H}).transpose(1, 2);
  d.mask = OptT(ctx, 3);
  at::Tensor past = OptT(ctx, 4);
  d.bias = OptT(ctx, 5);
  d.share_buffer = n.attr_i("past_present_share_buffer", 0) != 0 && past.defined();
  d.past_len = ctx.HasInput(6) ? HostInt(ctx.Input(6)) : (past.defined() ? past.size(3) : 0);
  d.beam = ctx.HasInput(7) ? HostInt(ctx.Input(7)) : 1;
  d.indirection = OptT(ctx, 8);
  d.filter = n.attr_f("mask_filter_value", -10000.f);
  d.scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  if (n.attr_i("do_rotary", 0) != 0) {
    // rotary position = past length, GPT-NeoX style halves, no cache input: angles from the default base
    int64_t rot = n.attr_i("rotary_embedding_dim", 0);
    if (rot == 0) rot = H;
    auto fopt = at::TensorOptions().dtype(at::kFloat).device(x.device());
    at::Tensor inv = at::pow(10000.0, -at::arange(0, rot, 2, fopt) / static_cast<double>(rot));
    at::Tensor ang = inv * static_cast<double>(d.past_len);
    at::Tensor c = at::cos(ang), s = at::sin(ang);
    auto rotate = [&](const at::Tensor& t) {
      at::Tensor tf = t.to(at::kFloat);
      at::Tensor a = tf.narrow(-1, 0, rot / 2), b = tf.narrow(-1, rot / 2, rot / 2);
      std::vector<at::Tensor> parts = {a * c - b * s, b * c + a * s};
      if (rot < H) parts.push_back(tf.narrow(-1, rot, H - rot));
      return at::cat(parts, -1).to(t.scalar_type());
    };
    d.q = rotate(d.q);
    d.k = rotate(d.k);
  }
  at::Tensor present;
  if (past.defined()) {
    d.past_k = past[0];
    d.past_v = past[1];
  }
  if (d.share_buffer) {
    RunDecoderStep(ctx, d, -1, nullptr);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, past);
  } else {
    // non-shared: build [2, B, N, T, H] so that both halves come out as one tensor
    const int64_t T = d.past_len + 1;
    present = at::empty({2, B, N, T, H}, d.k.options());
    if (d.past_len > 0) present.narrow(3, 0, d.past_len).copy_(past.narrow(3, 0, d.past_len));
    DecoderStep e = d;
    e.past_k = present[0];
    e.past_v = present[1];
    e.share_buffer = true;
    RunDecoderStep(ctx, e, -1, nullptr);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, present);
  }
}

// LongformerAttention (contrib_ops/cuda/bert/longformer_attention.cc), restated with a dense mask: a local token
// attends to the keys within `window` positions on either side and to every global token, with the regular
// projections; a global token attends to every token with the global projections.  `mask` is additive per key
// (0 = keep, large negative = padding).
void LongformerImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  auto project = [&](int wi, int bi) {
    at::Tensor p = at::matmul(x, ctx.RequiredInput(wi));
    if (ctx.HasInput(bi)) p = p + ctx.Input(bi);
    return p.to(at::kFloat);
  };
  at::Tensor y = contrib::LongformerCore(project(1, 2), project(4, 5), ctx.RequiredInput(3), ctx.RequiredInput(6), n.attr_i("num_heads", 1),
                                         n.attr_i("window", 1));
  ctx.SetOutput(0, y.to(x.scalar_type()).contiguous());
}

}  // namespace

namespace contrib {
// Sliding-window attention with global tokens on projected inputs: qkv / gqkv are [B, S, 3 * hidden] (float), mask is the
// additive key mask [B, S], global marks the tokens that attend to (and are attended by) everything.  Returns [B, S, hidden].
at::Tensor LongformerCore(const at::Tensor& qkv, const at::Tensor& gqkv, const at::Tensor& mask, const at::Tensor& global, int64_t N, int64_t w) {
  const int64_t B = qkv.size(0), S = qkv.size(1);
  const int64_t hidden = qkv.size(2) / 3, H = hidden / N;
  auto heads = [&](const at::Tensor& t, int64_t part) {
    return t.narrow(2, part * hidden, hidden).reshape({B, S, N, H}).transpose(1, 2);  // [B, N, S, H]
  };
  const double scale = 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor key_mask = mask.to(qkv.device(), at::kFloat).reshape({B, 1, 1, S});
  at::Tensor is_global = global.to(qkv.device()).ne(0);                                // [B, S]
  auto lopt = at::TensorOptions().dtype(at::kLong).device(qkv.device());
  at::Tensor pos = at::arange(S, lopt);
  at::Tensor in_window = (pos.unsqueeze(0) - pos.unsqueeze(1)).abs().le(w);          // [S, S]
  at::Tensor allowed = in_window.reshape({1, 1, S, S}).logical_or(is_global.reshape({B, 1, 1, S}));
  const float neg = -std::numeric_limits<float>::infinity();
  at::Tensor s_local = at::matmul(heads(qkv, 0) * scale, heads(qkv, 1).transpose(-1, -2)) + key_mask;
  s_local = s_local.masked_fill(allowed.logical_not(), neg);
  at::Tensor y_local = at::matmul(at::softmax(s_local, -1), heads(qkv, 2));
  at::Tensor s_glob = at::matmul(heads(gqkv, 0) * scale, heads(gqkv, 1).transpose(-1, -2)) + key_mask;
  at::Tensor y_glob = at::matmul(at::softmax(s_glob, -1), heads(gqkv, 2));
  at::Tensor y = at::where(is_global.reshape({B, 1, S, 1}), y_glob, y_local);
  return y.transpose(1, 2).reshape({B, S, hidden});
}
}  // namespace contrib

namespace {

// GatedRelativePositionBias (contrib_ops/cuda/bert/gated_relative_position_bias.cc; WavLM): per query a pair of gates
// from a small linear layer scales the shared relative position bias.
void GatedRelPosBiasImpl(Ctx& ctx) {
  const int64_t N = ctx.node().attr_i("num_heads", 1);
  at::Tensor q = ctx.RequiredInput(0).to(at::kFloat);
  ORTB_ENFORCE_ARG(!ctx.HasInput(6), "GatedRelativePositionBias: packed input (token_offset) is not supported");
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2) / N;
  q = (q + ctx.RequiredInput(1).to(at::kFloat)).reshape({B, S, N, H}).transpose(1, 2);           // [B, N, S, H]
  const at::Tensor& weight = ctx.RequiredInput(3);                                                // [H, D]
  const int64_t D = weight.size(1);
  at::Tensor g = at::matmul(q, weight.to(at::kFloat)) + ctx.RequiredInput(4).to(at::kFloat);     // [B, N, S, D]
  g = at::sigmoid(g.reshape({B, N, S, 2, D / 2}).sum(-1));                                       // [B, N, S, 2]
  at::Tensor gate_u = g.select(-1, 0), gate_r = g.select(-1, 1);
  at::Tensor eco = ctx.RequiredInput(5).to(at::kFloat).reshape({1, N, 1});
  at::Tensor gate = gate_u * (gate_r * eco - 1.0) + 2.0;                                          // [B, N, S]
  at::Tensor out = gate.unsqueeze(-1) * ctx.RequiredInput(2).to(at::kFloat);                      // x [1, N, S, S]
  ctx.SetOutput(0, out.to(ctx.RequiredInput(0).scalar_type()));
}

// MRotaryEmbedding: three position streams (temporal, height, width) pick the per-frequency angles; then the usual
// rotation.  mrope_layout 0 = contiguous sections, 1 = interleaved (H at 1, 4, 7 ..., W at 2, 5, 8 ...).
void MRotaryImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  at::Tensor x = ctx.RequiredInput(0);
  at::Tensor pos = ctx.RequiredInput(1).to(at::kLong).to(x.device());   // [3, B, S]
  const at::Tensor& cos_cache = ctx.RequiredInput(2);
  const at::Tensor& sin_cache = ctx.RequiredInput(3);
  const std::vector<int64_t> sec = n.attr_ints("mrope_section");
  ORTB_ENFORCE_ARG(sec.size() == 3, "MRotaryEmbedding: mrope_section needs three entries");
  const bool interleaved = n.attr_i("interleaved", 0) != 0;
  const int64_t layout = n.attr_i("mrope_layout", 0);
  const bool bnsh = x.dim() == 4;
  int64_t N = n.attr_i("num_heads", 0);
  const int64_t B = x.size(0), S = bnsh ? x.size(2) : x.size(1);
  const int64_t half = cos_cache.size(1), rot = 2 * half;
  ORTB_ENFORCE_ARG(sec[0] + sec[1] + sec[2] == half, "MRotaryEmbedding: sections must add up to half the rotary dimension");
  at::Tensor xs;  // [B, S, N, H]
  if (bnsh) {
    xs = x.transpose(1, 2);
  } else {
    int64_t H = n.attr_i("rotary_embedding_dim", 0) > 0 && N > 0 ? x.size(2) / N : rot;
    if (N == 0) N = x.size(2) / H;
    xs = x.reshape({B, S, N, x.size(2) / N});
  }
  const int64_t H = xs.size(3);
  // which stream feeds frequency d
  std::vector<int64_t> stream(half, 0);
  if (layout == 0) {
    for (int64_t d = 0; d < half; ++d) stream[d] = d < sec[0] ? 0 : (d < sec[0] + sec[1] ? 1 : 2);
  } else {
    for (int64_t d = 1; d < std::min(half, sec[1] * 3); d += 3) stream[d] = 1;
    for (int64_t d = 2; d < std::min(half, sec[2] * 3); d += 3) stream[d] = 2;
  }
  at::Tensor stream_t = at::tensor(stream, at::TensorOptions().dtype(at::kLong)).to(x.device());
  // cos / sin [B, S, half]: gather per stream, then pick per frequency
  at::Tensor cs = at::embedding(cos_cache.to(at::kFloat), pos);   // [3, B, S, half]
  at::Tensor sn = at::embedding(sin_cache.to(at::kFloat), pos);
  at::Tensor pick = stream_t.reshape({1, 1, 1, half}).expand({1, B, S, half});
  at::Tensor c = cs.gather(0, pick).squeeze(0).unsqueeze(2), s = sn.gather(0, pick).squeeze(0).unsqueeze(2);  // [B, S, 1, half]
  at::Tensor xf = xs.to(at::kFloat);
  at::Tensor a, b;
  if (interleaved) {
    at::Tensor pairs = xf.narrow(-1, 0, rot).reshape({B, S, xs.size(2), half, 2});
    a = pairs.select(-1, 0);
    b = pairs.select(-1, 1);
  } else {
    a = xf.narrow(-1, 0, half);
    b = xf.narrow(-1, half, half);
  }
  at::Tensor ra = a * c - b * s, rb = b * c + a * s;
  at::Tensor rotated = interleaved ? at::stack({ra, rb}, -1).reshape({B, S, xs.size(2), rot}) : at::cat({ra, rb}, -1);
  if (rot < H) rotated = at::cat({rotated, xf.narrow(-1, rot, H - rot)}, -1);
  const float scale = n.attr_f("scale", 1.0f);
  if (scale != 1.0f) rotated = rotated * scale;
  rotated = rotated.to(x.scalar_type());
  ctx.SetOutput(0, bnsh ? rotated.transpose(1, 2).contiguous() : rotated.reshape(x.sizes()));
}

}  // namespace

void RegisterContribKernels4Linear(KernelRegistry& r);

void RegisterContribKernels4(KernelRegistry& r) {
  r.RegisterFn(MS, "DecoderMaskedMultiHeadAttention", 1, kMax, DecoderMaskedMhaImpl, {7, 8});
  r.RegisterFn(MS, "DecoderMaskedSelfAttention", 1, kMax, DecoderMaskedSelfImpl, {6, 7});
  r.RegisterFn(MS, "LongformerAttention", 1, kMax, LongformerImpl);
  r.RegisterFn(MS, "GatedRelativePositionBias", 1, kMax, GatedRelPosBiasImpl);
  r.RegisterFn(MS, "MRotaryEmbedding", 1, kMax, MRotaryImpl);
  RegisterContribKernels4Linear(r);
}

}  // namespace ortb
