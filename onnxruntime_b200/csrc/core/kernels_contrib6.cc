// com.microsoft AttnLSTM: a one-layer LSTM whose cell is wrapped by a Bahdanau attention over a memory tensor
// (reference: onnxruntime/contrib_ops/cpu/attnlstm/deep_cpu_attn_lstm.cc, bahdanau_attention.cc, attention_wrapper.cc;
// semantics as documented in docs/ContribOperators.md).  Per time step and direction:
//   gates  = concat(X_t, ATTN_{t-1}) W^T + H_{t-1} R^T + Wb + Rb            (gate order i, o, f, c; peepholes P[iof])
//   C_t    = f (.) C_{t-1} + i (.) g(c),   H_t = o (.) h(C_t)
//   ALIGN  = softmax over memory steps of sum(V (.) tanh(M MW + H_t QW)),   CONTEXT = ALIGN . M (memory masked by its lengths)
//   ATTN_t = concat(H_t, CONTEXT) AW   (or CONTEXT when AW is absent)
// Default activations only (sigmoid, tanh, tanh); runs on whatever device the inputs live on.
#include <ATen/ATen.h>

#include <limits>

#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

void AttnLstmImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  ORTB_ENFORCE(!n.has_attr("activations") || n.attr_strings("activations").empty() ||
                   [&] {
                     for (size_t i = 0; i < n.attr_strings("activations").size(); ++i) {
                       const std::string a = n.attr_strings("activations")[i];
                       if (a != (i % 3 == 0 ? "Sigmoid" : "Tanh")) return false;
                     }
                     return true;
                   }(),
               "AttnLSTM: only the default activations (Sigmoid, Tanh, Tanh) are supported");
  const at::Tensor& X = ctx.RequiredInput(0);   // [S, B, I]
  const at::Tensor& W = ctx.RequiredInput(1);   // [D, 4H, I + A]
  const at::Tensor& R = ctx.RequiredInput(2);   // [D, 4H, H]
  ORTB_ENFORCE_ARG(ctx.HasInput(8) && ctx.HasInput(9) && ctx.HasInput(10) && ctx.HasInput(11), "AttnLSTM: QW, MW, V and M are required");
  const at::Tensor& QW = ctx.Input(8);          // [D, H, att]
  const at::Tensor& MW = ctx.Input(9);          // [D, mem_depth, att]
  const at::Tensor& V = ctx.Input(10);          // [D, att]
  const at::Tensor& M = ctx.Input(11);          // [B, mem_steps, mem_depth]
  const int64_t S = X.size(0), B = X.size(1), H = R.size(2), D = W.size(0);
  const std::string direction = n.attr_s("direction", "forward");
  ORTB_ENFORCE_ARG(D == (direction == "bidirectional" ? 2 : 1), "AttnLSTM: W has ", D, " directions for direction '", direction, "'");
  const float clip = n.has_attr("clip") ? n.attr_f("clip", 0.f) : 0.f;
  const bool input_forget = n.attr_i("input_forget", 0) != 0;
  at::Tensor lens = ctx.HasInput(4) ? ctx.Input(4).to(X.device(), at::kLong) : at::full({B}, S, at::TensorOptions().dtype(at::kLong).device(X.device()));
  at::Tensor values = M;
  at::Tensor mem_mask;  // [B, steps] true inside the memory
  if (ctx.HasInput(12)) {
    at::Tensor mlens = ctx.Input(12).to(X.device(), at::kLong);
    mem_mask = at::arange(M.size(1), mlens.options()).unsqueeze(0).lt(mlens.unsqueeze(1));
    values = M * mem_mask.unsqueeze(-1).to(M.scalar_type());
  }
  std::vector<at::Tensor> ys, yh, yc;
  for (int64_t d = 0; d < D; ++d) {
    const bool reverse = direction == "reverse" || d == 1;
    at::Tensor Wd = W[d], Rd = R[d];
    at::Tensor bias = ctx.HasInput(3) ? ctx.Input(3)[d].narrow(0, 0, 4 * H) + ctx.Input(3)[d].narrow(0, 4 * H, 4 * H) : at::zeros({4 * H}, X.options());
    at::Tensor Pi, Po, Pf;
    if (ctx.HasInput(7)) {
      Pi = ctx.Input(7)[d].narrow(0, 0, H);
      Po = ctx.Input(7)[d].narrow(0, H, H);
      Pf = ctx.Input(7)[d].narrow(0, 2 * H, H);
    }
    at::Tensor keys = at::matmul(values, MW[d]);  // [B, steps, att]
    const int64_t attn_size = ctx.HasInput(13) ? ctx.Input(13).size(2) : M.size(2);
    ORTB_ENFORCE_ARG(Wd.size(1) == X.size(2) + attn_size, "AttnLSTM: W's input size must be input_size + attention size (", X.size(2), " + ", attn_size, ")");
    at::Tensor h = ctx.HasInput(5) ? ctx.Input(5)[d] : at::zeros({B, H}, X.options());
    at::Tensor c = ctx.HasInput(6) ? ctx.Input(6)[d] : at::zeros({B, H}, X.options());
    at::Tensor attn = at::zeros({B, attn_size}, X.options());
    std::vector<at::Tensor> out(static_cast<size_t>(S));
    for (int64_t step = 0; step < S; ++step) {
      // a reversed direction walks every sequence from its own last valid step backwards
      at::Tensor t_idx = reverse ? at::clamp_min(lens - 1 - step, 0) : at::full({B}, step, lens.options());
      at::Tensor valid = (reverse ? lens.gt(step) : lens.gt(step)).unsqueeze(1);  // [B, 1]
      at::Tensor xt = X.permute({1, 0, 2}).gather(1, t_idx.reshape({B, 1, 1}).expand({B, 1, X.size(2)})).squeeze(1);
      at::Tensor gates = at::matmul(at::cat({xt, attn}, 1), Wd.t()) + at::matmul(h, Rd.t()) + bias;
      if (clip > 0) gates = at::clamp(gates, -clip, clip);
      at::Tensor gi = gates.narrow(1, 0, H), go = gates.narrow(1, H, H), gf = gates.narrow(1, 2 * H, H), gc = gates.narrow(1, 3 * H, H);
      if (Pi.defined()) {
        gi = gi + Pi * c;
        gf = gf + Pf * c;
      }
      at::Tensor it = at::sigmoid(gi);
      at::Tensor ft = input_forget ? 1 - it : at::sigmoid(gf);
      at::Tensor c_new = ft * c + it * at::tanh(gc);
      if (Po.defined()) go = go + Po * c_new;
      at::Tensor h_new = at::sigmoid(go) * at::tanh(c_new);
      // attention on the new hidden state
      at::Tensor pq = at::matmul(h_new, QW[d]).unsqueeze(1);                              // [B, 1, att]
      at::Tensor score = (at::tanh(keys + pq) * V[d]).sum(-1);                            // [B, steps]
      if (mem_mask.defined()) score = score.masked_fill(mem_mask.logical_not(), -std::numeric_limits<float>::infinity());
      at::Tensor align = at::softmax(score, -1);
      at::Tensor context = at::matmul(align.unsqueeze(1), values).squeeze(1);             // [B, mem_depth]
      at::Tensor attn_new = ctx.HasInput(13) ? at::matmul(at::cat({h_new, context}, 1), ctx.Input(13)[d]) : context;
      h = at::where(valid, h_new, h);
      c = at::where(valid, c_new, c);
      attn = at::where(valid, attn_new, attn);
      // outputs beyond a sequence's length are zero; a reversed direction writes to the step it read
      at::Tensor y = at::where(valid, h_new, at::zeros_like(h_new));
      if (!reverse) {
        out[static_cast<size_t>(step)] = y;
      } else {
        if (step == 0)
          for (auto& o : out) o = at::zeros({B, H}, X.options());
        for (int64_t b = 0; b < B; ++b) {
          const int64_t pos = t_idx[b].item<int64_t>();
          if (valid[b][0].item<bool>()) out[static_cast<size_t>(pos)][b] = y[b];
        }
      }
    }
    ys.push_back(at::stack(out, 0));  // [S, B, H]
    yh.push_back(h);
    yc.push_back(c);
  }
  ctx.SetOutput(0, at::stack(ys, 1));  // [S, D, B, H]
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, at::stack(yh, 0));
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, at::stack(yc, 0));
}

}  // namespace

void RegisterContribKernels6(KernelRegistry& r) { r.RegisterFn("com.microsoft", "AttnLSTM", 1, kMax, AttnLstmImpl, {4, 12}); }

}  // namespace ortb
