// GPU op wrappers, part 2: normalisation, rotary embedding, GroupQueryAttention,
// embedding gather, arg-max, bias/activation, and the row-parallel all-reduce.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>

#include <cmath>

#include "collective.h"
#include "contrib_math.h"
#include "cuda_ops.h"
#include "ortb200_kernels.h"
#include "session.h"

namespace ortb {

at::Tensor GemmAllReduce(OpKernelContext& ctx, const at::Tensor& partial, const at::Tensor& residual) {
  at::Tensor y = AllReduceSum(ctx.session(), partial);
  if (residual.defined()) y = y + residual;
  return y;
}

namespace {

using Ctx = OpKernelContext;
constexpr const char* MS = kMSDomain;

int DtypeCode(at::ScalarType t) {
  if (t == at::kHalf) return ORTB200_F16;
  if (t == at::kBFloat16) return ORTB200_BF16;
  if (t == at::kFloat) return ORTB200_F32;
  return -1;
}
bool HalfType(at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16; }
bool Aligned16(const at::Tensor& t) { return !t.defined() || (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0; }

// Runs the ATen-backed kernel of the same op (used when a shape / attribute is outside what the sm_100a kernel covers).
class WithFallback : public OpKernel {
 public:
  explicit WithFallback(const OpKernelInfo& info) : OpKernel(info) {
    const KernelDef* d = KernelRegistry::Generic().Find(info.node, info.graph);
    if (d) fallback_ = d->factory(info);
  }

 protected:
  void Fallback(Ctx& ctx) const {
    if (!fallback_) ORTB_THROW(NOT_IMPLEMENTED, "no fallback kernel for ", node_.op_type);
    fallback_->Compute(ctx);
  }
  std::unique_ptr<OpKernel> fallback_;
};

// LayerNormalization / SimplifiedLayerNormalization / RMSNormalization / Skip* variants.
class NormKernel final : public WithFallback {
 public:
  explicit NormKernel(const OpKernelInfo& info) : WithFallback(info) {
    const std::string& op = info.node.op_type;
    skip_ = op.rfind("Skip", 0) == 0;
    simplified_ = op.find("Simplified") != std::string::npos || op == "RMSNormalization";
    eps_ = info.node.attr_f("epsilon", 1e-5f);
    axis_ = info.node.attr_i("axis", -1);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int gi = skip_ ? 2 : 1;
    const at::Tensor& gamma = ctx.RequiredInput(gi);
    const int beta_idx = simplified_ ? -1 : gi + 1;
    const int bias_idx = skip_ ? (simplified_ ? 3 : 4) : -1;
    at::Tensor beta = beta_idx >= 0 && ctx.HasInput(beta_idx) ? ctx.Input(beta_idx) : at::Tensor();
    at::Tensor bias = bias_idx >= 0 && ctx.HasInput(bias_idx) ? ctx.Input(bias_idx) : at::Tensor();
    at::Tensor skip = skip_ ? ctx.RequiredInput(1) : at::Tensor();
    const int64_t H = x.size(-1);
    const int dt = DtypeCode(x.scalar_type());
    const bool last_axis = axis_ == -1 || axis_ == x.dim() - 1;
    const bool extra_outputs = (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) || (ctx.OutputCount() > 2 && ctx.OutputNeeded(2));
    const int64_t esz = static_cast<int64_t>(x.element_size());
    if (dt < 0 || !last_axis || extra_outputs || gamma.scalar_type() != x.scalar_type() || (H * esz) % 16 != 0 ||
        H * esz > 16 * 256 * 16 || (skip.defined() && skip.sizes() != x.sizes()) || gamma.numel() != H ||
        (beta.defined() && beta.scalar_type() != x.scalar_type()) || (bias.defined() && bias.scalar_type() != x.scalar_type())) {
      Fallback(ctx);
      return;
    }
    at::Tensor xc = x.contiguous(), sc = skip.defined() ? skip.contiguous() : skip;
    at::Tensor out = at::empty_like(xc);
    const bool want_sum = skip_ && ctx.OutputCount() > 3 && ctx.OutputNeeded(3);
    at::Tensor sum = want_sum ? at::empty_like(xc) : at::Tensor();
    if (!Aligned16(xc) || !Aligned16(sc) || !Aligned16(gamma) || !Aligned16(beta) || !Aligned16(bias)) {
      Fallback(ctx);
      return;
    }
    ortb200_norm_args a{};
    a.x = xc.data_ptr();
    a.skip = sc.defined() ? sc.data_ptr() : nullptr;
    a.bias = bias.defined() ? bias.data_ptr() : nullptr;
    a.gamma = gamma.data_ptr();
    a.beta = beta.defined() ? beta.data_ptr() : nullptr;
    a.out = out.data_ptr();
    a.sum_out = want_sum ? sum.data_ptr() : nullptr;
    a.rows = xc.numel() / H;
    a.hidden = static_cast<int>(H);
    a.epsilon = eps_;
    a.simplified = simplified_ ? 1 : 0;
    a.dtype = dt;
    CheckLaunch(ortb200_norm(&a, ctx.cuda_stream()), "ortb200_norm");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
    if (want_sum) ctx.SetOutput(3, sum);
  }

 private:
  bool skip_ = false, simplified_ = false;
  float eps_ = 1e-5f;
  int64_t axis_ = -1;
};

// Gather(axis=0) from a constant 2-D table (token embedding).
class EmbeddingGatherKernel final : public WithFallback {
 public:
  explicit EmbeddingGatherKernel(const OpKernelInfo& info) : WithFallback(info) {}
  void Compute(Ctx& ctx) const override {
    const at::Tensor& table = ctx.RequiredInput(0);
    const at::Tensor& ids = ctx.RequiredInput(1);
    const int64_t row_bytes = table.dim() == 2 ? table.size(1) * static_cast<int64_t>(table.element_size()) : 0;
    if (table.dim() != 2 || ids.scalar_type() != at::kLong || !ids.is_cuda() || row_bytes % 16 != 0 || !table.is_contiguous() ||
        !Aligned16(table) || node_.attr_i("axis", 0) != 0) {
      Fallback(ctx);
      return;
    }
    at::Tensor idc = ids.contiguous();
    std::vector<int64_t> shape = ids.sizes().vec();
    shape.push_back(table.size(1));
    at::Tensor out = at::empty(shape, table.options());
    CheckLaunch(ortb200_gather_rows(table.data_ptr(), idc.data_ptr<int64_t>(), out.data_ptr(), idc.numel(), table.size(0),
                                    static_cast<int>(table.size(1)), static_cast<int>(table.element_size()), ctx.cuda_stream()),
                "ortb200_gather_rows");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
  }
};

class ArgMaxKernel final : public WithFallback {
  mutable at::Tensor ws_;  // per-row merge slots + counters, kept zero between launches

 public:
  explicit ArgMaxKernel(const OpKernelInfo& info) : WithFallback(info) {}
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t axis = node_.attr_i("axis", 0);
    if (axis < 0) axis += x.dim();
    const int dt = DtypeCode(x.scalar_type());
    if (dt < 0 || axis != x.dim() - 1 || node_.attr_i("select_last_index", 0) != 0 || x.numel() == 0) {
      Fallback(ctx);
      return;
    }
    at::Tensor xc = x.contiguous();
    std::vector<int64_t> shape = x.sizes().vec();
    if (node_.attr_i("keepdims", 1)) shape.back() = 1;
    else shape.pop_back();
    at::Tensor out = at::empty(shape, x.options().dtype(at::kLong));
    const int64_t rows = xc.numel() / x.size(-1);
    if (!ws_.defined() || ws_.numel() < rows * 16 || ws_.device() != x.device())
      ws_ = at::zeros({std::max<int64_t>(rows, 64) * 16}, x.options().dtype(at::kByte));
    CheckLaunch(ortb200_argmax(xc.data_ptr(), out.data_ptr<int64_t>(), rows, x.size(-1), dt, ws_.data_ptr(), ws_.numel(),
                               ctx.cuda_stream()),
                "ortb200_argmax");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
  }
};

// FastGelu / BiasGelu / Gelu / QuickGelu / Relu-like activations with an optional 1-D bias.
class BiasActKernel final : public WithFallback {
 public:
  explicit BiasActKernel(const OpKernelInfo& info) : WithFallback(info) {
    const std::string& op = info.node.op_type;
    if (op == "FastGelu") act_ = ORTB200_ACT_FASTGELU;
    else if (op == "BiasGelu") act_ = ORTB200_ACT_GELU;
    else if (op == "Gelu") act_ = (info.node.domain.empty() && info.node.attr_s("approximate", "none") == "tanh") ? ORTB200_ACT_FASTGELU : ORTB200_ACT_GELU;
    else if (op == "QuickGelu") { act_ = ORTB200_ACT_QUICKGELU; alpha_ = info.node.attr_f("alpha", 1.702f); }
    else if (op == "Relu") act_ = ORTB200_ACT_RELU;
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor bias = ctx.HasInput(1) ? ctx.Input(1) : at::Tensor();
    const int dt = DtypeCode(x.scalar_type());
    if (dt < 0 || x.numel() == 0 || (bias.defined() && (bias.dim() != 1 || bias.numel() != x.size(-1) || bias.scalar_type() != x.scalar_type()))) {
      Fallback(ctx);
      return;
    }
    at::Tensor xc = x.contiguous();
    at::Tensor out = at::empty_like(xc);
    CheckLaunch(ortb200_bias_act(xc.data_ptr(), bias.defined() ? bias.data_ptr() : nullptr, out.data_ptr(), xc.numel() / x.size(-1),
                                 static_cast<int>(x.size(-1)), act_, alpha_, dt, ctx.cuda_stream()),
                "ortb200_bias_act");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
  }

 private:
  int act_ = ORTB200_ACT_NONE;
  float alpha_ = 1.702f;
};

// com.microsoft.RotaryEmbedding
class RotaryKernel final : public WithFallback {
 public:
  explicit RotaryKernel(const OpKernelInfo& info) : WithFallback(info) {}
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const at::Tensor& pos = ctx.RequiredInput(1);
    const at::Tensor& cos = ctx.RequiredInput(2);
    const at::Tensor& sin = ctx.RequiredInput(3);
    const int dt = DtypeCode(x.scalar_type());
    int64_t N = node_.attr_i("num_heads", 0);
    const int64_t rot = node_.attr_i("rotary_embedding_dim", 0);
    const bool bnsh = x.dim() == 4;
    if (dt < 0 || cos.scalar_type() != x.scalar_type() || node_.attr_f("scale", 1.f) != 1.f || node_.attr_i("is_packed_batching", 0) ||
        pos.scalar_type() != at::kLong || (!bnsh && rot > 0 && N == 0)) {
      Fallback(ctx);
      return;
    }
    int64_t B = x.size(0), S, H;
    if (bnsh) {
      N = x.size(1);
      S = x.size(2);
      H = x.size(3);
    } else {
      S = x.size(1);
      H = N > 0 ? x.size(2) / N : cos.size(1) * 2;
      if (N == 0) N = x.size(2) / H;
    }
    at::Tensor xc = x.contiguous();
    at::Tensor out = at::empty_like(xc);
    const int64_t* pid = nullptr;
    int64_t offset = 0;
    at::Tensor pc;
    if (pos.numel() == 1) {
      offset = pos.cpu().item<int64_t>();
    } else {
      pc = pos.to(x.device()).contiguous();
      pid = pc.data_ptr<int64_t>();
    }
    CheckLaunch(ortb200_rotary(xc.data_ptr(), out.data_ptr(), pid, offset, cos.data_ptr(), sin.data_ptr(), static_cast<int>(B),
                               static_cast<int>(S), static_cast<int>(N), static_cast<int>(H), static_cast<int>(rot),
                               node_.attr_i("interleaved", 0) != 0, bnsh ? 1 : 0, dt, ctx.cuda_stream()),
                "ortb200_rotary");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
  }
};

// com.microsoft.GroupQueryAttention
class GqaKernel final : public WithFallback {
 public:
  explicit GqaKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    N_ = n.attr_i("num_heads", 0);
    Nk_ = n.attr_i("kv_num_heads", 0);
    do_rotary_ = n.attr_i("do_rotary", 0) != 0;
    interleaved_ = n.attr_i("rotary_interleaved", 0) != 0;
    window_ = n.attr_i("local_window_size", -1);
    scale_ = n.attr_f("scale", 0.f);
    softcap_ = n.attr_f("softcap", 0.f);
    smooth_ = n.attr_i("smooth_softmax", 0) != 0;
    // the node that consumes the attention output (the output projection): with ortb200.attention_prefetch=1 its weights
    // are requested into the L2 while the decode kernel runs (off by default: measured 0.1 ms per step slower)
    if (!n.outputs.empty() && !n.outputs[0].empty()) {
      for (const auto& other : info.graph.Nodes()) {
        if (!other->inputs.empty() && other->inputs[0] == n.outputs[0]) {
          consumer_ = other->name;
          break;
        }
      }
    }
  }

  void Compute(Ctx& ctx) const override {
    const at::Tensor& query = ctx.RequiredInput(0);
    const bool packed = !ctx.HasInput(1);
    const int64_t B = query.size(0), S = query.size(1);
    const int64_t H = packed ? query.size(2) / (N_ + 2 * Nk_) : query.size(2) / N_;
    const int dt = DtypeCode(query.scalar_type());
    if (S > 1 && ctx.session()->config().Get("ortb200.math_attention", "0") == "1") {
      Fallback(ctx);  // fused attention kernels switched off (sdpa_kernel = MATH / ORT_DISABLE_FLASH_ATTENTION)
      return;
    }
    const at::Tensor& seqlens = ctx.RequiredInput(5);
    const int64_t total = ctx.RequiredInput(6).cpu().to(at::kLong).reshape({-1})[0].item<int64_t>();
    const bool has_past = ctx.HasInput(3) && ctx.HasInput(4);
    const bool unsupported = !HalfType(query.scalar_type()) || (H != 64 && H != 128) || ctx.HasInput(10) || ctx.HasInput(12) ||
                             ctx.HasInput(13) || ctx.HasInput(14) || ctx.HasInput(15) || smooth_ || seqlens.scalar_type() != at::kInt ||
                             (ctx.OutputCount() > 3 && ctx.OutputNeeded(3)) || (has_past && ctx.Input(3).scalar_type() != query.scalar_type()) ||
                             (do_rotary_ && (!ctx.HasInput(7) || ctx.Input(7).scalar_type() != query.scalar_type()));
    const bool first_prompt = (S == total);
    if (unsupported || (!first_prompt && !has_past)) {
      Fallback(ctx);
      return;
    }
    // present cache: reuse the past buffers when they have room (shared-buffer mode), else allocate
    at::Tensor kc, vc;
    if (has_past && ctx.Input(3).size(2) >= total && ctx.Input(3).is_contiguous() && ctx.Input(4).is_contiguous()) {
      kc = ctx.Input(3);
      vc = ctx.Input(4);
    } else if (first_prompt) {
      kc = at::zeros({B, Nk_, total, H}, query.options());
      vc = at::zeros({B, Nk_, total, H}, query.options());
    } else {
      Fallback(ctx);  // a past that must grow: the reference copies into a larger buffer
      return;
    }
    const int64_t Smax = kc.size(2);
    at::Tensor qc = query.contiguous();
    at::Tensor q_rot = at::empty({B, S, N_, H}, query.options());
    at::Tensor sl = seqlens.to(query.device()).contiguous();
    at::Tensor pos_ids;
    if (ctx.HasInput(9)) pos_ids = ctx.Input(9).to(query.device(), at::kLong).contiguous();

    // one-token steps: the tcgen05 decode kernel (head size 128) unpacks, rotates and appends by itself - one launch
    // fewer and no round trip of the rotated query (3.63 -> 3.56 ms per step on Llama-3-8B at batch 8).  The CUDA-core
    // kernel (head size 64) can do the same but was measured slower that way, so there it needs ortb200.fused_gqa_prep=1;
    // "0" switches the fusion off everywhere.
    const std::string fuse_cfg = ctx.session()->config().Get("ortb200.fused_gqa_prep", "auto");
    const bool tc_kernel = H == 128 && ctx.session()->config().Get("ortb200.decode_attention_algo", "0") != "1";
    const bool fuse_prep = S == 1 && !first_prompt && packed && !pos_ids.defined() &&
                           (!do_rotary_ || ctx.Input(7).size(1) * 2 == H) && (fuse_cfg == "1" || (fuse_cfg != "0" && tc_kernel));
    if (!fuse_prep) {
      ortb200_gqa_prep_args pa{};
      pa.qkv = qc.data_ptr();
      at::Tensor kin, vin;
      if (!packed) {
        kin = ctx.Input(1).contiguous();
        vin = ctx.RequiredInput(2).contiguous();
        pa.k = kin.data_ptr();
        pa.v = vin.data_ptr();
      }
      pa.q_out = q_rot.data_ptr();
      pa.k_cache = kc.data_ptr();
      pa.v_cache = vc.data_ptr();
      pa.seqlens_k = sl.data_ptr<int>();
      pa.cos_cache = do_rotary_ ? ctx.Input(7).data_ptr() : nullptr;
      pa.sin_cache = do_rotary_ ? ctx.RequiredInput(8).data_ptr() : nullptr;
      pa.position_ids = pos_ids.defined() ? pos_ids.data_ptr<int64_t>() : nullptr;
      pa.B = static_cast<int>(B); pa.S = static_cast<int>(S); pa.N = static_cast<int>(N_); pa.Nk = static_cast<int>(Nk_);
      pa.H = static_cast<int>(H); pa.Smax = static_cast<int>(Smax);
      pa.rot_dim = do_rotary_ ? static_cast<int>(ctx.Input(7).size(1) * 2) : 0;
      pa.cos_rows = do_rotary_ ? static_cast<int>(ctx.Input(7).size(0)) : 0;
      pa.interleaved = interleaved_ ? 1 : 0;
      pa.first_prompt = first_prompt ? 1 : 0;
      pa.do_rotary = do_rotary_ ? 1 : 0;
      pa.dtype = dt;
      pa.use_pdl = ctx.session()->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
      CheckLaunch(ortb200_gqa_prep(&pa, ctx.cuda_stream()), "ortb200_gqa_prep");
      ctx.session()->AddLaunches(1);
    }

    at::Tensor out;
    if (S == 1) {
      out = at::empty({B, 1, N_ * H}, query.options());
      at::Tensor& ws = ctx.session()->AttnWorkspace(ortb200_gqa_decode_workspace_bytes(static_cast<int>(B), static_cast<int>(N_), static_cast<int>(H)));
      ortb200_gqa_decode_args da{};
      da.q = q_rot.data_ptr();
      if (fuse_prep) {
        da.qkv = qc.data_ptr();
        da.cos_cache = do_rotary_ ? ctx.Input(7).data_ptr() : nullptr;
        da.sin_cache = do_rotary_ ? ctx.RequiredInput(8).data_ptr() : nullptr;
        da.do_rotary = do_rotary_ ? 1 : 0;
        da.rotary_interleaved = interleaved_ ? 1 : 0;
        da.cos_rows = do_rotary_ ? static_cast<int>(ctx.Input(7).size(0)) : 0;
      }
      da.k_cache = kc.data_ptr();
      da.v_cache = vc.data_ptr();
      da.seqlens_k = sl.data_ptr<int>();
      da.head_sink = ctx.HasInput(11) ? ctx.Input(11).data_ptr() : nullptr;
      da.out = out.data_ptr();
      da.workspace = ws.data_ptr();
      da.workspace_bytes = ws.numel();
      da.B = static_cast<int>(B); da.N = static_cast<int>(N_); da.Nk = static_cast<int>(Nk_); da.H = static_cast<int>(H);
      da.Smax = static_cast<int>(Smax);
      da.splits = 0;
      da.window = static_cast<int>(window_);
      da.scale = scale_;
      da.softcap = softcap_;
      da.dtype = dt;
      da.use_pdl = ctx.session()->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
      da.status = ctx.session()->StatusWord().data_ptr<int>();
      // "0" picks (the tcgen05 kernel where it applies), "1" forces the CUDA-core split-KV kernel
      da.algo = ctx.session()->config().Get("ortb200.decode_attention_algo", "0") == "1" ? 1 : 0;
      if (!consumer_.empty() && ctx.session()->config().Get("ortb200.attention_prefetch", "0") == "1") {
        const auto hint = ctx.session()->FindWeightHint(consumer_);
        da.prefetch = hint.first;
        da.prefetch_bytes = hint.second;
      }
      CheckLaunch(ortb200_gqa_decode(&da, ctx.cuda_stream()), "ortb200_gqa_decode");
      ctx.session()->AddLaunches(1);
    } else {
      out = PrefillAttention(ctx, q_rot, kc, vc, sl, first_prompt, B, S, H, total, dt).reshape({B, S, N_ * H});
    }
    ctx.SetOutput(0, out);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, kc);
    if (ctx.OutputCount() > 2) ctx.SetOutput(2, vc);
  }

 private:
  std::string consumer_;
  // q_rot [B,S,N,H]; caches [B,Nk,Smax,H] already hold the new tokens.
  at::Tensor PrefillAttention(Ctx& ctx, const at::Tensor& q_rot, const at::Tensor& kc, const at::Tensor& vc, const at::Tensor& sl,
                              bool first_prompt, int64_t B, int64_t S, int64_t H, int64_t total, int dt) const {
    at::Tensor out = at::empty({B, S, N_, H}, q_rot.options());
    ortb200_attn_prefill_args a{};
    a.q = q_rot.data_ptr();
    a.k = kc.data_ptr();
    a.v = vc.data_ptr();
    a.seqlens_k = sl.data_ptr<int>();
    a.head_sink = ctx.HasInput(11) ? ctx.Input(11).data_ptr() : nullptr;
    a.out = out.data_ptr();
    a.B = static_cast<int>(B); a.S = static_cast<int>(S); a.N = static_cast<int>(N_); a.Nk = static_cast<int>(Nk_);
    a.H = static_cast<int>(H);
    a.kv_len = static_cast<int>(kc.size(2));
    a.q_strides[0] = S * N_ * H; a.q_strides[1] = N_ * H; a.q_strides[2] = H;
    a.o_strides[0] = S * N_ * H; a.o_strides[1] = N_ * H; a.o_strides[2] = H;
    a.kv_strides[0] = kc.stride(0); a.kv_strides[1] = kc.stride(1); a.kv_strides[2] = kc.stride(2);
    a.first_prompt = first_prompt ? 1 : 0;
    a.causal = 1;
    a.window = static_cast<int>(window_);
    a.scale = scale_;
    a.softcap = softcap_;
    a.dtype = dt;
    a.status = ctx.session()->StatusWord().data_ptr<int>();
    (void)total;
    CheckLaunch(ortb200_attn_prefill(&a, ctx.cuda_stream()), "ortb200_attn_prefill");
    ctx.session()->AddLaunches(1);
    return out;
  }

  int64_t N_ = 0, Nk_ = 0, window_ = -1;
  bool do_rotary_ = false, interleaved_ = false, smooth_ = false;
  float scale_ = 0.f, softcap_ = 0.f;
};

template <typename K>
void Reg(KernelRegistry& r, const std::string& domain, const std::string& op, std::vector<int> host = {},
         std::function<bool(const Node&, const Graph&)> supports = nullptr) {
  KernelDef d;
  d.domain = domain;
  d.op_type = op;
  d.host_inputs = std::move(host);
  d.supports = std::move(supports);
  d.factory = [](const OpKernelInfo& info) { return std::make_unique<K>(info); };
  r.Register(std::move(d));
}

}  // namespace

void RegisterMoreCudaKernels(KernelRegistry& r) {
  Reg<NormKernel>(r, "", "LayerNormalization");
  Reg<NormKernel>(r, "", "SimplifiedLayerNormalization");
  Reg<NormKernel>(r, "", "RMSNormalization");
  Reg<NormKernel>(r, MS, "SkipLayerNormalization");
  Reg<NormKernel>(r, MS, "SkipSimplifiedLayerNormalization");
  Reg<EmbeddingGatherKernel>(r, "", "Gather", {}, [](const Node& n, const Graph& g) {
    const at::Tensor* t = g.GetConstant(n.input(0));
    return t != nullptr && t->dim() == 2 && n.attr_i("axis", 0) == 0;
  });
  Reg<ArgMaxKernel>(r, "", "ArgMax");
  Reg<BiasActKernel>(r, MS, "FastGelu");
  Reg<BiasActKernel>(r, MS, "BiasGelu");
  Reg<BiasActKernel>(r, MS, "Gelu");
  Reg<BiasActKernel>(r, MS, "QuickGelu");
  Reg<BiasActKernel>(r, "", "Gelu");
  Reg<RotaryKernel>(r, MS, "RotaryEmbedding");
  Reg<GqaKernel>(r, MS, "GroupQueryAttention", {6});
}

}  // namespace ortb
