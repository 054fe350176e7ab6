// GPU op wrappers, part 3: MatMulNBits, PagedAttention, BERT Attention / MultiHeadAttention.
//
// Reference counterparts: onnxruntime/contrib_ops/cuda/quantization/matmul_nbits.cc,
// contrib_ops/cuda/bert/paged_attention.cc, bert/attention.cc and bert/multihead_attention.cc.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>

#include <cmath>

#include "cuda_ops.h"
#include "ortb200_kernels.h"
#include "session.h"

namespace ortb {
namespace {

using Ctx = OpKernelContext;
constexpr const char* MS = kMSDomain;

int DtypeCode(at::ScalarType t) {
  if (t == at::kHalf) return ORTB200_F16;
  if (t == at::kBFloat16) return ORTB200_BF16;
  return -1;
}
bool HalfType(at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16; }

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

// ---------------------------------------------------------------------------------------------------------------
// MatMulNBits: the packed weights stay packed in device memory; each call expands them to [N, K] rows with the
// dequantisation kernel and runs the tcgen05 GEMM on the result (bias in the GEMM epilogue).
class MatMulNBitsKernel final : public WithFallback {
 public:
  explicit MatMulNBitsKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    K_ = n.attr_i("K", 0);
    N_ = n.attr_i("N", 0);
    bits_ = n.attr_i("bits", 4);
    block_ = n.attr_i("block_size", 32);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& a = ctx.RequiredInput(0);
    const at::Tensor& B = ctx.RequiredInput(1);
    const at::Tensor& scales = ctx.RequiredInput(2);
    at::Tensor zp = ctx.HasInput(3) ? ctx.Input(3) : at::Tensor();
    const int dt = DtypeCode(a.scalar_type());
    const bool zp_packed = zp.defined() && zp.scalar_type() == at::kByte;
    if (dt < 0 || scales.scalar_type() != a.scalar_type() || (bits_ != 4 && bits_ != 8) || block_ < 16 ||
        (block_ & (block_ - 1)) != 0 || K_ % 8 != 0 || ctx.HasInput(4) || !B.is_cuda() ||
        (zp.defined() && !zp_packed && zp.scalar_type() != a.scalar_type())) {
      Fallback(ctx);
      return;
    }
    at::Tensor Bc = B.contiguous(), sc = scales.contiguous();
    if (zp.defined()) zp = zp.contiguous();
    at::Tensor w = at::empty({N_, K_}, a.options());
    CheckLaunch(ortb200_nbits_dequant(Bc.data_ptr(), sc.data_ptr(), zp.defined() ? zp.data_ptr() : nullptr, zp_packed ? 1 : 0,
                                      w.data_ptr(), N_, static_cast<int>(K_), static_cast<int>(bits_), static_cast<int>(block_), K_,
                                      dt, ctx.cuda_stream()),
                "ortb200_nbits_dequant");
    ctx.session()->AddLaunches(1);
    at::Tensor x2 = a.reshape({-1, K_}).contiguous();
    at::Tensor bias = ctx.HasInput(5) ? ctx.Input(5) : at::Tensor();
    at::Tensor y = LaunchGemm(ctx, x2, w, N_, 0, bias, at::Tensor(), ORTB200_ACT_NONE, 1.f);
    std::vector<int64_t> shape = a.sizes().vec();
    shape.back() = N_;
    ctx.SetOutput(0, y.reshape(shape));
  }

 private:
  int64_t K_ = 0, N_ = 0, bits_ = 4, block_ = 32;
};

// ---------------------------------------------------------------------------------------------------------------
// PagedAttention, decode form (one new token per sequence): rotary + cache write, then the split-KV kernel reading
// the cache through the block table.  Other forms (prompt chunks) take the generic path.
class PagedAttentionKernel final : public WithFallback {
 public:
  explicit PagedAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    N_ = n.attr_i("num_heads", 0);
    Nk_ = n.attr_i("kv_num_heads", 0);
    do_rotary_ = n.attr_i("do_rotary", 0) != 0;
    interleaved_ = n.attr_i("rotary_interleaved", 0) != 0;
    window_ = n.attr_i("local_window_size", -1);
    scale_ = n.attr_f("scale", 0.f);
    softcap_ = n.attr_f("softcap", 0.f);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& query = ctx.RequiredInput(0);
    const at::Tensor& kc = ctx.RequiredInput(3);
    const at::Tensor& vc = ctx.RequiredInput(4);
    const at::Tensor& cum = ctx.RequiredInput(5);
    const at::Tensor& past = ctx.RequiredInput(6);
    const at::Tensor& table = ctx.RequiredInput(7);
    const int64_t T = query.size(0), B = past.numel();
    const int64_t H = kc.size(3), block_size = kc.size(1), num_blocks = kc.size(0);
    const bool packed = !ctx.HasInput(1);
    const int dt = DtypeCode(query.scalar_type());
    const bool decode = T == B;
    if (dt < 0 || !decode || (H != 64 && H != 128) || kc.scalar_type() != query.scalar_type() || !kc.is_contiguous() ||
        !vc.is_contiguous() || !cum.is_cuda() || !past.is_cuda() || !table.is_cuda() || cum.scalar_type() != at::kInt ||
        past.scalar_type() != at::kInt || table.scalar_type() != at::kInt ||
        (do_rotary_ && (!ctx.HasInput(8) || ctx.Input(8).scalar_type() != query.scalar_type()))) {
      Fallback(ctx);
      return;
    }
    at::Tensor qc = query.contiguous();
    at::Tensor q_rot = at::empty({T, N_, H}, query.options());
    at::Tensor tb = table.contiguous();
    ortb200_paged_prep_args pa{};
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
    pa.cu_seqlens = cum.data_ptr<int>();
    pa.past_seqlens = past.data_ptr<int>();
    pa.block_table = tb.data_ptr<int>();
    pa.cos_cache = do_rotary_ ? ctx.Input(8).data_ptr() : nullptr;
    pa.sin_cache = do_rotary_ ? ctx.RequiredInput(9).data_ptr() : nullptr;
    pa.T = static_cast<int>(T); pa.B = static_cast<int>(B); pa.N = static_cast<int>(N_); pa.Nk = static_cast<int>(Nk_);
    pa.H = static_cast<int>(H);
    pa.block_size = static_cast<int>(block_size); pa.max_blocks = static_cast<int>(tb.size(1)); pa.num_blocks = static_cast<int>(num_blocks);
    pa.rot_dim = do_rotary_ ? static_cast<int>(ctx.Input(8).size(1) * 2) : 0;
    pa.interleaved = interleaved_ ? 1 : 0;
    pa.do_rotary = do_rotary_ ? 1 : 0;
    pa.dtype = dt;
    pa.status = ctx.session()->StatusWord().data_ptr<int>();
    CheckLaunch(ortb200_paged_prep(&pa, ctx.cuda_stream()), "ortb200_paged_prep");

    at::Tensor out = at::empty({T, N_ * H}, query.options());
    at::Tensor& ws = ctx.session()->AttnWorkspace(ortb200_gqa_decode_workspace_bytes(static_cast<int>(B), static_cast<int>(N_), static_cast<int>(H)));
    ortb200_gqa_decode_args da{};
    da.q = q_rot.data_ptr();
    da.k_cache = kc.data_ptr();
    da.v_cache = vc.data_ptr();
    da.seqlens_k = past.data_ptr<int>();  // total length - 1 == past length for a one-token step
    da.out = out.data_ptr();
    da.workspace = ws.data_ptr();
    da.workspace_bytes = ws.numel();
    da.B = static_cast<int>(B); da.N = static_cast<int>(N_); da.Nk = static_cast<int>(Nk_); da.H = static_cast<int>(H);
    da.Smax = static_cast<int>(tb.size(1) * block_size);
    da.window = static_cast<int>(window_);
    da.scale = scale_;
    da.softcap = softcap_;
    da.dtype = dt;
    da.use_pdl = 0;
    da.status = pa.status;
    da.block_table = tb.data_ptr<int>();
    da.block_size = static_cast<int>(block_size);
    da.max_blocks = static_cast<int>(tb.size(1));
    CheckLaunch(ortb200_gqa_decode(&da, ctx.cuda_stream()), "ortb200_gqa_decode(paged)");
    ctx.session()->AddLaunches(2);
    ctx.SetOutput(0, out);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, kc);
    if (ctx.OutputCount() > 2) ctx.SetOutput(2, vc);
  }

 private:
  int64_t N_ = 0, Nk_ = 0, window_ = -1;
  bool do_rotary_ = false, interleaved_ = false;
  float scale_ = 0.f, softcap_ = 0.f;
};

// ---------------------------------------------------------------------------------------------------------------
// Encoder attention on the tcgen05 flash kernel.  q / k / v are views described by strides, so neither the packed
// QKV projection output nor separate Q, K, V activations are transposed or copied.
struct EncoderAttnCall {
  at::Tensor q, k, v;          // any layout reachable as (batch, token, head, dim) with dim contiguous
  int64_t B, S, T, N, H;
  at::Tensor lengths;          // optional int32 [B]: keys [0, len) are valid
  at::Tensor key_mask;         // optional int32 [B, T]
  bool causal;
  float scale;
};

at::Tensor RunEncoderAttention(Ctx& ctx, const EncoderAttnCall& c, int dt) {
  at::Tensor out = at::empty({c.B, c.S, c.N, c.H}, c.q.options());
  ortb200_attn_prefill_args a{};
  a.q = c.q.data_ptr();
  a.k = c.k.data_ptr();
  a.v = c.v.data_ptr();
  at::Tensor lens_m1;
  if (c.lengths.defined()) {
    lens_m1 = (c.lengths.to(at::kInt) - 1).contiguous();
    a.seqlens_k = lens_m1.data_ptr<int>();
  }
  if (c.key_mask.defined()) a.key_mask = c.key_mask.data_ptr<int>();
  a.out = out.data_ptr();
  a.B = static_cast<int>(c.B); a.S = static_cast<int>(c.S); a.N = static_cast<int>(c.N); a.Nk = static_cast<int>(c.N);
  a.H = static_cast<int>(c.H);
  a.kv_len = static_cast<int>(c.T);
  a.q_strides[0] = c.q.stride(0); a.q_strides[1] = c.q.stride(1); a.q_strides[2] = c.q.stride(2);
  a.o_strides[0] = out.stride(0); a.o_strides[1] = out.stride(1); a.o_strides[2] = out.stride(2);
  // keys are addressed as (batch, head, position)
  a.kv_strides[0] = c.k.stride(0); a.kv_strides[1] = c.k.stride(2); a.kv_strides[2] = c.k.stride(1);
  a.first_prompt = 1;
  a.causal = c.causal ? 1 : 0;
  a.window = -1;
  a.scale = c.scale;
  a.dtype = dt;
  a.status = ctx.session()->StatusWord().data_ptr<int>();
  CheckLaunch(ortb200_attn_prefill(&a, ctx.cuda_stream()), "ortb200_attn_prefill(encoder)");
  ctx.session()->AddLaunches(1);
  return out;
}

// true when q, k, v (as [B, tokens, N, H] views) are usable by the kernel: dim contiguous, strides multiples of 8,
// k and v with identical strides (one stride triple describes both)
bool ViewsOk(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  auto ok = [](const at::Tensor& t) {
    if (t.stride(3) != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride(i) % 8 != 0) return false;
    return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  return ok(q) && ok(k) && ok(v) && k.strides() == v.strides();
}

// mask_index -> (lengths | key mask).  Returns false for the forms the kernel does not take.
bool DecodeMask(const at::Tensor& m, int64_t B, int64_t T, at::Tensor* lengths, at::Tensor* key_mask) {
  if (m.dim() == 1 && m.size(0) == B) {
    *lengths = m;
    return true;
  }
  if (m.dim() == 2 && m.size(0) == B && m.size(1) == T) {
    *key_mask = m.ne(0).to(at::kInt).contiguous();
    return true;
  }
  return false;
}

class BertAttentionKernel final : public WithFallback {
 public:
  explicit BertAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    N_ = n.attr_i("num_heads", 1);
    causal_ = n.attr_i("unidirectional", 0) != 0;
    scale_ = n.attr_f("scale", 0.f);
    sizes_ = n.attr_ints("qkv_hidden_sizes");
    const at::Tensor* w = info.constant_input(1);
    if (w && w->dim() == 2 && HalfType(w->scalar_type()) && w->size(0) % 8 == 0) w_nk_ = w->t().contiguous();
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int dt = DtypeCode(x.scalar_type());
    const int64_t B = x.size(0), S = x.size(1);
    const int64_t W3 = w_nk_.defined() ? w_nk_.size(0) : 0;
    const bool equal_sizes = sizes_.empty() || (sizes_.size() == 3 && sizes_[0] == sizes_[1] && sizes_[1] == sizes_[2]);
    const int64_t H = W3 > 0 ? W3 / 3 / N_ : 0;
    at::Tensor lengths, key_mask;
    if (dt < 0 || !w_nk_.defined() || w_nk_.scalar_type() != x.scalar_type() || !equal_sizes || (H != 64 && H != 128) ||
        ctx.HasInput(4) || ctx.HasInput(5) || (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ||
        (ctx.HasInput(3) && !DecodeMask(ctx.Input(3), B, S, &lengths, &key_mask))) {
      Fallback(ctx);
      return;
    }
    at::Tensor bias = ctx.HasInput(2) ? ctx.Input(2) : at::Tensor();
    at::Tensor qkv = LaunchGemm(ctx, x.reshape({B * S, x.size(2)}).contiguous(), w_nk_, W3, 0, bias, at::Tensor(), ORTB200_ACT_NONE, 1.f);
    at::Tensor v5 = qkv.reshape({B, S, 3, N_, H});
    EncoderAttnCall c{v5.select(2, 0), v5.select(2, 1), v5.select(2, 2), B, S, S, N_, H, lengths, key_mask, causal_, scale_};
    ctx.SetOutput(0, RunEncoderAttention(ctx, c, dt).reshape({B, S, N_ * H}));
  }

 private:
  int64_t N_ = 1;
  bool causal_ = false;
  float scale_ = 0.f;
  std::vector<int64_t> sizes_;
  at::Tensor w_nk_;
};

class MultiHeadAttentionKernel final : public WithFallback {
 public:
  explicit MultiHeadAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    N_ = info.node.attr_i("num_heads", 1);
    causal_ = info.node.attr_i("unidirectional", 0) != 0;
    scale_ = info.node.attr_f("scale", 0.f);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& q_in = ctx.RequiredInput(0);
    const int dt = DtypeCode(q_in.scalar_type());
    const bool extra = ctx.HasInput(3) || ctx.HasInput(5) || ctx.HasInput(6) || ctx.HasInput(7) ||
                       (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) || (ctx.OutputCount() > 2 && ctx.OutputNeeded(2));
    if (dt < 0 || extra) {
      Fallback(ctx);
      return;
    }
    const int64_t B = q_in.size(0), S = q_in.size(1);
    at::Tensor q, k, v;
    if (q_in.dim() == 5) {  // packed QKV [B, S, N, 3, H]
      q = q_in.select(3, 0);
      k = q_in.select(3, 1);
      v = q_in.select(3, 2);
    } else if (q_in.dim() == 3 && ctx.HasInput(1) && ctx.Input(1).dim() == 5) {  // packed KV [B, T, N, 2, H]
      const at::Tensor& kv = ctx.Input(1);
      q = q_in.reshape({B, S, N_, -1});
      k = kv.select(3, 0);
      v = kv.select(3, 1);
    } else if (q_in.dim() == 3 && ctx.HasInput(1) && ctx.Input(1).dim() == 3 && ctx.HasInput(2)) {
      q = q_in.reshape({B, S, N_, -1});
      k = ctx.Input(1).reshape({B, ctx.Input(1).size(1), N_, -1});
      v = ctx.Input(2).reshape({B, ctx.Input(2).size(1), N_, -1});
    } else {
      Fallback(ctx);
      return;
    }
    const int64_t T = k.size(1), H = q.size(3);
    at::Tensor lengths, key_mask;
    if ((H != 64 && H != 128) || v.size(3) != H || (causal_ && S != T) || !ViewsOk(q, k, v) ||
        (ctx.HasInput(4) && !DecodeMask(ctx.Input(4), B, T, &lengths, &key_mask))) {
      Fallback(ctx);
      return;
    }
    EncoderAttnCall c{q, k, v, B, S, T, N_, H, lengths, key_mask, causal_, scale_};
    ctx.SetOutput(0, RunEncoderAttention(ctx, c, dt).reshape({B, S, N_ * H}));
  }

 private:
  int64_t N_ = 1;
  bool causal_ = false;
  float scale_ = 0.f;
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

void RegisterCudaKernels3(KernelRegistry& r) {
  Reg<MatMulNBitsKernel>(r, MS, "MatMulNBits");
  Reg<PagedAttentionKernel>(r, MS, "PagedAttention");
  Reg<BertAttentionKernel>(r, MS, "Attention");
  Reg<MultiHeadAttentionKernel>(r, MS, "MultiHeadAttention");
}

}  // namespace ortb
