// If / Loop / Scan.  Each body graph gets its own GraphExecutor, built on first
// use when the devices of the captured values and body inputs are known
// (reference: onnxruntime/core/providers/cpu/controlflow/{if,loop,scan_9}.cc,
// which create a sub-SessionState per body).
#include <ATen/ATen.h>

#include <ATen/CPUGeneratorImpl.h>

#include <algorithm>
#include <cmath>
#include <mutex>

#include "executor.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

struct Body {
  std::shared_ptr<Graph> graph;
  std::unique_ptr<GraphExecutor> exec;
  std::vector<std::string> implicit;  // captured value names
};

class ControlFlowBase : public OpKernel {
 public:
  explicit ControlFlowBase(const OpKernelInfo& info) : OpKernel(info), session_(info.session), parent_graph_(&info.graph) {}

 protected:
  void Prepare(Body& body, Ctx& ctx, const std::vector<Value>& body_inputs) const {
    if (body.exec) return;
    std::map<std::string, bool> outer_on_gpu;
    for (auto& name : body.implicit) {
      Value v = ctx.LookupValue(name);
      outer_on_gpu[name] = v.t.defined() && v.t.is_cuda();
    }
    const auto& ins = body.graph->Inputs();
    for (size_t i = 0; i < ins.size() && i < body_inputs.size(); ++i)
      outer_on_gpu["\x02input:" + ins[i].name] = body_inputs[i].t.defined() && body_inputs[i].t.is_cuda();
    auto ex = std::make_unique<GraphExecutor>(session_, body.graph.get(), &outer_on_gpu);
    ex->Build();
    body.exec = std::move(ex);
  }

  std::vector<Value> RunBody(Body& body, Ctx& ctx, const std::vector<Value>& inputs) const {
    Prepare(body, ctx, inputs);
    std::map<std::string, Value> outer;
    for (auto& name : body.exec->outer_names()) outer[name] = ctx.LookupValue(name);
    std::vector<Value> ordered(body.exec->input_names().size());
    const auto& gi = body.graph->Inputs();
    // executor inputs follow graph input order minus constant initializers
    size_t k = 0;
    for (size_t i = 0; i < gi.size() && k < ordered.size(); ++i) {
      if (body.exec->input_names()[k] != gi[i].name) continue;
      if (i < inputs.size()) ordered[k] = inputs[i];
      ++k;
    }
    static const RunOptions default_ro;
    const RunOptions& ro = ctx.run_options ? *ctx.run_options : default_ro;
    return body.exec->Run(ro, ordered, &outer, body.exec->output_names());
  }

  Body MakeBody(const std::string& attr) const {
    auto it = node_.subgraphs.find(attr);
    if (it == node_.subgraphs.end()) ORTB_THROW(INVALID_GRAPH, node_.op_type, " node '", node_.name, "' has no ", attr);
    Body b;
    b.graph = it->second;
    Node probe;
    probe.subgraphs[attr] = it->second;
    b.implicit = parent_graph_->ImplicitInputs(probe);
    return b;
  }

  at::Tensor ToSessionDevice(const at::Tensor& t) const {
    if (!t.defined() || !session_ || !session_->uses_gpu() || t.is_cuda()) return t;
    return t.to(session_->device());
  }

  InferenceSession* session_;
  const Graph* parent_graph_;
  mutable std::mutex mu_;
};

class IfKernel final : public ControlFlowBase {
 public:
  explicit IfKernel(const OpKernelInfo& info) : ControlFlowBase(info) {
    then_ = MakeBody("then_branch");
    else_ = MakeBody("else_branch");
  }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const bool cond = ctx.RequiredInput(0).cpu().reshape({-1})[0].item<bool>();
    Body& b = cond ? then_ : else_;
    std::vector<Value> outs = RunBody(b, ctx, {});
    for (int i = 0; i < ctx.OutputCount() && i < static_cast<int>(outs.size()); ++i) {
      if (outs[i].seq) ctx.SetOutputSeq(i, *outs[i].seq);
      else ctx.SetOutput(i, ToSessionDevice(outs[i].t));
    }
  }

 private:
  mutable Body then_, else_;
};

class LoopKernel final : public ControlFlowBase {
 public:
  explicit LoopKernel(const OpKernelInfo& info) : ControlFlowBase(info) { body_ = MakeBody("body"); }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    int64_t max_trip = std::numeric_limits<int64_t>::max();
    if (ctx.HasInput(0)) max_trip = ctx.Input(0).cpu().reshape({-1})[0].item<int64_t>();
    bool cond = true;
    if (ctx.HasInput(1)) cond = ctx.Input(1).cpu().reshape({-1})[0].item<bool>();
    const int n_carried = ctx.InputCount() - 2;
    std::vector<Value> carried;
    for (int i = 0; i < n_carried; ++i) carried.push_back(ctx.InputValue(2 + i));
    const int n_body_out = static_cast<int>(body_.graph->Outputs().size());
    const int n_scan = n_body_out - 1 - n_carried;
    ORTB_ENFORCE(n_scan >= 0, "Loop body has too few outputs");
    std::vector<std::vector<at::Tensor>> scans(n_scan);
    for (int64_t it = 0; it < max_trip && cond; ++it) {
      std::vector<Value> in(2 + n_carried);
      in[0].t = at::scalar_tensor(it, at::kLong);
      in[1].t = at::scalar_tensor(cond, at::kBool);
      for (int i = 0; i < n_carried; ++i) in[2 + i] = carried[i];
      std::vector<Value> out = RunBody(body_, ctx, in);
      cond = out[0].t.cpu().reshape({-1})[0].item<bool>();
      for (int i = 0; i < n_carried; ++i) carried[i] = out[1 + i];
      for (int i = 0; i < n_scan; ++i) scans[i].push_back(out[1 + n_carried + i].t);
    }
    for (int i = 0; i < n_carried; ++i) {
      if (carried[i].seq) ctx.SetOutputSeq(i, *carried[i].seq);
      else ctx.SetOutput(i, ToSessionDevice(carried[i].t));
    }
    for (int i = 0; i < n_scan; ++i) {
      if (scans[i].empty()) {
        ctx.SetOutput(n_carried + i, at::empty({0}, at::TensorOptions().device(ctx.device())));
      } else {
        ctx.SetOutput(n_carried + i, ToSessionDevice(at::stack(scans[i], 0)));
      }
    }
  }

 private:
  mutable Body body_;
};

// SequenceMap (opset 17): the body runs once per position of the first input sequence; further inputs are sequences of
// the same length (their elements at that position) or tensors (passed to every call); every body output becomes a sequence.
class SequenceMapKernel final : public ControlFlowBase {
 public:
  explicit SequenceMapKernel(const OpKernelInfo& info) : ControlFlowBase(info) { body_ = MakeBody("body"); }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const Value& first = ctx.InputValue(0);
    ORTB_ENFORCE_ARG(first.seq != nullptr, "SequenceMap: the first input must be a sequence");
    const size_t len = first.seq->size();
    const int n_in = ctx.InputCount(), n_out = static_cast<int>(body_.graph->Outputs().size());
    for (int i = 1; i < n_in; ++i) {
      const Value& v = ctx.InputValue(i);
      ORTB_ENFORCE_ARG(!v.seq || v.seq->size() == len, "SequenceMap: input sequences differ in length");
    }
    std::vector<std::vector<at::Tensor>> outs(static_cast<size_t>(n_out));
    for (size_t pos = 0; pos < len; ++pos) {
      std::vector<Value> in(static_cast<size_t>(n_in));
      for (int i = 0; i < n_in; ++i) {
        const Value& v = ctx.InputValue(i);
        if (v.seq) in[static_cast<size_t>(i)].t = (*v.seq)[pos];
        else in[static_cast<size_t>(i)] = v;
      }
      std::vector<Value> out = RunBody(body_, ctx, in);
      for (int k = 0; k < n_out; ++k) outs[static_cast<size_t>(k)].push_back(ToSessionDevice(out[static_cast<size_t>(k)].t));
    }
    for (int k = 0; k < n_out && k < ctx.OutputCount(); ++k) ctx.SetOutputSeq(k, outs[static_cast<size_t>(k)]);
  }

 private:
  mutable Body body_;
};

class ScanKernel final : public ControlFlowBase {
 public:
  explicit ScanKernel(const OpKernelInfo& info) : ControlFlowBase(info) { body_ = MakeBody("body"); }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const Node& n = ctx.node();
    const int64_t m = n.attr_i("num_scan_inputs", 0);
    const int total_in = ctx.InputCount();
    const int n_state = total_in - static_cast<int>(m);
    std::vector<int64_t> in_axes = n.attr_ints("scan_input_axes"), in_dirs = n.attr_ints("scan_input_directions");
    std::vector<int64_t> out_axes = n.attr_ints("scan_output_axes"), out_dirs = n.attr_ints("scan_output_directions");
    in_axes.resize(m, 0);
    in_dirs.resize(m, 0);
    const int n_body_out = static_cast<int>(body_.graph->Outputs().size());
    const int k = n_body_out - n_state;
    out_axes.resize(k, 0);
    out_dirs.resize(k, 0);
    std::vector<Value> state;
    for (int i = 0; i < n_state; ++i) state.push_back(ctx.InputValue(i));
    std::vector<at::Tensor> scan_in;
    int64_t len = -1;
    for (int64_t i = 0; i < m; ++i) {
      at::Tensor t = ctx.RequiredInput(n_state + static_cast<int>(i));
      int64_t ax = in_axes[i] < 0 ? in_axes[i] + t.dim() : in_axes[i];
      in_axes[i] = ax;
      if (len < 0) len = t.size(ax);
      ORTB_ENFORCE_ARG(t.size(ax) == len, "Scan inputs disagree on sequence length");
      scan_in.push_back(t);
    }
    std::vector<std::vector<at::Tensor>> outs(k);
    for (int64_t s = 0; s < len; ++s) {
      std::vector<Value> in(n_state + m);
      for (int i = 0; i < n_state; ++i) in[i] = state[i];
      for (int64_t i = 0; i < m; ++i) {
        const int64_t idx = in_dirs[i] ? len - 1 - s : s;
        in[n_state + i].t = scan_in[i].select(in_axes[i], idx).contiguous();
      }
      std::vector<Value> out = RunBody(body_, ctx, in);
      for (int i = 0; i < n_state; ++i) state[i] = out[i];
      for (int i = 0; i < k; ++i) outs[i].push_back(out[n_state + i].t);
    }
    for (int i = 0; i < n_state; ++i) ctx.SetOutput(i, ToSessionDevice(state[i].t));
    for (int i = 0; i < k; ++i) {
      if (outs[i].empty()) continue;
      if (out_dirs[i]) std::reverse(outs[i].begin(), outs[i].end());
      int64_t ax = out_axes[i];
      if (ax < 0) ax += outs[i][0].dim() + 1;
      ctx.SetOutput(n_state + i, ToSessionDevice(at::stack(outs[i], ax)));
    }
  }

 private:
  mutable Body body_;
};

// ---------------------------------------------------------------------------------------------------------------
// Generation as operators: com.microsoft GreedySearch / Sampling / BeamSearch drive a decoder body graph token by token
// (reference: onnxruntime/contrib_ops/cpu/transformers/greedy_search.cc, sampling.cc, beam_search.cc, beam_search_scorer.cc,
// logits_processor.h; device kernels contrib_ops/cuda/transformers/generation_cuda_impl.cu).
//   model_type 0 (GPT): the `decoder` body takes input_ids [R, S] int32, position_ids [R, S] int32, attention_mask
//     [R, total] int32 and one past state per layer [2, R, heads, past, head]; it returns logits [R, S, vocab] and the
//     present states, which the loop feeds back (beam search re-orders their rows).
//   model_type 1 (T5) and 2 (Whisper; also the WhisperBeamSearch operator): the `encoder` body runs once on the
//     encoder input (token ids, or audio features for Whisper), the encoder attention mask (T5 only) and the first
//     decoder tokens; it returns logits, encoder_hidden_states and per layer key / value of the decoder's self attention
//     and of the cross attention.  The `decoder` body then takes input_ids [R, 1], the encoder attention mask (T5 only),
//     encoder_hidden_states when it declares that input, the self-attention states of all layers and then the
//     cross-attention states of all layers; it returns logits and the new self-attention states.
// All tensor work is ATen on the body's device.
class GenerationKernel final : public ControlFlowBase {
 public:
  explicit GenerationKernel(const OpKernelInfo& info) : ControlFlowBase(info) {
    const Node& n = info.node;
    kind_ = n.op_type;
    model_type_ = n.attr_i("model_type", kind_ == "WhisperBeamSearch" ? 2 : 0);
    ORTB_ENFORCE_ARG(model_type_ >= 0 && model_type_ <= 2, kind_, ": model_type must be 0 (GPT), 1 (T5) or 2 (Whisper)");
    decoder_ = MakeBody("decoder");
    eos_ = n.attr_i("eos_token_id", -1);
    pad_ = n.attr_i("pad_token_id", 0);
    no_repeat_ngram_ = n.attr_i("no_repeat_ngram_size", 0);
    early_stopping_ = n.attr_i("early_stopping", 0) != 0;
    temperature_ = n.attr_f("temperature", 1.f);
    top_p_ = n.attr_f("top_p", 0.f);
    filter_value_ = n.attr_f("filter_value", -1e20f);
    min_tokens_to_keep_ = n.attr_i("min_tokens_to_keep", 1);
    presence_penalty_ = n.attr_f("presence_penalty", 0.f);
    seed_ = n.attr_i("seed", 0);
    const auto& ins = decoder_.graph->Inputs();
    if (model_type_ != 0) {
      ORTB_ENFORCE_ARG(kind_ == "BeamSearch" || kind_ == "WhisperBeamSearch" || kind_ == "GreedySearch", kind_,
                       ": encoder-decoder models are driven by BeamSearch, WhisperBeamSearch or GreedySearch");
      encoder_ = MakeBody("encoder");
      start_token_ = n.attr_i("decoder_start_token_id", 0);
      const int n_enc_out = static_cast<int>(encoder_.graph->Outputs().size());
      ORTB_ENFORCE_ARG(n_enc_out > 2 && (n_enc_out - 2) % 4 == 0, kind_,
                       ": the encoder body must return logits, encoder_hidden_states and four states per layer");
      layers_ = (n_enc_out - 2) / 4;
      const int fixed = static_cast<int>(ins.size()) - 4 * layers_;
      dec_has_mask_ = model_type_ == 1;
      const int base = dec_has_mask_ ? 2 : 1;
      ORTB_ENFORCE_ARG(fixed == base || fixed == base + 1, kind_, ": the decoder body's inputs do not match ", layers_, " layers");
      dec_has_hidden_ = fixed == base + 1;
      return;
    }
    ORTB_ENFORCE_ARG(ins.size() >= 3, kind_, ": the decoder body needs input_ids, position_ids, attention_mask and past states");
    layers_ = static_cast<int>(ins.size()) - 3;
    if (layers_ > 0) {
      const auto& d = ins[3].type.dims;
      ORTB_ENFORCE_ARG(d.size() == 5 && d[2].has_value && d[4].has_value, kind_, ": past states must be [2, batch, heads, past, head] with static heads and head size");
      heads_ = d[2].value;
      head_size_ = d[4].value;
      past_type_ = ToTorchType(ins[3].type.elem_type);
    }
  }

  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const bool beam = kind_ == "BeamSearch" || kind_ == "WhisperBeamSearch";
    const bool encdec = model_type_ != 0;
    const at::Tensor& enc_input = ctx.RequiredInput(0);
    at::Tensor ids;
    if (!encdec) {
      ids = enc_input.to(at::kLong);
    } else if (kind_ == "WhisperBeamSearch" && ctx.HasInput(10)) {
      ids = ctx.Input(10).to(enc_input.device(), at::kLong);   // forced decoder prompt
    } else {
      ids = at::full({enc_input.size(0), 1}, start_token_, at::TensorOptions().dtype(at::kLong).device(enc_input.device()));
    }
    ORTB_ENFORCE_ARG(ids.dim() == 2, kind_, ": input_ids must be [batch, sequence]");
    auto scalar_i = [&](int i, int64_t dflt) { return ctx.HasInput(i) ? ctx.Input(i).cpu().reshape({-1})[0].item<int64_t>() : dflt; };
    auto scalar_f = [&](int i, double dflt) { return ctx.HasInput(i) ? ctx.Input(i).cpu().to(at::kDouble).reshape({-1})[0].item<double>() : dflt; };
    const int64_t B = ids.size(0), S0 = ids.size(1);
    const int64_t max_length = scalar_i(1, S0 + 1), min_length = scalar_i(2, 0);
    // input layout: BeamSearch (ids, max, min, num_beams, num_return_sequences, length_penalty, repetition_penalty, vocab_mask,
    // prefix_vocab_mask, attention_mask); GreedySearch / Sampling (ids, max, min, repetition_penalty, vocab_mask, prefix_vocab_mask, attention_mask)
    const int64_t K = beam ? scalar_i(3, 1) : 1, nrs = beam ? scalar_i(4, 1) : 1;
    const double length_penalty = beam ? scalar_f(5, 1.0) : 1.0;
    const double rep_penalty = scalar_f(beam ? 6 : 3, 1.0);
    const int vm = beam ? 7 : 4, am = beam ? 9 : 6;
    ORTB_ENFORCE_ARG(K >= 1 && nrs >= 1 && nrs <= K && max_length > S0, kind_, ": invalid num_beams / num_return_sequences / max_length");
    at::Device dev = ids.device();
    at::Tensor vocab_mask = ctx.HasInput(vm) ? ctx.Input(vm).to(dev) : at::Tensor();
    at::Tensor mask, enc_mask;
    if (encdec) {
      // the attention_mask input belongs to the encoder; the decoder side attends to everything generated so far
      mask = at::ones({B, S0}, at::TensorOptions().dtype(at::kInt).device(dev));
      if (model_type_ == 1)
        enc_mask = ctx.HasInput(am) ? ctx.Input(am).to(dev, at::kInt) : at::ones({B, enc_input.size(1)}, at::TensorOptions().dtype(at::kInt).device(dev));
    } else {
      mask = ctx.HasInput(am) ? ctx.Input(am).to(dev, at::kInt) : at::ones({B, S0}, at::TensorOptions().dtype(at::kInt).device(dev));
    }
    const int64_t R = B * K;
    at::Tensor seqs = ids.repeat_interleave(K, 0);
    mask = mask.repeat_interleave(K, 0);
    // positions count the attended tokens (left padding keeps position 0 for the first real token)
    at::Tensor pos = (mask.to(at::kLong).cumsum(1) - 1).clamp_min(0);
    std::vector<at::Tensor> past(static_cast<size_t>(layers_));
    if (!encdec)
      for (auto& p : past) p = at::zeros({2, R, heads_, 0, head_size_}, at::TensorOptions().dtype(past_type_).device(dev));
    at::Tensor enc_hidden, enc_mask_rows;
    const int64_t reorder_dim = encdec ? 0 : 1;
    at::Tensor step_ids = seqs, step_pos = pos;
    at::Tensor beam_scores = at::zeros({B, K}, at::TensorOptions().dtype(at::kFloat).device(dev));
    if (K > 1) beam_scores.narrow(1, 1, K - 1).fill_(-1e9f);
    at::Tensor done = at::zeros({R}, at::TensorOptions().dtype(at::kBool).device(dev));
    std::vector<std::vector<std::pair<double, at::Tensor>>> finished(static_cast<size_t>(B));
    std::vector<bool> batch_done(static_cast<size_t>(B), false);
    at::Generator gen = at::detail::createCPUGenerator(static_cast<uint64_t>(seed_));
    int64_t V = 0;

    for (int64_t step = 0; seqs.size(1) < max_length; ++step) {
      at::Tensor logits;
      if (!encdec) {
        std::vector<Value> in(static_cast<size_t>(3 + layers_));
        in[0].t = step_ids.to(at::kInt);
        in[1].t = step_pos.to(at::kInt);
        in[2].t = mask;
        for (int l = 0; l < layers_; ++l) in[static_cast<size_t>(3 + l)].t = past[static_cast<size_t>(l)];
        std::vector<Value> out = RunBody(decoder_, ctx, in);
        ORTB_ENFORCE(static_cast<int>(out.size()) >= 1 + layers_, kind_, ": the decoder body returned too few outputs");
        logits = out[0].t;
        logits = logits.select(1, logits.size(1) - 1).to(at::kFloat).clone();   // [R, V]
        for (int l = 0; l < layers_; ++l) past[static_cast<size_t>(l)] = out[static_cast<size_t>(1 + l)].t;
      } else if (step == 0) {
        // encoder pass: also yields the logits of the first decoder position(s) and every layer's states
        std::vector<Value> in;
        in.emplace_back();
        in.back().t = enc_input;
        if (model_type_ == 1) {
          in.emplace_back();
          in.back().t = enc_mask;
        }
        in.emplace_back();
        in.back().t = ids.to(at::kInt);
        std::vector<Value> out = RunBody(encoder_, ctx, in);
        ORTB_ENFORCE(static_cast<int>(out.size()) >= 2 + 4 * layers_, kind_, ": the encoder body returned too few outputs");
        logits = out[0].t;
        logits = logits.select(1, logits.size(1) - 1).to(at::kFloat).repeat_interleave(K, 0);
        enc_hidden = out[1].t.repeat_interleave(K, 0);
        if (enc_mask.defined()) enc_mask_rows = enc_mask.repeat_interleave(K, 0);
        past.assign(static_cast<size_t>(4 * layers_), at::Tensor());
        for (int l = 0; l < layers_; ++l) {   // stored as the decoder wants them: all self states, then all cross states
          past[static_cast<size_t>(2 * l)] = out[static_cast<size_t>(2 + 4 * l)].t.repeat_interleave(K, 0);
          past[static_cast<size_t>(2 * l + 1)] = out[static_cast<size_t>(3 + 4 * l)].t.repeat_interleave(K, 0);
          past[static_cast<size_t>(2 * layers_ + 2 * l)] = out[static_cast<size_t>(4 + 4 * l)].t.repeat_interleave(K, 0);
          past[static_cast<size_t>(2 * layers_ + 2 * l + 1)] = out[static_cast<size_t>(5 + 4 * l)].t.repeat_interleave(K, 0);
        }
      } else {
        std::vector<Value> in;
        auto push = [&](const at::Tensor& t) {
          in.emplace_back();
          in.back().t = t;
        };
        push(step_ids.to(at::kInt));
        if (dec_has_mask_) push(enc_mask_rows);
        if (dec_has_hidden_) push(enc_hidden);
        for (auto& p : past) push(p);
        std::vector<Value> out = RunBody(decoder_, ctx, in);
        ORTB_ENFORCE(static_cast<int>(out.size()) >= 1 + 2 * layers_, kind_, ": the decoder body returned too few outputs");
        logits = out[0].t;
        logits = logits.select(1, logits.size(1) - 1).to(at::kFloat).clone();
        for (int i = 0; i < 2 * layers_; ++i) past[static_cast<size_t>(i)] = out[static_cast<size_t>(1 + i)].t;
      }
      V = logits.size(1);
      // ---- logits processors, in the reference's order
      const int64_t cur_len = seqs.size(1);
      if (eos_ >= 0 && cur_len < min_length) logits.select(1, eos_).fill_(-INFINITY);
      if (rep_penalty != 1.0) {
        at::Tensor seen = logits.gather(1, seqs);
        seen = at::where(seen < 0, seen * rep_penalty, seen / rep_penalty);
        logits.scatter_(1, seqs, seen);
      }
      if (presence_penalty_ != 0.f) {
        at::Tensor seen = at::zeros_like(logits).scatter_(1, seqs, 1.0);
        logits = logits - seen * presence_penalty_;
      }
      if (no_repeat_ngram_ > 0 && cur_len + 1 >= no_repeat_ngram_) BanRepeatedNgrams(logits, seqs, no_repeat_ngram_);
      if (vocab_mask.defined()) logits.masked_fill_(vocab_mask.reshape({1, -1}) == 0, -INFINITY);
      if (ctx.HasInput(vm + 1) && step == 0) logits.masked_fill_(ctx.Input(vm + 1).to(dev).repeat_interleave(K, 0) == 0, -INFINITY);

      at::Tensor next_tok, rows;
      if (!beam) {
        if (kind_ == "Sampling") {
          at::Tensor sc = temperature_ > 0.f && temperature_ != 1.f ? logits / temperature_ : logits;
          if (top_p_ > 0.f && top_p_ < 1.f) sc = TopPFilter(sc);
          at::Tensor probs = at::softmax(sc, -1).cpu();
          next_tok = at::multinomial(probs, 1, false, gen).reshape({-1}).to(dev);
        } else {
          next_tok = logits.argmax(-1);
        }
        next_tok = at::where(done, at::full_like(next_tok, pad_), next_tok);
        if (eos_ >= 0) done = done | (next_tok == eos_);
      } else {
        // ---- beam scorer: 2K candidates per batch entry so that finished beams can be replaced
        at::Tensor logp = at::log_softmax(logits, -1);
        at::Tensor cand = (beam_scores.reshape({R, 1}) + logp).reshape({B, K * V});
        auto top = at::topk(cand, 2 * K, 1);
        at::Tensor ts = std::get<0>(top).cpu(), ti = std::get<1>(top).cpu();
        at::Tensor new_scores = at::full({B, K}, -1e9f), new_src = at::zeros({B, K}, at::kLong), new_tok = at::full({B, K}, pad_, at::kLong);
        auto tsa = ts.accessor<float, 2>();
        auto tia = ti.accessor<int64_t, 2>();
        const int64_t gen_len = cur_len + 1 - S0;
        for (int64_t b = 0; b < B; ++b) {
          if (batch_done[static_cast<size_t>(b)]) continue;
          int64_t filled = 0;
          for (int64_t rank = 0; rank < 2 * K && filled < K; ++rank) {
            const int64_t src = tia[b][rank] / V, tok = tia[b][rank] % V;
            if (eos_ >= 0 && tok == eos_) {
              if (rank < K) {
                at::Tensor hyp = at::cat({seqs[b * K + src], at::full({1}, eos_, seqs.options())});
                finished[static_cast<size_t>(b)].emplace_back(tsa[b][rank] / std::pow(static_cast<double>(gen_len), length_penalty), hyp);
              }
              continue;
            }
            new_scores[b][filled] = tsa[b][rank];
            new_src[b][filled] = src;
            new_tok[b][filled] = tok;
            ++filled;
          }
          auto& fin = finished[static_cast<size_t>(b)];
          if (static_cast<int64_t>(fin.size()) >= K) {
            std::vector<double> sc;
            for (auto& f : fin) sc.push_back(f.first);
            std::sort(sc.begin(), sc.end());
            const double worst_kept = sc[sc.size() - static_cast<size_t>(K)];
            const double best_open = new_scores[b].max().item<float>() / std::pow(static_cast<double>(gen_len), length_penalty);
            if (early_stopping_ || worst_kept >= best_open) batch_done[static_cast<size_t>(b)] = true;
          }
        }
        rows = (at::arange(B, at::kLong).unsqueeze(1) * K + new_src).reshape({-1}).to(dev);
        seqs = seqs.index_select(0, rows);
        mask = mask.index_select(0, rows);
        pos = pos.index_select(0, rows);
        for (auto& p : past) p = p.index_select(reorder_dim, rows);
        beam_scores = new_scores.to(dev);
        next_tok = new_tok.reshape({-1}).to(dev);
      }
      seqs = at::cat({seqs, next_tok.unsqueeze(1)}, 1);
      mask = at::cat({mask, at::ones({R, 1}, mask.options())}, 1);
      step_pos = pos.select(1, pos.size(1) - 1).unsqueeze(1) + 1;
      pos = at::cat({pos, step_pos}, 1);
      step_ids = next_tok.unsqueeze(1);
      if (!beam && eos_ >= 0 && done.all().item<bool>()) break;
      if (beam && std::all_of(batch_done.begin(), batch_done.end(), [](bool d) { return d; })) break;
    }

    auto iopt = at::TensorOptions().dtype(at::kInt).device(dev);
    if (!beam) {
      at::Tensor outseq = at::full({B, max_length}, pad_, iopt);
      outseq.narrow(1, 0, seqs.size(1)).copy_(seqs.to(at::kInt));
      ctx.SetOutput(0, outseq);
      return;
    }
    const int64_t gen_len = std::max<int64_t>(seqs.size(1) - S0, 1);
    at::Tensor outseq = at::full({B, nrs, max_length}, pad_, iopt);
    at::Tensor outscore = at::zeros({B, nrs}, at::TensorOptions().dtype(at::kFloat));
    at::Tensor bs_cpu = beam_scores.cpu();
    for (int64_t b = 0; b < B; ++b) {
      auto hyps = finished[static_cast<size_t>(b)];
      for (int64_t k = 0; k < K; ++k)  // open beams count as hypotheses of the current length
        hyps.emplace_back(bs_cpu[b][k].item<float>() / std::pow(static_cast<double>(gen_len), length_penalty), seqs[b * K + k]);
      std::stable_sort(hyps.begin(), hyps.end(), [](const auto& x, const auto& y) { return x.first > y.first; });
      for (int64_t j = 0; j < nrs; ++j) {
        const at::Tensor& h = hyps[static_cast<size_t>(j)].second;
        const int64_t len = std::min<int64_t>(h.size(0), max_length);
        outseq[b][j].narrow(0, 0, len).copy_(h.narrow(0, 0, len).to(at::kInt));
        outscore[b][j] = hyps[static_cast<size_t>(j)].first;
      }
    }
    ctx.SetOutput(0, outseq);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, outscore.to(dev));
  }

 private:
  // tokens that would complete an n-gram already present in the row are banned
  static void BanRepeatedNgrams(at::Tensor& logits, const at::Tensor& seqs, int64_t n) {
    const int64_t L = seqs.size(1);
    if (n == 1) {
      logits.scatter_(1, seqs, -INFINITY);
      return;
    }
    at::Tensor grams = seqs.unfold(1, n, 1);                                   // [R, L - n + 1, n]
    at::Tensor tail = seqs.narrow(1, L - (n - 1), n - 1).unsqueeze(1);          // [R, 1, n - 1]
    at::Tensor hit = (grams.narrow(2, 0, n - 1) == tail).all(-1);              // [R, L - n + 1]
    at::Tensor last = grams.select(2, n - 1);
    at::Tensor ban = at::zeros_like(logits, at::kBool);
    ban.scatter_(1, at::where(hit, last, at::zeros_like(last)), hit);
    // position 0 of `ban` may have been written with false by the masked-out entries: restore real hits on token 0
    at::Tensor zero_hit = (hit & (last == 0)).any(1);
    ban.select(1, 0).copy_(zero_hit);
    logits.masked_fill_(ban, -INFINITY);
  }

  at::Tensor TopPFilter(const at::Tensor& logits) const {
    auto sorted = at::sort(logits, -1, /*descending=*/true);
    at::Tensor sl = std::get<0>(sorted), idx = std::get<1>(sorted);
    at::Tensor probs = at::softmax(sl, -1);
    at::Tensor drop = (probs.cumsum(-1) - probs) > top_p_;   // the token that crosses the threshold stays
    if (min_tokens_to_keep_ > 0) drop.narrow(1, 0, std::min<int64_t>(min_tokens_to_keep_, drop.size(1))).fill_(false);
    sl = sl.masked_fill(drop, filter_value_);
    return at::full_like(logits, filter_value_).scatter(1, idx, sl);
  }

  std::string kind_;
  mutable Body decoder_, encoder_;
  int64_t model_type_ = 0, start_token_ = 0;
  bool dec_has_mask_ = false, dec_has_hidden_ = false;
  int64_t eos_ = -1, pad_ = 0, no_repeat_ngram_ = 0, min_tokens_to_keep_ = 1, seed_ = 0, heads_ = 0, head_size_ = 0;
  bool early_stopping_ = false;
  float temperature_ = 1.f, top_p_ = 0.f, filter_value_ = -1e20f, presence_penalty_ = 0.f;
  int layers_ = 0;
  at::ScalarType past_type_ = at::kFloat;
};

template <typename K>
void RegisterClass(KernelRegistry& r, const std::string& op, int since, std::vector<int> host) {
  KernelDef d;
  d.domain = "";
  d.op_type = op;
  d.since_min = since;
  d.since_max = kMax;
  d.host_inputs = std::move(host);
  d.factory = [](const OpKernelInfo& info) { return std::make_unique<K>(info); };
  r.Register(std::move(d));
}

}  // namespace

void RegisterControlFlowKernels(KernelRegistry& r) {
  RegisterClass<IfKernel>(r, "If", 1, {0});
  RegisterClass<LoopKernel>(r, "Loop", 1, {0, 1});
  RegisterClass<ScanKernel>(r, "Scan", 9, {});
  RegisterClass<SequenceMapKernel>(r, "SequenceMap", 17, {});
  for (const char* op : {"GreedySearch", "Sampling", "BeamSearch", "WhisperBeamSearch"}) {
    KernelDef d;
    d.domain = kMSDomain;
    d.op_type = op;
    d.since_min = 1;
    d.since_max = kMax;
    d.factory = [](const OpKernelInfo& info) { return std::make_unique<GenerationKernel>(info); };
    r.Register(std::move(d));
  }
}

}  // namespace ortb
