// GPU-only lowering passes: rewrite GEMM chains onto the fused sm_100a kernels.
//
//  * GemmEpilogueFusion:  MatMul(x, W) [+ bias] [+ activation] [+ residual]
//        -> com.ortb200.FusedGemm(x, W, bias, residual) {activation}
//    one tcgen05 GEMM whose epilogue applies bias, activation and the residual
//    add (the reference runs cuBLAS followed by separate BiasGelu / Add kernels).
//  * SwiGLUFusion:  Mul(silu(MatMul(x, Wg)), MatMul(x, Wu)) -> com.ortb200.GemmSwiGLU(x, Wg, Wu)
//    one kernel with two TMEM accumulators sharing the activation tile.
//  * MatMulAllReduceFusion:  AllReduce(GEMM) -> the GEMM carries all_reduce=1 and
//    its kernel finishes the row-parallel sum over NVLink itself.
#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

constexpr const char* kFusedDomain = "com.ortb200";

bool IsHalfWeight2D(const Graph& g, const std::string& name) {
  const at::Tensor* w = g.GetConstant(name);
  if (!w || w->dim() != 2) return false;
  if (w->scalar_type() != at::kHalf && w->scalar_type() != at::kBFloat16) return false;
  return w->size(0) % 8 == 0;  // K: TMA row pitch must be a multiple of 16 bytes
}

Node* SoleConsumer(const Graph& g, const std::string& v) {
  if (g.IsGraphOutput(v)) return nullptr;
  auto cs = g.Consumers(v);
  return cs.size() == 1 ? cs[0] : nullptr;
}

// y * sigmoid(y) rooted at a Mul node; returns y's name
bool MatchSilu(const Graph& g, Node* mul, std::string* y, Node** sigmoid) {
  if (mul->op_type != "Mul" || !mul->domain.empty() || mul->inputs.size() != 2) return false;
  for (int s = 0; s < 2; ++s) {
    Node* sg = g.Producer(mul->inputs[s]);
    if (sg && sg->op_type == "Sigmoid" && sg->domain.empty() && sg->inputs[0] == mul->inputs[1 - s] &&
        g.NumConsumers(sg->outputs[0]) == 1) {
      *y = mul->inputs[1 - s];
      *sigmoid = sg;
      return true;
    }
  }
  return false;
}

int SwiGLUFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* top : g.Nodes()) {
    if (top->op_type != "Mul" || !top->domain.empty() || top->inputs.size() != 2) continue;
    for (int s = 0; s < 2; ++s) {
      Node* silu = g.Producer(top->inputs[s]);
      Node* up = g.Producer(top->inputs[1 - s]);
      if (!silu || !up) continue;
      std::string gate_out;
      Node* sig = nullptr;
      if (!MatchSilu(g, silu, &gate_out, &sig)) continue;
      Node* gate = g.Producer(gate_out);
      if (!gate || gate->op_type != "MatMul" || !gate->domain.empty() || up->op_type != "MatMul" || !up->domain.empty()) continue;
      if (gate->inputs[0] != up->inputs[0]) continue;
      if (!IsHalfWeight2D(g, gate->inputs[1]) || !IsHalfWeight2D(g, up->inputs[1])) continue;
      if (g.GetConstant(gate->inputs[1])->sizes() != g.GetConstant(up->inputs[1])->sizes()) continue;
      if (g.NumConsumers(gate_out) != 2 || g.NumConsumers(up->outputs[0]) != 1 || g.NumConsumers(silu->outputs[0]) != 1) continue;
      g.AddNode("GemmSwiGLU", {gate->inputs[0], gate->inputs[1], up->inputs[1]}, {top->outputs[0]}, kFusedDomain,
                g.UniqueName("GemmSwiGLU"));
      g.RemoveNode(top);
      g.RemoveNode(silu);
      g.RemoveNode(sig);
      g.RemoveNode(gate);
      g.RemoveNode(up);
      ++count;
      break;
    }
  }
  return count;
}

int GemmEpilogueFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* mm : g.Nodes()) {
    if (mm->op_type != "MatMul" || !mm->domain.empty()) continue;
    if (!IsHalfWeight2D(g, mm->inputs[1]) || g.GetConstant(mm->inputs[0])) continue;
    const int64_t N = g.GetConstant(mm->inputs[1])->size(1);
    std::vector<Node*> chain;
    std::string cur = mm->outputs[0];
    std::string bias, residual, act = "none";
    float alpha = 1.702f;
    Node* n = SoleConsumer(g, cur);
    // bias
    if (n && n->op_type == "Add" && n->domain.empty()) {
      for (int s = 0; s < 2; ++s) {
        int64_t len = 0;
        if (n->inputs[1 - s] == cur && IsConst1D(g, n->inputs[s], &len) && len == N) {
          bias = n->inputs[s];
          chain.push_back(n);
          cur = n->outputs[0];
          n = SoleConsumer(g, cur);
          break;
        }
      }
    }
    // activation
    if (n) {
      std::string a;
      if (n->domain == kMSDomain && n->op_type == "FastGelu" && !n->has_input(1)) a = "fastgelu";
      else if (n->domain == kMSDomain && n->op_type == "Gelu") a = "gelu";
      else if (n->domain.empty() && n->op_type == "Gelu") a = n->attr_s("approximate", "none") == "tanh" ? "fastgelu" : "gelu";
      else if (n->domain.empty() && n->op_type == "Relu") a = "relu";
      else if (n->domain == kMSDomain && n->op_type == "QuickGelu") { a = "quickgelu"; alpha = n->attr_f("alpha", 1.702f); }
      else if (bias.empty() && n->domain == kMSDomain && (n->op_type == "BiasGelu" || (n->op_type == "FastGelu" && n->has_input(1))) &&
               n->inputs[0] == cur) {
        int64_t len = 0;
        if (IsConst1D(g, n->inputs[1], &len) && len == N) {
          bias = n->inputs[1];
          a = n->op_type == "BiasGelu" ? "gelu" : "fastgelu";
        }
      }
      if (!a.empty() && !(a == "quickgelu" && std::abs(alpha - 1.702f) > 1e-4f)) {
        act = a;
        chain.push_back(n);
        cur = n->outputs[0];
        n = SoleConsumer(g, cur);
      }
    }
    // silu written as y * sigmoid(y): two consumers of cur
    if (act == "none" && !g.IsGraphOutput(cur) && g.NumConsumers(cur) == 2) {
      for (Node* cand : g.Consumers(cur)) {
        std::string y;
        Node* sig = nullptr;
        if (MatchSilu(g, cand, &y, &sig) && y == cur) {
          act = "silu";
          chain.push_back(sig);
          chain.push_back(cand);
          cur = cand->outputs[0];
          n = SoleConsumer(g, cur);
          break;
        }
      }
    }
    // residual
    if (n && n->op_type == "Add" && n->domain.empty() && n->inputs.size() == 2) {
      for (int s = 0; s < 2; ++s) {
        if (n->inputs[1 - s] == cur && !g.GetConstant(n->inputs[s]) && n->inputs[s] != cur) {
          residual = n->inputs[s];
          chain.push_back(n);
          cur = n->outputs[0];
          break;
        }
      }
    }
    if (chain.empty()) continue;
    std::vector<std::string> ins = {mm->inputs[0], mm->inputs[1], bias, residual};
    while (!ins.empty() && ins.back().empty()) ins.pop_back();
    Node* f = g.AddNode("FusedGemm", ins, {cur}, kFusedDomain, g.UniqueName("FusedGemm"));
    f->set_attr_s("activation", act);
    g.RemoveNode(mm);
    for (Node* x : chain) g.RemoveNode(x);
    ++count;
  }
  return count;
}

int MatMulAllReduceFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  if (c.world_size <= 1) return 0;
  for (Node* ar : g.Nodes()) {
    if (ar->op_type != "AllReduce" || ar->domain != kMSDomain || ar->inputs.size() != 1) continue;
    Node* p = g.Producer(ar->inputs[0]);
    if (!p || g.NumConsumers(p->outputs[0]) != 1) continue;
    if (p->domain.empty() && p->op_type == "MatMul" && IsHalfWeight2D(g, p->inputs[1]) && !g.GetConstant(p->inputs[0])) {
      Node* f = g.AddNode("FusedGemm", {p->inputs[0], p->inputs[1]}, {ar->outputs[0]}, kFusedDomain, g.UniqueName("GemmAllReduce"));
      f->set_attr_s("activation", "none");
      f->set_attr_i("all_reduce", 1);
      g.RemoveNode(p);
      g.RemoveNode(ar);
      ++count;
    } else if (p->domain == kFusedDomain && p->op_type == "FusedGemm" && !p->has_input(3) && !p->has_input(2) &&
               p->attr_s("activation", "none") == "none") {
      p->set_attr_i("all_reduce", 1);
      p->outputs[0] = ar->outputs[0];
      g.RemoveNode(ar);
      g.Invalidate();
      ++count;
    }
  }
  return count;
}

// AllGather(axis 0) -> MatMul with a constant 16-bit weight  ->  com.ortb200.AllGatherMatMul, which the GPU registry runs
// as one kernel (the shard is pushed to the peers by spare warps while the tensor cores start on the local rows).
int AllGatherMatMulFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  if (c.world_size <= 1) return 0;
  for (Node* ag : g.Nodes()) {
    if (ag->op_type != "AllGather" || ag->domain != kMSDomain || ag->inputs.size() != 1 || ag->attr_i("axis", 0) != 0) continue;
    Node* mm = SoleConsumer(g, ag->outputs[0]);
    if (!mm || !mm->domain.empty() || mm->op_type != "MatMul" || mm->inputs[0] != ag->outputs[0] || !IsHalfWeight2D(g, mm->inputs[1])) continue;
    if (g.IsGraphOutput(ag->outputs[0])) continue;
    g.AddNode("AllGatherMatMul", {ag->inputs[0], mm->inputs[1]}, {mm->outputs[0]}, kFusedDomain, g.UniqueName("AllGatherMatMul"));
    g.RemoveNode(mm);
    g.RemoveNode(ag);
    ++count;
  }
  return count;
}

// After MatMulAllReduceFusion: a residual Add directly behind an all-reducing GEMM is applied after the sum.
int AllReduceResidualFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* f : g.Nodes()) {
    if (f->domain != kFusedDomain || f->op_type != "FusedGemm" || f->attr_i("all_reduce", 0) == 0 || f->has_input(3)) continue;
    Node* add = SoleConsumer(g, f->outputs[0]);
    if (!add || add->op_type != "Add" || !add->domain.empty()) continue;
    for (int s = 0; s < 2; ++s) {
      if (add->inputs[1 - s] == f->outputs[0] && !g.GetConstant(add->inputs[s]) && add->inputs[s] != f->outputs[0]) {
        if (f->inputs.size() < 4) f->inputs.resize(4);
        f->inputs[3] = add->inputs[s];
        f->outputs[0] = add->outputs[0];
        g.RemoveNode(add);
        g.Invalidate();
        ++count;
        break;
      }
    }
  }
  return count;
}

// RMS normalisation folded into the GEMMs around it:
//   G1 = GEMM(a, W1);  (h, sum) = SkipSimplifiedLayerNormalization(G1, residual, gamma);  G2 = GEMM(h, W2)
//     -> sum = FusedGemm(a, W1, residual);  G2 = GEMM(sum, W2 * gamma){rms_eps}
//   h = SimplifiedLayerNormalization(x, gamma);  G2 = GEMM(h, W2)  ->  G2 = GEMM(x, W2 * gamma){rms_eps}
// The residual add rides in the epilogue of the first GEMM; 1 / rms(x) is a per-token factor that commutes with
// the second GEMM, whose kernel computes it while the weights stream.  Two launches per decoder layer disappear.
int RmsNormGemmFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* norm : g.Nodes()) {
    const bool skip = norm->domain == kMSDomain && norm->op_type == "SkipSimplifiedLayerNormalization";
    const bool plain = norm->domain.empty() && (norm->op_type == "SimplifiedLayerNormalization" || norm->op_type == "RMSNormalization");
    if (!skip && !plain) continue;
    if (plain && norm->attr_i("axis", -1) != -1) continue;
    if (skip && norm->has_input(3)) continue;
    const std::string gamma = norm->input(skip ? 2 : 1);
    int64_t K = 0;
    if (!IsConst1D(g, gamma, &K)) continue;
    const at::ScalarType gt = g.GetConstant(gamma)->scalar_type();
    if (gt != at::kHalf && gt != at::kBFloat16) continue;
    bool extra_used = false;
    for (size_t o = 1; o < norm->outputs.size(); ++o) {
      if (skip && o == 3) continue;
      if (norm->has_output(o) && (g.NumConsumers(norm->outputs[o]) > 0 || g.IsGraphOutput(norm->outputs[o]))) extra_used = true;
    }
    if (extra_used) continue;
    const std::string ln_out = norm->outputs[0];
    Node* cons = SoleConsumer(g, ln_out);
    if (!cons || cons->inputs.empty() || cons->inputs[0] != ln_out) continue;
    int kind = 0;  // 1 MatMul, 2 FusedGemm, 3 GemmSwiGLU
    if (cons->domain.empty() && cons->op_type == "MatMul" && IsHalfWeight2D(g, cons->inputs[1]) &&
        g.GetConstant(cons->inputs[1])->size(0) == K && g.GetConstant(cons->inputs[1])->scalar_type() == gt)
      kind = 1;
    else if (cons->domain == kFusedDomain && cons->op_type == "FusedGemm" && cons->attr_i("all_reduce", 0) == 0 &&
             cons->attr_f("rms_eps", 0.f) == 0.f && g.GetConstant(cons->inputs[1]) && g.GetConstant(cons->inputs[1])->size(0) == K)
      kind = 2;
    else if (cons->domain == kFusedDomain && cons->op_type == "GemmSwiGLU" && cons->attr_f("rms_eps", 0.f) == 0.f &&
             g.GetConstant(cons->inputs[1]) && g.GetConstant(cons->inputs[1])->size(0) == K)
      kind = 3;
    if (!kind) continue;
    std::string x_new = norm->inputs[0];
    if (skip) {
      Node* prod = g.Producer(norm->inputs[0]);
      if (!prod || g.NumConsumers(prod->outputs[0]) != 1 || g.IsGraphOutput(prod->outputs[0])) continue;
      const bool p_mm = prod->domain.empty() && prod->op_type == "MatMul" && IsHalfWeight2D(g, prod->inputs[1]) && !g.GetConstant(prod->inputs[0]);
      const bool p_fg = prod->domain == kFusedDomain && prod->op_type == "FusedGemm" && !prod->has_input(3);
      if (!p_mm && !p_fg) continue;
      const std::string sum = norm->has_output(3) ? norm->outputs[3] : g.UniqueName(ln_out + "_sum");
      if (p_mm) {
        Node* f = g.AddNode("FusedGemm", {prod->inputs[0], prod->inputs[1], "", norm->inputs[1]}, {sum}, kFusedDomain,
                            g.UniqueName("FusedGemm"));
        f->set_attr_s("activation", "none");
        g.RemoveNode(prod);
      } else {
        if (prod->inputs.size() < 4) prod->inputs.resize(4);
        prod->inputs[3] = norm->inputs[1];
        prod->outputs[0] = sum;
      }
      x_new = sum;
    }
    const float eps = norm->attr_f("epsilon", 1e-5f);
    if (kind == 1) {
      Node* f = g.AddNode("FusedGemm", {x_new, cons->inputs[1], "", "", gamma}, cons->outputs, kFusedDomain, g.UniqueName("FusedGemm"));
      f->set_attr_s("activation", "none");
      f->set_attr_f("rms_eps", eps);
      g.RemoveNode(cons);
    } else {
      const size_t gi = kind == 2 ? 4 : 3;
      if (cons->inputs.size() < gi + 1) cons->inputs.resize(gi + 1);
      cons->inputs[0] = x_new;
      cons->inputs[gi] = gamma;
      cons->set_attr_f("rms_eps", eps);
    }
    g.RemoveNode(norm);
    g.Invalidate();
    ++count;
  }
  return count;
}

// ---- 4-bit weights (com.microsoft.MatMulNBits) in the GPU lowering.
// (a) AllReduce(MatMulNBits(x, ...)) [+ residual Add]  ->  the MatMulNBits node carries all_reduce = 1 (and the residual
//     as input 6): the decode kernel finishes the row-parallel sum over NVLink itself, so a tensor-parallel decode step
//     holds no library collective and can be captured in a CUDA graph.
// (b) Mul(silu(MatMulNBits(x, Wg)), MatMulNBits(x, Wu))  ->  one MatMulNBits over the stacked gate | up rows followed by
//     com.ortb200.SwiGLU (a streaming kernel): two weight passes and three element-wise launches become two launches.
int NBitsAllReduceFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  if (c.world_size <= 1) return 0;
  for (Node* ar : g.Nodes()) {
    if (ar->op_type != "AllReduce" || ar->domain != kMSDomain || ar->inputs.size() != 1) continue;
    Node* p = g.Producer(ar->inputs[0]);
    if (!p || p->op_type != "MatMulNBits" || p->domain != kMSDomain || g.NumConsumers(p->outputs[0]) != 1 || p->has_input(5)) continue;
    std::string out = ar->outputs[0], residual;
    Node* add = SoleConsumer(g, out);
    if (add && add->op_type == "Add" && add->domain.empty() && add->inputs.size() == 2) {
      for (int s = 0; s < 2; ++s)
        if (add->inputs[1 - s] == out && !g.GetConstant(add->inputs[s]) && add->inputs[s] != out) residual = add->inputs[s];
    }
    p->set_attr_i("all_reduce", 1);
    if (!residual.empty()) {
      p->inputs.resize(7);
      p->inputs[6] = residual;
      p->outputs[0] = add->outputs[0];
      g.RemoveNode(add);
    } else {
      p->outputs[0] = out;
    }
    g.RemoveNode(ar);
    g.Invalidate();
    ++count;
  }
  return count;
}

int NBitsSwiGLUFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* top : g.Nodes()) {
    if (top->op_type != "Mul" || !top->domain.empty() || top->inputs.size() != 2) continue;
    for (int s = 0; s < 2; ++s) {
      Node* silu = g.Producer(top->inputs[s]);
      Node* up = g.Producer(top->inputs[1 - s]);
      if (!silu || !up) continue;
      std::string gate_out;
      Node* sig = nullptr;
      if (!MatchSilu(g, silu, &gate_out, &sig)) continue;
      Node* gate = g.Producer(gate_out);
      auto is_q = [&](Node* n) { return n && n->op_type == "MatMulNBits" && n->domain == kMSDomain && n->inputs.size() >= 3 && !n->has_input(3) && !n->has_input(4) && !n->has_input(5); };
      if (!is_q(gate) || !is_q(up) || gate->inputs[0] != up->inputs[0]) continue;
      if (gate->attr_i("K", 0) != up->attr_i("K", 0) || gate->attr_i("N", 0) != up->attr_i("N", 0) || gate->attr_i("bits", 4) != up->attr_i("bits", 4) ||
          gate->attr_i("block_size", 32) != up->attr_i("block_size", 32))
        continue;
      const at::Tensor *bg = g.GetConstant(gate->inputs[1]), *bu = g.GetConstant(up->inputs[1]);
      const at::Tensor *sg = g.GetConstant(gate->inputs[2]), *su = g.GetConstant(up->inputs[2]);
      if (!bg || !bu || !sg || !su || bg->sizes() != bu->sizes() || sg->sizes() != su->sizes()) continue;
      if (g.NumConsumers(gate_out) != 2 || g.NumConsumers(up->outputs[0]) != 1 || g.NumConsumers(silu->outputs[0]) != 1) continue;
      const int64_t I = gate->attr_i("N", 0);
      const std::string bn = g.UniqueName(gate->inputs[1] + "_gate_up"), sn = g.UniqueName(gate->inputs[2] + "_gate_up");
      g.AddInitializer(bn, at::cat({*bg, *bu}, 0).contiguous());
      g.AddInitializer(sn, at::cat({sg->reshape({I, -1}), su->reshape({I, -1})}, 0).contiguous());
      const std::string gu = g.UniqueName(top->outputs[0] + "_gate_up");
      Node* mm = g.AddNode("MatMulNBits", {gate->inputs[0], bn, sn}, {gu}, kMSDomain, g.UniqueName("MatMulNBits_gate_up"));
      mm->set_attr_i("K", gate->attr_i("K", 0));
      mm->set_attr_i("N", 2 * I);
      mm->set_attr_i("bits", gate->attr_i("bits", 4));
      mm->set_attr_i("block_size", gate->attr_i("block_size", 32));
      g.AddNode("SwiGLU", {gu}, {top->outputs[0]}, kFusedDomain, g.UniqueName("SwiGLU"));
      g.RemoveNode(top);
      g.RemoveNode(silu);
      g.RemoveNode(sig);
      g.RemoveNode(gate);
      g.RemoveNode(up);
      ++count;
      break;
    }
  }
  return count;
}

}  // namespace

void AddGpuPasses(std::vector<Pass>& v) {
  v.push_back({"NBitsSwiGLUFusion", 2, true, NBitsSwiGLUFusion});
  v.push_back({"NBitsAllReduceFusion", 2, true, NBitsAllReduceFusion});
  v.push_back({"SwiGLUFusion", 2, true, SwiGLUFusion});
  v.push_back({"AllGatherMatMulFusion", 2, true, AllGatherMatMulFusion});
  v.push_back({"MatMulAllReduceFusion", 2, true, MatMulAllReduceFusion});
  v.push_back({"AllReduceResidualFusion", 2, true, AllReduceResidualFusion});
  v.push_back({"GemmEpilogueFusion", 2, true, GemmEpilogueFusion});
  v.push_back({"RmsNormGemmFusion", 2, true, RmsNormGemmFusion});
}

}  // namespace opt
}  // namespace ortb
