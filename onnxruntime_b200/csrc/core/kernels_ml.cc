// ai.onnx.ml operators (numeric forms): tree ensembles, linear models, SVM regression, feature transforms.
// Reference kernels: onnxruntime/core/providers/cpu/ml/ (tree_ensemble_*.cc, linearclassifier.cc, linearregressor.cc,
// svmregressor.cc, scaler.cc, normalizer.cc, binarizer.cc, imputer.cc, onehotencoder.cc, array_feature_extractor.cc,
// feature_vectorizer.cc; score post-processing: ml_common.h).  These models are small and branchy: they run on the host
// in double precision, whatever device the session uses.  String labels / map types are not tensor types here.
#include <ATen/ATen.h>

#include <algorithm>
#include <cstdio>
#include <cmath>
#include <limits>
#include <map>

#include "kernel.h"
#include "string_table.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* ML = "ai.onnx.ml";

enum class Post { NONE, SOFTMAX, LOGISTIC, SOFTMAX_ZERO, PROBIT };

Post ParsePost(const std::string& s) {
  if (s == "SOFTMAX") return Post::SOFTMAX;
  if (s == "LOGISTIC") return Post::LOGISTIC;
  if (s == "SOFTMAX_ZERO") return Post::SOFTMAX_ZERO;
  if (s == "PROBIT") return Post::PROBIT;
  ORTB_ENFORCE_ARG(s.empty() || s == "NONE", "unknown post_transform '", s, "'");
  return Post::NONE;
}

double Logistic(double x) { return 1.0 / (1.0 + std::exp(-x)); }

// inverse of the standard normal CDF (Winitzki's approximation of erfinv, the form the reference uses)
double Probit(double p) {
  const double x = 2.0 * p - 1.0, sgn = x < 0 ? -1.0 : 1.0;
  const double ln = std::log((1.0 - x) * (1.0 + x));
  const double a = 0.147, t = 2.0 / (M_PI * a) + 0.5 * ln;
  return 1.41421356 * sgn * std::sqrt(std::sqrt(t * t - ln / a) - t);
}

// scores of one sample -> transformed scores (ml_common.h write_scores).  add_second_class: -1 none; 0 / 1 = a single
// score from all-positive weights becomes [1 - s, s]; 2 / 3 = from mixed weights becomes [-s, s].
std::vector<double> PostProcess(std::vector<double> s, Post post, int add_second_class) {
  if (s.size() >= 2) {
    switch (post) {
      case Post::PROBIT:
        for (auto& v : s) v = Probit(v);
        break;
      case Post::LOGISTIC:
        for (auto& v : s) v = Logistic(v);
        break;
      case Post::SOFTMAX:
      case Post::SOFTMAX_ZERO: {
        double mx = -std::numeric_limits<double>::infinity();
        for (double v : s) mx = std::max(mx, v);
        double sum = 0;
        for (auto& v : s) {
          if (post == Post::SOFTMAX_ZERO && v == 0.0) continue;  // zeros stay zero
          v = std::exp(v - mx);
          sum += v;
        }
        for (auto& v : s)
          if (!(post == Post::SOFTMAX_ZERO && v == 0.0)) v /= sum;
        break;
      }
      case Post::NONE:
        break;
    }
    return s;
  }
  if (s.size() == 1) {
    if (post == Post::PROBIT) return {Probit(s[0])};
    if (add_second_class >= 0) {
      const double v = s[0];
      if (post == Post::LOGISTIC) return {Logistic(-v), Logistic(v)};
      if (add_second_class <= 1) return {1.0 - v, v};
      return {-v, v};
    }
  }
  return s;
}

at::Tensor HostDouble(const at::Tensor& t) { return t.to(at::kCPU, at::kDouble).contiguous(); }

std::vector<double> AttrDoubles(const Node& n, const std::string& name) {
  std::vector<float> f = n.attr_floats(name);
  return std::vector<double>(f.begin(), f.end());
}

// ------------------------------------------------------------------------------------------------ tree ensembles
struct TreeEnsemble {
  struct TreeNode {
    int mode = 0;  // 0 leaf, 1 <=, 2 <, 3 >=, 4 >, 5 ==, 6 !=, 7 member of `members`
    std::vector<double> members;
    int64_t feature = 0;
    double value = 0;
    int64_t yes = -1, no = -1;  // indices into `nodes`
    bool missing_true = false;
    std::vector<std::pair<int64_t, double>> weights;  // leaf: (target or class index, weight)
  };
  std::vector<TreeNode> nodes;
  std::vector<int64_t> roots;
  int64_t n_outputs = 1;
  int aggregate = 0;  // 0 SUM, 1 AVERAGE, 2 MIN, 3 MAX
  Post post = Post::NONE;
  std::vector<double> base;
  bool weights_all_positive = true;

  void Build(const Node& n, bool classifier) {
    const char* prefix = classifier ? "class" : "target";
    const std::vector<int64_t> tree_ids = n.attr_ints("nodes_treeids"), node_ids = n.attr_ints("nodes_nodeids"),
                               features = n.attr_ints("nodes_featureids"), yes = n.attr_ints("nodes_truenodeids"),
                               no = n.attr_ints("nodes_falsenodeids"), miss = n.attr_ints("nodes_missing_value_tracks_true");
    const std::vector<double> values = AttrDoubles(n, "nodes_values");
    const std::vector<std::string> modes = n.attr_strings("nodes_modes");
    const size_t N = tree_ids.size();
    ORTB_ENFORCE_ARG(node_ids.size() == N && features.size() == N && yes.size() == N && no.size() == N && values.size() == N && modes.size() == N,
                     "tree ensemble: the nodes_* attributes differ in length");
    static const std::map<std::string, int> mode_of = {{"LEAF", 0}, {"BRANCH_LEQ", 1}, {"BRANCH_LT", 2}, {"BRANCH_GTE", 3},
                                                        {"BRANCH_GT", 4}, {"BRANCH_EQ", 5}, {"BRANCH_NEQ", 6}};
    std::map<std::pair<int64_t, int64_t>, int64_t> index;
    nodes.resize(N);
    for (size_t i = 0; i < N; ++i) index[{tree_ids[i], node_ids[i]}] = static_cast<int64_t>(i);
    std::vector<bool> is_child(N, false);
    for (size_t i = 0; i < N; ++i) {
      auto m = mode_of.find(modes[i]);
      ORTB_ENFORCE_ARG(m != mode_of.end(), "tree ensemble: unknown node mode '", modes[i], "'");
      TreeNode& t = nodes[i];
      t.mode = m->second;
      t.feature = features[i];
      t.value = values[i];
      t.missing_true = i < miss.size() && miss[i] != 0;
      if (t.mode != 0) {
        auto y = index.find({tree_ids[i], yes[i]}), f = index.find({tree_ids[i], no[i]});
        ORTB_ENFORCE_ARG(y != index.end() && f != index.end(), "tree ensemble: a branch points to a node that does not exist");
        t.yes = y->second;
        t.no = f->second;
        is_child[static_cast<size_t>(t.yes)] = is_child[static_cast<size_t>(t.no)] = true;
      }
    }
    for (size_t i = 0; i < N; ++i)
      if (!is_child[i]) roots.push_back(static_cast<int64_t>(i));
    const std::vector<int64_t> w_tree = n.attr_ints(std::string(prefix) + "_treeids"), w_node = n.attr_ints(std::string(prefix) + "_nodeids"),
                               w_id = n.attr_ints(std::string(prefix) + "_ids");
    const std::vector<double> w = AttrDoubles(n, std::string(prefix) + "_weights");
    ORTB_ENFORCE_ARG(w_tree.size() == w.size() && w_node.size() == w.size() && w_id.size() == w.size(), "tree ensemble: the leaf weight attributes differ in length");
    for (size_t i = 0; i < w.size(); ++i) {
      auto it = index.find({w_tree[i], w_node[i]});
      ORTB_ENFORCE_ARG(it != index.end(), "tree ensemble: a weight belongs to a node that does not exist");
      nodes[static_cast<size_t>(it->second)].weights.emplace_back(w_id[i], w[i]);
      if (w[i] < 0) weights_all_positive = false;
    }
    const std::string agg = n.attr_s("aggregate_function", "SUM");
    aggregate = agg == "AVERAGE" ? 1 : (agg == "MIN" ? 2 : (agg == "MAX" ? 3 : 0));
    post = ParsePost(n.attr_s("post_transform", "NONE"));
    base = AttrDoubles(n, "base_values");
  }

  // per-output aggregated scores of one sample (without base values)
  void Evaluate(const double* x, int64_t n_features, std::vector<double>* out) const {
    std::vector<bool> seen(static_cast<size_t>(n_outputs), false);
    out->assign(static_cast<size_t>(n_outputs), 0.0);
    for (int64_t root : roots) {
      int64_t i = root;
      while (nodes[static_cast<size_t>(i)].mode != 0) {
        const TreeNode& t = nodes[static_cast<size_t>(i)];
        ORTB_ENFORCE_ARG(t.feature >= 0 && t.feature < n_features, "tree ensemble: feature index ", t.feature, " out of range");
        const double v = x[t.feature];
        bool go;
        if (std::isnan(v)) {
          go = t.missing_true;
        } else {
          switch (t.mode) {
            case 1: go = v <= t.value; break;
            case 2: go = v < t.value; break;
            case 3: go = v >= t.value; break;
            case 4: go = v > t.value; break;
            case 5: go = v == t.value; break;
            case 7: go = std::find(t.members.begin(), t.members.end(), v) != t.members.end(); break;
            default: go = v != t.value; break;
          }
        }
        i = go ? t.yes : t.no;
      }
      for (auto& kv : nodes[static_cast<size_t>(i)].weights) {
        ORTB_ENFORCE_ARG(kv.first >= 0 && kv.first < n_outputs, "tree ensemble: target / class index out of range");
        double& acc = (*out)[static_cast<size_t>(kv.first)];
        const bool first = !seen[static_cast<size_t>(kv.first)];
        seen[static_cast<size_t>(kv.first)] = true;
        if (aggregate == 2) acc = first ? kv.second : std::min(acc, kv.second);
        else if (aggregate == 3) acc = first ? kv.second : std::max(acc, kv.second);
        else acc += kv.second;
      }
    }
    if (aggregate == 1 && !roots.empty())
      for (auto& v : *out) v /= static_cast<double>(roots.size());
  }
};

// ai.onnx.ml TreeEnsemble (opset 5): one operator for regression and classification scores, with tensor-valued
// attributes; interior nodes and leaves are numbered separately (nodes_trueleafs / nodes_falseleafs say which array a
// child index points into), set membership is a node mode, aggregate and post transform are integer codes.
class TreeEnsembleV5Kernel final : public OpKernel {
 public:
  explicit TreeEnsembleV5Kernel(const OpKernelInfo& info) : OpKernel(info) {
    const Node& n = info.node;
    auto doubles = [&](const char* name) {
      at::Tensor t = n.attr_tensor(name);
      std::vector<double> v;
      if (t.defined()) {
        t = t.to(at::kCPU, at::kDouble).contiguous().reshape({-1});
        v.assign(t.data_ptr<double>(), t.data_ptr<double>() + t.numel());
      }
      return v;
    };
    const std::vector<double> splits = doubles("nodes_splits"), weights = doubles("leaf_weights"), member_values = doubles("membership_values");
    std::vector<int64_t> modes;
    {
      at::Tensor m = n.attr_tensor("nodes_modes");
      ORTB_ENFORCE_ARG(m.defined(), "TreeEnsemble: nodes_modes is required");
      m = m.to(at::kCPU, at::kLong).contiguous().reshape({-1});
      modes.assign(m.data_ptr<int64_t>(), m.data_ptr<int64_t>() + m.numel());
    }
    const std::vector<int64_t> features = n.attr_ints("nodes_featureids"), yes = n.attr_ints("nodes_truenodeids"), no = n.attr_ints("nodes_falsenodeids"),
                               yes_leaf = n.attr_ints("nodes_trueleafs"), no_leaf = n.attr_ints("nodes_falseleafs"),
                               miss = n.attr_ints("nodes_missing_value_tracks_true"), targets = n.attr_ints("leaf_targetids"),
                               roots = n.attr_ints("tree_roots");
    const size_t M = modes.size(), L = weights.size();
    ORTB_ENFORCE_ARG(splits.size() == M && features.size() == M && yes.size() == M && no.size() == M && yes_leaf.size() == M && no_leaf.size() == M &&
                         targets.size() == L,
                     "TreeEnsemble: the nodes_* / leaf_* attributes differ in length");
    static const int mode_map[7] = {1, 2, 3, 4, 5, 6, 7};
    trees_.nodes.resize(M + L);
    size_t member_pos = 0;
    for (size_t i = 0; i < M; ++i) {
      auto& t = trees_.nodes[i];
      ORTB_ENFORCE_ARG(modes[i] >= 0 && modes[i] <= 6, "TreeEnsemble: unknown node mode ", modes[i]);
      t.mode = mode_map[modes[i]];
      t.feature = features[i];
      t.value = splits[i];
      t.missing_true = i < miss.size() && miss[i] != 0;
      auto child = [&](int64_t idx, int64_t is_leaf) {
        const int64_t limit = is_leaf ? static_cast<int64_t>(L) : static_cast<int64_t>(M);
        ORTB_ENFORCE_ARG(idx >= 0 && idx < limit, "TreeEnsemble: a branch points to a node that does not exist");
        return is_leaf ? static_cast<int64_t>(M) + idx : idx;
      };
      t.yes = child(yes[i], yes_leaf[i]);
      t.no = child(no[i], no_leaf[i]);
      if (t.mode == 7) {  // this node's set: the values up to the next NaN
        while (member_pos < member_values.size() && !std::isnan(member_values[member_pos])) t.members.push_back(member_values[member_pos++]);
        ++member_pos;
      }
    }
    for (size_t j = 0; j < L; ++j) trees_.nodes[M + j].weights.emplace_back(targets[j], weights[j]);
    for (int64_t r : roots) {
      // a tree that is a single leaf names the leaf array when there are no interior nodes at all
      ORTB_ENFORCE_ARG(r >= 0 && r < static_cast<int64_t>(M == 0 ? L : M), "TreeEnsemble: tree root out of range");
      trees_.roots.push_back(M == 0 ? static_cast<int64_t>(M) + r : r);
    }
    trees_.n_outputs = n.attr_i("n_targets", 1);
    static const int agg_map[4] = {1, 0, 2, 3};  // attribute: 0 AVERAGE, 1 SUM, 2 MIN, 3 MAX
    const int64_t agg = n.attr_i("aggregate_function", 1);
    ORTB_ENFORCE_ARG(agg >= 0 && agg <= 3, "TreeEnsemble: unknown aggregate_function ", agg);
    trees_.aggregate = agg_map[agg];
    static const Post posts[5] = {Post::NONE, Post::SOFTMAX, Post::LOGISTIC, Post::SOFTMAX_ZERO, Post::PROBIT};
    const int64_t post = n.attr_i("post_transform", 0);
    ORTB_ENFORCE_ARG(post >= 0 && post <= 4, "TreeEnsemble: unknown post_transform ", post);
    trees_.post = posts[post];
  }

  void Compute(Ctx& ctx) const override {
    const at::Tensor& x_in = ctx.RequiredInput(0);
    at::Tensor x = HostDouble(x_in.dim() == 1 ? x_in.unsqueeze(0) : x_in);
    ORTB_ENFORCE_ARG(x.dim() == 2, "TreeEnsemble: input must be [N, features]");
    const int64_t N = x.size(0), F = x.size(1), T = trees_.n_outputs;
    at::Tensor y = at::empty({N, T}, at::kDouble);
    std::vector<double> s;
    for (int64_t i = 0; i < N; ++i) {
      trees_.Evaluate(x.data_ptr<double>() + i * F, F, &s);
      std::vector<double> z = PostProcess(s, trees_.post, -1);
      for (int64_t k = 0; k < T; ++k) y.data_ptr<double>()[i * T + k] = z[static_cast<size_t>(k)];
    }
    ctx.SetOutput(0, y.to(x_in.is_floating_point() ? x_in.scalar_type() : at::kFloat).to(x_in.device()));
  }

 private:
  TreeEnsemble trees_;
};

class TreeEnsembleKernel final : public OpKernel {
 public:
  TreeEnsembleKernel(const OpKernelInfo& info, bool classifier) : OpKernel(info), classifier_(classifier) {
    const Node& n = info.node;
    if (classifier) {
      labels_ = n.attr_ints("classlabels_int64s");
      if (n.has_attr("classlabels_strings") && !n.attr_strings("classlabels_strings").empty()) {
        string_labels_ = true;  // labels travel as ids of the string table
        labels_.clear();
        for (auto& s : n.attr_strings("classlabels_strings")) labels_.push_back(InternString(s));
      }
      // weights may name fewer classes than there are labels (binary models carry the positive class only)
      std::vector<int64_t> ids = n.attr_ints("class_ids");
      int64_t distinct = 0;
      for (int64_t id : ids) distinct = std::max(distinct, id + 1);
      std::sort(ids.begin(), ids.end());
      ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
      binary_ = labels_.size() == 2 && ids.size() == 1;
      trees_.n_outputs = binary_ ? 1 : std::max<int64_t>(static_cast<int64_t>(labels_.size()), distinct);
      single_id_ = ids.empty() ? 0 : ids[0];
    } else {
      trees_.n_outputs = n.attr_i("n_targets", 1);
    }
    trees_.Build(n, classifier);
    if (binary_)  // all weights sit on one class id: fold it to output 0
      for (auto& t : trees_.nodes)
        for (auto& kv : t.weights) kv.first = 0;
  }

  void Compute(Ctx& ctx) const override {
    const at::Tensor& x_in = ctx.RequiredInput(0);
    at::Tensor x = HostDouble(x_in.dim() == 1 ? x_in.unsqueeze(0) : x_in);
    ORTB_ENFORCE_ARG(x.dim() == 2, "tree ensemble: input must be [N, features]");
    const int64_t N = x.size(0), F = x.size(1);
    const int64_t n_out = classifier_ ? (binary_ ? 2 : trees_.n_outputs) : trees_.n_outputs;
    at::Tensor scores = at::empty({N, n_out}, at::kFloat);
    at::Tensor labels = classifier_ ? at::empty({N}, at::kLong) : at::Tensor();
    std::vector<double> s;
    for (int64_t i = 0; i < N; ++i) {
      trees_.Evaluate(x.data_ptr<double>() + i * F, F, &s);
      for (size_t k = 0; k < s.size() && k < trees_.base.size(); ++k) s[k] += trees_.base[k];
      int add_second = -1;
      if (classifier_) {
        int64_t label;
        if (binary_) {
          const bool positive = trees_.weights_all_positive ? s[0] > 0.5 : s[0] > 0.0;
          add_second = trees_.weights_all_positive ? (positive ? 0 : 1) : (positive ? 2 : 3);
          label = positive ? labels_[1] : labels_[0];
        } else {
          const size_t best = static_cast<size_t>(std::max_element(s.begin(), s.end()) - s.begin());
          label = best < labels_.size() ? labels_[best] : static_cast<int64_t>(best);
        }
        labels.data_ptr<int64_t>()[i] = label;
      }
      std::vector<double> z = PostProcess(s, trees_.post, add_second);
      for (int64_t k = 0; k < n_out; ++k) scores.data_ptr<float>()[i * n_out + k] = static_cast<float>(k < static_cast<int64_t>(z.size()) ? z[static_cast<size_t>(k)] : 0.0);
    }
    if (classifier_) {
      if (string_labels_) ctx.SetOutputStrings(0, labels);
      else ctx.SetOutput(0, labels.to(x_in.device()));
      if (ctx.OutputCount() > 1) ctx.SetOutput(1, scores.to(x_in.device()));
    } else {
      ctx.SetOutput(0, scores.to(x_in.device()));
    }
  }

 private:
  bool classifier_, binary_ = false, string_labels_ = false;
  TreeEnsemble trees_;
  std::vector<int64_t> labels_;
  int64_t single_id_ = 0;
};

// ------------------------------------------------------------------------------------------------ linear models
void LinearImpl(Ctx& ctx, bool classifier) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = HostDouble(x_in.dim() == 1 ? x_in.unsqueeze(0) : x_in);
  const int64_t N = x.size(0), F = x.size(1);
  const std::vector<double> coef = AttrDoubles(n, "coefficients"), icpt = AttrDoubles(n, "intercepts");
  ORTB_ENFORCE_ARG(F > 0 && coef.size() % static_cast<size_t>(F) == 0, "linear model: coefficients do not match ", F, " features");
  const int64_t rows = static_cast<int64_t>(coef.size()) / F;
  at::Tensor W = at::tensor(coef, at::kDouble).reshape({rows, F});
  at::Tensor s = at::matmul(x, W.t());
  if (!icpt.empty()) s = s + at::tensor(icpt, at::kDouble).reshape({1, -1});
  const Post post = ParsePost(n.attr_s("post_transform", "NONE"));
  std::vector<int64_t> labels = classifier ? n.attr_ints("classlabels_ints") : std::vector<int64_t>();
  const bool string_labels = classifier && n.has_attr("classlabels_strings") && !n.attr_strings("classlabels_strings").empty();
  if (string_labels) {
    labels.clear();
    for (auto& s : n.attr_strings("classlabels_strings")) labels.push_back(InternString(s));
  }
  const bool binary = classifier && rows == 1 && labels.size() == 2;
  const int64_t n_out = binary ? 2 : rows;
  at::Tensor scores = at::empty({N, n_out}, at::kFloat);
  at::Tensor lab = classifier ? at::empty({N}, at::kLong) : at::Tensor();
  for (int64_t i = 0; i < N; ++i) {
    std::vector<double> row(s.data_ptr<double>() + i * rows, s.data_ptr<double>() + (i + 1) * rows);
    int add_second = -1;
    if (classifier) {
      if (binary) {
        const bool positive = row[0] > 0;
        add_second = positive ? 2 : 3;
        lab.data_ptr<int64_t>()[i] = positive ? labels[1] : labels[0];
      } else {
        const size_t best = static_cast<size_t>(std::max_element(row.begin(), row.end()) - row.begin());
        lab.data_ptr<int64_t>()[i] = best < labels.size() ? labels[best] : static_cast<int64_t>(best);
      }
    }
    std::vector<double> z = PostProcess(row, post, add_second);
    for (int64_t k = 0; k < n_out; ++k) scores.data_ptr<float>()[i * n_out + k] = static_cast<float>(z[static_cast<size_t>(k)]);
  }
  if (classifier) {
    if (string_labels) ctx.SetOutputStrings(0, lab);
    else ctx.SetOutput(0, lab.to(x_in.device()));
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, scores.to(x_in.device()));
  } else {
    ctx.SetOutput(0, scores.to(x_in.device()));
  }
}

// SVMRegressor: sum_i coef_i K(sv_i, x) + rho (support-vector form) or w . x + rho (n_supports = 0, linear kernel)
void SvmRegressorImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = HostDouble(x_in.dim() == 1 ? x_in.unsqueeze(0) : x_in);
  const int64_t F = x.size(1), nsv = n.attr_i("n_supports", 0);
  const std::vector<double> coef = AttrDoubles(n, "coefficients"), rho = AttrDoubles(n, "rho"), kp = AttrDoubles(n, "kernel_params");
  const std::string kernel = n.attr_s("kernel_type", "LINEAR");
  const double gamma = kp.size() > 0 ? kp[0] : 0.0, coef0 = kp.size() > 1 ? kp[1] : 0.0, degree = kp.size() > 2 ? kp[2] : 0.0;
  auto K = [&](const at::Tensor& a, const at::Tensor& b) {  // [N, F] x [S, F] -> [N, S]
    if (kernel == "RBF") return at::exp(-gamma * at::cdist(a, b, 2.0, 2).pow(2));
    at::Tensor dot = at::matmul(a, b.t());
    if (kernel == "POLY") return (gamma * dot + coef0).pow(degree);
    if (kernel == "SIGMOID") return at::tanh(gamma * dot + coef0);
    ORTB_ENFORCE_ARG(kernel == "LINEAR", "SVMRegressor: unknown kernel_type '", kernel, "'");
    return dot;
  };
  at::Tensor y;
  if (nsv > 0) {
    at::Tensor sv = at::tensor(AttrDoubles(n, "support_vectors"), at::kDouble).reshape({nsv, F});
    y = at::matmul(K(x, sv), at::tensor(coef, at::kDouble).reshape({nsv, 1}));
  } else {
    y = K(x, at::tensor(coef, at::kDouble).reshape({1, F}));
  }
  if (!rho.empty()) y = y + rho[0];
  if (n.attr_i("one_class", 0)) y = at::where(y > 0, at::ones_like(y), -at::ones_like(y));
  ctx.SetOutput(0, y.to(at::kFloat).to(x_in.device()));
}

// [N, F] x [S, F] -> [N, S] kernel matrix (kernel_params: gamma, coef0, degree)
at::Tensor SvmKernel(const std::string& kernel, const std::vector<double>& kp, const at::Tensor& a, const at::Tensor& b) {
  const double gamma = kp.size() > 0 ? kp[0] : 0.0, coef0 = kp.size() > 1 ? kp[1] : 0.0, degree = kp.size() > 2 ? kp[2] : 0.0;
  if (kernel == "RBF") return at::exp(-gamma * at::cdist(a, b, 2.0, 2).pow(2));
  at::Tensor dot = at::matmul(a, b.t());
  if (kernel == "POLY") return (gamma * dot + coef0).pow(degree);
  if (kernel == "SIGMOID") return at::tanh(gamma * dot + coef0);
  ORTB_ENFORCE_ARG(kernel == "LINEAR", "SVM: unknown kernel_type '", kernel, "'");
  return dot;
}

// Class probabilities from pairwise probabilities r[i][j] = P(class i | class i or j): the second method of Wu, Lin and
// Weng, "Probability estimates for multi-class classification by pairwise coupling" (2004), as in libsvm.
std::vector<double> CouplePairwise(int64_t k, const std::vector<double>& r) {
  std::vector<double> p(static_cast<size_t>(k), 1.0 / static_cast<double>(k)), Q(static_cast<size_t>(k * k), 0.0), Qp(static_cast<size_t>(k), 0.0);
  auto at = [k](int64_t i, int64_t j) { return static_cast<size_t>(i * k + j); };
  for (int64_t t = 0; t < k; ++t)
    for (int64_t j = 0; j < k; ++j) {
      if (j == t) continue;
      Q[at(t, t)] += r[at(j, t)] * r[at(j, t)];
      Q[at(t, j)] = -r[at(j, t)] * r[at(t, j)];
    }
  const double eps = 0.005 / static_cast<double>(k);
  for (int iter = 0; iter < 100; ++iter) {
    double pQp = 0;
    for (int64_t t = 0; t < k; ++t) {
      Qp[static_cast<size_t>(t)] = 0;
      for (int64_t j = 0; j < k; ++j) Qp[static_cast<size_t>(t)] += Q[at(t, j)] * p[static_cast<size_t>(j)];
      pQp += p[static_cast<size_t>(t)] * Qp[static_cast<size_t>(t)];
    }
    double worst = 0;
    for (int64_t t = 0; t < k; ++t) worst = std::max(worst, std::fabs(Qp[static_cast<size_t>(t)] - pQp));
    if (worst < eps) break;
    for (int64_t t = 0; t < k; ++t) {
      const double diff = (-Qp[static_cast<size_t>(t)] + pQp) / Q[at(t, t)];
      p[static_cast<size_t>(t)] += diff;
      pQp = (pQp + diff * (diff * Q[at(t, t)] + 2 * Qp[static_cast<size_t>(t)])) / ((1 + diff) * (1 + diff));
      for (int64_t j = 0; j < k; ++j) {
        Qp[static_cast<size_t>(j)] = (Qp[static_cast<size_t>(j)] + diff * Q[at(t, j)]) / (1 + diff);
        p[static_cast<size_t>(j)] /= (1 + diff);
      }
    }
  }
  return p;
}

// SVMClassifier.  With support vectors: one-vs-one decisions d(i, j) = sum over the support vectors of class i of
// coef[j - 1][v] K(x, v) + sum over those of class j of coef[i][v] K(x, v) + rho(i, j); d > 0 votes for i.  Scores are
// the decisions (more than two classes), [-d, d] (two classes; logistic of both with post_transform LOGISTIC) or, with
// prob_a / prob_b, the coupled class probabilities.  Without support vectors: one linear (kernelised) score per class.
void SvmClassifierImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = HostDouble(x_in.dim() == 1 ? x_in.unsqueeze(0) : x_in);
  const int64_t N = x.size(0), F = x.size(1);
  const std::vector<double> coef = AttrDoubles(n, "coefficients"), rho = AttrDoubles(n, "rho"), kp = AttrDoubles(n, "kernel_params"),
                            sv = AttrDoubles(n, "support_vectors"), prob_a = AttrDoubles(n, "prob_a"), prob_b = AttrDoubles(n, "prob_b");
  const std::vector<int64_t> per_class = n.attr_ints("vectors_per_class");
  const std::string kernel = n.attr_s("kernel_type", "LINEAR");
  const Post post = ParsePost(n.attr_s("post_transform", "NONE"));
  const bool string_labels = n.has_attr("classlabels_strings") && !n.attr_strings("classlabels_strings").empty();
  std::vector<int64_t> labels = n.attr_ints("classlabels_ints");
  if (string_labels) {
    labels.clear();
    for (auto& s : n.attr_strings("classlabels_strings")) labels.push_back(InternString(s));
  }
  const bool all_positive = std::all_of(coef.begin(), coef.end(), [](double v) { return v >= 0; });
  const bool svc = !sv.empty();
  const int64_t classes = svc ? static_cast<int64_t>(per_class.size()) : std::max<int64_t>(static_cast<int64_t>(labels.size()), 1);
  ORTB_ENFORCE_ARG(classes >= 1 && !rho.empty(), "SVMClassifier: needs classes and rho");
  at::Tensor lab = at::empty({N}, at::kLong);
  at::Tensor scores;
  auto pick = [&](size_t best, double max_weight, bool have_proba) -> int64_t {
    if (labels.size() == 2 && classes <= 2) {
      if (!have_proba && ((all_positive && max_weight >= 0.5) || (max_weight > 0 && !all_positive))) return labels[1];
      return labels[best];
    }
    if (classes <= 2) return max_weight > 0 ? (string_labels ? InternString("1") : 1) : (string_labels ? InternString("0") : 0);
    return best < labels.size() ? labels[best] : static_cast<int64_t>(best);
  };
  if (!svc) {
    ORTB_ENFORCE_ARG(static_cast<int64_t>(coef.size()) >= classes * F, "SVMClassifier: coefficients do not cover classes x features");
    at::Tensor W = at::tensor(coef, at::kDouble).narrow(0, 0, classes * F).reshape({classes, F});
    at::Tensor s = SvmKernel(kernel, kp, x, W) + rho[0];
    scores = at::empty({N, classes}, at::kFloat);
    for (int64_t i = 0; i < N; ++i) {
      std::vector<double> row(s.data_ptr<double>() + i * classes, s.data_ptr<double>() + (i + 1) * classes);
      const size_t best = static_cast<size_t>(std::max_element(row.begin(), row.end()) - row.begin());
      lab.data_ptr<int64_t>()[i] = classes == 2 ? pick(best, row[best], false) : (best < labels.size() ? labels[best] : static_cast<int64_t>(best));
      std::vector<double> z = PostProcess(row, post, -1);
      for (int64_t c = 0; c < classes; ++c) scores.data_ptr<float>()[i * classes + c] = static_cast<float>(z[static_cast<size_t>(c)]);
    }
  } else {
    int64_t V = 0;
    std::vector<int64_t> first;
    for (int64_t c : per_class) {
      first.push_back(V);
      V += c;
    }
    const int64_t pairs = classes * (classes - 1) / 2;
    ORTB_ENFORCE_ARG(static_cast<int64_t>(sv.size()) == V * F && static_cast<int64_t>(coef.size()) >= (classes - 1) * V &&
                         static_cast<int64_t>(rho.size()) >= pairs,
                     "SVMClassifier: support_vectors / coefficients / rho do not match vectors_per_class");
    const bool have_proba = !prob_a.empty();
    ORTB_ENFORCE_ARG(!have_proba || (static_cast<int64_t>(prob_a.size()) >= pairs && static_cast<int64_t>(prob_b.size()) >= pairs),
                     "SVMClassifier: prob_a / prob_b need one entry per pair of classes");
    at::Tensor Kx = SvmKernel(kernel, kp, x, at::tensor(sv, at::kDouble).reshape({V, F})).contiguous();  // [N, V]
    const int64_t width = have_proba ? classes : (classes > 2 ? pairs : 2);
    scores = at::empty({N, width}, at::kFloat);
    std::vector<double> dec(static_cast<size_t>(pairs));
    for (int64_t i = 0; i < N; ++i) {
      const double* k = Kx.data_ptr<double>() + i * V;
      std::vector<int64_t> votes(static_cast<size_t>(classes), 0);
      int64_t pidx = 0;
      for (int64_t a = 0; a < classes - 1; ++a)
        for (int64_t b = a + 1; b < classes; ++b, ++pidx) {
          double sum = rho[static_cast<size_t>(pidx)];
          for (int64_t m = 0; m < per_class[static_cast<size_t>(a)]; ++m) sum += coef[static_cast<size_t>((b - 1) * V + first[static_cast<size_t>(a)] + m)] * k[first[static_cast<size_t>(a)] + m];
          for (int64_t m = 0; m < per_class[static_cast<size_t>(b)]; ++m) sum += coef[static_cast<size_t>(a * V + first[static_cast<size_t>(b)] + m)] * k[first[static_cast<size_t>(b)] + m];
          dec[static_cast<size_t>(pidx)] = sum;
          ++votes[static_cast<size_t>(sum > 0 ? a : b)];
        }
      const size_t best = static_cast<size_t>(std::max_element(votes.begin(), votes.end()) - votes.begin());
      lab.data_ptr<int64_t>()[i] = pairs == 1 ? pick(best, 0.0, have_proba) : (best < labels.size() ? labels[best] : static_cast<int64_t>(best));
      std::vector<double> z;
      if (have_proba) {
        std::vector<double> r(static_cast<size_t>(classes * classes), 0.0);
        pidx = 0;
        for (int64_t a = 0; a < classes - 1; ++a)
          for (int64_t b = a + 1; b < classes; ++b, ++pidx) {
            const double v = dec[static_cast<size_t>(pidx)] * prob_a[static_cast<size_t>(pidx)] + prob_b[static_cast<size_t>(pidx)];
            const double pr = std::min(std::max(1.0 / (1.0 + std::exp(v)), 1e-7), 1.0 - 1e-7);
            r[static_cast<size_t>(a * classes + b)] = pr;
            r[static_cast<size_t>(b * classes + a)] = 1.0 - pr;
          }
        z = PostProcess(CouplePairwise(classes, r), post, -1);
      } else if (classes > 2) {
        z = PostProcess(dec, post, -1);
      } else {
        z = PostProcess({dec[0]}, post, post == Post::NONE ? 2 : 0);
      }
      for (int64_t c = 0; c < width; ++c) scores.data_ptr<float>()[i * width + c] = static_cast<float>(c < static_cast<int64_t>(z.size()) ? z[static_cast<size_t>(c)] : 0.0);
    }
  }
  if (string_labels) ctx.SetOutputStrings(0, lab);
  else ctx.SetOutput(0, lab.to(x_in.device()));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, scores.to(x_in.device()));
}

at::Tensor PerFeature(const std::vector<float>& v, const at::Tensor& like) {
  at::Tensor t = at::tensor(v, at::kFloat).to(like.device());
  return t.numel() == 1 ? t.reshape({}) : t;
}

}  // namespace

void RegisterMlKernels(KernelRegistry& r) {
  for (bool classifier : {false, true}) {
    KernelDef d;
    d.domain = ML;
    d.op_type = classifier ? "TreeEnsembleClassifier" : "TreeEnsembleRegressor";
    d.since_min = 1;
    d.since_max = kMax;
    d.factory = [classifier](const OpKernelInfo& info) { return std::make_unique<TreeEnsembleKernel>(info, classifier); };
    r.Register(std::move(d));
  }
  {
    KernelDef d;
    d.domain = ML;
    d.op_type = "TreeEnsemble";
    d.since_min = 5;
    d.since_max = kMax;
    d.factory = [](const OpKernelInfo& info) { return std::make_unique<TreeEnsembleV5Kernel>(info); };
    r.Register(std::move(d));
  }
  r.RegisterFn(ML, "LinearRegressor", 1, kMax, [](Ctx& ctx) { LinearImpl(ctx, false); });
  r.RegisterFn(ML, "LinearClassifier", 1, kMax, [](Ctx& ctx) { LinearImpl(ctx, true); });
  r.RegisterFn(ML, "SVMRegressor", 1, kMax, SvmRegressorImpl);
  r.RegisterFn(ML, "SVMClassifier", 1, kMax, SvmClassifierImpl);
  // ZipMap: the rows of [N, C] scores become N maps from class label to score
  r.RegisterFn(ML, "ZipMap", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor x = ctx.RequiredInput(0).to(at::kCPU, at::kFloat);
    if (x.dim() == 1) x = x.unsqueeze(0);
    ORTB_ENFORCE_ARG(x.dim() == 2, "ZipMap: input must be [C] or [N, C]");
    MapRows m;
    m.string_keys = n.has_attr("classlabels_strings") && !n.attr_strings("classlabels_strings").empty();
    std::vector<int64_t> keys = n.attr_ints("classlabels_int64s");
    if (m.string_keys) {
      keys.clear();
      for (auto& s : n.attr_strings("classlabels_strings")) keys.push_back(InternString(s));
    }
    ORTB_ENFORCE_ARG(static_cast<int64_t>(keys.size()) == x.size(1), "ZipMap: ", keys.size(), " class labels for ", x.size(1), " columns");
    m.keys = at::tensor(keys, at::kLong);
    m.values = x.contiguous();
    ctx.SetOutputMaps(0, std::move(m));
  });
  // CastMap: map<int64, string | float> -> [1, C] tensor.  DENSE: the values in ascending key order; SPARSE: position = key,
  // max_map entries, zeros elsewhere.  cast_to: TO_FLOAT / TO_INT64 / TO_STRING.
  r.RegisterFn(ML, "CastMap", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const MapRows* m = ctx.InputMaps(0);
    ORTB_ENFORCE_ARG(m != nullptr && !m->string_keys && m->values.size(0) == 1, "CastMap: the input must be one map with int64 keys");
    const std::string to = n.attr_s("cast_to", "TO_FLOAT"), form = n.attr_s("map_form", "DENSE");
    at::Tensor order = at::argsort(m->keys);
    at::Tensor keys = m->keys.index_select(0, order), vals = m->values[0].index_select(0, order);
    // every value as a double (strings are parsed) and as a string id (numbers are printed), then the asked-for one is used
    std::vector<std::string> text;
    at::Tensor numeric;
    if (m->string_values) {
      text = StringsOfTensor(vals);
      numeric = at::empty({vals.numel()}, at::kDouble);
      if (to != "TO_STRING")
        for (size_t i = 0; i < text.size(); ++i) numeric[static_cast<int64_t>(i)] = std::stod(text[i]);
    } else {
      numeric = vals.to(at::kDouble);
      if (to == "TO_STRING")
        for (int64_t i = 0; i < numeric.numel(); ++i) {
          const double v = numeric[i].item<double>();
          char buf[64];
          if (v == std::floor(v) && std::fabs(v) < 1e15) std::snprintf(buf, sizeof(buf), "%lld", static_cast<long long>(v));
          else std::snprintf(buf, sizeof(buf), "%g", v);
          text.emplace_back(buf);
        }
    }
    int64_t width = keys.numel();
    at::Tensor position = at::arange(width, at::kLong);
    if (form == "SPARSE") {
      width = n.attr_i("max_map", 1);
      position = keys;
      ORTB_ENFORCE_ARG(keys.numel() == 0 || (keys.min().item<int64_t>() >= 0 && keys.max().item<int64_t>() < width), "CastMap: a key lies outside [0, max_map)");
    }
    if (to == "TO_STRING") {
      at::Tensor ids = at::full({width}, InternString(form == "SPARSE" ? "0" : ""), at::kLong);
      std::vector<int64_t> v;
      for (auto& s : text) v.push_back(InternString(s));
      ids.index_put_({position}, at::tensor(v, at::kLong));
      ctx.SetOutputStrings(0, ids.reshape({1, width}));
      return;
    }
    at::Tensor out = at::zeros({width}, at::kDouble).index_put_({position}, numeric);
    ctx.SetOutput(0, out.reshape({1, width}).to(to == "TO_INT64" ? at::kLong : at::kFloat));
  });
  // DictVectorizer: map<string | int64, number> -> [1, vocabulary] tensor with the map's value at every vocabulary entry (0 when absent)
  r.RegisterFn(ML, "DictVectorizer", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const MapRows* m = ctx.InputMaps(0);
    ORTB_ENFORCE_ARG(m != nullptr && !m->string_values, "DictVectorizer: the input must be a map with numeric values");
    std::vector<int64_t> vocab = n.attr_ints("int64_vocabulary");
    if (m->string_keys) {
      vocab.clear();
      for (auto& s : n.attr_strings("string_vocabulary")) vocab.push_back(InternString(s));
    }
    at::Tensor hit = at::tensor(vocab, at::kLong).unsqueeze(1).eq(m->keys.unsqueeze(0)).to(at::kDouble);   // [V, C]
    at::Tensor out = at::matmul(m->values.to(at::kDouble), hit.t());                                         // [N, V]
    ctx.SetOutput(0, out.to(at::kFloat));
  });
  r.RegisterFn(ML, "Scaler", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0).to(at::kFloat);
    ctx.SetOutput(0, (x - PerFeature(ctx.node().attr_floats("offset"), x)) * PerFeature(ctx.node().attr_floats("scale"), x));
  });
  r.RegisterFn(ML, "Normalizer", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0).to(at::kFloat);
    const std::string norm = ctx.node().attr_s("norm", "MAX");
    at::Tensor d = norm == "L1" ? x.abs().sum(-1, true) : (norm == "L2" ? x.pow(2).sum(-1, true).sqrt() : x.abs().amax(-1, true));
    ctx.SetOutput(0, at::where(d == 0, x, x / d));
  });
  r.RegisterFn(ML, "Binarizer", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, (x > ctx.node().attr_f("threshold", 0.f)).to(x.scalar_type()));
  });
  r.RegisterFn(ML, "Imputer", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    if (x.is_floating_point()) {
      const float replaced = n.attr_f("replaced_value_float", 0.f);
      at::Tensor fill = PerFeature(n.attr_floats("imputed_value_floats"), x).to(x.scalar_type());
      at::Tensor hit = std::isnan(replaced) ? at::isnan(x) : (x == replaced);
      ctx.SetOutput(0, at::where(hit, fill.expand_as(x), x));
    } else {
      std::vector<int64_t> v = n.attr_ints("imputed_value_int64s");
      at::Tensor fill = at::tensor(v, at::kLong).to(x.device());
      if (fill.numel() == 1) fill = fill.reshape({});
      ctx.SetOutput(0, at::where(x == n.attr_i("replaced_value_int64", 0), fill.expand_as(x), x));
    }
  });
  r.RegisterFn(ML, "OneHotEncoder", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> cat_ids = n.attr_ints("cats_int64s");
    if (ctx.InputIsString(0)) {  // strings are ids of the string table: compare ids
      cat_ids.clear();
      for (auto& s : n.attr_strings("cats_strings")) cat_ids.push_back(InternString(s));
    }
    at::Tensor cats = at::tensor(cat_ids, at::kLong).to(x.device());
    at::Tensor hot = x.to(at::kLong).unsqueeze(-1) == cats;
    if (n.attr_i("zeros", 1) == 0) ORTB_ENFORCE_ARG(hot.any(-1).all().item<bool>(), "OneHotEncoder: a value is not among the categories (zeros = 0)");
    ctx.SetOutput(0, hot.to(at::kFloat));
  });
  r.RegisterFn(ML, "ArrayFeatureExtractor", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor idx = ctx.RequiredInput(1).to(x.device(), at::kLong).reshape({-1});
    at::Tensor y = x.index_select(x.dim() - 1, idx);
    ctx.SetOutput(0, x.dim() == 1 ? y.unsqueeze(0) : y);
  });
  r.RegisterFn(ML, "FeatureVectorizer", 1, kMax, [](Ctx& ctx) {
    std::vector<at::Tensor> parts;
    const std::vector<int64_t> dims = ctx.node().attr_ints("inputdimensions");
    for (int i = 0; i < ctx.InputCount(); ++i) {
      if (!ctx.HasInput(i)) continue;
      at::Tensor t = ctx.Input(i).to(at::kFloat);
      const int64_t width = i < static_cast<int>(dims.size()) ? dims[static_cast<size_t>(i)] : (t.dim() > 1 ? t.size(-1) : t.numel());
      t = t.dim() <= 1 ? t.reshape({1, -1}) : t.reshape({t.size(0), -1});
      parts.push_back(t.narrow(1, 0, std::min<int64_t>(width, t.size(1))));
    }
    ctx.SetOutput(0, at::cat(parts, 1));
  });
}

}  // namespace ortb
