// Shape / indexing / reduction / linear-algebra ONNX operators over ATen
// (device-agnostic).  Shape-like operands are declared as host inputs so the
// partitioner keeps them in CPU memory, as the reference's CUDA kernels do with
// InputMemoryType(OrtMemTypeCPUInput, i).
#include <ATen/ATen.h>

#include <algorithm>
#include <numeric>

#include "string_table.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

std::vector<int64_t> ToVec(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

int64_t NormAxis(int64_t axis, int64_t rank) {
  if (axis < 0) axis += rank;
  ORTB_ENFORCE_ARG(axis >= 0 && axis < std::max<int64_t>(rank, 1), "axis out of range");
  return axis;
}

at::Tensor FixNegative(const at::Tensor& idx, int64_t dim_size) {
  return at::where(idx < 0, idx + dim_size, idx);
}

std::vector<int64_t> AxesFrom(Ctx& ctx, int input_idx, const char* attr_name, int opset_input_since) {
  const Node& n = ctx.node();
  if (n.since_version >= opset_input_since) {
    if (ctx.HasInput(input_idx)) return ToVec(ctx.Input(input_idx));
    return {};
  }
  return n.attr_ints(attr_name);
}

using ReduceFn = std::function<at::Tensor(const at::Tensor&, at::IntArrayRef, bool)>;

void ReduceImpl(Ctx& ctx, int axes_input_since, const ReduceFn& fn) {
  const at::Tensor& x = ctx.RequiredInput(0);
  std::vector<int64_t> axes = AxesFrom(ctx, 1, "axes", axes_input_since);
  const bool keepdims = ctx.node().attr_i("keepdims", 1) != 0;
  if (axes.empty()) {
    if (ctx.node().attr_i("noop_with_empty_axes", 0) != 0) {
      ctx.SetOutput(0, x);
      return;
    }
    axes.resize(x.dim());
    std::iota(axes.begin(), axes.end(), 0);
  }
  for (auto& a : axes) a = NormAxis(a, x.dim());
  if (x.dim() == 0) {
    ctx.SetOutput(0, fn(x.reshape({1}), {0}, false).reshape({}));
    return;
  }
  ctx.SetOutput(0, fn(x, axes, keepdims));
}

void RegisterReduce(KernelRegistry& r, const std::string& name, int axes_input_since, ReduceFn fn) {
  r.RegisterFn("", name, 1, kMax, [axes_input_since, fn](Ctx& ctx) { ReduceImpl(ctx, axes_input_since, fn); }, {1});
}

at::Tensor AmaxMulti(const at::Tensor& x, at::IntArrayRef axes, bool keep, bool is_max) {
  return is_max ? at::amax(x, axes, keep) : at::amin(x, axes, keep);
}

at::Tensor ProdMulti(const at::Tensor& x, at::IntArrayRef axes, bool keep) {
  std::vector<int64_t> sorted(axes.begin(), axes.end());
  std::sort(sorted.begin(), sorted.end(), std::greater<int64_t>());
  at::Tensor y = x;
  for (int64_t a : sorted) y = at::prod(y, a, keep);
  return y;
}

void SoftmaxLike(Ctx& ctx, const std::function<at::Tensor(const at::Tensor&, int64_t)>& fn) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const Node& n = ctx.node();
  if (n.since_version >= 13) {
    ctx.SetOutput(0, fn(x, NormAxis(n.attr_i("axis", -1), x.dim())));
  } else {
    // legacy semantics: coerce to 2-D at `axis`, normalise the trailing block
    const int64_t axis = NormAxis(n.attr_i("axis", 1), x.dim());
    int64_t outer = 1;
    for (int64_t i = 0; i < axis; ++i) outer *= x.size(i);
    at::Tensor x2 = x.reshape({outer, -1});
    ctx.SetOutput(0, fn(x2, 1).reshape(x.sizes()));
  }
}

at::Tensor SliceImpl(at::Tensor x, const std::vector<int64_t>& starts, const std::vector<int64_t>& ends,
                     std::vector<int64_t> axes, std::vector<int64_t> steps) {
  const int64_t rank = x.dim();
  if (axes.empty()) {
    axes.resize(starts.size());
    std::iota(axes.begin(), axes.end(), 0);
  }
  if (steps.empty()) steps.assign(starts.size(), 1);
  ORTB_ENFORCE_ARG(starts.size() == ends.size() && starts.size() == axes.size() && steps.size() == axes.size(),
                   "Slice: starts/ends/axes/steps differ in length");
  for (size_t i = 0; i < axes.size(); ++i) {
    const int64_t ax = NormAxis(axes[i], rank);
    const int64_t dim = x.size(ax);
    const int64_t step = steps[i];
    ORTB_ENFORCE_ARG(step != 0, "Slice: step cannot be 0");
    int64_t s = starts[i], e = ends[i];
    if (s < 0) s += dim;
    if (e < 0) e += dim;
    if (step > 0) {
      s = std::min(std::max<int64_t>(s, 0), dim);
      e = std::min(std::max<int64_t>(e, 0), dim);
      x = at::slice(x, ax, s, std::max(s, e), step);
    } else {
      s = std::min(std::max<int64_t>(s, 0), dim - 1);
      e = std::min(std::max<int64_t>(e, -1), dim - 1);
      if (ends[i] < -dim) e = -1;  // "very negative" end means run through index 0
      std::vector<int64_t> idx;
      for (int64_t k = s; k > e; k += step) idx.push_back(k);
      at::Tensor index = at::tensor(idx, at::TensorOptions().dtype(at::kLong)).to(x.device());
      x = at::index_select(x, ax, index);
    }
  }
  return x;
}

std::vector<int64_t> ReshapeTarget(const at::Tensor& x, std::vector<int64_t> shape, bool allowzero) {
  for (size_t i = 0; i < shape.size(); ++i) {
    if (shape[i] == 0 && !allowzero) {
      ORTB_ENFORCE_ARG(static_cast<int64_t>(i) < x.dim(), "Reshape: 0 refers to a dimension the input does not have");
      shape[i] = x.size(i);
    }
  }
  return shape;
}

at::Tensor GatherND(const at::Tensor& data, const at::Tensor& indices_in, int64_t batch_dims) {
  at::Tensor indices = indices_in.to(at::kLong);
  const int64_t k = indices.size(-1);
  const int64_t r = data.dim();
  ORTB_ENFORCE_ARG(k <= r - batch_dims, "GatherND: last indices dim too large");
  // flatten batch dims
  int64_t batch = 1;
  for (int64_t i = 0; i < batch_dims; ++i) batch *= data.size(i);
  std::vector<int64_t> dshape = {batch};
  for (int64_t i = batch_dims; i < r; ++i) dshape.push_back(data.size(i));
  at::Tensor d = data.reshape(dshape);
  at::Tensor idx = indices.reshape({batch, -1, k});  // [batch, n, k]
  const int64_t n = idx.size(1);
  // linear index over the k indexed dims
  at::Tensor lin = at::zeros({batch, n}, idx.options());
  int64_t stride = 1;
  for (int64_t j = k - 1; j >= 0; --j) {
    at::Tensor ij = idx.select(2, j);
    ij = FixNegative(ij, d.size(1 + j));
    lin = lin + ij * stride;
    stride *= d.size(1 + j);
  }
  std::vector<int64_t> tail;
  int64_t tail_elems = 1;
  for (int64_t i = 1 + k; i < d.dim(); ++i) {
    tail.push_back(d.size(i));
    tail_elems *= d.size(i);
  }
  at::Tensor flat = d.reshape({batch, stride, tail_elems});
  at::Tensor g = at::gather(flat, 1, lin.unsqueeze(-1).expand({batch, n, tail_elems}));
  std::vector<int64_t> out_shape(indices.sizes().begin(), indices.sizes().end() - 1);
  out_shape.insert(out_shape.end(), tail.begin(), tail.end());
  return g.reshape(out_shape);
}

at::Tensor ScatterND(const at::Tensor& data, const at::Tensor& indices_in, const at::Tensor& updates,
                     const std::string& reduction) {
  at::Tensor out = data.clone();
  at::Tensor indices = indices_in.to(at::kLong);
  const int64_t k = indices.size(-1);
  at::Tensor idx = indices.reshape({-1, k});
  const int64_t n = idx.size(0);
  int64_t stride = 1;
  at::Tensor lin = at::zeros({n}, idx.options());
  for (int64_t j = k - 1; j >= 0; --j) {
    lin = lin + FixNegative(idx.select(1, j), data.size(j)) * stride;
    stride *= data.size(j);
  }
  int64_t tail_elems = 1;
  for (int64_t i = k; i < data.dim(); ++i) tail_elems *= data.size(i);
  at::Tensor flat = out.reshape({stride, tail_elems});
  at::Tensor upd = updates.reshape({n, tail_elems});
  at::Tensor index = lin.unsqueeze(-1).expand({n, tail_elems});
  if (reduction == "none") flat.scatter_(0, index, upd);
  else if (reduction == "add") flat.scatter_add_(0, index, upd);
  else if (reduction == "mul") flat.scatter_reduce_(0, index, upd, "prod");
  else if (reduction == "max") flat.scatter_reduce_(0, index, upd, "amax");
  else if (reduction == "min") flat.scatter_reduce_(0, index, upd, "amin");
  else ORTB_THROW(INVALID_ARGUMENT, "ScatterND: unknown reduction ", reduction);
  return flat.reshape(data.sizes());
}

at::Tensor ConstantValue(const Node& n) {
  if (n.has_attr("value")) return n.attr_tensor("value");  // a string tensor comes back as ids of the string table
  if (n.has_attr("sparse_value")) return n.attr_tensor("sparse_value");  // expanded: the kernels are dense
  if (n.has_attr("value_string")) return InternStrings({n.attr_s("value_string")}, {});
  if (n.has_attr("value_strings")) {
    const std::vector<std::string> v = n.attr_strings("value_strings");
    return InternStrings(v, {static_cast<int64_t>(v.size())});
  }
  if (n.has_attr("value_float")) return at::scalar_tensor(n.attr_f("value_float", 0.f), at::kFloat);
  if (n.has_attr("value_int")) return at::scalar_tensor(n.attr_i("value_int", 0), at::kLong);
  if (n.has_attr("value_floats")) return at::tensor(n.attr_floats("value_floats"), at::kFloat);
  if (n.has_attr("value_ints")) return at::tensor(n.attr_ints("value_ints"), at::kLong);
  ORTB_THROW(NOT_IMPLEMENTED, "Constant node '", n.name, "' has no supported value attribute");
}

class ConstantKernel final : public OpKernel {
 public:
  explicit ConstantKernel(const OpKernelInfo& info) : OpKernel(info) {
    value_ = ConstantValue(info.node).to(info.device);
    strings_ = ConstantHoldsStrings(info.node);
  }
  void Compute(Ctx& ctx) const override {
    if (strings_) ctx.SetOutputStrings(0, value_);
    else ctx.SetOutput(0, value_);
  }

 private:
  at::Tensor value_;
  bool strings_ = false;
};

}  // namespace

void RegisterTensorKernels(KernelRegistry& r) {
  // ---------------------------------------------------------------- shapes
  r.RegisterFn("", "Shape", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t rank = x.dim();
    int64_t start = ctx.node().attr_i("start", 0), end = ctx.node().attr_i("end", rank);
    if (start < 0) start += rank;
    if (end < 0) end += rank;
    start = std::min(std::max<int64_t>(start, 0), rank);
    end = std::min(std::max<int64_t>(end, 0), rank);
    std::vector<int64_t> dims;
    for (int64_t i = start; i < end; ++i) dims.push_back(x.size(i));
    ctx.SetOutput(0, at::tensor(dims, at::TensorOptions().dtype(at::kLong)));
  });
  r.RegisterFn("", "Size", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::scalar_tensor(ctx.RequiredInput(0).numel(), at::kLong));
  });
  r.RegisterFn("", "Reshape", 1, 4, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x.reshape(ReshapeTarget(x, ctx.node().attr_ints("shape"), false)));
  });
  r.RegisterFn("", "Reshape", 5, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x.reshape(ReshapeTarget(x, ToVec(ctx.RequiredInput(1)), ctx.node().attr_i("allowzero", 0) != 0)));
  }, {1});
  r.RegisterFn("", "Flatten", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t axis = ctx.node().attr_i("axis", 1);
    if (axis < 0) axis += x.dim();
    int64_t outer = 1;
    for (int64_t i = 0; i < axis; ++i) outer *= x.size(i);
    ctx.SetOutput(0, x.reshape({outer, outer == 0 ? 0 : (x.numel() / std::max<int64_t>(outer, 1))}));
  });
  r.RegisterFn("", "Squeeze", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> axes = AxesFrom(ctx, 1, "axes", 13);
    if (axes.empty()) {
      ctx.SetOutput(0, at::squeeze(x));
      return;
    }
    std::vector<int64_t> shape;
    std::vector<bool> drop(x.dim(), false);
    for (auto a : axes) drop[NormAxis(a, x.dim())] = true;
    for (int64_t i = 0; i < x.dim(); ++i) {
      if (drop[i]) ORTB_ENFORCE_ARG(x.size(i) == 1, "Squeeze: dimension ", i, " is not 1");
      else shape.push_back(x.size(i));
    }
    ctx.SetOutput(0, x.reshape(shape));
  }, {1});
  r.RegisterFn("", "Unsqueeze", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> axes = AxesFrom(ctx, 1, "axes", 13);
    const int64_t out_rank = x.dim() + static_cast<int64_t>(axes.size());
    for (auto& a : axes) a = NormAxis(a, out_rank);
    std::sort(axes.begin(), axes.end());
    at::Tensor y = x;
    for (auto a : axes) y = y.unsqueeze(a);
    ctx.SetOutput(0, y);
  }, {1});
  r.RegisterFn("", "Transpose", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> perm = ctx.node().attr_ints("perm");
    if (perm.empty()) {
      perm.resize(x.dim());
      std::iota(perm.rbegin(), perm.rend(), 0);
    }
    ctx.SetOutput(0, x.permute(perm).contiguous());
  });
  r.RegisterFn("", "Concat", 1, kMax, [](Ctx& ctx) {
    std::vector<at::Tensor> parts;
    for (int i = 0; i < ctx.InputCount(); ++i)
      if (ctx.HasInput(i)) parts.push_back(ctx.Input(i));
    ORTB_ENFORCE_ARG(!parts.empty(), "Concat needs at least one input");
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", 1), parts[0].dim());
    // mixed host/device operands (constants placed by first use) follow the first tensor
    for (auto& p : parts)
      if (p.device() != parts[0].device()) p = p.to(parts[0].device());
    ctx.SetOutput(0, at::cat(parts, axis));
  });
  r.RegisterFn("", "Split", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const Node& n = ctx.node();
    const int64_t axis = NormAxis(n.attr_i("axis", 0), x.dim());
    std::vector<int64_t> sizes;
    if (n.since_version >= 13) {
      if (ctx.HasInput(1)) sizes = ToVec(ctx.Input(1));
    } else {
      sizes = n.attr_ints("split");
    }
    const int64_t nout = n.has_attr("num_outputs") ? n.attr_i("num_outputs", 1) : ctx.OutputCount();
    if (sizes.empty()) {
      const int64_t dim = x.size(axis);
      const int64_t chunk = (dim + nout - 1) / nout;
      for (int64_t i = 0; i < nout; ++i) sizes.push_back(std::max<int64_t>(0, std::min(chunk, dim - i * chunk)));
    }
    std::vector<at::Tensor> parts = at::split_with_sizes(x, sizes, axis);
    for (int i = 0; i < ctx.OutputCount() && i < static_cast<int>(parts.size()); ++i) ctx.SetOutput(i, parts[i].contiguous());
  }, {1});
  r.RegisterFn("", "Slice", 1, 9, [](Ctx& ctx) {
    const Node& n = ctx.node();
    ctx.SetOutput(0, SliceImpl(ctx.RequiredInput(0), n.attr_ints("starts"), n.attr_ints("ends"), n.attr_ints("axes"), {}));
  });
  r.RegisterFn("", "Slice", 10, kMax, [](Ctx& ctx) {
    std::vector<int64_t> axes, steps;
    if (ctx.HasInput(3)) axes = ToVec(ctx.Input(3));
    if (ctx.HasInput(4)) steps = ToVec(ctx.Input(4));
    ctx.SetOutput(0, SliceImpl(ctx.RequiredInput(0), ToVec(ctx.RequiredInput(1)), ToVec(ctx.RequiredInput(2)), axes, steps)
                         .contiguous());
  }, {1, 2, 3, 4});
  r.RegisterFn("", "Expand", 8, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> shape = ToVec(ctx.RequiredInput(1));
    std::vector<int64_t> target = at::infer_size(x.sizes(), shape);
    ctx.SetOutput(0, x.expand(target).contiguous());
  }, {1});
  r.RegisterFn("", "Tile", 6, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, ctx.RequiredInput(0).repeat(ToVec(ctx.RequiredInput(1))));
  }, {1});
  r.RegisterFn("", "Pad", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const Node& n = ctx.node();
    std::vector<int64_t> pads, axes;
    at::Scalar value = 0;
    if (n.since_version >= 11 || !n.domain.empty()) {  // the com.microsoft form takes pads as an input, like opset 11
      pads = ToVec(ctx.RequiredInput(1));
      if (ctx.HasInput(2) && ctx.Input(2).numel() > 0) value = ctx.Input(2).cpu().reshape({-1})[0].item();
      if (ctx.HasInput(3)) axes = ToVec(ctx.Input(3));
    } else {
      pads = n.has_attr("pads") ? n.attr_ints("pads") : n.attr_ints("paddings");
      value = n.attr_f("value", 0.f);
    }
    const int64_t rank = x.dim();
    if (axes.empty()) {
      axes.resize(rank);
      std::iota(axes.begin(), axes.end(), 0);
    }
    ORTB_ENFORCE_ARG(pads.size() == axes.size() * 2, "Pad: pads must have 2 * len(axes) entries");
    std::vector<int64_t> begin(rank, 0), end(rank, 0);
    for (size_t i = 0; i < axes.size(); ++i) {
      const int64_t a = NormAxis(axes[i], rank);
      begin[a] = pads[i];
      end[a] = pads[i + axes.size()];
    }
    // ATen wants (last dim begin, last dim end, second-to-last begin, ...)
    std::vector<int64_t> tp;
    for (int64_t d = rank - 1; d >= 0; --d) {
      tp.push_back(begin[d]);
      tp.push_back(end[d]);
    }
    const std::string mode = n.attr_s("mode", "constant");
    if (mode == "constant") {
      ctx.SetOutput(0, at::constant_pad_nd(x, tp, value));
    } else {
      // drop leading zero pairs so that reflect/replicate see at most 3 padded dims
      while (tp.size() > 2 && tp[tp.size() - 1] == 0 && tp[tp.size() - 2] == 0) tp.resize(tp.size() - 2);
      const std::string tmode = mode == "reflect" ? "reflect" : (mode == "edge" ? "replicate" : "circular");
      const int64_t padded_dims = static_cast<int64_t>(tp.size() / 2);
      at::Tensor y = x;
      // torch needs (N, C, spatial...) for non-constant modes: add leading dims if necessary
      int64_t added = 0;
      while (y.dim() < padded_dims + 2) {
        y = y.unsqueeze(0);
        ++added;
      }
      if (y.dim() > padded_dims + 2) {
        // fold extra leading dims into one
        std::vector<int64_t> s = {-1, 1};
        for (int64_t d = y.dim() - padded_dims; d < y.dim(); ++d) s.push_back(y.size(d));
        at::Tensor folded = y.reshape(s);
        at::Tensor p = at::pad(folded, tp, tmode);
        std::vector<int64_t> os(x.sizes().begin(), x.sizes().end());
        for (int64_t d = 0; d < rank; ++d) os[d] = x.size(d) + begin[d] + end[d];
        ctx.SetOutput(0, p.reshape(os));
        return;
      }
      at::Tensor p = at::pad(y, tp, tmode);
      for (int64_t i = 0; i < added; ++i) p = p.squeeze(0);
      ctx.SetOutput(0, p);
    }
  }, {1, 2, 3});
  r.RegisterFn("", "Range", 11, kMax, [](Ctx& ctx) {
    const at::Tensor& s = ctx.RequiredInput(0);
    const at::Scalar start = s.cpu().item(), limit = ctx.RequiredInput(1).cpu().item(), delta = ctx.RequiredInput(2).cpu().item();
    ctx.SetOutput(0, at::arange(start, limit, delta, at::TensorOptions().dtype(s.scalar_type()).device(ctx.device())));
  }, {0, 1, 2});
  r.RegisterFn("", "ConstantOfShape", 9, kMax, [](Ctx& ctx) {
    std::vector<int64_t> shape = ToVec(ctx.RequiredInput(0));
    at::Tensor v = ctx.node().attr_tensor("value");
    if (!v.defined()) v = at::zeros({1}, at::kFloat);
    ctx.SetOutput(0, at::full(shape, v.reshape({-1})[0].item(), at::TensorOptions().dtype(v.scalar_type()).device(ctx.device())));
  }, {0});
  {
    KernelDef d;
    d.domain = "";
    d.op_type = "Constant";
    d.factory = [](const OpKernelInfo& info) { return std::make_unique<ConstantKernel>(info); };
    r.Register(std::move(d));
  }
  r.RegisterFn("", "Trilu", 14, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t k = ctx.HasInput(1) ? ctx.Input(1).cpu().item<int64_t>() : 0;
    ctx.SetOutput(0, ctx.node().attr_i("upper", 1) ? at::triu(x, k) : at::tril(x, k));
  }, {1});
  r.RegisterFn("", "EyeLike", 9, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t k = ctx.node().attr_i("k", 0);
    at::ScalarType dt = ctx.node().has_attr("dtype") ? ToTorchType(static_cast<int32_t>(ctx.node().attr_i("dtype", 1))) : x.scalar_type();
    at::Tensor out = at::zeros({x.size(0), x.size(1)}, x.options().dtype(dt));
    out.diagonal(k).fill_(1);
    ctx.SetOutput(0, out);
  });

  // ------------------------------------------------------- gather / scatter
  r.RegisterFn("", "Gather", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor idx = ctx.RequiredInput(1).to(at::kLong);
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
    if (idx.device() != x.device()) idx = idx.to(x.device());
    at::Tensor flat = FixNegative(idx.reshape({-1}), x.size(axis));
    at::Tensor g = at::index_select(x, axis, flat);
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().begin() + axis);
    shape.insert(shape.end(), idx.sizes().begin(), idx.sizes().end());
    shape.insert(shape.end(), x.sizes().begin() + axis + 1, x.sizes().end());
    ctx.SetOutput(0, g.reshape(shape));
  });
  r.RegisterFn("", "GatherElements", 11, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
    ctx.SetOutput(0, at::gather(x, axis, FixNegative(ctx.RequiredInput(1).to(at::kLong), x.size(axis))));
  });
  r.RegisterFn("", "GatherND", 11, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, GatherND(ctx.RequiredInput(0), ctx.RequiredInput(1), ctx.node().attr_i("batch_dims", 0)));
  });
  auto scatter_elements = [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
    at::Tensor idx = FixNegative(ctx.RequiredInput(1).to(at::kLong), x.size(axis));
    const at::Tensor& upd = ctx.RequiredInput(2);
    const std::string red = ctx.node().attr_s("reduction", "none");
    at::Tensor out = x.clone();
    if (red == "none") out.scatter_(axis, idx, upd);
    else if (red == "add") out.scatter_add_(axis, idx, upd);
    else if (red == "mul") out.scatter_reduce_(axis, idx, upd, "prod");
    else if (red == "max") out.scatter_reduce_(axis, idx, upd, "amax");
    else if (red == "min") out.scatter_reduce_(axis, idx, upd, "amin");
    else ORTB_THROW(INVALID_ARGUMENT, "ScatterElements: unknown reduction ", red);
    ctx.SetOutput(0, out);
  };
  r.RegisterFn("", "ScatterElements", 11, kMax, scatter_elements);
  r.RegisterFn("", "Scatter", 9, 10, scatter_elements);
  r.RegisterFn("", "ScatterND", 11, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, ScatterND(ctx.RequiredInput(0), ctx.RequiredInput(1), ctx.RequiredInput(2),
                               ctx.node().attr_s("reduction", "none")));
  });
  r.RegisterFn("", "OneHot", 9, kMax, [](Ctx& ctx) {
    at::Tensor idx = ctx.RequiredInput(0).to(at::kLong);
    const int64_t depth = ctx.RequiredInput(1).cpu().to(at::kLong).reshape({-1})[0].item<int64_t>();
    const at::Tensor& values = ctx.RequiredInput(2);
    int64_t axis = ctx.node().attr_i("axis", -1);
    if (axis < 0) axis += idx.dim() + 1;
    idx = FixNegative(idx, depth);
    at::Tensor valid = (idx >= 0).logical_and(idx < depth);
    at::Tensor oh = at::one_hot(at::where(valid, idx, at::zeros_like(idx)), depth).to(at::kBool).logical_and(valid.unsqueeze(-1));
    at::Tensor v = values.to(idx.device());
    at::Tensor out = at::where(oh, v[1], v[0]);
    if (axis != idx.dim()) out = out.movedim(-1, axis).contiguous();
    ctx.SetOutput(0, out);
  }, {1});
  r.RegisterFn("", "NonZero", 9, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::nonzero(ctx.RequiredInput(0)).t().contiguous());
  });
  r.RegisterFn("", "Compress", 9, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor cond = ctx.RequiredInput(1).to(at::kBool);
    at::Tensor idx = at::nonzero(cond).reshape({-1}).to(x.device());
    if (ctx.node().has_attr("axis")) {
      ctx.SetOutput(0, at::index_select(x, NormAxis(ctx.node().attr_i("axis", 0), x.dim()), idx));
    } else {
      ctx.SetOutput(0, at::index_select(x.reshape({-1}), 0, idx));
    }
  });
  r.RegisterFn("", "TopK", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const Node& n = ctx.node();
    const int64_t k = n.since_version >= 10 ? ctx.RequiredInput(1).cpu().to(at::kLong).reshape({-1})[0].item<int64_t>() : n.attr_i("k", 1);
    const int64_t axis = NormAxis(n.attr_i("axis", -1), x.dim());
    auto res = at::topk(x, k, axis, n.attr_i("largest", 1) != 0, true);
    ctx.SetOutput(0, std::get<0>(res));
    ctx.SetOutput(1, std::get<1>(res));
  }, {1});
  r.RegisterFn("", "CumSum", 11, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t axis = NormAxis(ctx.RequiredInput(1).cpu().to(at::kLong).reshape({-1})[0].item<int64_t>(), x.dim());
    const bool exclusive = ctx.node().attr_i("exclusive", 0) != 0, reverse = ctx.node().attr_i("reverse", 0) != 0;
    at::Tensor y = reverse ? at::flip(x, {axis}) : x;
    at::Tensor c = at::cumsum(y, axis);
    if (exclusive) c = c - y;
    ctx.SetOutput(0, reverse ? at::flip(c, {axis}) : c);
  }, {1});
  r.RegisterFn("", "DepthToSpace", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t b = ctx.node().attr_i("blocksize", 1);
    const int64_t N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
    at::Tensor y;
    if (ctx.node().attr_s("mode", "DCR") == "DCR") y = x.reshape({N, b, b, C / (b * b), H, W}).permute({0, 3, 4, 1, 5, 2});
    else y = x.reshape({N, C / (b * b), b, b, H, W}).permute({0, 1, 4, 2, 5, 3});
    ctx.SetOutput(0, y.reshape({N, C / (b * b), H * b, W * b}));
  });
  r.RegisterFn("", "SpaceToDepth", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t b = ctx.node().attr_i("blocksize", 1);
    const int64_t N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
    at::Tensor y = x.reshape({N, C, H / b, b, W / b, b}).permute({0, 3, 5, 1, 2, 4});
    ctx.SetOutput(0, y.reshape({N, C * b * b, H / b, W / b}));
  });
  r.RegisterFn("", "ReverseSequence", 10, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> lens = ToVec(ctx.RequiredInput(1));
    const int64_t batch_axis = ctx.node().attr_i("batch_axis", 1), time_axis = ctx.node().attr_i("time_axis", 0);
    at::Tensor out = x.clone();
    for (int64_t b = 0; b < static_cast<int64_t>(lens.size()); ++b) {
      at::Tensor src = x.select(batch_axis, b);
      at::Tensor dst = out.select(batch_axis, b);
      const int64_t t_ax = time_axis > batch_axis ? time_axis - 1 : time_axis;
      dst.narrow(t_ax, 0, lens[b]).copy_(at::flip(src.narrow(t_ax, 0, lens[b]), {t_ax}));
    }
    ctx.SetOutput(0, out);
  }, {1});

  // ------------------------------------------------------------ reductions
  RegisterReduce(r, "ReduceSum", 13, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::sum(x, a, k); });
  RegisterReduce(r, "ReduceMean", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::mean(x, a, k); });
  RegisterReduce(r, "ReduceMax", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return AmaxMulti(x, a, k, true); });
  RegisterReduce(r, "ReduceMin", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return AmaxMulti(x, a, k, false); });
  RegisterReduce(r, "ReduceProd", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return ProdMulti(x, a, k); });
  RegisterReduce(r, "ReduceL1", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::sum(at::abs(x), a, k); });
  RegisterReduce(r, "ReduceL2", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::sqrt(at::sum(x * x, a, k)); });
  RegisterReduce(r, "ReduceSumSquare", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::sum(x * x, a, k); });
  RegisterReduce(r, "ReduceLogSum", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::log(at::sum(x, a, k)); });
  RegisterReduce(r, "ReduceLogSumExp", 18, [](const at::Tensor& x, at::IntArrayRef a, bool k) { return at::logsumexp(x, a, k); });
  auto arg_reduce = [](bool is_max) {
    return [is_max](Ctx& ctx) {
      const at::Tensor& x = ctx.RequiredInput(0);
      const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
      const bool keep = ctx.node().attr_i("keepdims", 1) != 0;
      if (ctx.node().attr_i("select_last_index", 0) != 0) {
        at::Tensor f = at::flip(x, {axis});
        at::Tensor i = is_max ? at::argmax(f, axis, keep) : at::argmin(f, axis, keep);
        ctx.SetOutput(0, (x.size(axis) - 1) - i);
      } else {
        ctx.SetOutput(0, is_max ? at::argmax(x, axis, keep) : at::argmin(x, axis, keep));
      }
    };
  };
  r.RegisterFn("", "ArgMax", 1, kMax, arg_reduce(true));
  r.RegisterFn("", "ArgMin", 1, kMax, arg_reduce(false));

  r.RegisterFn("", "Softmax", 1, kMax, [](Ctx& ctx) {
    SoftmaxLike(ctx, [](const at::Tensor& x, int64_t a) { return at::softmax(x, a); });
  });
  r.RegisterFn("", "LogSoftmax", 1, kMax, [](Ctx& ctx) {
    SoftmaxLike(ctx, [](const at::Tensor& x, int64_t a) { return at::log_softmax(x, a); });
  });
  r.RegisterFn("", "Hardmax", 1, kMax, [](Ctx& ctx) {
    SoftmaxLike(ctx, [](const at::Tensor& x, int64_t a) {
      at::Tensor idx = at::argmax(x, a, true);
      return at::zeros_like(x).scatter_(a, idx, 1);
    });
  });

  // --------------------------------------------------------- linear algebra
  r.RegisterFn("", "MatMul", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    const at::Tensor& b = ctx.RequiredInput(1);
    ctx.SetOutput(0, at::matmul(a, b));
  });
  r.RegisterFn("", "Gemm", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor a = ctx.RequiredInput(0), b = ctx.RequiredInput(1);
    if (n.attr_i("transA", 0)) a = a.t();
    if (n.attr_i("transB", 0)) b = b.t();
    const float alpha = n.attr_f("alpha", 1.f), beta = n.attr_f("beta", 1.f);
    at::Tensor y = at::matmul(a, b);
    if (alpha != 1.f) y = y * alpha;
    if (ctx.HasInput(2)) y = y + (beta == 1.f ? ctx.Input(2) : ctx.Input(2) * beta);
    ctx.SetOutput(0, y);
  });
  r.RegisterFn("", "Einsum", 12, kMax, [](Ctx& ctx) {
    std::vector<at::Tensor> ops;
    for (int i = 0; i < ctx.InputCount(); ++i) ops.push_back(ctx.RequiredInput(i));
    ctx.SetOutput(0, at::einsum(ctx.node().attr_s("equation"), ops));
  });
  r.RegisterFn("", "MatMulInteger", 10, kMax, [](Ctx& ctx) {
    at::Tensor a = ctx.RequiredInput(0).to(at::kInt), b = ctx.RequiredInput(1).to(at::kInt);
    if (ctx.HasInput(2)) {
      at::Tensor za = ctx.Input(2).to(at::kInt);
      a = a - (za.dim() == 1 && za.numel() > 1 ? za.unsqueeze(-1) : za);
    }
    if (ctx.HasInput(3)) b = b - ctx.Input(3).to(at::kInt);
    if (a.is_cuda()) ctx.SetOutput(0, at::matmul(a.to(at::kFloat), b.to(at::kFloat)).to(at::kInt));
    else ctx.SetOutput(0, at::matmul(a, b));
  });

  // ---------------------------------------------------------------- copies
  r.RegisterFn("", "MemcpyToHost", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, ctx.RequiredInput(0).cpu()); });
  r.RegisterFn("", "MemcpyFromHost", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, ctx.RequiredInput(0).to(ctx.device(), /*non_blocking=*/true));
  });

  // ------------------------------------------------------------- sequences
  r.RegisterFn("", "SequenceConstruct", 11, kMax, [](Ctx& ctx) {
    std::vector<at::Tensor> s;
    for (int i = 0; i < ctx.InputCount(); ++i) s.push_back(ctx.RequiredInput(i));
    ctx.SetOutputSeq(0, std::move(s));
  });
  r.RegisterFn("", "SequenceEmpty", 11, kMax, [](Ctx& ctx) { ctx.SetOutputSeq(0, {}); });
  r.RegisterFn("", "SequenceLength", 11, kMax, [](Ctx& ctx) {
    auto& s = ctx.InputValue(0).seq;
    ORTB_ENFORCE_ARG(s != nullptr, "SequenceLength expects a sequence");
    ctx.SetOutput(0, at::scalar_tensor(static_cast<int64_t>(s->size()), at::kLong));
  });
  r.RegisterFn("", "SequenceAt", 11, kMax, [](Ctx& ctx) {
    auto& s = ctx.InputValue(0).seq;
    ORTB_ENFORCE_ARG(s != nullptr, "SequenceAt expects a sequence");
    int64_t i = ctx.RequiredInput(1).cpu().item<int64_t>();
    if (i < 0) i += static_cast<int64_t>(s->size());
    ORTB_ENFORCE_ARG(i >= 0 && i < static_cast<int64_t>(s->size()), "SequenceAt: index out of range");
    ctx.SetOutput(0, (*s)[i]);
  }, {1});
  r.RegisterFn("", "SequenceInsert", 11, kMax, [](Ctx& ctx) {
    auto& s = ctx.InputValue(0).seq;
    ORTB_ENFORCE_ARG(s != nullptr, "SequenceInsert expects a sequence");
    std::vector<at::Tensor> out = *s;
    int64_t pos = static_cast<int64_t>(out.size());
    if (ctx.HasInput(2)) {
      pos = ctx.Input(2).cpu().item<int64_t>();
      if (pos < 0) pos += static_cast<int64_t>(out.size());
    }
    out.insert(out.begin() + pos, ctx.RequiredInput(1));
    ctx.SetOutputSeq(0, std::move(out));
  }, {2});
  r.RegisterFn("", "SequenceErase", 11, kMax, [](Ctx& ctx) {
    auto& s = ctx.InputValue(0).seq;
    ORTB_ENFORCE_ARG(s != nullptr && !s->empty(), "SequenceErase expects a non-empty sequence");
    std::vector<at::Tensor> out = *s;
    int64_t pos = static_cast<int64_t>(out.size()) - 1;
    if (ctx.HasInput(1)) {
      pos = ctx.Input(1).cpu().item<int64_t>();
      if (pos < 0) pos += static_cast<int64_t>(out.size());
    }
    out.erase(out.begin() + pos);
    ctx.SetOutputSeq(0, std::move(out));
  }, {1});
  r.RegisterFn("", "ConcatFromSequence", 11, kMax, [](Ctx& ctx) {
    auto& s = ctx.InputValue(0).seq;
    ORTB_ENFORCE_ARG(s != nullptr && !s->empty(), "ConcatFromSequence expects a non-empty sequence");
    const int64_t axis = ctx.node().attr_i("axis", 0);
    ctx.SetOutput(0, ctx.node().attr_i("new_axis", 0) ? at::stack(*s, axis) : at::cat(*s, axis));
  });
  r.RegisterFn("", "SplitToSequence", 11, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
    std::vector<at::Tensor> parts;
    if (ctx.HasInput(1)) {
      std::vector<int64_t> sp = ToVec(ctx.Input(1));
      if (ctx.Input(1).dim() == 0) parts = at::split(x, sp[0], axis);
      else parts = at::split_with_sizes(x, sp, axis);
    } else {
      parts = at::split(x, 1, axis);
      if (!ctx.node().attr_i("keepdims", 1))
        for (auto& p : parts) p = p.squeeze(axis);
    }
    ctx.SetOutputSeq(0, std::move(parts));
  }, {1});
}

}  // namespace ortb
