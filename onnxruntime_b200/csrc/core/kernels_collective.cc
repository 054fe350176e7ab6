// Collective contrib operators on torch.distributed process groups: AllReduce,
// AllGather, AllToAll, ShardedMoE and the Distributed* family.  These are the
// library-collective BASELINE implementations (NCCL on GPUs, gloo on CPU
// ranks); the fused compute+collective kernels in kernels_cuda.cc take over
// the tensor-parallel hot paths on the GPU.
//
// Reference: onnxruntime/contrib_ops/cuda/collective/{nccl_kernels.cc,
// sharded_moe.cc,distributed_matmul.cc,sharding.cc}.  The reference bootstraps
// NCCL through MPI or a TCP rendezvous; here the process group comes from
// torch.distributed and is looked up by name.
#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>

#include "collective.h"
#include "contrib_math.h"
#include "kernel.h"
#include "session.h"
#include "sharding_spec.h"

namespace ortb {

c10::intrusive_ptr<c10d::ProcessGroup> GroupOf(InferenceSession* s) {
  if (!s || s->world_size <= 1 || s->dist_group.empty()) return nullptr;
  ++s->library_collective_calls;
  return c10d::resolve_process_group(s->dist_group);
}

at::Tensor AllReduceSum(InferenceSession* s, const at::Tensor& t) {
  auto pg = GroupOf(s);
  if (!pg) return t;
  at::Tensor buf = t.contiguous().clone();
  std::vector<at::Tensor> v{buf};
  pg->allreduce(v)->wait();
  return buf;
}

at::Tensor AllGatherAxis(InferenceSession* s, const at::Tensor& t, int64_t axis) {
  auto pg = GroupOf(s);
  if (!pg) return t;
  const int64_t w = pg->getSize();
  at::Tensor in = t.contiguous();
  if (in.dim() == 0) in = in.reshape({1});
  if (axis < 0) axis += in.dim();
  // the flat form (leading dimension multiplied by the group size) is the one every backend accepts
  std::vector<int64_t> flat = in.sizes().vec();
  flat[0] *= w;
  at::Tensor out = at::empty(flat, in.options());
  pg->_allgather_base(out, in)->wait();
  if (axis == 0) return out;
  std::vector<int64_t> shape = in.sizes().vec();
  shape.insert(shape.begin(), w);
  out = out.reshape(shape);
  // [w, d0, .., da, ..] -> [d0, .., w*da, ..]
  return out.movedim(0, axis).flatten(axis, axis + 1).contiguous();
}

at::Tensor AllToAllEqual(InferenceSession* s, const at::Tensor& t) {
  auto pg = GroupOf(s);
  if (!pg) return t;
  at::Tensor in = t.contiguous();
  at::Tensor out = at::empty_like(in);
  std::vector<int64_t> none;
  pg->alltoall_base(out, in, none, none)->wait();
  return out;
}

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

at::Tensor Shard(const at::Tensor& full, const TensorPartitionSpec& spec, int64_t rank) {
  const int ax = spec.ShardedAxis();
  if (ax < 0) return full;
  const int64_t n = spec.NumShards();
  const int64_t idx = spec.ShardIndexOf(spec.Mesh().elements[rank % spec.Mesh().Size()]);
  const int64_t sz = full.size(ax) / n;
  return full.narrow(ax, idx * sz, sz).contiguous();
}

at::Tensor Gather(InferenceSession* s, const at::Tensor& shard, const TensorPartitionSpec& spec) {
  const int ax = spec.ShardedAxis();
  if (ax < 0) return shard;
  return AllGatherAxis(s, shard, ax);
}

struct Specs {
  std::vector<TensorPartitionSpec> in, out;
};

Specs ParseSpecs(const Node& n) {
  Specs sp;
  auto parse = [&](const char* elems_attr, const char* shapes_attr, const char* specs_attr, std::vector<TensorPartitionSpec>& dst) {
    std::vector<std::string> elems = n.attr_strings(elems_attr), shapes = n.attr_strings(shapes_attr),
                             specs = n.attr_strings(specs_attr);
    for (size_t i = 0; i < specs.size(); ++i) {
      const std::string& e = elems.size() == specs.size() ? elems[i] : elems.at(0);
      const std::string& sh = shapes.size() == specs.size() ? shapes[i] : shapes.at(0);
      dst.push_back(TensorPartitionSpec::Parse(specs[i], DeviceMesh::Parse(e, sh)));
    }
  };
  parse("input_device_mesh_elements", "input_device_mesh_shapes", "input_shard_specs", sp.in);
  parse("output_device_mesh_elements", "output_device_mesh_shapes", "output_shard_specs", sp.out);
  return sp;
}

// Every Distributed* op can be evaluated as: gather the sharded operands, run the plain op, shard the result.
// DistributedMatMul short-cuts the two tensor-parallel cases that need no gather.
class DistributedOp final : public OpKernel {
 public:
  DistributedOp(const OpKernelInfo& info, std::string plain_op) : OpKernel(info), plain_op_(std::move(plain_op)) {
    specs_ = ParseSpecs(info.node);
    plain_ = info.node;
    plain_.op_type = plain_op_;
    plain_.domain = "";
    plain_.since_version = 18;
    for (const char* a : {"input_device_mesh_elements", "input_device_mesh_shapes", "input_shard_specs",
                          "output_device_mesh_elements", "output_device_mesh_shapes", "output_shard_specs"})
      plain_.attrs.erase(a);
    const KernelDef* d = KernelRegistry::Generic().Find(plain_, info.graph);
    ORTB_ENFORCE(d != nullptr, "no kernel for ", plain_op_);
    OpKernelInfo pinfo{plain_, info.graph, info.session, info.device, info.config, [](int) { return nullptr; }};
    kernel_ = d->factory(pinfo);
  }

  void Compute(Ctx& ctx) const override {
    InferenceSession* s = ctx.session();
    const int64_t rank = s ? s->rank : 0;
    const int nin = ctx.InputCount();
    ORTB_ENFORCE_ARG(static_cast<int>(specs_.in.size()) >= nin, "input_shard_specs is shorter than the input list");
    if (plain_op_ == "MatMul" && nin == 2) {
      const auto& sa = specs_.in[0];
      const auto& sb = specs_.in[1];
      const auto& sy = specs_.out.at(0);
      const at::Tensor& a = ctx.RequiredInput(0);
      const at::Tensor& b = ctx.RequiredInput(1);
      const int a_ax = sa.ShardedAxis(), b_ax = sb.ShardedAxis(), y_ax = sy.ShardedAxis();
      const int a_rank = static_cast<int>(sa.Rank()), b_rank = static_cast<int>(sb.Rank()), y_rank = static_cast<int>(sy.Rank());
      // column-parallel: A replicated, B sharded on its last axis, Y sharded on its last axis
      if (a_ax < 0 && b_ax == b_rank - 1 && y_ax == y_rank - 1) {
        ctx.SetOutput(0, at::matmul(a, b));
        return;
      }
      // row-parallel: A sharded on K (last axis), B sharded on K (second-to-last), Y replicated -> partial sums
      if (a_ax == a_rank - 1 && b_ax == b_rank - 2 && y_ax < 0) {
        ctx.SetOutput(0, AllReduceSum(s, at::matmul(a, b)));
        return;
      }
      // data-parallel rows: A sharded on a batch/row axis, B replicated, Y sharded the same way
      if (a_ax >= 0 && a_ax < a_rank - 1 && b_ax < 0 && y_ax == a_ax + (y_rank - a_rank)) {
        ctx.SetOutput(0, at::matmul(a, b));
        return;
      }
    }
    std::vector<Value> in(nin), out(ctx.OutputCount());
    for (int i = 0; i < nin; ++i)
      if (ctx.HasInput(i)) in[i].t = Gather(s, ctx.Input(i), specs_.in[i]);
    std::vector<bool> needed(ctx.OutputCount(), true);
    OpKernelContext sub(plain_, s, ctx.device(), in, out, needed);
    kernel_->Compute(sub);
    for (int i = 0; i < ctx.OutputCount(); ++i) {
      if (!out[i].t.defined()) continue;
      ctx.SetOutput(i, i < static_cast<int>(specs_.out.size()) ? Shard(out[i].t, specs_.out[i], rank) : out[i].t);
    }
  }

 private:
  std::string plain_op_;
  Specs specs_;
  Node plain_;
  std::unique_ptr<OpKernel> kernel_;
};

void RegisterDistributed(KernelRegistry& r, const std::string& op, const std::string& plain, std::vector<int> host) {
  KernelDef d;
  d.domain = MS;
  d.op_type = op;
  d.host_inputs = std::move(host);
  d.factory = [plain](const OpKernelInfo& info) { return std::make_unique<DistributedOp>(info, plain); };
  r.Register(std::move(d));
}

// ShardedMoE: fc1 [E_local, H, I_local], fc2 [E_local, I_local, H], fc3 [E_local, H, I_local]; input and output replicated.
class ShardedMoeKernel final : public OpKernel {
 public:
  explicit ShardedMoeKernel(const OpKernelInfo& info) : OpKernel(info) {
    attrs_ = contrib::ParseMoeAttrs(info.node);
    start_ = info.node.attr_i("local_experts_start_index", 0);
    tensor_shards_ = info.node.attr_i("tensor_shards", 1);
    tokens_sharded_ = info.node.attr_i("tokens_sharded", 0) != 0;
  }
  void Compute(Ctx& ctx) const override {
    InferenceSession* s = ctx.session();
    const at::Tensor& x = ctx.RequiredInput(0);
    if (tokens_sharded_ && s && s->world_size > 1) {
      ComputeTokenSharded(ctx);
      return;
    }
    at::Tensor x2 = x.reshape({-1, x.size(-1)});
    auto opt = [&](int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); };
    // to the [E, out, in] layout of the dense MoE math
    at::Tensor fc1 = ctx.RequiredInput(2).transpose(1, 2), fc2 = ctx.RequiredInput(4).transpose(1, 2);
    at::Tensor fc3 = ctx.HasInput(6) ? ctx.Input(6).transpose(1, 2) : at::Tensor();
    const int64_t e_local = fc1.size(0);
    at::Tensor fc2_bias = opt(5);
    const int64_t world = s ? s->world_size : 1;
    if (fc2_bias.defined()) {
      if (fc2_bias.size(0) != e_local) fc2_bias = fc2_bias.narrow(0, start_, e_local);
      // with tensor-sharded experts every rank adds the bias to its partial sum: scale it so the sum is right
      if (tensor_shards_ > 1) fc2_bias = fc2_bias / static_cast<double>(tensor_shards_);
    }
    at::Tensor partial = contrib::MoeForward(x2, ctx.RequiredInput(1).reshape({x2.size(0), -1}), fc1, opt(3), fc2, fc2_bias,
                                             fc3, opt(7), attrs_, start_, start_ + e_local);
    at::Tensor y = world > 1 ? AllReduceSum(s, partial.to(at::kFloat)).to(x.scalar_type()) : partial;
    ctx.SetOutput(0, y.reshape(x.sizes()));
  }

  // tokens_sharded = 1 (an attribute of this runtime, not of the reference): every rank holds its own tokens.  A token's row
  // (with its router logits) travels once to every rank that owns one of its top-k experts (all-to-all dispatch), that rank
  // adds up its experts' weighted outputs for the row, and the partial sums travel back (all-to-all combine) to be added per
  // token.  Rows per (source, destination) pair vary, so both exchanges are padded to the largest pair count, which the ranks
  // learn from an all-gather of their count vectors.  Experts must be split evenly over the ranks, rank r owning the r-th part.
  void ComputeTokenSharded(Ctx& ctx) const {
    InferenceSession* s = ctx.session();
    const int64_t world = s->world_size;
    const at::Tensor& x_in = ctx.RequiredInput(0);
    at::Tensor x = x_in.reshape({-1, x_in.size(-1)}).to(at::kFloat);
    at::Tensor logits = ctx.RequiredInput(1).reshape({x.size(0), -1}).to(at::kFloat);
    const int64_t T = x.size(0), H = x.size(1), E = logits.size(1);
    auto opt = [&](int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); };
    at::Tensor fc1 = ctx.RequiredInput(2).transpose(1, 2), fc2 = ctx.RequiredInput(4).transpose(1, 2);
    at::Tensor fc3 = ctx.HasInput(6) ? ctx.Input(6).transpose(1, 2) : at::Tensor();
    const int64_t e_local = fc1.size(0);
    ORTB_ENFORCE_ARG(e_local * world == E && start_ == s->rank * e_local, "ShardedMoE (tokens_sharded): experts must be split evenly, rank r owning part r");
    ORTB_ENFORCE_ARG(tensor_shards_ == 1, "ShardedMoE (tokens_sharded): tensor-sharded experts are not supported in this mode");
    auto lopt = at::TensorOptions().dtype(at::kLong).device(x.device());
    // which ranks does every token need?
    at::Tensor owner = std::get<1>(logits.topk(attrs_.k, 1)).floor_divide(e_local);                   // [T, k]
    at::Tensor need = at::zeros({T, world}, lopt.dtype(at::kBool)).scatter_(1, owner, true);          // [T, world]
    at::Tensor counts = need.sum(0).to(at::kLong);                                                   // rows this rank sends to every rank
    at::Tensor all_counts = AllGatherAxis(s, counts.reshape({1, world}), 0).to(at::kCPU);            // [source, destination]
    const int64_t cap = std::max<int64_t>(all_counts.max().item<int64_t>(), 1);
    // dispatch: [destination, cap, H + E], rows beyond a pair's count are zero
    at::Tensor send = at::zeros({world, cap, H + E}, x.options());
    std::vector<at::Tensor> rows_for(static_cast<size_t>(world));
    at::Tensor payload = at::cat({x, logits}, 1);
    for (int64_t d = 0; d < world; ++d) {
      rows_for[static_cast<size_t>(d)] = need.select(1, d).nonzero().reshape({-1});
      const int64_t n = rows_for[static_cast<size_t>(d)].numel();
      if (n > 0) send[d].narrow(0, 0, n).copy_(payload.index_select(0, rows_for[static_cast<size_t>(d)]));
    }
    at::Tensor recv = AllToAllEqual(s, send.reshape({world * cap, H + E})).reshape({world, cap, H + E});
    // this rank's experts on everything it received (padding rows included: their results are never read)
    at::Tensor got = recv.reshape({world * cap, H + E});
    at::Tensor fc2_bias = opt(5);
    if (fc2_bias.defined() && fc2_bias.size(0) != e_local) fc2_bias = fc2_bias.narrow(0, start_, e_local);
    at::Tensor partial = contrib::MoeForward(got.narrow(1, 0, H), got.narrow(1, H, E), fc1, opt(3), fc2, fc2_bias, fc3, opt(7), attrs_, start_,
                                             start_ + e_local).to(at::kFloat);
    // combine: the partial sums go back to where the rows came from
    at::Tensor back = AllToAllEqual(s, partial.reshape({world * cap, H})).reshape({world, cap, H});
    at::Tensor out = at::zeros({T, H}, x.options());
    for (int64_t d = 0; d < world; ++d) {
      const at::Tensor& rows = rows_for[static_cast<size_t>(d)];
      if (rows.numel() > 0) out.index_add_(0, rows, back[d].narrow(0, 0, rows.numel()));
    }
    ctx.SetOutput(0, out.to(x_in.scalar_type()).reshape(x_in.sizes()));
  }

 private:
  contrib::MoeAttrs attrs_;
  int64_t start_ = 0, tensor_shards_ = 1;
  bool tokens_sharded_ = false;
};

}  // namespace

void RegisterCollectiveKernels(KernelRegistry& r) {
  r.RegisterFn(MS, "AllReduce", 1, kMax, [](Ctx& ctx) {
    for (int i = 0; i < ctx.InputCount() && i < ctx.OutputCount(); ++i)
      if (ctx.HasInput(i)) ctx.SetOutput(i, AllReduceSum(ctx.session(), ctx.Input(i)));
  });
  r.RegisterFn(MS, "AllGather", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, AllGatherAxis(ctx.session(), ctx.RequiredInput(0), ctx.node().attr_i("axis", 0)));
  });
  // all-gather along axis 0, then MatMul (+ bias): the generic form of the fused GPU kernel
  r.RegisterFn("com.ortb200", "AllGatherMatMul", 1, kMax, [](Ctx& ctx) {
    at::Tensor y = at::matmul(AllGatherAxis(ctx.session(), ctx.RequiredInput(0), 0), ctx.RequiredInput(1));
    ctx.SetOutput(0, ctx.HasInput(2) ? y + ctx.Input(2) : y);
  });
  r.RegisterFn(MS, "AllToAll", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, AllToAllEqual(ctx.session(), ctx.RequiredInput(0))); });
  {
    KernelDef d;
    d.domain = MS;
    d.op_type = "ShardedMoE";
    d.factory = [](const OpKernelInfo& info) { return std::make_unique<ShardedMoeKernel>(info); };
    r.Register(std::move(d));
  }
  RegisterDistributed(r, "DistributedMatMul", "MatMul", {});
  RegisterDistributed(r, "DistributedSlice", "Slice", {1, 2, 3, 4});
  RegisterDistributed(r, "DistributedReshape", "Reshape", {1});
  RegisterDistributed(r, "DistributedExpand", "Expand", {1});
  RegisterDistributed(r, "DistributedReduceSum", "ReduceSum", {1});
  RegisterDistributed(r, "DistributedReduceMax", "ReduceMax", {1});
  RegisterDistributed(r, "DistributedReduceMean", "ReduceMean", {1});
  RegisterDistributed(r, "DistributedSqueeze", "Squeeze", {1});
  RegisterDistributed(r, "DistributedUnsqueeze", "Unsqueeze", {1});
}

}  // namespace ortb
