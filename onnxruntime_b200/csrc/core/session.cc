#include "session.h"
#include "allocation_planner.h"

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGraph.h>
#include <ATen/Parallel.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <unistd.h>

#include <cstdlib>
#include <ctime>
#include <fstream>
#include <iomanip>
#include <set>
#include <sstream>
#include <thread>

#include "ep_context.h"
#include "executor.h"
#include "shape_inference.h"
#include "threadpool.h"

namespace ortb {

// ---------------------------------------------------------------- Profiler
void Profiler::Start(const std::string& prefix) {
  std::time_t t = std::time(nullptr);
  std::tm tm_buf;
  localtime_r(&t, &tm_buf);
  std::ostringstream ss;
  ss << prefix << "_" << std::put_time(&tm_buf, "%Y-%m-%d_%H-%M-%S") << ".json";
  path_ = ss.str();
  t0_ = std::chrono::steady_clock::now();
  enabled_ = true;
  events_.clear();
}

int64_t Profiler::NowUs() const {
  return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0_).count();
}

void Profiler::Record(const std::string& cat, const std::string& name, int64_t ts_us, int64_t dur_us,
                      std::map<std::string, std::string> args) {
  if (!enabled_) return;
  std::lock_guard<std::mutex> lk(mu_);
  if (events_.size() >= max_events_) return;  // capped like the reference's max_num_events_
  events_.push_back({cat, name, ts_us, dur_us, std::move(args)});
}

static std::string JsonEscape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o.push_back('\\'); o.push_back(c); }
    else if (c == '\n') o += "\\n";
    else if (static_cast<unsigned char>(c) < 0x20) o += ' ';
    else o.push_back(c);
  }
  return o;
}

std::string Profiler::End() {
  if (!enabled_) return "";
  std::lock_guard<std::mutex> lk(mu_);
  std::ofstream f(path_);
  const int pid = static_cast<int>(::getpid());
  f << "[\n";
  for (size_t i = 0; i < events_.size(); ++i) {
    auto& e = events_[i];
    f << "{\"cat\" : \"" << e.cat << "\",\"pid\" :" << pid << ",\"tid\" :" << 0 << ",\"dur\" :" << e.dur_us
      << ",\"ts\" :" << e.ts_us << ",\"ph\" : \"X\",\"name\" :\"" << JsonEscape(e.name) << "\",\"args\" : {";
    bool first = true;
    for (auto& kv : e.args) {
      if (!first) f << ",";
      first = false;
      f << "\"" << JsonEscape(kv.first) << "\" : \"" << JsonEscape(kv.second) << "\"";
    }
    f << "}}" << (i + 1 < events_.size() ? ",\n" : "\n");
  }
  f << "]\n";
  enabled_ = false;
  return path_;
}

// ------------------------------------------------------- InferenceSession
struct InferenceSession::CapturedGraph {
  at::cuda::CUDAGraph graph;
  std::vector<Value> slots;            // slot vector captured with the graph (static addresses)
  std::vector<at::Tensor> static_in;   // per runtime input: tensor whose storage the graph reads
  std::vector<std::vector<int64_t>> in_shapes;
  bool captured = false;
  bool bound_at_capture = false;       // inputs were IOBinding buffers, used in place
  int warm_runs = 0;
};

InferenceSession::InferenceSession(const SessionOptions& so)
    : so_(so), logger_(so.logid, so.log_severity_level, so.log_verbosity_level) {
  EnsureKernelsRegistered();
  if (so_.enable_profiling) {
    profiler_.Start(so_.profile_file_prefix);
    profiling_start_ns_ =
        std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
  }
}

InferenceSession::~InferenceSession() {
  cuda_graphs_.clear();
  exec_.reset();
}

void InferenceSession::Load(const std::string& path) {
  if (model_) ORTB_THROW(MODEL_LOADED, "This session already contains a loaded model.");
  const int64_t t0 = profiler_.NowUs();
  model_ = Model::Load(path);
  model_path_ = path;
  loaded_from_context_ = ExpandContextModel(model_, model_->model_dir);
  profiler_.Record("Session", "model_loading_uri", t0, profiler_.NowUs() - t0);
}

void InferenceSession::LoadFromBytes(const std::string& bytes) {
  if (model_) ORTB_THROW(MODEL_LOADED, "This session already contains a loaded model.");
  const int64_t t0 = profiler_.NowUs();
  model_ = Model::LoadFromBytes(std::make_shared<std::string>(bytes), "");
  loaded_from_context_ = ExpandContextModel(model_, "");
  profiler_.Record("Session", "model_loading_array", t0, profiler_.NowUs() - t0);
}

// ep.context_enable: store the prepared graph as a one-node EPContext model (ep_context.h)
void InferenceSession::WriteContextModel() {
  std::string out = so_.config.Get("ep.context_file_path");
  if (out.empty()) {
    ORTB_ENFORCE_ARG(!model_path_.empty(), "ep.context_file_path is required when the model was loaded from memory");
    const size_t dot = model_path_.rfind(".onnx");
    out = (dot == std::string::npos ? model_path_ : model_path_.substr(0, dot)) + "_ctx.onnx";
  }
  const bool embed = so_.config.Get("ep.context_embed_mode", "1") != "0";
  const size_t slash = out.find_last_of('/');
  const std::string dir = slash == std::string::npos ? "." : out.substr(0, slash);
  std::string base = slash == std::string::npos ? out : out.substr(slash + 1);
  const size_t dot = base.rfind(".onnx");
  const std::string side_name = (dot == std::string::npos ? base : base.substr(0, dot)) + "_ortb200.bin";
  std::string side;
  const std::string bytes = MakeContextModel(*model_, embed, side_name, &side);
  std::ofstream f(out, std::ios::binary);
  if (!f) ORTB_THROW(FAIL, "cannot open ", out, " for writing");
  f.write(bytes.data(), static_cast<std::streamsize>(bytes.size()));
  if (!embed) {
    std::ofstream sf(dir + "/" + side_name, std::ios::binary);
    if (!sf) ORTB_THROW(FAIL, "cannot open ", dir + "/" + side_name, " for writing");
    sf.write(side.data(), static_cast<std::streamsize>(side.size()));
  }
  ORTB_LOG(logger_, kInfo) << "compiled model written to " << out << (embed ? " (payload embedded)" : " (payload in " + side_name + ")");
}

static void ApplyFreeDimOverrides(Graph& g, const SessionOptions& so) {
  if (so.free_dim_by_name.empty() && so.free_dim_by_denotation.empty()) return;
  for (auto& v : g.Inputs()) {
    for (auto& d : v.type.dims) {
      if (d.has_value) continue;
      auto it = so.free_dim_by_name.find(d.param);
      if (!d.param.empty() && it != so.free_dim_by_name.end()) {
        d.has_value = true;
        d.value = it->second;
        continue;
      }
      auto dt = so.free_dim_by_denotation.find(d.denotation);
      if (!d.denotation.empty() && dt != so.free_dim_by_denotation.end()) {
        d.has_value = true;
        d.value = dt->second;
      }
    }
  }
}

void InferenceSession::Initialize(const std::vector<std::pair<std::string, ProviderOptions>>& providers,
                                  const std::vector<std::string>& disabled_optimizers) {
  if (!model_) ORTB_THROW(NO_MODEL, "Model was not loaded.");
  if (initialized_) ORTB_THROW(MODEL_LOADED, "Session has already been initialized.");
  const int64_t t0 = profiler_.NowUs();

  providers_.clear();
  device_ = c10::Device(c10::kCPU);
  for (auto& p : providers) {
    if (p.first == kCudaEP) {
      int dev_id = 0;
      auto it = p.second.find("device_id");
      if (it != p.second.end()) dev_id = std::stoi(it->second);
      if (!at::hasCUDA() || dev_id >= static_cast<int>(at::cuda::device_count()))
        ORTB_THROW(EP_FAIL, "CUDAExecutionProvider: no usable CUDA device ", dev_id);
      device_ = c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(dev_id));
      auto g = p.second.find("enable_cuda_graph");
      enable_cuda_graph_ = g != p.second.end() && (g->second == "1" || g->second == "true" || g->second == "True");
      providers_.push_back(kCudaEP);
      provider_options_[kCudaEP] = p.second;
      provider_options_[kCudaEP]["device_id"] = std::to_string(dev_id);
    } else if (p.first == kCpuEP) {
      providers_.push_back(kCpuEP);
      provider_options_[kCpuEP] = p.second;
    } else {
      ORTB_THROW(INVALID_ARGUMENT, "Unknown execution provider ", p.first);
    }
  }
  if (std::find(providers_.begin(), providers_.end(), kCpuEP) == providers_.end()) {
    providers_.push_back(kCpuEP);  // the CPU provider is always present, last
    provider_options_[kCpuEP];
  }

  Graph& g = model_->MainGraph();
  // session-supplied initializers
  for (auto& kv : so_.initializers) {
    if (!g.IsInitializer(kv.first)) ORTB_THROW(INVALID_ARGUMENT, "add_initializer: '", kv.first, "' is not an initializer of the model");
    g.AddInitializer(kv.first, kv.second);
    g.PendingExternal().erase(kv.first);
  }
  for (auto& kv : so_.external_initializers) {
    if (!g.IsInitializer(kv.first))
      ORTB_THROW(INVALID_ARGUMENT, "add_external_initializers: '", kv.first, "' is not an initializer of the model");
    g.AddInitializer(kv.first, kv.second);
    g.PendingExternal().erase(kv.first);
  }
  for (auto& name : g.PendingExternal()) {
    ORTB_THROW(INVALID_ARGUMENT, "initializer '", name, "' expects its data from the session (add_external_initializers)");
  }
  ApplyFreeDimOverrides(g, so_);

  c10::cuda::OptionalCUDAGuard guard;
  if (device_.is_cuda()) guard.set_device(device_);

  std::set<std::string> disabled(disabled_optimizers.begin(), disabled_optimizers.end());
  {
    std::istringstream ss(so_.config.Get("optimization.disable_specified_optimizers"));
    std::string tok;
    while (std::getline(ss, tok, ',')) if (!tok.empty()) disabled.insert(tok);
  }
  const size_t nodes_before = g.Nodes().size();
  // a compiled (EP context) model holds the graph as an earlier session prepared it: nothing left to optimize
  OptimizeGraph(g, loaded_from_context_ ? 0 : so_.graph_optimization_level, disabled, device_.is_cuda(), so_.config, world_size);
  ORTB_LOG(logger_, kInfo) << "graph optimization level " << so_.graph_optimization_level << ": " << nodes_before << " -> "
                           << g.Nodes().size() << " nodes";

  {
    // static type / shape inference over the optimized graph: gives get_outputs() its shapes when the file declares none
    // and fills value_info for tools; schema violations are worth a warning (strict mode makes them errors)
    const bool strict = so_.config.Get("session.strict_shape_type_inference", "0") == "1";
    InferenceReport rep = InferShapes(g, strict);
    for (auto& p : rep.problems) ORTB_LOG(logger_, kWarning) << "shape inference: " << p;
    ORTB_LOG(logger_, kInfo) << "shape inference: " << rep.inferred << " of " << rep.nodes << " nodes fully resolved";
  }
  if (!so_.optimized_model_filepath.empty()) model_->Save(so_.optimized_model_filepath);
  if (so_.config.Get("ep.context_enable", "0") == "1" && !loaded_from_context_) WriteContextModel();

  ApplyThreadingAndWarnings();
  auto exec = std::make_unique<GraphExecutor>(this, &g, nullptr);
  exec->Build();
  input_names_ = exec->input_names();
  output_names_ = exec->output_names();
  input_device_ = exec->input_devices();
  graph_capturable_ = exec->capturable();
  input_index_.clear();
  input_info_.assign(input_names_.size(), nullptr);
  for (size_t i = 0; i < input_names_.size(); ++i) {
    input_index_[input_names_[i]] = i;
    for (auto& vi : g.Inputs())
      if (vi.name == input_names_[i]) input_info_[i] = &vi;
  }
  exec_ = std::move(exec);
  initialized_ = true;
  {
    // nodes that could not be placed on the first provider are worth a warning (they force device <-> host copies)
    size_t on_cpu = 0, total = 0;
    std::string example;
    for (auto& t : NodeAssignments()) {
      ++total;
      if (std::get<2>(t) == kCpuEP) {
        ++on_cpu;
        if (example.empty()) example = std::get<1>(t) + " (" + std::get<0>(t) + ")";
      }
    }
    ORTB_LOG(logger_, kInfo) << "session initialized: " << total << " nodes, providers " << providers_.front()
                             << (providers_.size() > 1 ? " + " + providers_.back() : std::string()) << ", device " << device_.str();
    if (device_.is_cuda() && on_cpu > 0) {
      ORTB_LOG(logger_, kWarning) << on_cpu << " of " << total << " nodes run on the CPU provider, e.g. " << example;
      if (so_.config.Get("session.disable_cpu_ep_fallback", "0") == "1") {
        initialized_ = false;
        ORTB_THROW(FAIL, "session.disable_cpu_ep_fallback is set and ", on_cpu, " nodes were placed on the CPU provider, e.g. ", example);
      }
    }
  }
  profiler_.Record("Session", "session_initialization", t0, profiler_.NowUs() - t0);
}

// Options of the reference that map onto something here are applied; the rest is accepted (scripts written for the
// reference keep working) but reported, so that nobody tunes a knob that does nothing.
void InferenceSession::ApplyThreadingAndWarnings() {
  // intra-op parallelism of the host kernels is ATen's pool (process-wide, like the reference's global thread pools)
  if (so_.intra_op_num_threads > 0) {
    at::set_num_threads(so_.intra_op_num_threads);
    ORTB_LOG(logger_, kInfo) << "intra_op_num_threads=" << so_.intra_op_num_threads << " applied to the host math pool (process-wide)";
  }
  if (so_.execution_mode == 1) {
    int n = so_.inter_op_num_threads > 0 ? so_.inter_op_num_threads : static_cast<int>(std::thread::hardware_concurrency());
    if (n < 1) n = 1;
    if (device_.is_cuda()) {
      ORTB_LOG(logger_, kWarning) << "execution_mode=ORT_PARALLEL has no effect on a GPU session: device work is ordered by one stream";
    } else {
      inter_op_pool_ = std::make_shared<ThreadPool>(n - 1, "inter-op");  // the calling thread is the n-th lane
    }
  } else if (so_.inter_op_num_threads > 1) {
    ORTB_LOG(logger_, kWarning) << "inter_op_num_threads is only used with execution_mode=ORT_PARALLEL";
  }
  if (!so_.enable_mem_reuse || !so_.enable_cpu_mem_arena)
    ORTB_LOG(logger_, kWarning) << "enable_mem_reuse / enable_cpu_mem_arena have no effect: tensors come from PyTorch's caching "
                                   "allocators (see memory.enable_memory_arena_shrinkage to give memory back); enable_mem_pattern "
                                   "controls the tracing of memory patterns (get_memory_plans)";
  if (so_.use_deterministic_compute) {
    // every kernel of this library sums in a fixed order; ATen needs to be told
    at::globalContext().setDeterministicAlgorithms(true, /*warn_only=*/true);
  }
  if (so_.execution_order != 0)
    ORTB_LOG(logger_, kWarning) << "execution_order is ignored: nodes run in a stable topological order";
  // session configuration keys: known ones are honoured where they apply, unknown ones are reported once
  static const std::set<std::string> known = {
      "session.graph_optimizations_loop_level", "optimization.disable_specified_optimizers", "session.disable_cpu_ep_fallback",
      "session.disable_prepacking", "session.use_device_allocator_for_initializers", "session.use_env_allocators",
      "session.set_denormal_as_zero", "session.intra_op.allow_spinning", "session.inter_op.allow_spinning",
      "session.record_ep_graph_assignment_info", "session.load_model_format", "session.save_model_format",
      "optimization.enable_gelu_approximation", "optimization.minimal_build_optimizations", "ep.context_enable",
      "ep.context_file_path", "ep.context_embed_mode", "session.use_ort_model_bytes_directly", "session.strict_shape_type_inference",
      "session.qdqisint8allowed", "session.enable_dq_matmulnbits_fusion", "session.qdq_matmulnbits_accuracy_level",
      "session.dynamic_block_base", "session.force_spinning_stop", "session.collect_node_memory_stats_to_file",
      "session.disable_quant_qdq", "ep.context_node_name_prefix", "session.enable_quant_qdq_cleanup"};
  for (auto& kv : so_.config.entries) {
    if (kv.first.rfind("ortb200.", 0) == 0 || kv.first.rfind("ep.cuda.", 0) == 0) continue;
    if (!known.count(kv.first)) ORTB_LOG(logger_, kWarning) << "session config entry '" << kv.first << "' is not known to this runtime and is ignored";
  }
  if (so_.config.Get("session.set_denormal_as_zero", "0") == "1") at::globalContext().setFlushDenormal(true);
  // Attention kernel selection of the reference (contrib_ops/cpu/bert/attention_common.h: ORT_DISABLE_FLASH_ATTENTION ...,
  // provider option sdpa_kernel with bit 16 = MATH): with the fused families switched off, prompt-sized attention runs on
  // the unfused ATen path and decode attention on the CUDA-core split-KV kernel instead of the tcgen05 kernels.
  {
    auto env_is_one = [](const char* name) {
      const char* v = std::getenv(name);
      return v != nullptr && std::string(v) == "1";
    };
    bool math_only = env_is_one("ORT_DISABLE_FLASH_ATTENTION");
    auto cuda_opts = provider_options_.find(kCudaEP);
    if (cuda_opts != provider_options_.end()) {
      auto sd = cuda_opts->second.find("sdpa_kernel");
      if (sd != cuda_opts->second.end()) {
        int bits = 0;
        try {
          bits = std::stoi(sd->second);
        } catch (const std::exception&) {
          ORTB_LOG(logger_, kWarning) << "sdpa_kernel must be an integer bit mask; got '" << sd->second << "'";
        }
        if (bits != 0 && (bits & ~16) == 0) math_only = true;
      }
    }
    if (math_only) {
      so_.config.entries.emplace("ortb200.math_attention", "1");
      so_.config.entries.emplace("ortb200.decode_attention_algo", "1");
      ORTB_LOG(logger_, kInfo) << "fused attention kernels are switched off for this session";
    }
  }
  static const std::set<std::string> cuda_known = {"device_id", "enable_cuda_graph", "gpu_mem_limit", "arena_extend_strategy",
      "cudnn_conv_algo_search", "do_copy_in_default_stream", "user_compute_stream", "tunable_op_enable", "tunable_op_tuning_enable",
      "tunable_op_max_tuning_duration_ms", "prefer_nhwc", "use_ep_level_unified_stream", "use_tf32", "fuse_conv_bias", "sdpa_kernel",
      "cudnn_conv_use_max_workspace", "cudnn_conv1d_pad_to_nc1d", "enable_cudnn", "enable_skip_layer_norm_strict_mode", "has_user_compute_stream",
      "gpu_external_alloc", "gpu_external_free", "gpu_external_empty_cache"};
  auto po = provider_options_.find(kCudaEP);
  if (po != provider_options_.end()) {
    for (auto& kv : po->second) {
      if (!cuda_known.count(kv.first)) {
        ORTB_LOG(logger_, kWarning) << "CUDA provider option '" << kv.first << "' is not known and is ignored";
      } else if (kv.first == "tunable_op_enable") {
        tunable_op_enable = kv.second == "1" || kv.second == "true" || kv.second == "True";
      } else if (kv.first == "tunable_op_tuning_enable") {
        tunable_op_tuning_enable = kv.second == "1" || kv.second == "true" || kv.second == "True";
      } else if (kv.first == "tunable_op_max_tuning_duration_ms") {
        const int ms = std::stoi(kv.second);
        if (ms > 0) tunable_op_max_tuning_duration_ms = ms;
      } else if (kv.first == "use_tf32") {
        at::globalContext().setAllowTF32CuBLAS(kv.second == "1");
      } else if (kv.first == "gpu_mem_limit" && device_.is_cuda()) {
        // a byte budget becomes a fraction of the device for the caching allocator
        const double limit = std::stod(kv.second);
        size_t free_b = 0, total_b = 0;
        if (limit > 0 && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && total_b > 0 && limit < static_cast<double>(total_b))
          c10::cuda::CUDACachingAllocator::setMemoryFraction(limit / static_cast<double>(total_b), device_.index());
      } else if (kv.first != "device_id" && kv.first != "enable_cuda_graph") {
        ORTB_LOG(logger_, kInfo) << "CUDA provider option '" << kv.first << "' is accepted; it selects between library code paths the "
                                    "reference has and this runtime does not";
      }
    }
  }
}

std::vector<std::string> InferenceSession::Providers() const { return providers_; }

static NodeArgMeta MetaOf(const ValueInfo& v) {
  NodeArgMeta m;
  m.name = v.name;
  const pb::TypeProto* t = &v.type;
  std::string wrap_open, wrap_close;
  if (t->which == 4) { wrap_open = "seq("; wrap_close = ")"; if (t->elem) t = t->elem.get(); }
  else if (t->which == 9) { wrap_open = "optional("; wrap_close = ")"; if (t->elem) t = t->elem.get(); }
  m.type = wrap_open + "tensor(" + pb::DataTypeName(t->elem_type) + ")" + wrap_close;
  m.has_shape = t->has_shape;
  for (auto& d : t->dims) {
    m.shape.push_back(d.has_value ? d.value : -1);
    m.sym.push_back(d.has_value ? "" : d.param);
  }
  return m;
}

std::vector<NodeArgMeta> InferenceSession::InputsMeta() const {
  std::vector<NodeArgMeta> out;
  const Graph& g = *model_->graph_;
  for (auto& v : g.Inputs())
    if (!g.IsInitializer(v.name)) out.push_back(MetaOf(v));
  return out;
}

std::vector<NodeArgMeta> InferenceSession::OutputsMeta() const {
  std::vector<NodeArgMeta> out;
  for (auto& v : model_->graph_->Outputs()) out.push_back(MetaOf(v));
  return out;
}

std::vector<NodeArgMeta> InferenceSession::OverridableInitializersMeta() const {
  std::vector<NodeArgMeta> out;
  const Graph& g = *model_->graph_;
  for (auto& v : g.Inputs())
    if (g.IsInitializer(v.name) && !g.IsConstant(v.name)) out.push_back(MetaOf(v));
  return out;
}

std::vector<std::tuple<std::string, std::string, std::string>> InferenceSession::NodeAssignments() const {
  std::vector<std::tuple<std::string, std::string, std::string>> out;
  GraphExecutor* ex = exec_.get();
  if (!ex) return out;
  for (auto& st : ex->steps()) out.emplace_back(st.node->name, st.node->op_type, st.node->ep);
  return out;
}

at::Tensor& InferenceSession::GemmWorkspace(int64_t nbytes) {
  if (!gemm_ws_.defined() || gemm_ws_.numel() < nbytes) {
    const int64_t sz = std::max<int64_t>(nbytes, 64 << 20);
    gemm_ws_ = at::zeros({sz}, at::TensorOptions().dtype(at::kByte).device(device_));
  }
  return gemm_ws_;
}

at::Tensor& InferenceSession::AttnWorkspace(int64_t nbytes) {
  if (!attn_ws_.defined() || attn_ws_.numel() < nbytes) {
    const int64_t sz = std::max<int64_t>(nbytes, 8 << 20);
    attn_ws_ = at::zeros({sz}, at::TensorOptions().dtype(at::kByte).device(device_));
  }
  return attn_ws_;
}

at::Tensor& InferenceSession::StatusWord() {
  if (!status_word_.defined()) status_word_ = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(device_));
  return status_word_;
}

void InferenceSession::CheckDeviceStatus() {
  if (!status_word_.defined()) return;
  const int code = status_word_.cpu().data_ptr<int>()[0];
  if (code != 0) {
    status_word_.zero_();
    ORTB_THROW(EP_FAIL, "a GPU kernel reported status ", code, " (a bounded wait ran out); the run's outputs are invalid");
  }
}

static void ValidateFeed(const ValueInfo& vi, const at::Tensor& t, bool is_string) {
  if (vi.type.which != 1) return;
  if (is_string || vi.type.elem_type == pb::STRING) {
    if (!is_string || (vi.type.elem_type != 0 && vi.type.elem_type != pb::STRING))
      ORTB_THROW(INVALID_ARGUMENT, "Unexpected input data type. Actual: (tensor(", is_string ? "string" : pb::DataTypeName(ToOnnxType(t.scalar_type())),
                 ")) , expected: (tensor(", pb::DataTypeName(vi.type.elem_type), ")) for input '", vi.name, "'");
  } else if (vi.type.elem_type != 0) {
    at::ScalarType want = ToTorchType(vi.type.elem_type);
    if (want != t.scalar_type())
      ORTB_THROW(INVALID_ARGUMENT, "Unexpected input data type. Actual: (tensor(", pb::DataTypeName(ToOnnxType(t.scalar_type())),
                 ")) , expected: (tensor(", pb::DataTypeName(vi.type.elem_type), ")) for input '", vi.name, "'");
  }
  if (vi.type.has_shape) {
    if (static_cast<int64_t>(vi.type.dims.size()) != t.dim())
      ORTB_THROW(INVALID_ARGUMENT, "Invalid rank for input: ", vi.name, " Got: ", t.dim(), " Expected: ", vi.type.dims.size(),
                 " Please fix either the inputs/outputs or the model.");
    for (size_t i = 0; i < vi.type.dims.size(); ++i)
      if (vi.type.dims[i].has_value && vi.type.dims[i].value != t.size(i))
        ORTB_THROW(INVALID_ARGUMENT, "Got invalid dimensions for input: ", vi.name, " for the following indices\n index: ", i,
                   " Got: ", t.size(i), " Expected: ", vi.type.dims[i].value,
                   "\n Please fix either the inputs/outputs or the model.");
  }
}

namespace {
bool AliasesAny(const at::Tensor& t, const std::vector<at::Tensor>& pool) {
  for (auto& p : pool)
    if (p.defined() && p.is_alias_of(t)) return true;
  return false;
}
}  // namespace

std::vector<Value> InferenceSession::RunImpl(const RunOptions& ro, const std::vector<std::string>& feed_names,
                                             const std::vector<Value>& feeds,
                                             const std::vector<std::string>& output_names_in,
                                             const std::vector<Value>* bound_outputs) {
  if (!initialized_) ORTB_THROW(FAIL, "Session not initialized.");
  ORTB_ENFORCE_ARG(feed_names.size() == feeds.size(), "feed names and values differ in length");
  std::lock_guard<std::mutex> run_lock(run_mu_);
  GraphExecutor* ex = exec_.get();
  const int64_t t_run0 = profiler_.NowUs();
  // a run may carry its own id and threshold (RunOptions.logid / log_severity_level)
  logging::Logger run_logger(ro.logid.empty() ? logger_.id() : ro.logid, ro.log_severity_level >= 0 ? ro.log_severity_level : logger_.threshold(),
                             ro.log_verbosity_level > 0 ? ro.log_verbosity_level : logger_.verbosity());
  ORTB_VLOG(run_logger, 1) << "run: " << feed_names.size() << " feeds, " << output_names_in.size() << " requested outputs";
  c10::cuda::OptionalCUDAGuard guard;
  if (device_.is_cuda()) guard.set_device(device_);

  std::vector<std::string> output_names = output_names_in.empty() ? output_names_ : output_names_in;
  for (auto& n : output_names)
    if (std::find(output_names_.begin(), output_names_.end(), n) == output_names_.end())
      ORTB_THROW(INVALID_ARGUMENT, "Invalid output name:", n);

  // order the feeds as the plan expects and validate them
  const Graph& g = *model_->graph_;
  std::vector<Value> inputs(input_names_.size());
  for (size_t i = 0; i < feed_names.size(); ++i) {
    auto it = input_index_.find(feed_names[i]);
    if (it == input_index_.end()) ORTB_THROW(INVALID_ARGUMENT, "Invalid input name: ", feed_names[i]);
    const size_t idx = it->second;
    if (feeds[i].t.defined()) {
      if (input_info_[idx]) ValidateFeed(*input_info_[idx], feeds[i].t, feeds[i].is_string);
      const c10::Device want = input_device_[idx];
      inputs[idx].t = feeds[i].t.device() == want ? feeds[i].t : feeds[i].t.to(want, /*non_blocking=*/true);
      inputs[idx].is_string = feeds[i].is_string;
    } else {
      inputs[idx] = feeds[i];
    }
  }
  for (size_t i = 0; i < inputs.size(); ++i)
    if (!inputs[i].defined() && !g.IsInitializer(input_names_[i]))
      ORTB_THROW(INVALID_ARGUMENT, "Required inputs ([", input_names_[i], "]) are missing from input feed.");

  std::vector<Value> results;
  int64_t graph_id = -1;
  // memory pattern of this set of input shapes: traced on its first eager run, planned afterwards
  std::string pattern;
  bool trace_memory = false;
  if (so_.enable_mem_pattern) {
    std::ostringstream key;
    for (size_t i = 0; i < inputs.size(); ++i)
      if (inputs[i].t.defined()) key << input_names_[i] << inputs[i].t.sizes() << ";";
    pattern = key.str();
    trace_memory = memory_plans_.count(pattern) == 0 && memory_plans_.size() < 16;
  }
  auto run_eager = [&]() {
    if (trace_memory) ex->BeginMemoryTrace();
    std::vector<Value> r;
    try {
      r = ex->Run(ro, inputs, nullptr, output_names);
    } catch (...) {
      if (trace_memory) ex->EndMemoryTrace();
      throw;
    }
    if (trace_memory) {
      memory_plans_[pattern] = PlanBuffers(ex->EndMemoryTrace(), pattern);
      trace_memory = false;
      const MemoryPlan& mp = memory_plans_[pattern];
      ORTB_VLOG(run_logger, 1) << "memory pattern " << pattern << ": host " << mp.peak_bytes[0] << " of " << mp.total_bytes[0]
                               << " bytes, device " << mp.peak_bytes[1] << " of " << mp.total_bytes[1] << " bytes";
    }
    return r;
  };
  if (enable_cuda_graph_ && graph_capturable_) {
    const std::string id = ro.config.Get("gpu_graph_id", "0");
    graph_id = std::stoll(id);
    if (uncapturable_graph_ids_.count(graph_id)) graph_id = -1;
  }

  if (graph_id >= 0 && !(cuda_graphs_.count(graph_id) && cuda_graphs_[graph_id]->captured)) {
    // one eager run first (lazy initialisation, workspace allocation); it also shows whether the step calls a
    // library collective, which is left out of graph capture (the process-group's own streams and watchdog do
    // not belong inside a capture) - such a step keeps running eagerly
    const int64_t lib_before = library_collective_calls;
    results = run_eager();
    cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(device_.index()).stream());
    CheckDeviceStatus();
    if (library_collective_calls != lib_before) {
      uncapturable_graph_ids_.insert(graph_id);
      graph_id = -1;
    }
  }

  if (graph_id >= 0) {
    auto& cg_ptr = cuda_graphs_[graph_id];
    if (!cg_ptr) cg_ptr = std::make_unique<CapturedGraph>();
    CapturedGraph& cg = *cg_ptr;
    if (!cg.captured) {
      cg.static_in.clear();
      cg.in_shapes.clear();
      // Addresses are frozen into the graph.  Buffers bound through IOBinding are used in place (the caller fixed their
      // addresses on purpose: a KV cache is updated where it lies), as the reference requires for graph replay.
      // Tensors handed to a plain run() are copied into buffers the session owns, so that a later run with other
      // tensors never writes into the first call's arguments.
      cg.bound_at_capture = bound_outputs != nullptr;
      for (auto& v : inputs) {
        at::Tensor t = v.t;
        if (t.defined() && !cg.bound_at_capture) t = t.clone();
        cg.static_in.push_back(t);
        cg.in_shapes.push_back(t.defined() ? t.sizes().vec() : std::vector<int64_t>{});
      }
      cg.slots = ex->NewSlots();
      for (size_t i = 0; i < inputs.size(); ++i) {
        const int s = ex->SlotOf(input_names_[i]);
        if (inputs[i].t.defined()) cg.slots[s].t = cg.static_in[i];
        else if (inputs[i].defined()) cg.slots[s] = inputs[i];
      }
      c10::cuda::CUDAStream side = c10::cuda::getStreamFromPool(false, device_.index());
      {
        c10::cuda::CUDAStreamGuard sg(side);
        cg.graph.capture_begin();
        const int64_t launches_before = launch_count_;
        try {
          ex->ExecuteSteps(ro, cg.slots);
          last_run_launches_ = launch_count_ - launches_before;
        } catch (...) {
          cg.graph.capture_end();
          cuda_graphs_.erase(graph_id);
          throw;
        }
        cg.graph.capture_end();
      }
      cg.captured = true;
      cg.graph.replay();  // the capture itself executed nothing
    } else {
      for (size_t i = 0; i < inputs.size(); ++i) {
        if (!inputs[i].t.defined()) continue;
        ORTB_ENFORCE_ARG(cg.static_in[i].defined() && inputs[i].t.sizes().vec() == cg.in_shapes[i], "input '", input_names_[i],
                         "' changed shape after CUDA graph capture; use a different gpu_graph_id per shape");
        ORTB_ENFORCE_ARG(inputs[i].t.scalar_type() == cg.static_in[i].scalar_type() && inputs[i].t.device() == cg.static_in[i].device(),
                         "input '", input_names_[i], "' changed type or device after CUDA graph capture");
        if (inputs[i].t.data_ptr() != cg.static_in[i].data_ptr()) cg.static_in[i].copy_(inputs[i].t, true);
      }
      cg.graph.replay();
    }
    results.clear();
    for (auto& n : output_names) results.push_back(cg.slots[ex->SlotOf(n)]);
    for (size_t i = 0; i < results.size(); ++i) {
      if (!results[i].t.defined()) continue;
      const at::Tensor b = bound_outputs ? (*bound_outputs)[i].t : at::Tensor();
      if (b.defined()) {
        if (b.data_ptr() != results[i].t.data_ptr()) const_cast<at::Tensor&>(b).copy_(results[i].t, true);
        results[i].t = b;
      } else if (!bound_outputs || !AliasesAny(results[i].t, cg.static_in)) {
        // the graph's own output buffer is overwritten by the next replay: hand out a copy (an output that is one of
        // the bound input buffers, such as an in-place KV cache, is returned as it is)
        results[i].t = results[i].t.clone();
      }
    }
  } else if (bound_outputs) {
    // run with caller-provided output buffers placed in their slots
    std::vector<Value> slots = ex->NewSlots();
    for (size_t i = 0; i < inputs.size(); ++i)
      if (inputs[i].defined()) slots[ex->SlotOf(input_names_[i])] = inputs[i];
    for (size_t i = 0; i < output_names.size(); ++i)
      if ((*bound_outputs)[i].t.defined()) slots[ex->SlotOf(output_names[i])] = (*bound_outputs)[i];
    const int64_t launches_before = launch_count_;
    ex->ExecuteSteps(ro, slots);
    last_run_launches_ = launch_count_ - launches_before;
    for (auto& n : output_names) results.push_back(slots[ex->SlotOf(n)]);
  } else {
    const int64_t launches_before = launch_count_;
    results = run_eager();
    last_run_launches_ = launch_count_ - launches_before;
  }
  if (profiler_.enabled()) {
    if (device_.is_cuda()) cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(device_.index()).stream());
    profiler_.Record("Session", "model_run", t_run0, profiler_.NowUs() - t_run0);
  }
  // run option memory.enable_memory_arena_shrinkage ("cpu:0;gpu:0"): hand cached device memory back after this run
  // (reference: onnxruntime/core/session/inference_session.cc:4147 ShrinkMemoryArenas)
  if (device_.is_cuda() && ro.config.Get("memory.enable_memory_arena_shrinkage").find("gpu") != std::string::npos) {
    cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(device_.index()).stream());
    c10::cuda::CUDACachingAllocator::emptyCache();
  }
  return results;
}

std::vector<Value> InferenceSession::Run(const RunOptions& ro, const std::vector<std::string>& feed_names,
                                         const std::vector<Value>& feeds, const std::vector<std::string>& output_names) {
  return RunImpl(ro, feed_names, feeds, output_names, nullptr);
}

void InferenceSession::RunWithBinding(const RunOptions& ro, IOBinding& b) {
  std::vector<std::string> names = b.out_names_;
  std::vector<Value> res = RunImpl(ro, b.in_names_, b.in_values_, names, &b.out_values_);
  b.results_.clear();
  for (size_t i = 0; i < res.size(); ++i) {
    Value v = res[i];
    if (!b.out_values_[i].t.defined() && v.t.defined() && v.t.device() != b.out_devices_[i])
      v.t = v.t.to(b.out_devices_[i]);
    b.results_.push_back(v);
  }
}

std::string InferenceSession::EndProfiling() { return profiler_.End(); }

// ------------------------------------------------------------------ IOBinding
void IOBinding::BindInput(const std::string& name, const at::Tensor& t) {
  auto& names = session_->input_names_;
  auto it = std::find(names.begin(), names.end(), name);
  if (it == names.end()) ORTB_THROW(INVALID_ARGUMENT, "Failed to find input name in the model input def list: ", name);
  // the copy to the device the consuming node is planned on happens here, once
  const c10::Device want = session_->input_device_[static_cast<size_t>(it - names.begin())];
  Value v;
  v.t = t.device() == want ? t : t.to(want);
  for (size_t i = 0; i < in_names_.size(); ++i)
    if (in_names_[i] == name) {
      in_values_[i] = v;
      return;
    }
  in_names_.push_back(name);
  in_values_.push_back(v);
}

void IOBinding::BindOutput(const std::string& name, const at::Tensor& t) {
  auto& names = session_->output_names_;
  if (std::find(names.begin(), names.end(), name) == names.end())
    ORTB_THROW(INVALID_ARGUMENT, "Failed to find output name in the model output def list: ", name);
  Value v;
  v.t = t;
  for (size_t i = 0; i < out_names_.size(); ++i)
    if (out_names_[i] == name) {
      out_values_[i] = v;
      out_devices_[i] = t.device();
      return;
    }
  out_names_.push_back(name);
  out_values_.push_back(v);
  out_devices_.push_back(t.device());
}

void IOBinding::BindOutputToDevice(const std::string& name, c10::Device device) {
  auto& names = session_->output_names_;
  if (std::find(names.begin(), names.end(), name) == names.end())
    ORTB_THROW(INVALID_ARGUMENT, "Failed to find output name in the model output def list: ", name);
  for (size_t i = 0; i < out_names_.size(); ++i)
    if (out_names_[i] == name) {
      out_values_[i] = Value();
      out_devices_[i] = device;
      return;
    }
  out_names_.push_back(name);
  out_values_.emplace_back();
  out_devices_.push_back(device);
}

void IOBinding::SynchronizeInputs() {
  if (session_->device_.is_cuda())
    cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(session_->device_.index()).stream());
}

void IOBinding::SynchronizeOutputs() {
  if (session_->device_.is_cuda()) {
    cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(session_->device_.index()).stream());
    if (session_->config().Get("ortb200.check_status_every_run", "0") == "1") session_->CheckDeviceStatus();
  }
}

}  // namespace ortb
