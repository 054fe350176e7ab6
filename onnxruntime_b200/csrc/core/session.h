// InferenceSession: load -> optimize -> partition -> plan -> run.
//
// Mirrors the life cycle of the reference's InferenceSession
// (onnxruntime/core/session/inference_session.cc: Load :1155, Initialize :2405,
// TransformGraph :1523, Run :3274) with a different execution model: the
// optimized graph is lowered once into a flat launch program (one Step per
// node with pre-resolved value slots and a release list), and on the GPU the
// whole program is captured into a CUDA graph and replayed.
#pragma once
#include <atomic>
#include <chrono>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "allocation_planner.h"
#include "logging.h"
#include "graph.h"
#include "kernel.h"

namespace ortb {

struct SessionOptions {
  bool enable_cpu_mem_arena = true;
  bool enable_mem_pattern = true;
  bool enable_mem_reuse = true;
  bool enable_profiling = false;
  std::string profile_file_prefix = "onnxruntime_profile_";
  std::string optimized_model_filepath;
  std::string logid;
  int log_severity_level = -1;      // -1: the process default (logging::Manager)
  int log_verbosity_level = 0;
  int intra_op_num_threads = 0;
  int inter_op_num_threads = 0;
  int execution_mode = 0;           // 0 sequential, 1 parallel
  int execution_order = 0;          // 0 default, 1 priority-based, 2 memory-efficient
  int graph_optimization_level = 99;  // 0 none, 1 basic, 2 extended, 3 layout, 99 all
  bool use_deterministic_compute = false;
  bool use_per_session_threads = true;
  ConfigOptions config;
  std::map<std::string, int64_t> free_dim_by_name, free_dim_by_denotation;
  std::map<std::string, at::Tensor> initializers;           // add_initializer: overrides by name
  std::map<std::string, at::Tensor> external_initializers;  // add_external_initializers
};

struct RunOptions {
  int log_severity_level = -1;
  int log_verbosity_level = 0;
  std::string logid;
  std::shared_ptr<std::atomic<bool>> terminate = std::make_shared<std::atomic<bool>>(false);
  bool only_execute_path_to_fetches = false;
  ConfigOptions config;
};

using ProviderOptions = std::map<std::string, std::string>;

struct NodeArgMeta {
  std::string name;
  std::string type;  // "tensor(float)"
  // -1 entries are unknown; `sym` holds the symbolic name for those
  std::vector<int64_t> shape;
  std::vector<std::string> sym;
  bool has_shape = false;
};

struct ProfileEvent {
  std::string cat, name;
  int64_t ts_us = 0, dur_us = 0;
  std::map<std::string, std::string> args;
};

class Profiler {
 public:
  void Start(const std::string& prefix);
  bool enabled() const { return enabled_; }
  int64_t NowUs() const;
  void Record(const std::string& cat, const std::string& name, int64_t ts_us, int64_t dur_us,
              std::map<std::string, std::string> args = {});
  std::string End();  // writes the chrome-trace JSON file, returns its path
  size_t NumEvents() const { return events_.size(); }

 private:
  bool enabled_ = false;
  std::string path_;
  std::vector<ProfileEvent> events_;
  std::chrono::steady_clock::time_point t0_;
  std::mutex mu_;
  size_t max_events_ = 1000000;
};

struct Step {
  const Node* node = nullptr;
  std::unique_ptr<OpKernel> kernel;
  std::vector<int> in_slots, out_slots;  // -1 = absent
  std::vector<bool> out_needed;
  std::vector<int> release;  // slots whose last use is this step
  c10::Device device = c10::Device(c10::kCPU);
  bool on_gpu = false;
};

class IOBinding;
class GraphExecutor;

class InferenceSession {
 public:
  explicit InferenceSession(const SessionOptions& so);
  ~InferenceSession();

  void Load(const std::string& path);
  void LoadFromBytes(const std::string& bytes);
  // providers in priority order with their options; names of optimizers to skip
  void Initialize(const std::vector<std::pair<std::string, ProviderOptions>>& providers,
                  const std::vector<std::string>& disabled_optimizers);

  std::vector<Value> Run(const RunOptions& ro, const std::vector<std::string>& feed_names,
                         const std::vector<Value>& feeds, const std::vector<std::string>& output_names);
  void RunWithBinding(const RunOptions& ro, IOBinding& binding);

  std::vector<NodeArgMeta> InputsMeta() const;
  std::vector<NodeArgMeta> OutputsMeta() const;
  std::vector<NodeArgMeta> OverridableInitializersMeta() const;
  const Model& model() const { return *model_; }
  Model& model() { return *model_; }
  std::vector<std::string> Providers() const;
  std::map<std::string, ProviderOptions> ProviderOptionsMap() const { return provider_options_; }
  std::string EndProfiling();
  int64_t ProfilingStartTimeNs() const { return profiling_start_ns_; }
  c10::Device device() const { return device_; }
  bool uses_gpu() const { return device_.is_cuda(); }
  const SessionOptions& options() const { return so_; }
  const ConfigOptions& config() const { return so_.config; }
  // inter-op pool: present when execution_mode is parallel (ExecutionMode::ORT_PARALLEL), null otherwise
  class ThreadPool* InterOpPool() const { return inter_op_pool_.get(); }
  // per-node provider assignment: (node name, op type, provider)
  std::vector<std::tuple<std::string, std::string, std::string>> NodeAssignments() const;
  Profiler& profiler() { return profiler_; }
  const logging::Logger& logger() const { return logger_; }
  int NumCapturedGraphs() const { return static_cast<int>(cuda_graphs_.size()); }
  int64_t KernelLaunchCount() const { return launch_count_; }
  // one plan per input-shape pattern seen so far (SessionOptions.enable_mem_pattern)
  const std::map<std::string, MemoryPlan>& MemoryPlans() const { return memory_plans_; }
  // launches issued by the most recent execution of the step list (eager run or graph capture)
  int64_t LastRunLaunchCount() const { return last_run_launches_; }
  void AddLaunches(int64_t n) { launch_count_ += n; }
  // Device memory a kernel streams on every run (its pre-packed weights), by node name.  A kernel that leaves the
  // memory system idle (decode attention) asks the L2 for the next node's weights while it runs.
  void RegisterWeightHint(const std::string& node_name, const void* ptr, int64_t bytes) { weight_hints_[node_name] = {ptr, bytes}; }
  std::pair<const void*, int64_t> FindWeightHint(const std::string& node_name) const {
    auto it = weight_hints_.find(node_name);
    return it == weight_hints_.end() ? std::pair<const void*, int64_t>{nullptr, 0} : it->second;
  }
  // device scratch shared by the GPU kernels (split-K partials, counters), zero-initialised
  at::Tensor& GemmWorkspace(int64_t nbytes);
  at::Tensor& AttnWorkspace(int64_t nbytes);
  at::Tensor& StatusWord();
  // Check the device status word (bounded waits); throws EP_FAIL when a kernel reported a timeout.
  void CheckDeviceStatus();
  // Symmetric workspace for the fused compute+collective kernels: base address of every rank's buffer as mapped
  // into this process (index = rank), and its size.  Empty = not available (collectives go through the process group).
  // TunableOp (CUDA provider options tunable_op_enable / tunable_op_tuning_enable / tunable_op_max_tuning_duration_ms;
  // reference: onnxruntime/core/framework/tunable.h, core/providers/cuda/tunable/cuda_tuning_context.cc): per GEMM
  // signature the launch configuration that measured fastest on this device.  Results can be exported and loaded
  // again (get_tuning_results / set_tuning_results), so a deployment tunes once.
  struct TunedGemm {
    int force_splits = 0, force_bn = 0, force_tile_rows = 0;
    float microseconds = 0.f;  // 0 when the entry was loaded, not measured
  };
  std::map<std::string, TunedGemm> tuning_results;
  bool tunable_op_enable = false, tunable_op_tuning_enable = false;
  int tunable_op_max_tuning_duration_ms = 200;  // per signature

  std::vector<void*> symm_peers;
  int64_t symm_bytes = 0;
  void* symm_multicast = nullptr;  // NVLS multicast address of the workspace (0: none)
  // the multicast address to hand to a kernel, honouring ortb200.nvls = "0"
  void* NvlsPointer() const { return so_.config.Get("ortb200.nvls", "1") == "0" ? nullptr : symm_multicast; }
  int64_t library_collective_calls = 0;  // process-group collectives issued so far (the in-kernel ones do not count)
  std::set<int64_t> uncapturable_graph_ids_;
  std::string dist_group;  // torch.distributed group name used by collective ops ("" = default)
  int rank = 0, world_size = 1;

 private:
  friend class IOBinding;
  std::vector<Value> RunImpl(const RunOptions& ro, const std::vector<std::string>& feed_names,
                             const std::vector<Value>& feeds, const std::vector<std::string>& output_names,
                             const std::vector<Value>* bound_outputs);

  struct CapturedGraph;
  void ApplyThreadingAndWarnings();
  void WriteContextModel();
  std::string model_path_;
  bool loaded_from_context_ = false;
  std::shared_ptr<class ThreadPool> inter_op_pool_;
  SessionOptions so_;
  std::shared_ptr<Model> model_;
  bool initialized_ = false;
  c10::Device device_ = c10::Device(c10::kCPU);
  std::vector<std::string> providers_;
  std::map<std::string, ProviderOptions> provider_options_;
  bool enable_cuda_graph_ = false;

  // plan
  std::unique_ptr<GraphExecutor> exec_;
  std::vector<c10::Device> input_device_;  // per runtime input: where the plan wants it
  std::vector<std::string> input_names_, output_names_;
  bool graph_capturable_ = false;

  std::map<int64_t, std::unique_ptr<CapturedGraph>> cuda_graphs_;
  std::map<std::string, std::pair<const void*, int64_t>> weight_hints_;
  Profiler profiler_;
  logging::Logger logger_;
  int64_t profiling_start_ns_ = 0;
  int64_t launch_count_ = 0;
  int64_t last_run_launches_ = 0;
  std::map<std::string, MemoryPlan> memory_plans_;
  std::map<std::string, size_t> input_index_;
  std::vector<const ValueInfo*> input_info_;
  at::Tensor gemm_ws_, attn_ws_, status_word_;
  std::mutex run_mu_;
};

// Named inputs/outputs bound to caller-owned buffers (reference: onnxruntime/core/session/IOBinding.cc).
class IOBinding {
 public:
  explicit IOBinding(InferenceSession* s) : session_(s) {}
  void BindInput(const std::string& name, const at::Tensor& t);
  void BindOutput(const std::string& name, const at::Tensor& t);           // pre-allocated
  void BindOutputToDevice(const std::string& name, c10::Device device);    // session allocates there
  void ClearInputs() { in_names_.clear(); in_values_.clear(); }
  void ClearOutputs() { out_names_.clear(); out_values_.clear(); out_devices_.clear(); results_.clear(); }
  void SynchronizeInputs();
  void SynchronizeOutputs();
  const std::vector<std::string>& OutputNames() const { return out_names_; }
  const std::vector<Value>& Results() const { return results_; }

  std::vector<std::string> in_names_, out_names_;
  std::vector<Value> in_values_, out_values_;
  std::vector<c10::Device> out_devices_;
  std::vector<Value> results_;
  InferenceSession* session_;
};

// Optimizer entry point (optimizer.cc).  level: 0 none, 1 basic, 2 extended, 99 all.
// `gpu` enables the fusions that only the GPU provider has kernels for.
struct OptimizerStats {
  std::map<std::string, int> applied;  // pass name -> number of rewrites
};
OptimizerStats OptimizeGraph(Graph& g, int level, const std::set<std::string>& disabled, bool gpu,
                             const ConfigOptions& config, int world_size);
// Evaluate one node on CPU with constant inputs (used by constant folding).
std::vector<at::Tensor> EvaluateNodeOnCpu(const Node& node, const Graph& g, const std::vector<at::Tensor>& inputs);

}  // namespace ortb
