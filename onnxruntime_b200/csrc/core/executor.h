// GraphExecutor: partitions one Graph between host and GPU, inserts the copies,
// creates the kernels and runs the resulting launch program.  The main graph
// and every control-flow body own one executor each.
//
// Design notes (what replaces which part of the reference):
//  * partitioning  -> GraphPartitioner::Partition (core/framework/graph_partitioner.cc:1451)
//    plus GetCpuPreferredNodes (fallback_cpu_capability.cc:44): a node runs on
//    the GPU unless every dynamic input already lives on the host (shape
//    arithmetic stays on the CPU);
//  * copy insertion -> MemcpyTransformer (core/optimizer/transformer_memcpy.cc:101);
//  * plan + release list -> SequentialPlanner (core/framework/allocation_planner.cc:1867-1996);
//  * step loop -> StreamExecutionContext::RunSince (stream_execution_context.cc:180).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "allocation_planner.h"
#include "debug_node_io.h"
#include "session.h"

namespace ortb {

class GraphExecutor {
 public:
  // `outer_on_gpu`: location of values visible from enclosing graphs (name -> true when on GPU)
  GraphExecutor(InferenceSession* session, Graph* graph, const std::map<std::string, bool>* outer_on_gpu);
  void Build();

  // inputs aligned with input_names(); outer values by name (control-flow bodies)
  std::vector<Value> Run(const RunOptions& ro, const std::vector<Value>& inputs,
                         const std::map<std::string, Value>* outer, const std::vector<std::string>& output_names);

  const std::vector<std::string>& input_names() const { return input_names_; }
  const std::vector<std::string>& output_names() const { return output_names_; }
  const std::vector<c10::Device>& input_devices() const { return input_device_; }
  const std::vector<std::string>& outer_names() const { return outer_names_; }
  bool capturable() const { return capturable_; }
  const std::vector<Step>& steps() const { return steps_; }
  bool ValueOnGpu(const std::string& name) const;
  Graph* graph() const { return graph_; }
  // Run only the step loop over a prepared slot vector (used inside CUDA-graph capture).
  void ExecuteSteps(const RunOptions& ro, std::vector<Value>& slots);
  // true when ExecutionMode::ORT_PARALLEL can apply: every step runs on the host
  bool parallel_ok() const { return parallel_ok_; }
  std::vector<Value> NewSlots() const { return constant_slots_; }
  int SlotOf(const std::string& name) const;
  // Memory-pattern tracing: between the two calls every step records what its outputs allocated.
  void BeginMemoryTrace();
  std::vector<PlannedBuffer> EndMemoryTrace();

 private:
  void Partition();
  void InsertCopies();
  void BuildStepGraph();
  void RunStep(const RunOptions& ro, const Step& st, std::vector<Value>& slots, OpKernelContext::Lookup* lookup, int node_index);
  void ExecuteStepsParallel(const RunOptions& ro, std::vector<Value>& slots, OpKernelContext::Lookup* lookup, class ThreadPool* pool);
  int NewSlot(const std::string& name);

  InferenceSession* session_;
  Graph* graph_;
  std::map<std::string, bool> outer_on_gpu_;
  std::map<std::string, bool> on_gpu_;  // value name -> location
  std::vector<Step> steps_;
  std::map<std::string, int> slot_of_;
  std::vector<std::string> slot_names_;
  std::vector<Value> constant_slots_;
  std::vector<std::string> input_names_, output_names_, outer_names_;
  std::vector<int> input_slot_, outer_slot_;
  std::vector<c10::Device> input_device_;
  bool capturable_ = false;
  bool parallel_ok_ = false, nvtx_ = true;
  std::vector<std::vector<int>> step_deps_, step_succ_;  // step index -> steps it waits for / steps waiting for it
  const std::map<std::string, Value>* current_outer_ = nullptr;
  struct SlotTrace {
    int64_t bytes = -1;  // -1: not produced by a step during the trace
    int step = -1;
    bool on_gpu = false;
  };
  std::vector<SlotTrace> trace_;
  bool tracing_ = false;
  NodeDumpOptions dump_ = NodeDumpOptions::FromEnvironment();
};

}  // namespace ortb
