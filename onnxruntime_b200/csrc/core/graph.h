// In-memory graph IR: Model / Graph / Node with name-keyed values.
//
// Plays the role of the reference's onnxruntime/core/graph (graph.cc, model.cc,
// graph_viewer.cc, graph_utils.cc) in a much smaller form: values are
// identified by name, initializers are torch tensors, producer/consumer maps
// are derived lazily, and the optimizer edits the node list directly.
#pragma once
#include <ATen/ATen.h>

#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "onnx_pb.h"

namespace ortb {

constexpr const char* kOnnxDomain = "";
constexpr const char* kMSDomain = "com.microsoft";
constexpr const char* kCpuEP = "CPUExecutionProvider";
constexpr const char* kCudaEP = "CUDAExecutionProvider";

// ONNX element type <-> torch scalar type.  Sub-byte types map to Byte (packed).
at::ScalarType ToTorchType(int32_t onnx_type);
int32_t ToOnnxType(at::ScalarType t);

// TensorProto <-> torch tensor (CPU).  `model_dir` resolves external data files.
at::Tensor TensorFromProto(const pb::TensorProto& t, const std::string& model_dir);
pb::TensorProto TensorToProto(const at::Tensor& t, const std::string& name);

struct ValueInfo {
  std::string name;
  pb::TypeProto type;
};

class Graph;

struct Node {
  int id = -1;
  std::string name, op_type, domain;
  std::vector<std::string> inputs, outputs;  // "" marks an omitted optional
  std::map<std::string, pb::AttributeProto> attrs;
  std::map<std::string, std::shared_ptr<Graph>> subgraphs;  // attribute name -> body
  std::string ep;  // execution provider assigned by the partitioner
  int since_version = 0;
  bool removed = false;  // set by Graph::RemoveNode; the object lives on until Graph::PurgeRemoved()

  bool has_attr(const std::string& n) const { return attrs.count(n) != 0; }
  int64_t attr_i(const std::string& n, int64_t dflt) const;
  float attr_f(const std::string& n, float dflt) const;
  std::string attr_s(const std::string& n, const std::string& dflt = "") const;
  std::vector<int64_t> attr_ints(const std::string& n) const;
  std::vector<float> attr_floats(const std::string& n) const;
  std::vector<std::string> attr_strings(const std::string& n) const;
  at::Tensor attr_tensor(const std::string& n) const;  // undefined tensor when absent
  void set_attr_i(const std::string& n, int64_t v);
  void set_attr_f(const std::string& n, float v);
  void set_attr_s(const std::string& n, const std::string& v);
  void set_attr_ints(const std::string& n, const std::vector<int64_t>& v);
  void set_attr_floats(const std::string& n, const std::vector<float>& v);
  void set_attr_strings(const std::string& n, const std::vector<std::string>& v);
  void set_attr_tensor(const std::string& n, const at::Tensor& t);

  const std::string& input(size_t i) const {
    static const std::string empty;
    return i < inputs.size() ? inputs[i] : empty;
  }
  bool has_input(size_t i) const { return i < inputs.size() && !inputs[i].empty(); }
  bool has_output(size_t i) const { return i < outputs.size() && !outputs[i].empty(); }
};

// a Constant node whose value is a tensor of strings (value_string / value_strings, or a STRING tensor in `value`)
bool ConstantHoldsStrings(const Node& n);

class Graph {
 public:
  Graph() = default;
  static std::shared_ptr<Graph> FromProto(const pb::GraphProto& g, const std::map<std::string, int64_t>& opsets,
                                          const std::string& model_dir, Graph* parent = nullptr);
  pb::GraphProto ToProto() const;

  // ---- nodes
  Node* AddNode(const std::string& op_type, const std::vector<std::string>& inputs,
                const std::vector<std::string>& outputs, const std::string& domain = "",
                const std::string& name = "");
  // Unlinks `n` from the graph.  The object itself is only marked (`removed`, operator type "<removed>") and is
  // released by PurgeRemoved(), so loops over a snapshot of Nodes() may still read it.
  void RemoveNode(Node* n);
  void PurgeRemoved();
  std::vector<Node*> Nodes() const;             // live nodes, insertion order
  std::vector<Node*> TopologicalOrder() const;  // Kahn's algorithm, stable; throws INVALID_GRAPH on a cycle
  size_t NumNodes() const;
  // Re-orders the stored node list topologically.
  void SortNodes();

  // ---- values
  bool IsInitializer(const std::string& name) const { return initializers_.count(name) != 0; }
  // constant == initializer that is not also a graph input (cannot be overridden at run time)
  bool IsConstant(const std::string& name) const;
  const at::Tensor* GetInitializer(const std::string& name) const;
  const at::Tensor* GetConstant(const std::string& name) const;
  void AddInitializer(const std::string& name, const at::Tensor& t);
  void RemoveInitializer(const std::string& name);
  const std::map<std::string, at::Tensor>& Initializers() const { return initializers_; }
  // initializers that hold strings (ids of the string table); GetConstant() hides them from the graph rewrites
  // initializers declared as UINT4 / INT4: held one value per byte (uint8 / int8) and packed again when the graph is saved
  int32_t FourBitTypeOf(const std::string& name) const {
    auto it = four_bit_values_.find(name);
    return it == four_bit_values_.end() ? 0 : it->second;
  }
  void MarkFourBitValue(const std::string& name, int32_t elem_type) { four_bit_values_[name] = elem_type; }
  bool IsStringValue(const std::string& name) const { return string_values_.count(name) != 0; }
  void MarkStringValue(const std::string& name) { string_values_.insert(name); }
  // names of initializers whose data is supplied by the session (external initializers)
  std::set<std::string>& PendingExternal() { return pending_external_; }

  bool IsGraphInput(const std::string& name) const;
  bool IsGraphOutput(const std::string& name) const;
  std::vector<ValueInfo>& Inputs() { return inputs_; }
  std::vector<ValueInfo>& Outputs() { return outputs_; }
  const std::vector<ValueInfo>& Inputs() const { return inputs_; }
  const std::vector<ValueInfo>& Outputs() const { return outputs_; }
  std::map<std::string, ValueInfo>& ValueInfos() { return value_info_; }
  // graph inputs that are not initializers
  std::vector<const ValueInfo*> RuntimeInputs() const;

  Node* Producer(const std::string& value) const;
  std::vector<Node*> Consumers(const std::string& value) const;
  size_t NumConsumers(const std::string& value) const;  // graph outputs count as one consumer
  void ReplaceAllUses(const std::string& old_name, const std::string& new_name);
  std::string UniqueName(const std::string& prefix);
  // true when `name` is visible here or in an enclosing graph
  bool IsOuterScopeValue(const std::string& name) const;

  int64_t Opset(const std::string& domain) const;
  std::map<std::string, int64_t>& Opsets() { return opsets_; }
  const std::string& Name() const { return name_; }
  Graph* Parent() const { return parent_; }
  // Removes nodes whose outputs are unused and initializers nobody reads.
  int RemoveDeadNodes();
  // Values referenced by subgraphs of `n` that are defined outside them.
  std::vector<std::string> ImplicitInputs(const Node& n) const;
  void Invalidate() { dirty_ = true; }

 private:
  void RebuildIndex() const;

  std::string name_;
  std::vector<std::unique_ptr<Node>> nodes_;
  std::vector<std::unique_ptr<Node>> graveyard_;  // removed nodes awaiting PurgeRemoved()
  std::map<std::string, at::Tensor> initializers_;
  std::set<std::string> string_values_;
  std::map<std::string, int32_t> four_bit_values_;
  std::set<std::string> pending_external_;
  std::vector<ValueInfo> inputs_, outputs_;
  std::map<std::string, ValueInfo> value_info_;
  std::map<std::string, int64_t> opsets_;
  Graph* parent_ = nullptr;
  int next_unique_ = 0;

  mutable bool dirty_ = true;
  mutable std::unordered_map<std::string, Node*> producer_;
  mutable std::unordered_map<std::string, std::vector<Node*>> consumers_;
};

class Model {
 public:
  static std::shared_ptr<Model> Load(const std::string& path);
  static std::shared_ptr<Model> LoadFromBytes(std::shared_ptr<const std::string> bytes, const std::string& model_dir = "");
  std::string Serialize() const;  // ModelProto bytes of the current graph
  void Save(const std::string& path) const;

  Graph& MainGraph() { return *graph_; }
  std::shared_ptr<Graph> graph_;
  int64_t ir_version = 8;
  std::string producer_name, producer_version, domain, doc_string, graph_name;
  int64_t model_version = 0;
  std::map<std::string, std::string> metadata;
  std::vector<pb::FunctionProto> functions;
  std::string model_dir;
};

}  // namespace ortb
