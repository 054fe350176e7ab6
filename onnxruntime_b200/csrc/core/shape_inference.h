// Static type and shape inference with one function per operator, and the operator schema table behind it.
//
// Plays the role of Graph::Resolve's inference step in the reference (onnxruntime/core/graph/graph.cc:3212-3787,
// which calls ONNX's per-operator inference functions) and of the contrib operator schemas
// (onnxruntime/core/graph/contrib_ops/bert_defs.cc, contrib_defs.cc, quantization_defs.cc, collective_defs.cc).
// Dimensions are values or names; unknown dimensions get a fresh name, so equal symbols mean equal sizes.  Small
// integer tensors (what Shape / Gather / Concat / arithmetic produce on the way to a Reshape) are tracked by value,
// which is what makes the exported transformer graphs resolve without running them.
#pragma once
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "graph.h"

namespace ortb {

struct OpSchema {
  std::string domain, op_type;
  int min_inputs = 0, max_inputs = 1 << 20;
  int min_outputs = 1, max_outputs = 1 << 20;
  std::function<void(class InferenceContext&)> infer;  // may be empty: the operator is known, its shapes are not derived
};

// Read-only view of one node during inference plus the place to write its output types.
class InferenceContext {
 public:
  const Node& node;
  size_t NumInputs() const { return node.inputs.size(); }
  bool HasInput(size_t i) const { return i < node.inputs.size() && !node.inputs[i].empty() && Type(i) != nullptr; }
  const pb::TypeProto* Type(size_t i) const;                 // null when unknown
  bool HasShape(size_t i) const { return Type(i) && Type(i)->has_shape; }
  const std::vector<pb::Dimension>& Dims(size_t i) const;    // requires HasShape(i)
  int Rank(size_t i) const { return HasShape(i) ? static_cast<int>(Dims(i).size()) : -1; }
  int32_t ElemType(size_t i) const { return Type(i) ? Type(i)->elem_type : 0; }
  // value of a small integer tensor input (constant initializer or derived), as dimensions; null when unknown
  const std::vector<pb::Dimension>* IntValue(size_t i) const;
  // constant initializer feeding input i (null otherwise)
  const at::Tensor* Constant(size_t i) const;

  void SetOutput(size_t i, int32_t elem_type, const std::vector<pb::Dimension>& dims);
  void SetOutputType(size_t i, int32_t elem_type);           // type known, shape unknown
  void SetOutputIntValue(size_t i, const std::vector<pb::Dimension>& value);
  void PassThrough(size_t in = 0, size_t out = 0);           // same type and shape
  pb::Dimension FreshDim();

  // internal
  InferenceContext(const Node& n, const Graph& g, std::map<std::string, pb::TypeProto>& types,
                   std::map<std::string, std::vector<pb::Dimension>>& values, int& counter)
      : node(n), graph_(g), types_(types), values_(values), counter_(counter) {}

 private:
  const Graph& graph_;
  std::map<std::string, pb::TypeProto>& types_;
  std::map<std::string, std::vector<pb::Dimension>>& values_;
  int& counter_;
};

const OpSchema* FindSchema(const std::string& domain, const std::string& op_type);
std::vector<const OpSchema*> AllSchemas();

struct InferenceReport {
  int nodes = 0, inferred = 0;            // nodes visited / nodes whose every output got a shape
  std::vector<std::string> problems;      // schema violations ("MatMul node 'x' has 1 inputs, expected 2..2")
};

// Fills graph.ValueInfos() (and the shapes of graph outputs that were declared without one) from the inputs,
// initializers and per-operator functions.  Never throws on an operator it does not know: that value stays unknown.
// `strict`: schema violations raise INVALID_GRAPH instead of being reported.
InferenceReport InferShapes(Graph& g, bool strict = false);

}  // namespace ortb
