#include "ep_context.h"

#include <fstream>
#include <sstream>

#include "common.h"
#include "onnx_pb.h"

namespace ortb {

namespace {

pb::AttributeProto IntAttr(const std::string& name, int64_t v) {
  pb::AttributeProto a;
  a.name = name;
  a.type = 2;  // INT
  a.i = v;
  return a;
}

pb::AttributeProto StrAttr(const std::string& name, const std::string& v) {
  pb::AttributeProto a;
  a.name = name;
  a.type = 3;  // STRING
  a.s = v;
  return a;
}

}  // namespace

std::string MakeContextModel(const Model& model, bool embed, const std::string& side_file_name, std::string* side_bytes) {
  const std::string payload = model.Serialize();
  Graph& g = *model.graph_;
  pb::ModelProto mp;
  mp.ir_version = model.ir_version;
  mp.producer_name = model.producer_name;
  mp.producer_version = model.producer_version;
  mp.domain = model.domain;
  mp.doc_string = model.doc_string;
  mp.model_version = model.model_version;
  mp.has_graph = true;
  mp.graph.name = model.graph_name.empty() ? "ep_context" : model.graph_name;
  pb::NodeProto node;
  node.op_type = "EPContext";
  node.domain = kMSDomain;
  node.name = "ortb200_context_0";
  for (const ValueInfo* vi : g.RuntimeInputs()) {
    pb::ValueInfoProto p;
    p.name = vi->name;
    p.type = vi->type;
    mp.graph.input.push_back(p);
    node.input.push_back(vi->name);
  }
  for (const ValueInfo& vi : g.Outputs()) {
    pb::ValueInfoProto p;
    p.name = vi.name;
    p.type = vi.type;
    mp.graph.output.push_back(p);
    node.output.push_back(vi.name);
  }
  node.attribute.push_back(IntAttr("main_context", 1));
  node.attribute.push_back(IntAttr("embed_mode", embed ? 1 : 0));
  node.attribute.push_back(StrAttr("source", kEpContextSource));
  node.attribute.push_back(StrAttr("ep_sdk_version", "0.1.0"));
  node.attribute.push_back(StrAttr("partition_name", "ortb200_partition_0"));
  if (embed) {
    node.attribute.push_back(StrAttr("ep_cache_context", payload));
  } else {
    ORTB_ENFORCE_ARG(side_bytes != nullptr && !side_file_name.empty(), "a side file is needed when the payload is not embedded");
    node.attribute.push_back(StrAttr("ep_cache_context", side_file_name));
    *side_bytes = payload;
  }
  mp.graph.node.push_back(std::move(node));
  bool has_ms = false;
  for (auto& kv : g.Opsets()) {
    mp.opset_import.push_back({kv.first, kv.second});
    has_ms = has_ms || kv.first == kMSDomain;
  }
  if (!has_ms) mp.opset_import.push_back({kMSDomain, 1});
  for (auto& kv : model.metadata) mp.metadata_props.push_back({kv.first, kv.second});
  return pb::SerializeModel(mp);
}

bool ExpandContextModel(std::shared_ptr<Model>& model, const std::string& model_dir) {
  Graph& g = model->MainGraph();
  auto nodes = g.Nodes();
  if (nodes.size() != 1) {
    for (Node* n : nodes)
      if (n->op_type == "EPContext" && n->domain == kMSDomain && n->attr_s("source") == kEpContextSource)
        ORTB_THROW(NOT_IMPLEMENTED, "EPContext node '", n->name, "' beside other nodes: only whole-graph context models are supported");
    return false;
  }
  Node* n = nodes[0];
  if (n->op_type != "EPContext" || n->domain != kMSDomain) return false;
  const std::string source = n->attr_s("source");
  if (source != kEpContextSource)
    ORTB_THROW(NOT_IMPLEMENTED, "EPContext node '", n->name, "' was compiled by '", source, "'; this runtime loads its own context models only");
  std::string payload = n->attr_s("ep_cache_context");
  if (n->attr_i("embed_mode", 1) == 0) {
    ORTB_ENFORCE_ARG(payload.find("..") == std::string::npos && !payload.empty() && payload[0] != '/',
                     "EPContext: the side file must be a relative path below the model's directory");
    const std::string path = (model_dir.empty() ? std::string(".") : model_dir) + "/" + payload;
    std::ifstream f(path, std::ios::binary);
    if (!f) ORTB_THROW(NO_SUCHFILE, "EPContext: cannot open the context file ", path);
    std::ostringstream ss;
    ss << f.rdbuf();
    payload = ss.str();
  }
  ORTB_ENFORCE_ARG(!payload.empty(), "EPContext node without a payload");
  std::shared_ptr<Model> inner = Model::LoadFromBytes(std::make_shared<std::string>(std::move(payload)), model_dir);
  // the outer file's metadata wins where it says something (the payload was written from the same model)
  for (auto& kv : model->metadata) inner->metadata[kv.first] = kv.second;
  model = inner;
  return true;
}

}  // namespace ortb
