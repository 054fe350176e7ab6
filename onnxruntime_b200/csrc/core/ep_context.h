// Compiled ("EP context") models: the graph as the session prepared it - optimized, fused and lowered for the target
// device - stored as the payload of one com.microsoft EPContext node, so that a later session skips that work.
//
// Contract of the reference (onnxruntime/core/framework/graph_partitioner.cc CreateEpContextModel,
// include/onnxruntime/core/session/onnxruntime_session_options_config_keys.h "ep.context_*", docs EPContext design):
//   ep.context_enable = "1"        write the compiled model when the session is created
//   ep.context_file_path           where (default: "<model>_ctx.onnx" beside the input model)
//   ep.context_embed_mode = "1"    payload inside the node (attribute ep_cache_context); "0": in a side file whose
//                                  name, relative to the context model, is the attribute's value
// EPContext node attributes written here: main_context = 1, embed_mode, ep_cache_context, source = "ortb200",
// ep_sdk_version, partition_name.  A model whose only node is such an EPContext node is expanded when it is loaded.
#pragma once
#include <memory>
#include <string>

#include "graph.h"

namespace ortb {

constexpr const char* kEpContextSource = "ortb200";

// Serialized context model for `model` as it stands.  embed = false puts the payload into *side_bytes and the name
// `side_file_name` into the node.
std::string MakeContextModel(const Model& model, bool embed, const std::string& side_file_name, std::string* side_bytes);

// When `model` is a context model of this runtime, replaces it by the model in its payload and returns true.
// `model_dir` resolves the side file of embed_mode 0.
bool ExpandContextModel(std::shared_ptr<Model>& model, const std::string& model_dir);

}  // namespace ortb
