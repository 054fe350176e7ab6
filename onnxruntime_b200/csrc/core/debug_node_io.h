// Node input / output dumping for debugging, driven by the reference's environment variables
// (onnxruntime/core/framework/debug_node_inputs_outputs_utils.h:13-74):
//   ORT_DEBUG_NODE_IO_DUMP_SHAPE_DATA=1         shapes and types of every node's inputs and outputs
//   ORT_DEBUG_NODE_IO_DUMP_NODE_PLACEMENT=1     the provider each node runs on
//   ORT_DEBUG_NODE_IO_DUMP_INPUT_DATA=1 / ORT_DEBUG_NODE_IO_DUMP_OUTPUT_DATA=1   values (a snippet: first and last items)
//   ORT_DEBUG_NODE_IO_DUMP_STATISTICS_DATA=1    min / max / mean / count of NaN and Inf per tensor
//   ORT_DEBUG_NODE_IO_DUMP_HALF_CONVERSION_OVERFLOW=1  float tensors with values beyond ORT_DEBUG_NODE_IO_HALF_OVERFLOW_THRESHOLD (65504)
//   ORT_DEBUG_NODE_IO_NAME_FILTER / ORT_DEBUG_NODE_IO_OP_TYPE_FILTER   ';'-separated substrings / operator types
//   ORT_DEBUG_NODE_IO_DUMP_DATA_DESTINATION=stdout|files, ORT_DEBUG_NODE_IO_OUTPUT_DIR, ORT_DEBUG_NODE_IO_SNIPPET_EDGE_ITEMS
// The reference compiles this in with a build flag; here it is always available and costs one flag test per node when
// no variable is set.  Destination "sqlite" is not offered.
#pragma once
#include <string>
#include <vector>

#include "kernel.h"

namespace ortb {

struct NodeDumpOptions {
  bool any = false;
  bool shapes = false, placement = false, input_data = false, output_data = false, statistics = false, half_overflow = false;
  bool to_files = false;
  std::string output_dir = ".";
  std::vector<std::string> name_filter, op_filter;
  int edge_items = 3;
  double half_threshold = 65504.0;

  static NodeDumpOptions FromEnvironment();
  bool Matches(const Node& n) const;
};

// Writes the requested facts about one executed node.  Synchronises with the device when values are read.
void DumpNodeIO(const NodeDumpOptions& opt, const Node& node, const std::vector<Value>& inputs, const std::vector<Value>& outputs);

}  // namespace ortb
