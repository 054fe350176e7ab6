// Sharding-spec algebra of the Distributed* operators: a device mesh and a
// per-axis partition spec written as "RS[0]" (axis 0 replicated, axis 1
// sharded along mesh axis 0).  Same string grammar and attribute names as the
// reference (onnxruntime/contrib_ops/cuda/collective/sharding_spec.h:18-486);
// like the reference, one sharded tensor axis on a 1-D mesh is what the
// operators support.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "common.h"

namespace ortb {

struct DeviceMesh {
  std::vector<int64_t> elements;  // device ids in row-major order
  std::vector<int64_t> shape;
  static DeviceMesh Parse(const std::string& elements, const std::string& shape);  // "[0,1,2,3]", "[4]"
  int64_t Size() const { return static_cast<int64_t>(elements.size()); }
};

struct AxisPartitionSpec {
  bool sharded = false;
  int mesh_axis = -1;
};

class TensorPartitionSpec {
 public:
  static TensorPartitionSpec Parse(const std::string& spec, const DeviceMesh& mesh);
  static TensorPartitionSpec Replica(size_t rank, const DeviceMesh& mesh);
  std::string ToString() const;
  size_t Rank() const { return axes_.size(); }
  bool HasShard() const { return ShardedAxis() >= 0; }
  int ShardedAxis() const;          // tensor axis that is sharded, -1 when fully replicated
  int64_t NumShards() const;        // number of shards along the sharded axis (1 when replicated)
  const DeviceMesh& Mesh() const { return mesh_; }
  const std::vector<AxisPartitionSpec>& Axes() const { return axes_; }
  std::vector<int64_t> ShardShape(const std::vector<int64_t>& full) const;
  std::vector<int64_t> FullShape(const std::vector<int64_t>& shard) const;
  // index of `device_id` along the sharded mesh axis
  int64_t ShardIndexOf(int64_t device_id) const;

 private:
  std::vector<AxisPartitionSpec> axes_;
  DeviceMesh mesh_;
};

std::vector<int64_t> ParseIntList(const std::string& text);  // "[0, 1, 2]"

}  // namespace ortb
