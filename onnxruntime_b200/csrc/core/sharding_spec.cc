#include "sharding_spec.h"

#include <cctype>
#include <sstream>

namespace ortb {

std::vector<int64_t> ParseIntList(const std::string& text) {
  std::vector<int64_t> out;
  std::string cur;
  for (char c : text) {
    if (std::isdigit(static_cast<unsigned char>(c)) || c == '-') {
      cur.push_back(c);
    } else {
      if (!cur.empty()) out.push_back(std::stoll(cur));
      cur.clear();
      if (!(c == '[' || c == ']' || c == ',' || std::isspace(static_cast<unsigned char>(c))))
        ORTB_THROW(INVALID_ARGUMENT, "unexpected character '", c, "' in integer list \"", text, "\"");
    }
  }
  if (!cur.empty()) out.push_back(std::stoll(cur));
  return out;
}

DeviceMesh DeviceMesh::Parse(const std::string& elements, const std::string& shape) {
  DeviceMesh m;
  m.elements = ParseIntList(elements);
  m.shape = ParseIntList(shape);
  int64_t n = 1;
  for (auto d : m.shape) n *= d;
  ORTB_ENFORCE_ARG(n == static_cast<int64_t>(m.elements.size()), "device mesh shape ", shape, " does not match ",
                   m.elements.size(), " elements");
  return m;
}

TensorPartitionSpec TensorPartitionSpec::Parse(const std::string& spec, const DeviceMesh& mesh) {
  TensorPartitionSpec s;
  s.mesh_ = mesh;
  size_t i = 0;
  int shards = 0;
  while (i < spec.size()) {
    const char c = spec[i];
    if (c == 'R') {
      s.axes_.push_back({false, -1});
      ++i;
    } else if (c == 'S') {
      ORTB_ENFORCE_ARG(i + 1 < spec.size() && spec[i + 1] == '[', "sharding spec \"", spec, "\": S must be followed by [mesh axis]");
      const size_t close = spec.find(']', i);
      ORTB_ENFORCE_ARG(close != std::string::npos, "sharding spec \"", spec, "\": missing ]");
      const int axis = std::stoi(spec.substr(i + 2, close - i - 2));
      ORTB_ENFORCE_ARG(axis >= 0 && axis < static_cast<int>(mesh.shape.size()), "sharding spec \"", spec, "\": mesh axis ",
                       axis, " out of range");
      s.axes_.push_back({true, axis});
      ++shards;
      i = close + 1;
    } else if (std::isspace(static_cast<unsigned char>(c))) {
      ++i;
    } else {
      ORTB_THROW(INVALID_ARGUMENT, "sharding spec \"", spec, "\": unexpected character '", c, "'");
    }
  }
  ORTB_ENFORCE_ARG(shards <= 1, "sharding spec \"", spec, "\": at most one sharded tensor axis is supported");
  return s;
}

TensorPartitionSpec TensorPartitionSpec::Replica(size_t rank, const DeviceMesh& mesh) {
  TensorPartitionSpec s;
  s.mesh_ = mesh;
  s.axes_.assign(rank, AxisPartitionSpec{});
  return s;
}

std::string TensorPartitionSpec::ToString() const {
  std::ostringstream ss;
  for (auto& a : axes_) {
    if (a.sharded) ss << "S[" << a.mesh_axis << "]";
    else ss << "R";
  }
  return ss.str();
}

int TensorPartitionSpec::ShardedAxis() const {
  for (size_t i = 0; i < axes_.size(); ++i)
    if (axes_[i].sharded) return static_cast<int>(i);
  return -1;
}

int64_t TensorPartitionSpec::NumShards() const {
  const int ax = ShardedAxis();
  if (ax < 0) return 1;
  return mesh_.shape[axes_[ax].mesh_axis];
}

std::vector<int64_t> TensorPartitionSpec::ShardShape(const std::vector<int64_t>& full) const {
  ORTB_ENFORCE_ARG(full.size() == axes_.size(), "shape rank ", full.size(), " does not match spec ", ToString());
  std::vector<int64_t> out = full;
  const int ax = ShardedAxis();
  if (ax >= 0) {
    ORTB_ENFORCE_ARG(full[ax] % NumShards() == 0, "dimension ", full[ax], " is not divisible into ", NumShards(), " shards");
    out[ax] = full[ax] / NumShards();
  }
  return out;
}

std::vector<int64_t> TensorPartitionSpec::FullShape(const std::vector<int64_t>& shard) const {
  ORTB_ENFORCE_ARG(shard.size() == axes_.size(), "shape rank ", shard.size(), " does not match spec ", ToString());
  std::vector<int64_t> out = shard;
  const int ax = ShardedAxis();
  if (ax >= 0) out[ax] = shard[ax] * NumShards();
  return out;
}

int64_t TensorPartitionSpec::ShardIndexOf(int64_t device_id) const {
  const int ax = ShardedAxis();
  if (ax < 0) return 0;
  // position of the device in the mesh, then its coordinate along the sharded mesh axis
  int64_t linear = -1;
  for (size_t i = 0; i < mesh_.elements.size(); ++i)
    if (mesh_.elements[i] == device_id) linear = static_cast<int64_t>(i);
  ORTB_ENFORCE_ARG(linear >= 0, "device ", device_id, " is not part of the mesh");
  const int mesh_axis = axes_[ax].mesh_axis;
  int64_t stride = 1;
  for (size_t i = mesh_.shape.size(); i-- > static_cast<size_t>(mesh_axis) + 1;) stride *= mesh_.shape[i];
  return (linear / stride) % mesh_.shape[mesh_axis];
}

}  // namespace ortb
