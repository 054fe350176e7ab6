// Process-group helpers shared by the collective kernels (baseline paths) and the GPU kernels.
#pragma once
#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>

namespace ortb {

class InferenceSession;

// nullptr when the session is not distributed (world size 1 or no group name).
c10::intrusive_ptr<c10d::ProcessGroup> GroupOf(InferenceSession* s);
at::Tensor AllReduceSum(InferenceSession* s, const at::Tensor& t);             // returns a new tensor
at::Tensor AllGatherAxis(InferenceSession* s, const at::Tensor& t, int64_t axis);
at::Tensor AllToAllEqual(InferenceSession* s, const at::Tensor& t);           // equal splits along the flattened dim

}  // namespace ortb
