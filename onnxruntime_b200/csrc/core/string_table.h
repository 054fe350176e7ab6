// String tensors.  A tensor of strings is carried as an int64 tensor of ids into a process-wide, append-only table
// of distinct strings (id 0 is the empty string), together with a flag on the Value that holds it.  Every operator
// that only moves elements (Reshape, Gather, Concat, Identity ...) therefore works on string tensors as it is, Equal
// compares ids, and only the operators that look inside the strings go through the table.
// Reference: std::string tensors of onnxruntime/core/framework/tensor.h and data_types.h.
#pragma once
#include <ATen/ATen.h>

#include <string>
#include <vector>

namespace ortb {

int64_t InternString(const std::string& s);
const std::string& StringOfId(int64_t id);  // throws on an id that was never handed out
// ids of `strings` as an int64 CPU tensor of `shape` (numel must match)
at::Tensor InternStrings(const std::vector<std::string>& strings, at::IntArrayRef shape);
// the strings of an id tensor, row-major
std::vector<std::string> StringsOfTensor(const at::Tensor& ids);

}  // namespace ortb
