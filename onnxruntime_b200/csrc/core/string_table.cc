#include "string_table.h"

#include <deque>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>

#include "common.h"

namespace ortb {

namespace {
struct Table {
  std::shared_mutex mu;
  std::deque<std::string> strings;  // deque: references stay valid while the table grows
  std::unordered_map<std::string, int64_t> ids;
  Table() {
    strings.emplace_back("");
    ids.emplace("", 0);
  }
};
Table& table() {
  static Table* t = new Table();  // never destroyed: tensors may outlive static destruction order
  return *t;
}
}  // namespace

int64_t InternString(const std::string& s) {
  Table& t = table();
  {
    std::shared_lock<std::shared_mutex> lock(t.mu);
    auto it = t.ids.find(s);
    if (it != t.ids.end()) return it->second;
  }
  std::unique_lock<std::shared_mutex> lock(t.mu);
  auto it = t.ids.find(s);
  if (it != t.ids.end()) return it->second;
  const int64_t id = static_cast<int64_t>(t.strings.size());
  t.strings.push_back(s);
  t.ids.emplace(s, id);
  return id;
}

const std::string& StringOfId(int64_t id) {
  Table& t = table();
  std::shared_lock<std::shared_mutex> lock(t.mu);
  ORTB_ENFORCE_ARG(id >= 0 && id < static_cast<int64_t>(t.strings.size()), "string tensor holds id ", id, ", which names no string");
  return t.strings[static_cast<size_t>(id)];
}

at::Tensor InternStrings(const std::vector<std::string>& strings, at::IntArrayRef shape) {
  at::Tensor ids = at::empty(shape, at::kLong);
  ORTB_ENFORCE_ARG(ids.numel() == static_cast<int64_t>(strings.size()), "string tensor: ", strings.size(), " strings for shape ", shape);
  int64_t* p = ids.data_ptr<int64_t>();
  for (size_t i = 0; i < strings.size(); ++i) p[i] = InternString(strings[i]);
  return ids;
}

std::vector<std::string> StringsOfTensor(const at::Tensor& ids_in) {
  at::Tensor ids = ids_in.to(at::kCPU, at::kLong).contiguous();
  std::vector<std::string> out;
  out.reserve(static_cast<size_t>(ids.numel()));
  const int64_t* p = ids.data_ptr<int64_t>();
  for (int64_t i = 0; i < ids.numel(); ++i) out.push_back(StringOfId(p[i]));
  return out;
}

}  // namespace ortb
