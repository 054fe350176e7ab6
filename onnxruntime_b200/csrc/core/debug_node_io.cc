#include "debug_node_io.h"

#include <ATen/ATen.h>

#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>

namespace ortb {

namespace {

bool EnvFlag(const char* name) {
  const char* v = std::getenv(name);
  return v != nullptr && std::string(v) != "0" && std::string(v) != "";
}

std::vector<std::string> EnvList(const char* name) {
  std::vector<std::string> out;
  const char* v = std::getenv(name);
  if (v == nullptr) return out;
  std::istringstream ss(v);
  std::string tok;
  while (std::getline(ss, tok, ';'))
    if (!tok.empty()) out.push_back(tok);
  return out;
}

std::string SafeFileName(std::string s) {
  for (char& c : s)
    if (!(std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '-' || c == '.')) c = '_';
  return s;
}

void Describe(std::ostream& os, const NodeDumpOptions& opt, const std::string& label, const std::string& name, const Value& v, bool data) {
  os << "  " << label << " '" << name << "'";
  if (!v.t.defined()) {
    os << (v.defined() ? " <sequence>" : " <absent>") << "\n";
    return;
  }
  const at::Tensor& t = v.t;
  os << " " << c10::toString(t.scalar_type()) << " " << t.sizes() << " on " << t.device() << "\n";
  if (t.numel() == 0 || !(data || opt.statistics || opt.half_overflow)) return;
  at::Tensor host = t.detach().to(at::kCPU);
  const bool numeric = host.is_floating_point() || at::isIntegralType(host.scalar_type(), /*includeBool=*/true);
  if (!numeric) return;
  at::Tensor f = host.to(at::kDouble).reshape({-1});
  if (opt.statistics) {
    at::Tensor finite = at::isfinite(f);
    const int64_t nan = at::isnan(f).sum().item<int64_t>(), inf = at::isinf(f).sum().item<int64_t>();
    os << "    statistics: ";
    if (finite.any().item<bool>()) {
      at::Tensor g = f.masked_select(finite);
      os << "min " << g.min().item<double>() << " max " << g.max().item<double>() << " mean " << g.mean().item<double>();
    } else {
      os << "no finite value";
    }
    os << " nan " << nan << " inf " << inf << " count " << f.numel() << "\n";
  }
  if (opt.half_overflow && host.scalar_type() == at::kFloat) {
    const int64_t over = (f.abs() > opt.half_threshold).sum().item<int64_t>();
    if (over > 0) os << "    half conversion overflow: " << over << " values beyond " << opt.half_threshold << "\n";
  }
  if (data) {
    const int64_t n = f.numel(), e = opt.edge_items;
    os << "    data: [";
    for (int64_t i = 0; i < n; ++i) {
      if (n > 2 * e && i == e) {
        os << " ...";
        i = n - e - 1;
        continue;
      }
      os << (i ? " " : "") << f[i].item<double>();
    }
    os << "]\n";
  }
}

}  // namespace

NodeDumpOptions NodeDumpOptions::FromEnvironment() {
  NodeDumpOptions o;
  o.shapes = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_SHAPE_DATA");
  o.placement = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_NODE_PLACEMENT");
  o.input_data = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_INPUT_DATA");
  o.output_data = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_OUTPUT_DATA");
  o.statistics = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_STATISTICS_DATA");
  o.half_overflow = EnvFlag("ORT_DEBUG_NODE_IO_DUMP_HALF_CONVERSION_OVERFLOW");
  o.any = o.shapes || o.placement || o.input_data || o.output_data || o.statistics || o.half_overflow;
  o.name_filter = EnvList("ORT_DEBUG_NODE_IO_NAME_FILTER");
  o.op_filter = EnvList("ORT_DEBUG_NODE_IO_OP_TYPE_FILTER");
  if (const char* d = std::getenv("ORT_DEBUG_NODE_IO_DUMP_DATA_DESTINATION")) o.to_files = std::string(d) == "files";
  if (const char* d = std::getenv("ORT_DEBUG_NODE_IO_OUTPUT_DIR")) o.output_dir = d;
  if (const char* d = std::getenv("ORT_DEBUG_NODE_IO_SNIPPET_EDGE_ITEMS")) o.edge_items = std::max(1, std::atoi(d));
  if (const char* d = std::getenv("ORT_DEBUG_NODE_IO_HALF_OVERFLOW_THRESHOLD")) o.half_threshold = std::atof(d);
  return o;
}

bool NodeDumpOptions::Matches(const Node& n) const {
  if (!op_filter.empty()) {
    bool hit = false;
    for (auto& f : op_filter) hit = hit || n.op_type == f;
    if (!hit) return false;
  }
  if (!name_filter.empty()) {
    bool hit = false;
    for (auto& f : name_filter) hit = hit || n.name.find(f) != std::string::npos;
    if (!hit) return false;
  }
  return true;
}

void DumpNodeIO(const NodeDumpOptions& opt, const Node& node, const std::vector<Value>& inputs, const std::vector<Value>& outputs) {
  if (!opt.any || !opt.Matches(node)) return;
  std::ostringstream os;
  os << "node '" << node.name << "' (" << (node.domain.empty() ? "" : node.domain + "::") << node.op_type << ")";
  if (opt.placement) os << " on " << (node.ep.empty() ? kCpuEP : node.ep);
  os << "\n";
  const bool describe = opt.shapes || opt.input_data || opt.output_data || opt.statistics || opt.half_overflow;
  if (describe) {
    for (size_t i = 0; i < inputs.size(); ++i)
      if (i < node.inputs.size() && !node.inputs[i].empty()) Describe(os, opt, "input", node.inputs[i], inputs[i], opt.input_data);
    for (size_t i = 0; i < outputs.size(); ++i)
      if (i < node.outputs.size() && !node.outputs[i].empty()) Describe(os, opt, "output", node.outputs[i], outputs[i], opt.output_data);
  }
  if (opt.to_files) {
    std::ofstream f(opt.output_dir + "/" + SafeFileName(node.name.empty() ? node.op_type : node.name) + ".txt", std::ios::app);
    if (f) {
      f << os.str();
      return;
    }
  }
  std::cout << os.str() << std::flush;
}

}  // namespace ortb
