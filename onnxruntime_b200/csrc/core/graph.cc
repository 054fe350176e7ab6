#include "graph.h"
#include "string_table.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>

namespace ortb {

const char* StatusCodeName(StatusCode c) {
  switch (c) {
    case StatusCode::OK: return "OK";
    case StatusCode::FAIL: return "FAIL";
    case StatusCode::INVALID_ARGUMENT: return "INVALID_ARGUMENT";
    case StatusCode::NO_SUCHFILE: return "NO_SUCHFILE";
    case StatusCode::NO_MODEL: return "NO_MODEL";
    case StatusCode::ENGINE_ERROR: return "ENGINE_ERROR";
    case StatusCode::RUNTIME_EXCEPTION: return "RUNTIME_EXCEPTION";
    case StatusCode::INVALID_PROTOBUF: return "INVALID_PROTOBUF";
    case StatusCode::MODEL_LOADED: return "MODEL_LOADED";
    case StatusCode::NOT_IMPLEMENTED: return "NOT_IMPLEMENTED";
    case StatusCode::INVALID_GRAPH: return "INVALID_GRAPH";
    case StatusCode::EP_FAIL: return "EP_FAIL";
    case StatusCode::MODEL_LOAD_CANCELED: return "MODEL_LOAD_CANCELED";
    case StatusCode::MODEL_REQUIRES_COMPILATION: return "MODEL_REQUIRES_COMPILATION";
    case StatusCode::NOT_FOUND: return "NOT_FOUND";
  }
  return "UNKNOWN";
}

std::string Status::ToString() const {
  if (IsOK()) return "OK";
  return MakeString("[ONNXRuntimeError] : ", static_cast<int>(code_), " : ", StatusCodeName(code_), " : ", msg_);
}

// --------------------------------------------------------------- type mapping
at::ScalarType ToTorchType(int32_t t) {
  switch (t) {
    case pb::FLOAT: return at::kFloat;
    case pb::UINT8: return at::kByte;
    case pb::INT8: return at::kChar;
    case pb::UINT16: return at::kUInt16;
    case pb::INT16: return at::kShort;
    case pb::INT32: return at::kInt;
    case pb::INT64: return at::kLong;
    case pb::BOOL: return at::kBool;
    case pb::FLOAT16: return at::kHalf;
    case pb::DOUBLE: return at::kDouble;
    case pb::UINT32: return at::kUInt32;
    case pb::UINT64: return at::kUInt64;
    case pb::COMPLEX64: return at::kComplexFloat;
    case pb::COMPLEX128: return at::kComplexDouble;
    case pb::BFLOAT16: return at::kBFloat16;
    case pb::FLOAT8E4M3FN: return at::kFloat8_e4m3fn;
    case pb::FLOAT8E4M3FNUZ: return at::kFloat8_e4m3fnuz;
    case pb::FLOAT8E5M2: return at::kFloat8_e5m2;
    case pb::FLOAT8E5M2FNUZ: return at::kFloat8_e5m2fnuz;
    case pb::UINT4: case pb::INT4: case pb::FLOAT4E2M1: return at::kByte;
    default: ORTB_THROW(NOT_IMPLEMENTED, "ONNX element type ", t, " has no tensor representation");
  }
}

int32_t ToOnnxType(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return pb::FLOAT;
    case at::kByte: return pb::UINT8;
    case at::kChar: return pb::INT8;
    case at::kUInt16: return pb::UINT16;
    case at::kShort: return pb::INT16;
    case at::kInt: return pb::INT32;
    case at::kLong: return pb::INT64;
    case at::kBool: return pb::BOOL;
    case at::kHalf: return pb::FLOAT16;
    case at::kDouble: return pb::DOUBLE;
    case at::kUInt32: return pb::UINT32;
    case at::kUInt64: return pb::UINT64;
    case at::kComplexFloat: return pb::COMPLEX64;
    case at::kComplexDouble: return pb::COMPLEX128;
    case at::kBFloat16: return pb::BFLOAT16;
    case at::kFloat8_e4m3fn: return pb::FLOAT8E4M3FN;
    case at::kFloat8_e4m3fnuz: return pb::FLOAT8E4M3FNUZ;
    case at::kFloat8_e5m2: return pb::FLOAT8E5M2;
    case at::kFloat8_e5m2fnuz: return pb::FLOAT8E5M2FNUZ;
    default: ORTB_THROW(NOT_IMPLEMENTED, "torch dtype has no ONNX element type");
  }
}

namespace {

struct MappedFile {
  void* addr = nullptr;
  size_t size = 0;
  ~MappedFile() {
    if (addr) munmap(addr, size);
  }
};

std::shared_ptr<MappedFile> MapFile(const std::string& path) {
  int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) ORTB_THROW(NO_SUCHFILE, "cannot open external data file ", path);
  struct stat st;
  if (fstat(fd, &st) != 0) {
    ::close(fd);
    ORTB_THROW(FAIL, "fstat failed for ", path);
  }
  auto mf = std::make_shared<MappedFile>();
  mf->size = static_cast<size_t>(st.st_size);
  if (mf->size) {
    mf->addr = mmap(nullptr, mf->size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (mf->addr == MAP_FAILED) {
      mf->addr = nullptr;
      ::close(fd);
      ORTB_THROW(FAIL, "mmap failed for ", path);
    }
  }
  ::close(fd);
  return mf;
}

int64_t NumElements(const std::vector<int64_t>& dims) {
  int64_t n = 1;
  for (auto d : dims) {
    ORTB_ENFORCE_ARG(d >= 0, "negative dimension in tensor");
    n *= d;
  }
  return n;
}

}  // namespace

at::Tensor TensorFromProto(const pb::TensorProto& t, const std::string& model_dir) {
  if (t.data_type == pb::STRING) return InternStrings(t.string_data, t.dims);  // ids; the caller marks the value as strings
  const at::ScalarType st = ToTorchType(t.data_type);
  const bool sub_byte = (t.data_type == pb::UINT4 || t.data_type == pb::INT4 || t.data_type == pb::FLOAT4E2M1);
  std::vector<int64_t> dims = t.dims;
  int64_t numel = NumElements(dims);
  int64_t nbytes;
  if (sub_byte) {
    nbytes = (numel + 1) / 2;
    dims = {nbytes};  // packed storage, two elements per byte
  } else {
    nbytes = numel * static_cast<int64_t>(c10::elementSize(st));
  }
  at::Tensor out = at::empty(dims, at::TensorOptions().dtype(st));

  if (t.data_location == 1) {
    std::string location;
    int64_t offset = 0, length = -1;
    for (auto& e : t.external_data) {
      if (e.key == "location") location = e.value;
      else if (e.key == "offset") offset = std::stoll(e.value);
      else if (e.key == "length") length = std::stoll(e.value);
    }
    ORTB_ENFORCE_ARG(!location.empty(), "external tensor '", t.name, "' has no location");
    // A location may not escape the model directory and may not be an in-memory address tag.
    ORTB_ENFORCE_ARG(location[0] != '/' && location.find("..") == std::string::npos && location[0] != '*',
                     "external data location '", location, "' is not a relative path inside the model directory");
    const std::string path = model_dir.empty() ? location : model_dir + "/" + location;
    auto mf = MapFile(path);
    if (length < 0) length = nbytes;
    ORTB_ENFORCE_ARG(length >= nbytes && offset >= 0 && static_cast<size_t>(offset + nbytes) <= mf->size,
                     "external data for '", t.name, "' is out of range of ", path);
    std::memcpy(out.data_ptr(), static_cast<const char*>(mf->addr) + offset, nbytes);
    return out;
  }

  if (t.has_raw) {
    ORTB_ENFORCE_ARG(static_cast<int64_t>(t.raw_size) == nbytes, "raw_data of tensor '", t.name, "' has ", t.raw_size,
                     " bytes, expected ", nbytes);
    if (nbytes) std::memcpy(out.data_ptr(), t.raw, nbytes);
    return out;
  }

  auto need = [&](size_t have) {
    ORTB_ENFORCE_ARG(static_cast<int64_t>(have) == numel || (numel == 0 && have == 0), "tensor '", t.name, "' has ",
                     have, " typed values, expected ", numel);
  };
  switch (t.data_type) {
    case pb::FLOAT:
      need(t.float_data.size());
      if (numel) std::memcpy(out.data_ptr(), t.float_data.data(), numel * 4);
      break;
    case pb::DOUBLE:
      need(t.double_data.size());
      if (numel) std::memcpy(out.data_ptr(), t.double_data.data(), numel * 8);
      break;
    case pb::INT64:
      need(t.int64_data.size());
      if (numel) std::memcpy(out.data_ptr(), t.int64_data.data(), numel * 8);
      break;
    case pb::UINT64:
      need(t.uint64_data.size());
      if (numel) std::memcpy(out.data_ptr(), t.uint64_data.data(), numel * 8);
      break;
    case pb::UINT32: {
      need(t.uint64_data.size());
      auto* p = static_cast<uint32_t*>(out.data_ptr());
      for (int64_t i = 0; i < numel; ++i) p[i] = static_cast<uint32_t>(t.uint64_data[i]);
      break;
    }
    case pb::INT32:
      need(t.int32_data.size());
      if (numel) std::memcpy(out.data_ptr(), t.int32_data.data(), numel * 4);
      break;
    case pb::COMPLEX64:
      ORTB_ENFORCE_ARG(static_cast<int64_t>(t.float_data.size()) == numel * 2, "complex64 tensor size");
      if (numel) std::memcpy(out.data_ptr(), t.float_data.data(), numel * 8);
      break;
    case pb::COMPLEX128:
      ORTB_ENFORCE_ARG(static_cast<int64_t>(t.double_data.size()) == numel * 2, "complex128 tensor size");
      if (numel) std::memcpy(out.data_ptr(), t.double_data.data(), numel * 16);
      break;
    case pb::UINT4: case pb::INT4: case pb::FLOAT4E2M1: {
      ORTB_ENFORCE_ARG(static_cast<int64_t>(t.int32_data.size()) == nbytes, "packed 4-bit tensor size");
      auto* p = static_cast<uint8_t*>(out.data_ptr());
      for (int64_t i = 0; i < nbytes; ++i) p[i] = static_cast<uint8_t>(t.int32_data[i]);
      break;
    }
    default: {
      // 8/16-bit types and bool store their bit patterns in int32_data
      need(t.int32_data.size());
      const size_t es = c10::elementSize(st);
      auto* p = static_cast<uint8_t*>(out.data_ptr());
      for (int64_t i = 0; i < numel; ++i) {
        const uint32_t v = static_cast<uint32_t>(t.int32_data[i]);
        if (es == 1) p[i] = static_cast<uint8_t>(v);
        else if (es == 2) reinterpret_cast<uint16_t*>(p)[i] = static_cast<uint16_t>(v);
        else ORTB_THROW(INVALID_ARGUMENT, "unexpected typed storage for element type ", t.data_type);
      }
    }
  }
  return out;
}

pb::TensorProto TensorToProto(const at::Tensor& t_in, const std::string& name) {
  at::Tensor t = t_in.detach().cpu().contiguous();
  pb::TensorProto p;
  p.name = name;
  p.data_type = ToOnnxType(t.scalar_type());
  p.dims = t.sizes().vec();
  p.set_raw(std::string(static_cast<const char*>(t.data_ptr()), t.nbytes()));
  return p;
}

// ------------------------------------------------------------------- Node
static const pb::AttributeProto* FindAttr(const Node& n, const std::string& name) {
  auto it = n.attrs.find(name);
  return it == n.attrs.end() ? nullptr : &it->second;
}

int64_t Node::attr_i(const std::string& n, int64_t dflt) const {
  auto* a = FindAttr(*this, n);
  if (!a) return dflt;
  if (a->type == pb::ATTR_INT) return a->i;
  if (a->type == pb::ATTR_FLOAT) return static_cast<int64_t>(a->f);
  return dflt;
}
float Node::attr_f(const std::string& n, float dflt) const {
  auto* a = FindAttr(*this, n);
  if (!a) return dflt;
  if (a->type == pb::ATTR_FLOAT) return a->f;
  if (a->type == pb::ATTR_INT) return static_cast<float>(a->i);
  return dflt;
}
std::string Node::attr_s(const std::string& n, const std::string& dflt) const {
  auto* a = FindAttr(*this, n);
  return (a && a->type == pb::ATTR_STRING) ? a->s : dflt;
}
std::vector<int64_t> Node::attr_ints(const std::string& n) const {
  auto* a = FindAttr(*this, n);
  if (!a) return {};
  if (a->type == pb::ATTR_INT) return {a->i};
  return a->ints;
}
std::vector<float> Node::attr_floats(const std::string& n) const {
  auto* a = FindAttr(*this, n);
  if (!a) return {};
  if (a->type == pb::ATTR_FLOAT) return {a->f};
  return a->floats;
}
std::vector<std::string> Node::attr_strings(const std::string& n) const {
  auto* a = FindAttr(*this, n);
  return a ? a->strings : std::vector<std::string>{};
}
at::Tensor DenseFromSparseProto(const pb::SparseTensorProto& s) {
  at::Tensor values = TensorFromProto(s.values, "").reshape({-1});
  at::Tensor idx = TensorFromProto(s.indices, "").to(at::kLong);
  at::Tensor dense = at::zeros({NumElements(s.dims)}, values.options());
  if (idx.dim() == 2) {  // [nnz, rank] coordinates -> linear positions
    ORTB_ENFORCE_ARG(idx.size(1) == static_cast<int64_t>(s.dims.size()), "sparse tensor '", s.values.name, "': indices do not match the rank");
    at::Tensor lin = at::zeros({idx.size(0)}, at::kLong);
    int64_t stride = 1;
    for (int64_t d = static_cast<int64_t>(s.dims.size()) - 1; d >= 0; --d) {
      lin = lin + idx.select(1, d) * stride;
      stride *= s.dims[static_cast<size_t>(d)];
    }
    idx = lin;
  }
  ORTB_ENFORCE_ARG(idx.numel() == values.numel(), "sparse tensor '", s.values.name, "': ", idx.numel(), " indices for ", values.numel(), " values");
  if (idx.numel() > 0) {
    ORTB_ENFORCE_ARG(idx.min().item<int64_t>() >= 0 && idx.max().item<int64_t>() < dense.numel(), "sparse tensor '", s.values.name, "': index out of range");
    dense.index_put_({idx.reshape({-1})}, values);
  }
  return dense.reshape(s.dims);
}

bool ConstantHoldsStrings(const Node& n) {
  if (n.has_attr("value_string") || n.has_attr("value_strings")) return true;
  auto* a = FindAttr(n, "value");
  return a && a->t && a->t->data_type == pb::STRING;
}
at::Tensor Node::attr_tensor(const std::string& n) const {
  auto* a = FindAttr(*this, n);
  if (a && a->sparse_tensor) return DenseFromSparseProto(*a->sparse_tensor);  // Constant.sparse_value
  if (!a || !a->t) return at::Tensor();
  return TensorFromProto(*a->t, "");
}
void Node::set_attr_i(const std::string& n, int64_t v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_INT; a.i = v; attrs[n] = a;
}
void Node::set_attr_f(const std::string& n, float v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_FLOAT; a.f = v; attrs[n] = a;
}
void Node::set_attr_s(const std::string& n, const std::string& v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_STRING; a.s = v; attrs[n] = a;
}
void Node::set_attr_ints(const std::string& n, const std::vector<int64_t>& v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_INTS; a.ints = v; attrs[n] = a;
}
void Node::set_attr_floats(const std::string& n, const std::vector<float>& v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_FLOATS; a.floats = v; attrs[n] = a;
}
void Node::set_attr_strings(const std::string& n, const std::vector<std::string>& v) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_STRINGS; a.strings = v; attrs[n] = a;
}
void Node::set_attr_tensor(const std::string& n, const at::Tensor& t) {
  pb::AttributeProto a; a.name = n; a.type = pb::ATTR_TENSOR;
  a.t = std::make_shared<pb::TensorProto>(TensorToProto(t, ""));
  attrs[n] = a;
}

// ------------------------------------------------------------------ Graph
std::shared_ptr<Graph> Graph::FromProto(const pb::GraphProto& g, const std::map<std::string, int64_t>& opsets,
                                        const std::string& model_dir, Graph* parent) {
  auto out = std::make_shared<Graph>();
  out->name_ = g.name;
  out->opsets_ = opsets;
  out->parent_ = parent;
  for (auto& t : g.initializer) {
    ORTB_ENFORCE_ARG(!t.name.empty(), "initializer without a name");
    bool pending = false;
    if (t.data_location == 1) {
      // External initializers may be supplied by the session instead of a file.
      pending = true;
      for (auto& e : t.external_data)
        if (e.key == "location" && e.value.rfind("*session*", 0) != 0) pending = false;
    }
    if (pending) {
      out->pending_external_.insert(t.name);
      out->initializers_[t.name] = at::empty({0}, at::TensorOptions().dtype(ToTorchType(t.data_type)));
      ValueInfo vi;
      vi.name = t.name;
      vi.type.which = 1;
      vi.type.elem_type = t.data_type;
      vi.type.has_shape = true;
      for (auto d : t.dims) {
        pb::Dimension dim;
        dim.has_value = true;
        dim.value = d;
        vi.type.dims.push_back(dim);
      }
      out->value_info_[t.name] = vi;
    } else {
      out->initializers_[t.name] = TensorFromProto(t, model_dir);
      if (t.data_type == pb::STRING) out->string_values_.insert(t.name);
      if (t.data_type == pb::UINT4 || t.data_type == pb::INT4) {
        // two values per byte, low nibble first -> one value per byte with the declared shape
        at::Tensor packed = out->initializers_[t.name].to(at::kInt);
        at::Tensor v = at::stack({at::bitwise_and(packed, 15), at::bitwise_right_shift(packed, 4)}, 1).reshape({-1}).narrow(0, 0, NumElements(t.dims));
        if (t.data_type == pb::INT4) v = at::bitwise_xor(v, 8) - 8;  // sign extension
        out->initializers_[t.name] = v.to(t.data_type == pb::INT4 ? at::kChar : at::kByte).reshape(t.dims).contiguous();
        out->four_bit_values_[t.name] = t.data_type;
      }
      if (t.data_type == pb::UINT4 || t.data_type == pb::INT4 || t.data_type == pb::FLOAT4E2M1) {
        ValueInfo vi;
        vi.name = t.name;
        vi.type.which = 1;
        vi.type.elem_type = t.data_type;
        vi.type.has_shape = true;
        for (auto d : t.dims) {
          pb::Dimension dim;
          dim.has_value = true;
          dim.value = d;
          vi.type.dims.push_back(dim);
        }
        out->value_info_[t.name] = vi;
      }
    }
  }
  // sparse initializers: the kernels are dense, so they are expanded here
  for (auto& s : g.sparse_initializer) {
    ORTB_ENFORCE_ARG(!s.values.name.empty(), "sparse initializer without a name");
    out->initializers_[s.values.name] = DenseFromSparseProto(s);
  }
  for (auto& v : g.input) out->inputs_.push_back({v.name, v.type});
  for (auto& v : g.output) out->outputs_.push_back({v.name, v.type});
  for (auto& v : g.value_info) out->value_info_[v.name] = {v.name, v.type};
  std::set<std::string> seen_outputs;
  for (auto& n : g.node) {
    Node* node = out->AddNode(n.op_type, n.input, n.output, n.domain == "ai.onnx" ? "" : n.domain, n.name);
    for (auto& o : n.output) {
      if (o.empty()) continue;
      if (!seen_outputs.insert(o).second)
        ORTB_THROW(INVALID_GRAPH, "value '", o, "' is produced by more than one node (graph is not in SSA form)");
    }
    for (auto& a : n.attribute) {
      if (a.type == pb::ATTR_GRAPH && a.g) {
        node->subgraphs[a.name] = Graph::FromProto(*a.g, opsets, model_dir, out.get());
      } else if (a.type == pb::ATTR_GRAPHS) {
        ORTB_NOT_IMPLEMENTED("attribute '", a.name, "' of node '", n.name, "' holds a list of graphs");
      } else {
        // Tensor attributes are read at run time (ConstantOfShape, Constant ...), long after the parsed model bytes
        // are gone: give each its own copy of the bytes its raw_data view points at.
        pb::AttributeProto& held = node->attrs[a.name];
        held = a;
        auto own = [](pb::TensorProto& t) {
          if (t.has_raw) t.set_raw(std::string(t.raw, t.raw_size));
        };
        if (held.t) {
          held.t = std::make_shared<pb::TensorProto>(*held.t);
          own(*held.t);
        }
        for (auto& t : held.tensors) own(t);
      }
    }
    node->since_version = static_cast<int>(out->Opset(node->domain));
  }
  return out;
}

pb::GraphProto Graph::ToProto() const {
  pb::GraphProto g;
  g.name = name_;
  for (Node* n : TopologicalOrder()) {
    pb::NodeProto np;
    np.name = n->name;
    np.op_type = n->op_type;
    np.domain = n->domain;
    np.input = n->inputs;
    np.output = n->outputs;
    for (auto& kv : n->attrs) np.attribute.push_back(kv.second);
    for (auto& kv : n->subgraphs) {
      pb::AttributeProto a;
      a.name = kv.first;
      a.type = pb::ATTR_GRAPH;
      a.g = std::make_shared<pb::GraphProto>(kv.second->ToProto());
      np.attribute.push_back(std::move(a));
    }
    g.node.push_back(std::move(np));
  }
  for (auto& kv : initializers_) {
    if (pending_external_.count(kv.first) && kv.second.numel() == 0) continue;
    if (four_bit_values_.count(kv.first)) {
      pb::TensorProto p;
      p.name = kv.first;
      p.data_type = four_bit_values_.at(kv.first);
      p.dims = kv.second.sizes().vec();
      at::Tensor v = at::bitwise_and(kv.second.to(at::kCPU, at::kInt).reshape({-1}), 15);
      if (v.numel() % 2) v = at::cat({v, at::zeros({1}, v.options())});
      v = v.reshape({-1, 2});
      at::Tensor packed = at::bitwise_or(v.select(1, 0), at::bitwise_left_shift(v.select(1, 1), 4)).to(at::kByte).contiguous();
      p.set_raw(std::string(static_cast<const char*>(packed.data_ptr()), static_cast<size_t>(packed.numel())));
      g.initializer.push_back(std::move(p));
      continue;
    }
    if (string_values_.count(kv.first)) {
      pb::TensorProto p;
      p.name = kv.first;
      p.data_type = pb::STRING;
      p.dims = kv.second.sizes().vec();
      p.string_data = StringsOfTensor(kv.second);
      g.initializer.push_back(std::move(p));
      continue;
    }
    g.initializer.push_back(TensorToProto(kv.second, kv.first));
  }
  for (auto& v : inputs_) {
    pb::ValueInfoProto p;
    p.name = v.name;
    p.type = v.type;
    g.input.push_back(std::move(p));
  }
  for (auto& v : outputs_) {
    pb::ValueInfoProto p;
    p.name = v.name;
    p.type = v.type;
    g.output.push_back(std::move(p));
  }
  for (auto& kv : value_info_) {
    pb::ValueInfoProto p;
    p.name = kv.second.name;
    p.type = kv.second.type;
    g.value_info.push_back(std::move(p));
  }
  return g;
}

Node* Graph::AddNode(const std::string& op_type, const std::vector<std::string>& inputs,
                     const std::vector<std::string>& outputs, const std::string& domain, const std::string& name) {
  auto n = std::make_unique<Node>();
  n->id = static_cast<int>(nodes_.size());
  n->op_type = op_type;
  n->domain = domain;
  n->inputs = inputs;
  n->outputs = outputs;
  n->name = name.empty() ? MakeString(op_type, "_", n->id) : name;
  n->since_version = static_cast<int>(Opset(domain));
  Node* raw = n.get();
  nodes_.push_back(std::move(n));
  dirty_ = true;
  return raw;
}

void Graph::RemoveNode(Node* n) {
  if (!n) return;
  ORTB_ENFORCE(n->id >= 0 && n->id < static_cast<int>(nodes_.size()) && nodes_[n->id].get() == n, "foreign node");
  // Tombstone: a pass may still hold this pointer in a snapshot of the node list, so the object stays alive (with an
  // operator type nothing matches) until PurgeRemoved() runs between passes.
  n->removed = true;
  n->op_type = "<removed>";
  n->inputs.clear();
  n->outputs.clear();
  graveyard_.push_back(std::move(nodes_[n->id]));
  dirty_ = true;
}

void Graph::PurgeRemoved() { graveyard_.clear(); }

std::vector<Node*> Graph::Nodes() const {
  std::vector<Node*> out;
  out.reserve(nodes_.size());
  for (auto& n : nodes_)
    if (n) out.push_back(n.get());
  return out;
}

size_t Graph::NumNodes() const {
  size_t c = 0;
  for (auto& n : nodes_)
    if (n) ++c;
  return c;
}

std::vector<std::string> Graph::ImplicitInputs(const Node& n) const {
  std::vector<std::string> out;
  std::set<std::string> seen;
  std::function<void(const Graph&)> visit = [&](const Graph& sg) {
    std::set<std::string> local;
    for (auto& v : sg.inputs_) local.insert(v.name);
    for (auto& kv : sg.initializers_) local.insert(kv.first);
    for (Node* m : sg.Nodes())
      for (auto& o : m->outputs)
        if (!o.empty()) local.insert(o);
    auto use = [&](const std::string& v) {
      if (v.empty() || local.count(v)) return;
      if (seen.insert(v).second) out.push_back(v);
    };
    for (Node* m : sg.Nodes()) {
      for (auto& i : m->inputs) use(i);
      if (!m->subgraphs.empty()) {
        // values the nested bodies need that are not defined in `sg`
        for (auto& v : sg.ImplicitInputs(*m)) use(v);
      }
    }
    for (auto& o : sg.outputs_) use(o.name);
  };
  for (auto& kv : n.subgraphs) visit(*kv.second);
  return out;
}

void Graph::RebuildIndex() const {
  producer_.clear();
  consumers_.clear();
  for (auto& n : nodes_) {
    if (!n) continue;
    for (auto& o : n->outputs)
      if (!o.empty()) producer_[o] = n.get();
    for (auto& i : n->inputs)
      if (!i.empty()) consumers_[i].push_back(n.get());
    if (!n->subgraphs.empty())
      for (auto& v : ImplicitInputs(*n)) consumers_[v].push_back(n.get());
  }
  dirty_ = false;
}

Node* Graph::Producer(const std::string& value) const {
  if (dirty_) RebuildIndex();
  auto it = producer_.find(value);
  return it == producer_.end() ? nullptr : it->second;
}

std::vector<Node*> Graph::Consumers(const std::string& value) const {
  if (dirty_) RebuildIndex();
  auto it = consumers_.find(value);
  return it == consumers_.end() ? std::vector<Node*>{} : it->second;
}

size_t Graph::NumConsumers(const std::string& value) const {
  size_t c = Consumers(value).size();
  if (IsGraphOutput(value)) ++c;
  return c;
}

std::vector<Node*> Graph::TopologicalOrder() const {
  if (dirty_) RebuildIndex();
  std::vector<Node*> live = Nodes();
  std::unordered_map<Node*, int> indeg;
  std::unordered_map<Node*, std::vector<Node*>> succ;
  for (Node* n : live) {
    indeg[n];
    std::set<Node*> preds;
    auto add_dep = [&](const std::string& v) {
      if (v.empty()) return;
      auto it = producer_.find(v);
      if (it != producer_.end() && it->second != n) preds.insert(it->second);
    };
    for (auto& i : n->inputs) add_dep(i);
    if (!n->subgraphs.empty())
      for (auto& v : ImplicitInputs(*n)) add_dep(v);
    for (Node* p : preds) {
      succ[p].push_back(n);
      indeg[n]++;
    }
  }
  // stable: ready nodes are emitted in original (id) order
  std::set<std::pair<int, Node*>> ready;
  for (Node* n : live)
    if (indeg[n] == 0) ready.insert({n->id, n});
  std::vector<Node*> order;
  order.reserve(live.size());
  while (!ready.empty()) {
    auto it = ready.begin();
    Node* n = it->second;
    ready.erase(it);
    order.push_back(n);
    for (Node* s : succ[n])
      if (--indeg[s] == 0) ready.insert({s->id, s});
  }
  if (order.size() != live.size()) ORTB_THROW(INVALID_GRAPH, "graph '", name_, "' contains a cycle");
  return order;
}

void Graph::SortNodes() {
  std::vector<Node*> order = TopologicalOrder();
  std::vector<std::unique_ptr<Node>> sorted;
  sorted.reserve(order.size());
  for (Node* n : order) {
    sorted.push_back(std::move(nodes_[n->id]));
  }
  nodes_ = std::move(sorted);
  for (size_t i = 0; i < nodes_.size(); ++i) nodes_[i]->id = static_cast<int>(i);
  dirty_ = true;
}

bool Graph::IsConstant(const std::string& name) const {
  if (!IsInitializer(name)) return false;
  if (pending_external_.count(name)) return true;
  // IR >= 4 allows initializers that are not graph inputs; those that are inputs can be overridden
  return !IsGraphInput(name);
}

const at::Tensor* Graph::GetInitializer(const std::string& name) const {
  auto it = initializers_.find(name);
  return it == initializers_.end() ? nullptr : &it->second;
}

const at::Tensor* Graph::GetConstant(const std::string& name) const {
  if (name.empty() || !IsConstant(name) || pending_external_.count(name) || string_values_.count(name)) return nullptr;
  return GetInitializer(name);
}

void Graph::AddInitializer(const std::string& name, const at::Tensor& t) {
  initializers_[name] = t;
  dirty_ = true;
}

void Graph::RemoveInitializer(const std::string& name) {
  initializers_.erase(name);
  pending_external_.erase(name);
  value_info_.erase(name);
  dirty_ = true;
}

bool Graph::IsGraphInput(const std::string& name) const {
  for (auto& v : inputs_)
    if (v.name == name) return true;
  return false;
}

bool Graph::IsGraphOutput(const std::string& name) const {
  for (auto& v : outputs_)
    if (v.name == name) return true;
  return false;
}

std::vector<const ValueInfo*> Graph::RuntimeInputs() const {
  std::vector<const ValueInfo*> out;
  for (auto& v : inputs_)
    if (!IsInitializer(v.name)) out.push_back(&v);
  return out;
}

void Graph::ReplaceAllUses(const std::string& old_name, const std::string& new_name) {
  for (auto& n : nodes_) {
    if (!n) continue;
    for (auto& i : n->inputs)
      if (i == old_name) i = new_name;
    for (auto& kv : n->subgraphs) kv.second->ReplaceAllUses(old_name, new_name);
  }
  for (auto& o : outputs_)
    if (o.name == old_name) o.name = new_name;
  dirty_ = true;
}

std::string Graph::UniqueName(const std::string& prefix) {
  if (dirty_) RebuildIndex();
  while (true) {
    std::string cand = MakeString(prefix, "_ortb", next_unique_++);
    if (!producer_.count(cand) && !initializers_.count(cand) && !IsGraphInput(cand) && !consumers_.count(cand)) return cand;
  }
}

bool Graph::IsOuterScopeValue(const std::string& name) const {
  for (const Graph* g = parent_; g; g = g->parent_) {
    if (g->IsInitializer(name) || g->IsGraphInput(name) || g->Producer(name)) return true;
  }
  return false;
}

int64_t Graph::Opset(const std::string& domain) const {
  auto it = opsets_.find(domain == "ai.onnx" ? "" : domain);
  if (it != opsets_.end()) return it->second;
  if (domain == kMSDomain) return 1;
  if (domain.empty()) return 17;
  return 1;
}

int Graph::RemoveDeadNodes() {
  int removed = 0;
  bool changed = true;
  while (changed) {
    changed = false;
    if (dirty_) RebuildIndex();
    for (auto& n : nodes_) {
      if (!n) continue;
      bool used = false;
      for (auto& o : n->outputs) {
        if (o.empty()) continue;
        if (IsGraphOutput(o) || consumers_.count(o)) {
          used = true;
          break;
        }
      }
      if (!used) {
        RemoveNode(n.get());
        ++removed;
        changed = true;
        dirty_ = true;
        break;
      }
    }
  }
  if (dirty_) RebuildIndex();
  std::vector<std::string> dead_inits;
  for (auto& kv : initializers_)
    if (!consumers_.count(kv.first) && !IsGraphOutput(kv.first)) dead_inits.push_back(kv.first);
  for (auto& n : dead_inits) {
    // keep initializers that subgraphs may read through outer scope: consumers_ already covers them
    RemoveInitializer(n);
  }
  return removed;
}

// ------------------------------------------------------------------ Model
namespace {

// Expand calls to model-local functions (FunctionProto) into plain nodes.
void InlineFunctions(pb::ModelProto& m) {
  if (m.functions.empty()) return;
  std::map<std::pair<std::string, std::string>, const pb::FunctionProto*> table;
  for (auto& f : m.functions) table[{f.domain, f.name}] = &f;
  int counter = 0;
  std::function<void(pb::GraphProto&, int)> expand = [&](pb::GraphProto& g, int depth) {
    ORTB_ENFORCE(depth < 32, "function inlining recursion too deep");
    bool again = true;
    while (again) {
      again = false;
      std::vector<pb::NodeProto> out_nodes;
      for (auto& n : g.node) {
        auto it = table.find({n.domain, n.op_type});
        if (it == table.end()) {
          for (auto& a : n.attribute)
            if (a.g) expand(*a.g, depth + 1);
          out_nodes.push_back(n);
          continue;
        }
        again = true;
        const pb::FunctionProto& f = *it->second;
        const std::string prefix = MakeString("_inl", counter++, "_", n.name, "_");
        std::map<std::string, std::string> rename;
        for (size_t i = 0; i < f.input.size(); ++i) rename[f.input[i]] = i < n.input.size() ? n.input[i] : "";
        for (size_t i = 0; i < f.output.size(); ++i) rename[f.output[i]] = i < n.output.size() ? n.output[i] : "";
        std::map<std::string, const pb::AttributeProto*> call_attrs;
        for (auto& a : n.attribute) call_attrs[a.name] = &a;
        for (auto fn : f.node) {
          for (auto& v : fn.input) {
            if (v.empty()) continue;
            auto r = rename.find(v);
            v = r != rename.end() ? r->second : prefix + v;
          }
          for (auto& v : fn.output) {
            if (v.empty()) continue;
            auto r = rename.find(v);
            if (r != rename.end() && !r->second.empty()) v = r->second;
            else v = prefix + v;
          }
          fn.name = prefix + fn.name;
          std::vector<pb::AttributeProto> attrs;
          for (auto& a : fn.attribute) {
            if (!a.ref_attr_name.empty()) {
              auto c = call_attrs.find(a.ref_attr_name);
              const pb::AttributeProto* src = c != call_attrs.end() ? c->second : nullptr;
              if (!src)
                for (auto& d : f.attribute_proto)
                  if (d.name == a.ref_attr_name) src = &d;
              if (!src) continue;  // optional attribute not provided
              pb::AttributeProto copy = *src;
              copy.name = a.name;
              copy.ref_attr_name.clear();
              attrs.push_back(std::move(copy));
            } else {
              attrs.push_back(a);
            }
          }
          fn.attribute = std::move(attrs);
          out_nodes.push_back(std::move(fn));
        }
      }
      g.node = std::move(out_nodes);
    }
  };
  expand(m.graph, 0);
}

std::shared_ptr<Model> BuildModel(pb::ModelProto& mp, const std::string& model_dir) {
  if (!mp.has_graph) ORTB_THROW(INVALID_PROTOBUF, "ModelProto has no graph (not an ONNX model?)");
  InlineFunctions(mp);
  auto m = std::make_shared<Model>();
  m->ir_version = mp.ir_version;
  m->producer_name = mp.producer_name;
  m->producer_version = mp.producer_version;
  m->domain = mp.domain;
  m->doc_string = mp.doc_string;
  m->model_version = mp.model_version;
  m->graph_name = mp.graph.name;
  m->model_dir = model_dir;
  for (auto& e : mp.metadata_props) m->metadata[e.key] = e.value;
  std::map<std::string, int64_t> opsets;
  for (auto& o : mp.opset_import) {
    const std::string d = o.domain == "ai.onnx" ? "" : o.domain;
    auto it = opsets.find(d);
    if (it == opsets.end() || it->second < o.version) opsets[d] = o.version;
  }
  m->graph_ = Graph::FromProto(mp.graph, opsets, model_dir);
  m->graph_->TopologicalOrder();  // validates acyclicity
  return m;
}

}  // namespace

std::shared_ptr<Model> Model::Load(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) ORTB_THROW(NO_SUCHFILE, "Load model from ", path, " failed: file doesn't exist");
  auto bytes = std::make_shared<std::string>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  std::string dir = ".";
  auto slash = path.find_last_of('/');
  if (slash != std::string::npos) dir = path.substr(0, slash);
  return LoadFromBytes(bytes, dir);
}

std::shared_ptr<Model> Model::LoadFromBytes(std::shared_ptr<const std::string> bytes, const std::string& model_dir) {
  pb::ModelProto mp;
  pb::ParseModel(bytes, &mp);
  return BuildModel(mp, model_dir);
}

std::string Model::Serialize() const {
  pb::ModelProto mp;
  mp.ir_version = ir_version;
  mp.producer_name = producer_name;
  mp.producer_version = producer_version;
  mp.domain = domain;
  mp.doc_string = doc_string;
  mp.model_version = model_version;
  mp.has_graph = true;
  mp.graph = graph_->ToProto();
  if (mp.graph.name.empty()) mp.graph.name = graph_name;
  for (auto& kv : graph_->Opsets()) mp.opset_import.push_back({kv.first, kv.second});
  for (auto& kv : metadata) mp.metadata_props.push_back({kv.first, kv.second});
  return pb::SerializeModel(mp);
}

void Model::Save(const std::string& path) const {
  std::ofstream f(path, std::ios::binary);
  if (!f) ORTB_THROW(FAIL, "cannot open ", path, " for writing");
  const std::string bytes = Serialize();
  f.write(bytes.data(), static_cast<std::streamsize>(bytes.size()));
}

}  // namespace ortb
