// Hand-written protobuf wire-format reader and writer for the ONNX schema
// (ModelProto and everything it contains).  There is no protoc-generated code
// and no dependency on libprotobuf: messages are plain structs.
//
// Field numbers follow onnx.proto (cross-checked against the schema embedded
// in the reference at js/web/lib/onnxjs/ort-schema/protobuf/onnx.js:
// ModelProto :2030, GraphProto :3017, TensorProto :3579, NodeProto :1306,
// AttributeProto :264).  Unknown fields are skipped, truncated or malformed
// input raises INVALID_PROTOBUF.
//
// Large tensors are not copied while parsing: TensorProto::raw points into the
// source buffer, which the ModelProto keeps alive.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace ortb {
namespace pb {

enum DataType : int32_t {
  UNDEFINED = 0, FLOAT = 1, UINT8 = 2, INT8 = 3, UINT16 = 4, INT16 = 5, INT32 = 6, INT64 = 7, STRING = 8, BOOL = 9,
  FLOAT16 = 10, DOUBLE = 11, UINT32 = 12, UINT64 = 13, COMPLEX64 = 14, COMPLEX128 = 15, BFLOAT16 = 16,
  FLOAT8E4M3FN = 17, FLOAT8E4M3FNUZ = 18, FLOAT8E5M2 = 19, FLOAT8E5M2FNUZ = 20, UINT4 = 21, INT4 = 22, FLOAT4E2M1 = 23,
};

enum AttrType : int32_t {
  ATTR_UNDEFINED = 0, ATTR_FLOAT = 1, ATTR_INT = 2, ATTR_STRING = 3, ATTR_TENSOR = 4, ATTR_GRAPH = 5, ATTR_FLOATS = 6,
  ATTR_INTS = 7, ATTR_STRINGS = 8, ATTR_TENSORS = 9, ATTR_GRAPHS = 10, ATTR_SPARSE_TENSOR = 11, ATTR_TYPE_PROTO = 13,
};

struct StringStringEntry {
  std::string key, value;
};

struct OperatorSetId {
  std::string domain;
  int64_t version = 0;
};

struct TensorProto {
  std::vector<int64_t> dims;
  int32_t data_type = 0;
  std::string name;
  std::string doc_string;
  // raw_data: a view (into the parsed buffer) or owned bytes
  const char* raw = nullptr;
  size_t raw_size = 0;
  std::string raw_owned;
  bool has_raw = false;
  std::vector<float> float_data;
  std::vector<int32_t> int32_data;
  std::vector<int64_t> int64_data;
  std::vector<double> double_data;
  std::vector<uint64_t> uint64_data;
  std::vector<std::string> string_data;
  std::vector<StringStringEntry> external_data;
  int32_t data_location = 0;  // 0 DEFAULT, 1 EXTERNAL

  void set_raw(std::string bytes) {
    raw_owned = std::move(bytes);
    raw = raw_owned.data();
    raw_size = raw_owned.size();
    has_raw = true;
  }
  TensorProto() = default;
  TensorProto(const TensorProto& o) { *this = o; }
  TensorProto& operator=(const TensorProto& o);
  TensorProto(TensorProto&& o) noexcept { *this = std::move(o); }
  TensorProto& operator=(TensorProto&& o) noexcept;
};

struct Dimension {
  bool has_value = false;
  int64_t value = 0;
  std::string param;      // symbolic name when !has_value (may be empty = unknown)
  std::string denotation;
};

struct TypeProto {
  // which: 0 = not set, 1 = tensor, 4 = sequence, 5 = map, 8 = sparse tensor, 9 = optional
  int which = 0;
  int32_t elem_type = 0;
  bool has_shape = false;
  std::vector<Dimension> dims;
  std::shared_ptr<TypeProto> elem;  // sequence / optional element, map value
  int32_t map_key_type = 0;
  std::string denotation;
};

struct ValueInfoProto {
  std::string name;
  TypeProto type;
  std::string doc_string;
};

struct GraphProto;

// COO sparse tensor: `indices` are linear positions [nnz] or coordinates [nnz, rank] into a tensor of shape `dims`
struct SparseTensorProto {
  TensorProto values, indices;
  std::vector<int64_t> dims;
};

struct AttributeProto {
  std::string name;
  int32_t type = 0;
  float f = 0.f;
  int64_t i = 0;
  std::string s;
  std::shared_ptr<TensorProto> t;
  std::shared_ptr<SparseTensorProto> sparse_tensor;
  std::shared_ptr<GraphProto> g;
  std::vector<float> floats;
  std::vector<int64_t> ints;
  std::vector<std::string> strings;
  std::vector<TensorProto> tensors;
  std::vector<std::shared_ptr<GraphProto>> graphs;
  std::string ref_attr_name;
  std::string doc_string;
  std::shared_ptr<TypeProto> tp;
};

struct NodeProto {
  std::vector<std::string> input, output;
  std::string name, op_type, domain, doc_string, overload;
  std::vector<AttributeProto> attribute;
  std::vector<StringStringEntry> metadata_props;
};

struct GraphProto {
  std::vector<NodeProto> node;
  std::string name, doc_string;
  std::vector<TensorProto> initializer;
  std::vector<SparseTensorProto> sparse_initializer;  // read only: the loader expands them into dense initializers
  std::vector<ValueInfoProto> input, output, value_info;
};

struct FunctionProto {
  std::string name, domain, doc_string, overload;
  std::vector<std::string> input, output, attribute;
  std::vector<AttributeProto> attribute_proto;
  std::vector<NodeProto> node;
  std::vector<OperatorSetId> opset_import;
};

struct ModelProto {
  int64_t ir_version = 0;
  std::string producer_name, producer_version, domain, doc_string;
  int64_t model_version = 0;
  GraphProto graph;
  bool has_graph = false;
  std::vector<OperatorSetId> opset_import;
  std::vector<StringStringEntry> metadata_props;
  std::vector<FunctionProto> functions;
  // keeps the parsed bytes alive for TensorProto::raw views
  std::shared_ptr<const std::string> backing;
};

// Parse; throws OrtError(INVALID_PROTOBUF) on malformed input.
void ParseModel(std::shared_ptr<const std::string> bytes, ModelProto* out);
void ParseModel(const char* data, size_t size, ModelProto* out);  // copies nothing; caller keeps data alive
void ParseTensor(const char* data, size_t size, TensorProto* out);
void ParseGraph(const char* data, size_t size, GraphProto* out);

std::string SerializeModel(const ModelProto& m);
std::string SerializeTensor(const TensorProto& t);
std::string SerializeGraph(const GraphProto& g);

size_t ElementSize(int32_t data_type);  // bytes per element; 0 for string / sub-byte types
const char* DataTypeName(int32_t data_type);  // "float", "float16", ...

}  // namespace pb
}  // namespace ortb
