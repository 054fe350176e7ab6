#include "onnx_pb.h"

#include <cstring>

#include "common.h"

namespace ortb {
namespace pb {

TensorProto& TensorProto::operator=(const TensorProto& o) {
  if (this == &o) return *this;
  dims = o.dims; data_type = o.data_type; name = o.name; doc_string = o.doc_string;
  raw_owned = o.raw_owned; has_raw = o.has_raw; raw_size = o.raw_size;
  raw = (o.raw == o.raw_owned.data() && !o.raw_owned.empty()) ? raw_owned.data() : o.raw;
  float_data = o.float_data; int32_data = o.int32_data; int64_data = o.int64_data; double_data = o.double_data;
  uint64_data = o.uint64_data; string_data = o.string_data; external_data = o.external_data;
  data_location = o.data_location;
  return *this;
}

TensorProto& TensorProto::operator=(TensorProto&& o) noexcept {
  if (this == &o) return *this;
  const bool owned = (o.raw == o.raw_owned.data() && !o.raw_owned.empty());
  dims = std::move(o.dims); data_type = o.data_type; name = std::move(o.name); doc_string = std::move(o.doc_string);
  raw_owned = std::move(o.raw_owned); has_raw = o.has_raw; raw_size = o.raw_size;
  raw = owned ? raw_owned.data() : o.raw;
  float_data = std::move(o.float_data); int32_data = std::move(o.int32_data); int64_data = std::move(o.int64_data);
  double_data = std::move(o.double_data); uint64_data = std::move(o.uint64_data);
  string_data = std::move(o.string_data); external_data = std::move(o.external_data);
  data_location = o.data_location;
  return *this;
}

namespace {

// ------------------------------------------------------------------ reader
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  int depth;

  Reader(const char* d, size_t n, int depth_ = 0)
      : p(reinterpret_cast<const uint8_t*>(d)), end(reinterpret_cast<const uint8_t*>(d) + n), depth(depth_) {
    if (depth > 64) ORTB_THROW(INVALID_PROTOBUF, "protobuf nesting too deep");
  }
  bool done() const { return p >= end; }

  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (true) {
      if (p >= end) ORTB_THROW(INVALID_PROTOBUF, "truncated varint");
      const uint8_t b = *p++;
      if (shift < 64) v |= static_cast<uint64_t>(b & 0x7F) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
      if (shift > 70) ORTB_THROW(INVALID_PROTOBUF, "varint too long");
    }
    return v;
  }
  uint32_t fixed32() {
    if (end - p < 4) ORTB_THROW(INVALID_PROTOBUF, "truncated fixed32");
    uint32_t v;
    std::memcpy(&v, p, 4);
    p += 4;
    return v;
  }
  uint64_t fixed64() {
    if (end - p < 8) ORTB_THROW(INVALID_PROTOBUF, "truncated fixed64");
    uint64_t v;
    std::memcpy(&v, p, 8);
    p += 8;
    return v;
  }
  // returns a view of a length-delimited field
  std::pair<const char*, size_t> bytes() {
    const uint64_t n = varint();
    if (n > static_cast<uint64_t>(end - p)) ORTB_THROW(INVALID_PROTOBUF, "length-delimited field overruns buffer");
    const char* s = reinterpret_cast<const char*>(p);
    p += n;
    return {s, static_cast<size_t>(n)};
  }
  std::string str() {
    auto b = bytes();
    return std::string(b.first, b.second);
  }
  bool next(uint32_t* field, uint32_t* wire) {
    if (done()) return false;
    const uint64_t key = varint();
    *field = static_cast<uint32_t>(key >> 3);
    *wire = static_cast<uint32_t>(key & 7);
    if (*field == 0) ORTB_THROW(INVALID_PROTOBUF, "field number 0");
    return true;
  }
  void skip(uint32_t wire) {
    switch (wire) {
      case 0: varint(); break;
      case 1: fixed64(); break;
      case 2: bytes(); break;
      case 5: fixed32(); break;
      default: ORTB_THROW(INVALID_PROTOBUF, "unsupported wire type ", wire);
    }
  }
  void expect(uint32_t wire, uint32_t want, const char* what) {
    if (wire != want) ORTB_THROW(INVALID_PROTOBUF, "wrong wire type for ", what);
  }
};

float as_float(uint32_t v) {
  float f;
  std::memcpy(&f, &v, 4);
  return f;
}
double as_double(uint64_t v) {
  double d;
  std::memcpy(&d, &v, 8);
  return d;
}

template <typename T, typename F>
void read_repeated_varint(Reader& r, uint32_t wire, std::vector<T>* out, F conv) {
  if (wire == 2) {
    auto b = r.bytes();
    Reader sub(b.first, b.second, r.depth + 1);
    while (!sub.done()) out->push_back(conv(sub.varint()));
  } else if (wire == 0) {
    out->push_back(conv(r.varint()));
  } else {
    ORTB_THROW(INVALID_PROTOBUF, "bad wire type for repeated varint");
  }
}

void read_repeated_float(Reader& r, uint32_t wire, std::vector<float>* out) {
  if (wire == 2) {
    auto b = r.bytes();
    if (b.second % 4) ORTB_THROW(INVALID_PROTOBUF, "packed float size");
    const size_t n = b.second / 4, old = out->size();
    out->resize(old + n);
    std::memcpy(out->data() + old, b.first, b.second);
  } else if (wire == 5) {
    out->push_back(as_float(r.fixed32()));
  } else {
    ORTB_THROW(INVALID_PROTOBUF, "bad wire type for repeated float");
  }
}

void read_repeated_double(Reader& r, uint32_t wire, std::vector<double>* out) {
  if (wire == 2) {
    auto b = r.bytes();
    if (b.second % 8) ORTB_THROW(INVALID_PROTOBUF, "packed double size");
    const size_t n = b.second / 8, old = out->size();
    out->resize(old + n);
    std::memcpy(out->data() + old, b.first, b.second);
  } else if (wire == 1) {
    out->push_back(as_double(r.fixed64()));
  } else {
    ORTB_THROW(INVALID_PROTOBUF, "bad wire type for repeated double");
  }
}

void parse_ss(const char* d, size_t n, int depth, StringStringEntry* e) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 2) e->key = r.str();
    else if (f == 2 && w == 2) e->value = r.str();
    else r.skip(w);
  }
}

void parse_opset(const char* d, size_t n, int depth, OperatorSetId* o) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 2) o->domain = r.str();
    else if (f == 2 && w == 0) o->version = static_cast<int64_t>(r.varint());
    else r.skip(w);
  }
}

void parse_tensor(const char* d, size_t n, int depth, TensorProto* t) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    switch (f) {
      case 1: read_repeated_varint(r, w, &t->dims, [](uint64_t v) { return static_cast<int64_t>(v); }); break;
      case 2: r.expect(w, 0, "TensorProto.data_type"); t->data_type = static_cast<int32_t>(r.varint()); break;
      case 4: read_repeated_float(r, w, &t->float_data); break;
      case 5: read_repeated_varint(r, w, &t->int32_data, [](uint64_t v) { return static_cast<int32_t>(v); }); break;
      case 6: r.expect(w, 2, "TensorProto.string_data"); t->string_data.push_back(r.str()); break;
      case 7: read_repeated_varint(r, w, &t->int64_data, [](uint64_t v) { return static_cast<int64_t>(v); }); break;
      case 8: r.expect(w, 2, "TensorProto.name"); t->name = r.str(); break;
      case 9: {
        r.expect(w, 2, "TensorProto.raw_data");
        auto b = r.bytes();
        t->raw = b.first;
        t->raw_size = b.second;
        t->has_raw = true;
        break;
      }
      case 10: read_repeated_double(r, w, &t->double_data); break;
      case 11: read_repeated_varint(r, w, &t->uint64_data, [](uint64_t v) { return v; }); break;
      case 12: r.expect(w, 2, "TensorProto.doc_string"); t->doc_string = r.str(); break;
      case 13: {
        r.expect(w, 2, "TensorProto.external_data");
        auto b = r.bytes();
        StringStringEntry e;
        parse_ss(b.first, b.second, depth + 1, &e);
        t->external_data.push_back(std::move(e));
        break;
      }
      case 14: r.expect(w, 0, "TensorProto.data_location"); t->data_location = static_cast<int32_t>(r.varint()); break;
      default: r.skip(w);
    }
  }
}

void parse_type(const char* d, size_t n, int depth, TypeProto* t);

void parse_shape(const char* d, size_t n, int depth, TypeProto* t) {
  Reader r(d, n, depth);
  uint32_t f, w;
  t->has_shape = true;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 2) {
      auto b = r.bytes();
      Reader dr(b.first, b.second, depth + 1);
      Dimension dim;
      uint32_t df, dw;
      while (dr.next(&df, &dw)) {
        if (df == 1 && dw == 0) { dim.has_value = true; dim.value = static_cast<int64_t>(dr.varint()); }
        else if (df == 2 && dw == 2) dim.param = dr.str();
        else if (df == 3 && dw == 2) dim.denotation = dr.str();
        else dr.skip(dw);
      }
      t->dims.push_back(std::move(dim));
    } else {
      r.skip(w);
    }
  }
}

void parse_type_tensor(const char* d, size_t n, int depth, TypeProto* t) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 0) t->elem_type = static_cast<int32_t>(r.varint());
    else if (f == 2 && w == 2) { auto b = r.bytes(); parse_shape(b.first, b.second, depth + 1, t); }
    else r.skip(w);
  }
}

void parse_type_wrapped(const char* d, size_t n, int depth, TypeProto* t) {
  // Sequence / Optional: field 1 = elem_type (TypeProto)
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 2) {
      auto b = r.bytes();
      t->elem = std::make_shared<TypeProto>();
      parse_type(b.first, b.second, depth + 1, t->elem.get());
    } else {
      r.skip(w);
    }
  }
}

void parse_type_map(const char* d, size_t n, int depth, TypeProto* t) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 0) t->map_key_type = static_cast<int32_t>(r.varint());
    else if (f == 2 && w == 2) {
      auto b = r.bytes();
      t->elem = std::make_shared<TypeProto>();
      parse_type(b.first, b.second, depth + 1, t->elem.get());
    } else r.skip(w);
  }
}

void parse_type(const char* d, size_t n, int depth, TypeProto* t) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (w != 2) { r.skip(w); continue; }
    auto b = r.bytes();
    switch (f) {
      case 1: t->which = 1; parse_type_tensor(b.first, b.second, depth + 1, t); break;
      case 4: t->which = 4; parse_type_wrapped(b.first, b.second, depth + 1, t); break;
      case 5: t->which = 5; parse_type_map(b.first, b.second, depth + 1, t); break;
      case 6: t->denotation = std::string(b.first, b.second); break;
      case 8: t->which = 8; parse_type_tensor(b.first, b.second, depth + 1, t); break;
      case 9: t->which = 9; parse_type_wrapped(b.first, b.second, depth + 1, t); break;
      default: break;
    }
  }
}

void parse_value_info(const char* d, size_t n, int depth, ValueInfoProto* v) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 1 && w == 2) v->name = r.str();
    else if (f == 2 && w == 2) { auto b = r.bytes(); parse_type(b.first, b.second, depth + 1, &v->type); }
    else if (f == 3 && w == 2) v->doc_string = r.str();
    else r.skip(w);
  }
}

void parse_graph(const char* d, size_t n, int depth, GraphProto* g);
void parse_sparse_tensor(const char* d, size_t n, int depth, SparseTensorProto* s);

void parse_attribute(const char* d, size_t n, int depth, AttributeProto* a) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    switch (f) {
      case 1: r.expect(w, 2, "AttributeProto.name"); a->name = r.str(); break;
      case 2: r.expect(w, 5, "AttributeProto.f"); a->f = as_float(r.fixed32()); break;
      case 3: r.expect(w, 0, "AttributeProto.i"); a->i = static_cast<int64_t>(r.varint()); break;
      case 4: r.expect(w, 2, "AttributeProto.s"); a->s = r.str(); break;
      case 5: {
        r.expect(w, 2, "AttributeProto.t");
        auto b = r.bytes();
        a->t = std::make_shared<TensorProto>();
        parse_tensor(b.first, b.second, depth + 1, a->t.get());
        break;
      }
      case 6: {
        r.expect(w, 2, "AttributeProto.g");
        auto b = r.bytes();
        a->g = std::make_shared<GraphProto>();
        parse_graph(b.first, b.second, depth + 1, a->g.get());
        break;
      }
      case 7: read_repeated_float(r, w, &a->floats); break;
      case 8: read_repeated_varint(r, w, &a->ints, [](uint64_t v) { return static_cast<int64_t>(v); }); break;
      case 9: r.expect(w, 2, "AttributeProto.strings"); a->strings.push_back(r.str()); break;
      case 10: {
        r.expect(w, 2, "AttributeProto.tensors");
        auto b = r.bytes();
        a->tensors.emplace_back();
        parse_tensor(b.first, b.second, depth + 1, &a->tensors.back());
        break;
      }
      case 11: {
        r.expect(w, 2, "AttributeProto.graphs");
        auto b = r.bytes();
        a->graphs.push_back(std::make_shared<GraphProto>());
        parse_graph(b.first, b.second, depth + 1, a->graphs.back().get());
        break;
      }
      case 22: {
        r.expect(w, 2, "AttributeProto.sparse_tensor");
        auto b = r.bytes();
        a->sparse_tensor = std::make_shared<SparseTensorProto>();
        parse_sparse_tensor(b.first, b.second, depth + 1, a->sparse_tensor.get());
        break;
      }
      case 13: r.expect(w, 2, "AttributeProto.doc_string"); a->doc_string = r.str(); break;
      case 14: {
        r.expect(w, 2, "AttributeProto.tp");
        auto b = r.bytes();
        a->tp = std::make_shared<TypeProto>();
        parse_type(b.first, b.second, depth + 1, a->tp.get());
        break;
      }
      case 20: r.expect(w, 0, "AttributeProto.type"); a->type = static_cast<int32_t>(r.varint()); break;
      case 21: r.expect(w, 2, "AttributeProto.ref_attr_name"); a->ref_attr_name = r.str(); break;
      default: r.skip(w);
    }
  }
  if (a->type == 0) {
    // proto2-era writers may omit `type`; infer it
    if (a->t) a->type = ATTR_TENSOR;
    else if (a->g) a->type = ATTR_GRAPH;
    else if (!a->floats.empty()) a->type = ATTR_FLOATS;
    else if (!a->ints.empty()) a->type = ATTR_INTS;
    else if (!a->strings.empty()) a->type = ATTR_STRINGS;
    else if (!a->tensors.empty()) a->type = ATTR_TENSORS;
    else if (!a->graphs.empty()) a->type = ATTR_GRAPHS;
    else if (!a->s.empty()) a->type = ATTR_STRING;
  }
}

void parse_node(const char* d, size_t n, int depth, NodeProto* node) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (w != 2) { r.skip(w); continue; }
    switch (f) {
      case 1: node->input.push_back(r.str()); break;
      case 2: node->output.push_back(r.str()); break;
      case 3: node->name = r.str(); break;
      case 4: node->op_type = r.str(); break;
      case 5: {
        auto b = r.bytes();
        node->attribute.emplace_back();
        parse_attribute(b.first, b.second, depth + 1, &node->attribute.back());
        break;
      }
      case 6: node->doc_string = r.str(); break;
      case 7: node->domain = r.str(); break;
      case 8: node->overload = r.str(); break;
      case 9: {
        auto b = r.bytes();
        StringStringEntry e;
        parse_ss(b.first, b.second, depth + 1, &e);
        node->metadata_props.push_back(std::move(e));
        break;
      }
      default: r.bytes();
    }
  }
}

void parse_sparse_tensor(const char* d, size_t n, int depth, SparseTensorProto* s) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (f == 3) {
      read_repeated_varint(r, w, &s->dims, [](uint64_t v) { return static_cast<int64_t>(v); });
    } else if ((f == 1 || f == 2) && w == 2) {
      auto b = r.bytes();
      parse_tensor(b.first, b.second, depth + 1, f == 1 ? &s->values : &s->indices);
    } else {
      r.skip(w);
    }
  }
}

void parse_graph(const char* d, size_t n, int depth, GraphProto* g) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (w != 2) { r.skip(w); continue; }
    auto b = r.bytes();
    switch (f) {
      case 1: g->node.emplace_back(); parse_node(b.first, b.second, depth + 1, &g->node.back()); break;
      case 2: g->name = std::string(b.first, b.second); break;
      case 5: g->initializer.emplace_back(); parse_tensor(b.first, b.second, depth + 1, &g->initializer.back()); break;
      case 10: g->doc_string = std::string(b.first, b.second); break;
      case 11: g->input.emplace_back(); parse_value_info(b.first, b.second, depth + 1, &g->input.back()); break;
      case 12: g->output.emplace_back(); parse_value_info(b.first, b.second, depth + 1, &g->output.back()); break;
      case 13: g->value_info.emplace_back(); parse_value_info(b.first, b.second, depth + 1, &g->value_info.back()); break;
      case 15: g->sparse_initializer.emplace_back(); parse_sparse_tensor(b.first, b.second, depth + 1, &g->sparse_initializer.back()); break;
      default: break;
    }
  }
}

void parse_function(const char* d, size_t n, int depth, FunctionProto* fn) {
  Reader r(d, n, depth);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    if (w != 2) { r.skip(w); continue; }
    auto b = r.bytes();
    switch (f) {
      case 1: fn->name = std::string(b.first, b.second); break;
      case 4: fn->input.emplace_back(b.first, b.second); break;
      case 5: fn->output.emplace_back(b.first, b.second); break;
      case 6: fn->attribute.emplace_back(b.first, b.second); break;
      case 7: fn->node.emplace_back(); parse_node(b.first, b.second, depth + 1, &fn->node.back()); break;
      case 8: fn->doc_string = std::string(b.first, b.second); break;
      case 9: fn->opset_import.emplace_back(); parse_opset(b.first, b.second, depth + 1, &fn->opset_import.back()); break;
      case 10: fn->domain = std::string(b.first, b.second); break;
      case 11: fn->attribute_proto.emplace_back(); parse_attribute(b.first, b.second, depth + 1, &fn->attribute_proto.back()); break;
      case 13: fn->overload = std::string(b.first, b.second); break;
      default: break;
    }
  }
}

// ------------------------------------------------------------------ writer
struct Writer {
  std::string out;
  void varint(uint64_t v) {
    while (v >= 0x80) {
      out.push_back(static_cast<char>((v & 0x7F) | 0x80));
      v >>= 7;
    }
    out.push_back(static_cast<char>(v));
  }
  void key(uint32_t field, uint32_t wire) { varint((static_cast<uint64_t>(field) << 3) | wire); }
  void f_varint(uint32_t field, uint64_t v) { key(field, 0); varint(v); }
  void f_int64(uint32_t field, int64_t v) { f_varint(field, static_cast<uint64_t>(v)); }
  void f_bytes(uint32_t field, const char* d, size_t n) { key(field, 2); varint(n); out.append(d, n); }
  void f_str(uint32_t field, const std::string& s) { f_bytes(field, s.data(), s.size()); }
  void f_str_opt(uint32_t field, const std::string& s) { if (!s.empty()) f_str(field, s); }
  void f_float(uint32_t field, float v) { key(field, 5); out.append(reinterpret_cast<const char*>(&v), 4); }
  void f_msg(uint32_t field, const std::string& sub) { f_str(field, sub); }
  template <typename T>
  void f_packed_varint(uint32_t field, const std::vector<T>& v) {
    if (v.empty()) return;
    Writer sub;
    for (auto x : v) sub.varint(static_cast<uint64_t>(static_cast<int64_t>(x)));
    f_msg(field, sub.out);
  }
  void f_packed_float(uint32_t field, const std::vector<float>& v) {
    if (v.empty()) return;
    f_bytes(field, reinterpret_cast<const char*>(v.data()), v.size() * 4);
  }
  void f_packed_double(uint32_t field, const std::vector<double>& v) {
    if (v.empty()) return;
    f_bytes(field, reinterpret_cast<const char*>(v.data()), v.size() * 8);
  }
};

std::string ser_ss(const StringStringEntry& e) {
  Writer w;
  w.f_str(1, e.key);
  w.f_str(2, e.value);
  return std::move(w.out);
}

std::string ser_opset(const OperatorSetId& o) {
  Writer w;
  w.f_str_opt(1, o.domain);
  w.f_int64(2, o.version);
  return std::move(w.out);
}

std::string ser_tensor(const TensorProto& t) {
  Writer w;
  w.f_packed_varint(1, t.dims);
  if (t.data_type) w.f_varint(2, static_cast<uint64_t>(t.data_type));
  w.f_packed_float(4, t.float_data);
  w.f_packed_varint(5, t.int32_data);
  for (auto& s : t.string_data) w.f_str(6, s);
  w.f_packed_varint(7, t.int64_data);
  w.f_str_opt(8, t.name);
  if (t.has_raw) w.f_bytes(9, t.raw, t.raw_size);
  w.f_packed_double(10, t.double_data);
  w.f_packed_varint(11, t.uint64_data);
  w.f_str_opt(12, t.doc_string);
  for (auto& e : t.external_data) w.f_msg(13, ser_ss(e));
  if (t.data_location) w.f_varint(14, static_cast<uint64_t>(t.data_location));
  return std::move(w.out);
}

std::string ser_type(const TypeProto& t);

std::string ser_type_tensor(const TypeProto& t) {
  Writer w;
  if (t.elem_type) w.f_varint(1, static_cast<uint64_t>(t.elem_type));
  if (t.has_shape) {
    Writer sh;
    for (auto& d : t.dims) {
      Writer dw;
      if (d.has_value) dw.f_int64(1, d.value);
      else if (!d.param.empty()) dw.f_str(2, d.param);
      dw.f_str_opt(3, d.denotation);
      sh.f_msg(1, dw.out);
    }
    w.f_msg(2, sh.out);
  }
  return std::move(w.out);
}

std::string ser_type(const TypeProto& t) {
  Writer w;
  switch (t.which) {
    case 1: w.f_msg(1, ser_type_tensor(t)); break;
    case 8: w.f_msg(8, ser_type_tensor(t)); break;
    case 4:
    case 9: {
      Writer sub;
      if (t.elem) sub.f_msg(1, ser_type(*t.elem));
      w.f_msg(static_cast<uint32_t>(t.which), sub.out);
      break;
    }
    case 5: {
      Writer sub;
      sub.f_varint(1, static_cast<uint64_t>(t.map_key_type));
      if (t.elem) sub.f_msg(2, ser_type(*t.elem));
      w.f_msg(5, sub.out);
      break;
    }
    default: break;
  }
  w.f_str_opt(6, t.denotation);
  return std::move(w.out);
}

std::string ser_value_info(const ValueInfoProto& v) {
  Writer w;
  w.f_str(1, v.name);
  if (v.type.which) w.f_msg(2, ser_type(v.type));
  w.f_str_opt(3, v.doc_string);
  return std::move(w.out);
}

std::string ser_graph(const GraphProto& g);

std::string ser_attribute(const AttributeProto& a) {
  Writer w;
  w.f_str(1, a.name);
  switch (a.type) {
    case ATTR_FLOAT: w.f_float(2, a.f); break;
    case ATTR_INT: w.f_int64(3, a.i); break;
    case ATTR_STRING: w.f_str(4, a.s); break;
    case ATTR_TENSOR: if (a.t) w.f_msg(5, ser_tensor(*a.t)); break;
    case ATTR_GRAPH: if (a.g) w.f_msg(6, ser_graph(*a.g)); break;
    case ATTR_FLOATS: w.f_packed_float(7, a.floats); break;
    case ATTR_INTS: w.f_packed_varint(8, a.ints); break;
    case ATTR_STRINGS: for (auto& s : a.strings) w.f_str(9, s); break;
    case ATTR_TENSORS: for (auto& t : a.tensors) w.f_msg(10, ser_tensor(t)); break;
    case ATTR_GRAPHS: for (auto& g : a.graphs) if (g) w.f_msg(11, ser_graph(*g)); break;
    case ATTR_TYPE_PROTO: if (a.tp) w.f_msg(14, ser_type(*a.tp)); break;
    default: break;
  }
  w.f_str_opt(13, a.doc_string);
  w.f_varint(20, static_cast<uint64_t>(a.type));
  w.f_str_opt(21, a.ref_attr_name);
  return std::move(w.out);
}

std::string ser_node(const NodeProto& n) {
  Writer w;
  for (auto& s : n.input) w.f_str(1, s);
  for (auto& s : n.output) w.f_str(2, s);
  w.f_str_opt(3, n.name);
  w.f_str(4, n.op_type);
  for (auto& a : n.attribute) w.f_msg(5, ser_attribute(a));
  w.f_str_opt(6, n.doc_string);
  w.f_str_opt(7, n.domain);
  w.f_str_opt(8, n.overload);
  for (auto& e : n.metadata_props) w.f_msg(9, ser_ss(e));
  return std::move(w.out);
}

std::string ser_graph(const GraphProto& g) {
  Writer w;
  for (auto& n : g.node) w.f_msg(1, ser_node(n));
  w.f_str_opt(2, g.name);
  for (auto& t : g.initializer) w.f_msg(5, ser_tensor(t));
  w.f_str_opt(10, g.doc_string);
  for (auto& v : g.input) w.f_msg(11, ser_value_info(v));
  for (auto& v : g.output) w.f_msg(12, ser_value_info(v));
  for (auto& v : g.value_info) w.f_msg(13, ser_value_info(v));
  return std::move(w.out);
}

std::string ser_function(const FunctionProto& fn) {
  Writer w;
  w.f_str(1, fn.name);
  for (auto& s : fn.input) w.f_str(4, s);
  for (auto& s : fn.output) w.f_str(5, s);
  for (auto& s : fn.attribute) w.f_str(6, s);
  for (auto& n : fn.node) w.f_msg(7, ser_node(n));
  w.f_str_opt(8, fn.doc_string);
  for (auto& o : fn.opset_import) w.f_msg(9, ser_opset(o));
  w.f_str_opt(10, fn.domain);
  for (auto& a : fn.attribute_proto) w.f_msg(11, ser_attribute(a));
  w.f_str_opt(13, fn.overload);
  return std::move(w.out);
}

}  // namespace

void ParseModel(const char* data, size_t size, ModelProto* m) {
  Reader r(data, size);
  uint32_t f, w;
  while (r.next(&f, &w)) {
    switch (f) {
      case 1: r.expect(w, 0, "ModelProto.ir_version"); m->ir_version = static_cast<int64_t>(r.varint()); break;
      case 2: r.expect(w, 2, "producer_name"); m->producer_name = r.str(); break;
      case 3: r.expect(w, 2, "producer_version"); m->producer_version = r.str(); break;
      case 4: r.expect(w, 2, "domain"); m->domain = r.str(); break;
      case 5: r.expect(w, 0, "model_version"); m->model_version = static_cast<int64_t>(r.varint()); break;
      case 6: r.expect(w, 2, "doc_string"); m->doc_string = r.str(); break;
      case 7: {
        r.expect(w, 2, "graph");
        auto b = r.bytes();
        parse_graph(b.first, b.second, 1, &m->graph);
        m->has_graph = true;
        break;
      }
      case 8: {
        r.expect(w, 2, "opset_import");
        auto b = r.bytes();
        m->opset_import.emplace_back();
        parse_opset(b.first, b.second, 1, &m->opset_import.back());
        break;
      }
      case 14: {
        r.expect(w, 2, "metadata_props");
        auto b = r.bytes();
        m->metadata_props.emplace_back();
        parse_ss(b.first, b.second, 1, &m->metadata_props.back());
        break;
      }
      case 25: {
        r.expect(w, 2, "functions");
        auto b = r.bytes();
        m->functions.emplace_back();
        parse_function(b.first, b.second, 1, &m->functions.back());
        break;
      }
      default: r.skip(w);
    }
  }
}

void ParseModel(std::shared_ptr<const std::string> bytes, ModelProto* out) {
  out->backing = bytes;
  ParseModel(bytes->data(), bytes->size(), out);
}

void ParseTensor(const char* data, size_t size, TensorProto* out) { parse_tensor(data, size, 0, out); }
void ParseGraph(const char* data, size_t size, GraphProto* out) { parse_graph(data, size, 0, out); }

std::string SerializeModel(const ModelProto& m) {
  Writer w;
  if (m.ir_version) w.f_int64(1, m.ir_version);
  w.f_str_opt(2, m.producer_name);
  w.f_str_opt(3, m.producer_version);
  w.f_str_opt(4, m.domain);
  if (m.model_version) w.f_int64(5, m.model_version);
  w.f_str_opt(6, m.doc_string);
  if (m.has_graph) w.f_msg(7, ser_graph(m.graph));
  for (auto& o : m.opset_import) w.f_msg(8, ser_opset(o));
  for (auto& e : m.metadata_props) w.f_msg(14, ser_ss(e));
  for (auto& f : m.functions) w.f_msg(25, ser_function(f));
  return std::move(w.out);
}

std::string SerializeTensor(const TensorProto& t) { return ser_tensor(t); }
std::string SerializeGraph(const GraphProto& g) { return ser_graph(g); }

size_t ElementSize(int32_t dt) {
  switch (dt) {
    case FLOAT: case INT32: case UINT32: return 4;
    case UINT8: case INT8: case BOOL: case FLOAT8E4M3FN: case FLOAT8E4M3FNUZ: case FLOAT8E5M2: case FLOAT8E5M2FNUZ: return 1;
    case UINT16: case INT16: case FLOAT16: case BFLOAT16: return 2;
    case INT64: case UINT64: case DOUBLE: case COMPLEX64: return 8;
    case COMPLEX128: return 16;
    default: return 0;
  }
}

const char* DataTypeName(int32_t dt) {
  switch (dt) {
    case FLOAT: return "float";
    case UINT8: return "uint8";
    case INT8: return "int8";
    case UINT16: return "uint16";
    case INT16: return "int16";
    case INT32: return "int32";
    case INT64: return "int64";
    case STRING: return "string";
    case BOOL: return "bool";
    case FLOAT16: return "float16";
    case DOUBLE: return "double";
    case UINT32: return "uint32";
    case UINT64: return "uint64";
    case COMPLEX64: return "complex64";
    case COMPLEX128: return "complex128";
    case BFLOAT16: return "bfloat16";
    case FLOAT8E4M3FN: return "float8e4m3fn";
    case FLOAT8E4M3FNUZ: return "float8e4m3fnuz";
    case FLOAT8E5M2: return "float8e5m2";
    case FLOAT8E5M2FNUZ: return "float8e5m2fnuz";
    case UINT4: return "uint4";
    case INT4: return "int4";
    case FLOAT4E2M1: return "float4e2m1";
    default: return "undefined";
  }
}

}  // namespace pb
}  // namespace ortb
