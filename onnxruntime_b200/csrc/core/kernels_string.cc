// Operators on tensors of strings: StringNormalizer, StringConcat, StringSplit, RegexFullMatch, casts between strings
// and numbers, ai.onnx.ml CategoryMapper, contrib Tokenizer.  A string tensor is an int64 tensor of ids of the string
// table (string_table.h); these kernels look the strings up, work on them on the host and intern their results.
// Reference kernels: onnxruntime/core/providers/cpu/nn/string_normalizer.cc, cpu/text/string_concat.cc,
// string_split.cc, regex_full_match.cc, cpu/tensor/cast_op.cc (string branches), cpu/ml/category_mapper.cc,
// contrib_ops/cpu/tokenizer.cc.
#include <ATen/ATen.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <regex>
#include <set>

#include "kernel.h"
#include "string_table.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

void RequireStrings(const Ctx& ctx, int i) {
  ORTB_ENFORCE(ctx.InputIsString(i), ctx.node().op_type, ": input ", i, " must be a tensor of strings");
}

// ASCII case mapping; bytes of multi-byte UTF-8 sequences are left alone
std::string ChangeCase(std::string s, bool upper) {
  for (auto& c : s) {
    const unsigned char u = static_cast<unsigned char>(c);
    if (u < 0x80) c = static_cast<char>(upper ? std::toupper(u) : std::tolower(u));
  }
  return s;
}

// code points of a UTF-8 string as byte ranges [begin, end)
std::vector<std::pair<size_t, size_t>> Utf8Chars(const std::string& s) {
  std::vector<std::pair<size_t, size_t>> out;
  for (size_t i = 0; i < s.size();) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    size_t len = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1;
    len = std::min(len, s.size() - i);
    out.emplace_back(i, i + len);
    i += len;
  }
  return out;
}

void StringNormalizerImpl(Ctx& ctx) {
  RequireStrings(ctx, 0);
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  ORTB_ENFORCE_ARG(x.dim() == 1 || (x.dim() == 2 && x.size(0) == 1), "StringNormalizer: input must be [C] or [1, C]");
  const std::string action = n.attr_s("case_change_action", "NONE");
  const bool case_sensitive = n.attr_i("is_case_sensitive", 0) != 0;
  std::set<std::string> stop;
  for (auto& w : n.attr_strings("stopwords")) stop.insert(case_sensitive ? w : ChangeCase(w, false));
  std::vector<std::string> out;
  for (auto& s : StringsOfTensor(x)) {
    if (stop.count(case_sensitive ? s : ChangeCase(s, false))) continue;
    out.push_back(action == "LOWER" ? ChangeCase(s, false) : (action == "UPPER" ? ChangeCase(s, true) : s));
  }
  if (out.empty()) out.push_back("");  // everything filtered: one empty string
  const int64_t C = static_cast<int64_t>(out.size());
  ctx.SetOutputStrings(0, InternStrings(out, x.dim() == 1 ? std::vector<int64_t>{C} : std::vector<int64_t>{1, C}));
}

void StringConcatImpl(Ctx& ctx) {
  RequireStrings(ctx, 0);
  RequireStrings(ctx, 1);
  std::vector<at::Tensor> both = at::broadcast_tensors({ctx.RequiredInput(0).cpu(), ctx.RequiredInput(1).cpu()});
  std::vector<std::string> a = StringsOfTensor(both[0]), b = StringsOfTensor(both[1]);
  for (size_t i = 0; i < a.size(); ++i) a[i] += b[i];
  ctx.SetOutputStrings(0, InternStrings(a, both[0].sizes()));
}

// whitespace split (no delimiter): runs of blanks separate, leading / trailing blanks ignored; with a delimiter: every
// occurrence separates (empty pieces are kept).  maxsplit bounds the number of splits.
std::vector<std::string> SplitOne(const std::string& s, const std::string& delim, int64_t maxsplit) {
  std::vector<std::string> out;
  int64_t splits = 0;
  if (delim.empty()) {
    size_t i = 0;
    while (i < s.size()) {
      while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
      if (i >= s.size()) break;
      if (maxsplit >= 0 && splits == maxsplit) {
        out.push_back(s.substr(i));
        return out;
      }
      size_t j = i;
      while (j < s.size() && !std::isspace(static_cast<unsigned char>(s[j]))) ++j;
      out.push_back(s.substr(i, j - i));
      ++splits;
      i = j;
    }
    return out;
  }
  size_t pos = 0;
  while (true) {
    const size_t hit = (maxsplit >= 0 && splits == maxsplit) ? std::string::npos : s.find(delim, pos);
    if (hit == std::string::npos) {
      out.push_back(s.substr(pos));
      return out;
    }
    out.push_back(s.substr(pos, hit - pos));
    pos = hit + delim.size();
    ++splits;
  }
}

void StringSplitImpl(Ctx& ctx) {
  RequireStrings(ctx, 0);
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  const std::string delim = n.attr_s("delimiter", "");
  const int64_t maxsplit = n.has_attr("maxsplit") ? n.attr_i("maxsplit", -1) : -1;
  std::vector<std::vector<std::string>> pieces;
  size_t widest = 0;
  for (auto& s : StringsOfTensor(x)) {
    pieces.push_back(SplitOne(s, delim, maxsplit));
    widest = std::max(widest, pieces.back().size());
  }
  std::vector<std::string> flat;
  at::Tensor counts = at::empty(x.sizes(), at::kLong);
  for (size_t i = 0; i < pieces.size(); ++i) {
    counts.data_ptr<int64_t>()[i] = static_cast<int64_t>(pieces[i].size());
    for (size_t k = 0; k < widest; ++k) flat.push_back(k < pieces[i].size() ? pieces[i][k] : std::string());
  }
  std::vector<int64_t> shape = x.sizes().vec();
  shape.push_back(static_cast<int64_t>(widest));
  ctx.SetOutputStrings(0, InternStrings(flat, shape));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, counts);
}

void RegexFullMatchImpl(Ctx& ctx) {
  RequireStrings(ctx, 0);
  const at::Tensor& x = ctx.RequiredInput(0);
  std::regex re;
  try {
    re = std::regex(ctx.node().attr_s("pattern", ""), std::regex::ECMAScript);
  } catch (const std::regex_error& e) {
    ORTB_THROW(INVALID_ARGUMENT, "RegexFullMatch: bad pattern: ", e.what());
  }
  at::Tensor y = at::empty(x.sizes(), at::kBool);
  const std::vector<std::string> s = StringsOfTensor(x);
  for (size_t i = 0; i < s.size(); ++i) y.data_ptr<bool>()[i] = std::regex_match(s[i], re);
  ctx.SetOutput(0, y.to(x.device()));
}

// number -> text the way the ONNX Cast operator asks for: integers plainly, floats in their shortest round-trip form
std::string NumberToString(double v, bool integral) {
  char buf[64];
  if (integral) {
    std::snprintf(buf, sizeof(buf), "%lld", static_cast<long long>(v));
    return buf;
  }
  if (std::isnan(v)) return "NaN";
  if (std::isinf(v)) return v > 0 ? "INF" : "-INF";
  for (int prec = 1; prec <= 9; ++prec) {  // float32 sources: 9 significant digits always round-trip
    std::snprintf(buf, sizeof(buf), "%.*g", prec, v);
    if (static_cast<float>(std::strtod(buf, nullptr)) == static_cast<float>(v)) break;
  }
  return buf;
}

void CategoryMapperImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  const std::vector<std::string> names = n.attr_strings("cats_strings");
  const std::vector<int64_t> ints = n.attr_ints("cats_int64s");
  ORTB_ENFORCE_ARG(names.size() == ints.size(), "CategoryMapper: cats_strings and cats_int64s differ in length");
  at::Tensor flat = x.to(at::kCPU, at::kLong).contiguous();
  at::Tensor out = at::empty(x.sizes(), at::kLong);
  const int64_t* src = flat.data_ptr<int64_t>();
  int64_t* dst = out.data_ptr<int64_t>();
  std::map<int64_t, int64_t> table;
  if (ctx.InputIsString(0)) {
    for (size_t i = 0; i < names.size(); ++i) table[InternString(names[i])] = ints[i];
    const int64_t dflt = n.attr_i("default_int64", -1);
    for (int64_t i = 0; i < flat.numel(); ++i) {
      auto it = table.find(src[i]);
      dst[i] = it == table.end() ? dflt : it->second;
    }
    ctx.SetOutput(0, out.to(x.device()));
  } else {
    for (size_t i = 0; i < names.size(); ++i) table[ints[i]] = InternString(names[i]);
    const int64_t dflt = InternString(n.attr_s("default_string", "_Unused"));
    for (int64_t i = 0; i < flat.numel(); ++i) {
      auto it = table.find(src[i]);
      dst[i] = it == table.end() ? dflt : it->second;
    }
    ctx.SetOutputStrings(0, out);
  }
}

// contrib Tokenizer: splits every string of X ([C] or [N, C]) into tokens, by separators (regular expressions tried in
// the given order at every position) or by a token expression (every match is a token); tokens shorter than mincharnum
// characters are dropped; with mark = 1 every row starts with \x02 and ends with \x03; rows are padded with pad_value.
void TokenizerImpl(Ctx& ctx) {
  RequireStrings(ctx, 0);
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  ORTB_ENFORCE_ARG(x.dim() == 1 || x.dim() == 2, "Tokenizer: input must be [C] or [N, C]");
  const bool mark = n.attr_i("mark", 0) != 0;
  const int64_t min_chars = std::max<int64_t>(n.attr_i("mincharnum", 1), 1);
  const std::string pad = n.attr_s("pad_value", "");
  const std::vector<std::string> seps = n.attr_strings("separators");
  const std::string token_exp = n.attr_s("tokenexp", "");
  std::vector<std::regex> sep_re;
  std::regex tok_re;
  const bool char_tokens = seps.size() == 1 && seps[0].empty();  // one empty separator: every character is a token
  try {
    for (auto& s : seps)
      if (!s.empty()) sep_re.emplace_back(s, std::regex::ECMAScript);
    if (!token_exp.empty()) tok_re = std::regex(token_exp, std::regex::ECMAScript);
  } catch (const std::regex_error& e) {
    ORTB_THROW(INVALID_ARGUMENT, "Tokenizer: bad regular expression: ", e.what());
  }
  ORTB_ENFORCE_ARG(char_tokens || !sep_re.empty() || !token_exp.empty(), "Tokenizer: needs separators or tokenexp");
  auto tokenize = [&](const std::string& s) {
    std::vector<std::string> toks;
    auto keep = [&](const std::string& t) {
      if (static_cast<int64_t>(Utf8Chars(t).size()) >= min_chars) toks.push_back(t);
    };
    if (char_tokens) {
      for (auto& r : Utf8Chars(s)) keep(s.substr(r.first, r.second - r.first));
    } else if (!token_exp.empty()) {
      for (auto it = std::sregex_iterator(s.begin(), s.end(), tok_re); it != std::sregex_iterator(); ++it)
        if (it->length() > 0) keep(it->str());
    } else {
      size_t start = 0, i = 0;
      while (i < s.size()) {
        size_t len = 0;
        for (auto& re : sep_re) {
          std::smatch m;
          if (std::regex_search(s.begin() + static_cast<std::ptrdiff_t>(i), s.end(), m, re, std::regex_constants::match_continuous) && m.length() > 0) {
            len = static_cast<size_t>(m.length());
            break;
          }
        }
        if (len > 0) {
          if (i > start) keep(s.substr(start, i - start));
          i += len;
          start = i;
        } else {
          ++i;
        }
      }
      if (start < s.size()) keep(s.substr(start));
    }
    return toks;
  };
  std::vector<std::vector<std::string>> rows;
  size_t widest = 0;
  for (auto& s : StringsOfTensor(x)) {
    rows.push_back(tokenize(s));
    widest = std::max(widest, rows.back().size());
  }
  const size_t width = widest + (mark ? 2 : 0);
  std::vector<std::string> flat;
  for (auto& r : rows) {
    size_t written = 0;
    if (mark) flat.emplace_back("\x02"), ++written;
    for (auto& t : r) flat.push_back(t), ++written;
    if (mark) flat.emplace_back("\x03"), ++written;
    for (; written < width; ++written) flat.push_back(pad);
  }
  std::vector<int64_t> shape = x.sizes().vec();
  shape.push_back(static_cast<int64_t>(width));
  ctx.SetOutputStrings(0, InternStrings(flat, shape));
}

}  // namespace

// Cast with a string on either side (called by the Cast kernel); returns false when neither side is a string.
bool CastWithStrings(OpKernelContext& ctx, int32_t to) {
  const bool from_string = ctx.InputIsString(0);
  if (!from_string && to != pb::STRING) return false;
  const at::Tensor& x = ctx.RequiredInput(0);
  if (from_string && to == pb::STRING) {
    ctx.SetOutputStrings(0, x);
    return true;
  }
  if (from_string) {
    const std::vector<std::string> s = StringsOfTensor(x);
    at::Tensor v = at::empty(x.sizes(), at::kDouble);
    for (size_t i = 0; i < s.size(); ++i) {
      char* end = nullptr;
      std::string t = s[i];
      if (t == "INF" || t == "+INF") t = "inf";
      if (t == "-INF") t = "-inf";
      v.data_ptr<double>()[i] = std::strtod(t.c_str(), &end);
      ORTB_ENFORCE_ARG(end != t.c_str() && *end == '\0', "Cast: '", s[i], "' is not a number");
    }
    ctx.SetOutput(0, v.to(ToTorchType(to)).to(x.device()));
    return true;
  }
  const bool integral = !x.is_floating_point();
  at::Tensor v = x.to(at::kCPU, at::kDouble).contiguous();
  std::vector<std::string> out;
  for (int64_t i = 0; i < v.numel(); ++i) out.push_back(NumberToString(v.data_ptr<double>()[i], integral));
  ctx.SetOutputStrings(0, InternStrings(out, x.sizes()));
  return true;
}

void RegisterStringKernels(KernelRegistry& r) {
  r.RegisterFn("", "StringNormalizer", 10, kMax, StringNormalizerImpl);
  r.RegisterFn("", "StringConcat", 20, kMax, StringConcatImpl);
  r.RegisterFn("", "StringSplit", 20, kMax, StringSplitImpl);
  r.RegisterFn("", "RegexFullMatch", 20, kMax, RegexFullMatchImpl);
  r.RegisterFn("ai.onnx.ml", "CategoryMapper", 1, kMax, CategoryMapperImpl);
  r.RegisterFn("com.microsoft", "Tokenizer", 1, kMax, TokenizerImpl);
}

}  // namespace ortb
