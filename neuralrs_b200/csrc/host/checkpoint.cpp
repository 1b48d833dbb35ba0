// The reference's checkpoint formats (src/serialize.rs) in host C++: positional text (:81-136) and
// safetensors (:197-238; the layout is the published one of the `safetensors` crate the reference links,
// 0.8.0: u64 header length, JSON header in name order padded with spaces to 8 bytes, raw little-endian data).
// No GPU code here: the trainer-level entry points in trainer.cu move the bytes to and from the device.
#include "checkpoint.h"

#include <algorithm>
#include <charconv>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>

#include "../nrs_internal.h"
#include "graph.h"
#include "nrs_checkpoint.h"

namespace nrs {
namespace checkpoint {
namespace {

[[noreturn]] void fail(int code, const std::string& m) { throw Error(code, m); }

bool ends_with(const std::string& s, const char* suffix) {
  const size_t n = std::strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

// Writes `bytes` to "<path>.tmp" and renames it over `path` (src/serialize.rs:92-101, :214-216).
void atomic_write(const std::string& path, const std::string& bytes) {
  const std::string tmp = path + ".tmp";
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) fail(NRS_ERR_ARG, "save: cannot create " + tmp);
    f.write(bytes.data(), (std::streamsize)bytes.size());
    f.flush();
    if (!f) fail(NRS_ERR_ARG, "save: write to " + tmp + " failed");
  }
  if (std::rename(tmp.c_str(), path.c_str()) != 0) fail(NRS_ERR_ARG, "save: rename to " + path + " failed");
}

std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) fail(NRS_ERR_ARG, "load: cannot open " + path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

size_t numel(const std::vector<int64_t>& shape) {
  size_t n = 1;
  for (int64_t d : shape) {
    if (d < 0) fail(NRS_ERR_SHAPE, "save: negative extent");
    n *= (size_t)d;
  }
  return n;
}

// ------------------------------------------------------------------ text

std::string text_bytes(const std::vector<Tensor>& tensors) {
  std::string out = "tensors " + std::to_string(tensors.size()) + "\n";
  for (const Tensor& t : tensors) {
    out += "len " + std::to_string(t.data.size()) + "\n";
    for (float v : t.data) {
      out += format_f32(v);
      out += '\n';
    }
  }
  return out;
}

float parse_f32(const std::string& line, const char* what) {
  // Rust's f32::from_str: decimal or exponent form, "inf"/"infinity"/"nan" in any case, optional sign.
  const char* s = line.c_str();
  char* end = nullptr;
  const float v = std::strtof(s, &end);
  if (end == s || *end != '\0' || line.empty() || std::isspace((unsigned char)line[0])) fail(NRS_ERR_ARG, std::string(what) + ": malformed value `" + line + "`");
  return v;
}

size_t header_count(const std::string& line, const char* what) {
  std::istringstream ss(line);
  std::string word;
  long long n = -1;
  if (!(ss >> word >> n) || n < 0) fail(NRS_ERR_ARG, std::string("load_tensors: malformed ") + what);
  return (size_t)n;
}

std::vector<Tensor> load_text(const std::string& path) {
  std::ifstream f(path);
  if (!f) fail(NRS_ERR_ARG, "load_tensors: cannot open " + path);
  std::string line;
  if (!std::getline(f, line)) fail(NRS_ERR_ARG, "load_tensors: missing header");
  const size_t n = header_count(line, "header");
  std::vector<Tensor> out;
  for (size_t i = 0; i < n; ++i) {
    if (!std::getline(f, line)) fail(NRS_ERR_ARG, "load_tensors: file ends before all tensors were read");
    const size_t len = header_count(line, "tensor header");
    Tensor t;
    t.name = "tensor_" + std::to_string(i);
    t.shape = {(int64_t)len};
    t.data.reserve(len);
    for (size_t k = 0; k < len; ++k) {
      if (!std::getline(f, line)) fail(NRS_ERR_ARG, "load_tensors: file ends mid-tensor");
      if (!line.empty() && line.back() == '\r') line.pop_back();
      t.data.push_back(parse_f32(line, "load_tensors"));
    }
    out.push_back(std::move(t));
  }
  return out;
}

// ----------------------------------------------------------- safetensors

std::string json_string(const std::string& s) {
  std::string o = "\"";
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      case '\b': o += "\\b"; break;
      case '\f': o += "\\f"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof buf, "\\u%04x", c);
          o += buf;
        } else {
          o += (char)c;
        }
    }
  }
  return o + "\"";
}

std::string safetensors_bytes(const std::vector<Tensor>& tensors) {
  std::vector<const Tensor*> order;
  for (const Tensor& t : tensors) {
    if (numel(t.shape) != t.data.size()) fail(NRS_ERR_SHAPE, "save: tensor shape does not match its data length (" + t.name + ")");
    order.push_back(&t);
  }
  // the crate orders by (dtype alignment descending, name); every tensor here is F32
  std::stable_sort(order.begin(), order.end(), [](const Tensor* a, const Tensor* b) { return a->name < b->name; });
  for (size_t i = 1; i < order.size(); ++i)
    if (order[i]->name == order[i - 1]->name) fail(NRS_ERR_ARG, "save: duplicate tensor name " + order[i]->name);
  std::string header = "{";
  size_t offset = 0;
  for (size_t i = 0; i < order.size(); ++i) {
    const Tensor& t = *order[i];
    if (i) header += ',';
    header += json_string(t.name) + ":{\"dtype\":\"F32\",\"shape\":[";
    for (size_t d = 0; d < t.shape.size(); ++d) header += (d ? "," : "") + std::to_string(t.shape[d]);
    const size_t bytes = t.data.size() * 4;
    header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + bytes) + "]}";
    offset += bytes;
  }
  header += "}";
  while (header.size() % 8 != 0) header += ' ';
  std::string out;
  out.reserve(8 + header.size() + offset);
  const uint64_t n = header.size();
  for (int b = 0; b < 8; ++b) out += (char)((n >> (8 * b)) & 0xff);
  out += header;
  for (const Tensor* t : order) {
    static_assert(sizeof(float) == 4, "f32");
    // little-endian hosts only (x86-64 / aarch64-le): the in-memory bytes are the file bytes
    out.append(reinterpret_cast<const char*>(t->data.data()), t->data.size() * 4);
  }
  return out;
}

// A recursive-descent reader for the header: objects, arrays, strings, integers, true/false/null.
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const char* key) const {
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JsonReader {
  const std::string& s;
  size_t i = 0;
  int depth = 0;
  explicit JsonReader(const std::string& src) : s(src) {}
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  [[noreturn]] void bad(const char* what) { fail(NRS_ERR_ARG, std::string("load: not a valid safetensors file (header: ") + what + ")"); }
  char peek() { ws(); if (i >= s.size()) bad("truncated"); return s[i]; }
  void expect(char c) { if (peek() != c) bad("unexpected character"); ++i; }
  std::string string() {
    expect('"');
    std::string o;
    while (true) {
      if (i >= s.size()) bad("unterminated string");
      char c = s[i++];
      if (c == '"') break;
      if (c != '\\') { o += c; continue; }
      if (i >= s.size()) bad("unterminated escape");
      c = s[i++];
      switch (c) {
        case '"': o += '"'; break;
        case '\\': o += '\\'; break;
        case '/': o += '/'; break;
        case 'n': o += '\n'; break;
        case 'r': o += '\r'; break;
        case 't': o += '\t'; break;
        case 'b': o += '\b'; break;
        case 'f': o += '\f'; break;
        case 'u': {
          if (i + 4 > s.size()) bad("short \\u escape");
          unsigned cp = 0;
          for (int k = 0; k < 4; ++k) {
            const char h = s[i++];
            cp = cp * 16 + (unsigned)(h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 99);
            if (cp > 0xffff * 16u) bad("bad \\u escape");
          }
          // basic multilingual plane only (surrogate pairs are kept as two 3-byte sequences)
          if (cp < 0x80) o += (char)cp;
          else if (cp < 0x800) { o += (char)(0xc0 | (cp >> 6)); o += (char)(0x80 | (cp & 0x3f)); }
          else { o += (char)(0xe0 | (cp >> 12)); o += (char)(0x80 | ((cp >> 6) & 0x3f)); o += (char)(0x80 | (cp & 0x3f)); }
          break;
        }
        default: bad("unknown escape");
      }
    }
    return o;
  }
  Json value() {
    if (++depth > 32) bad("nesting too deep");
    Json j;
    const char c = peek();
    if (c == '{') {
      j.kind = Json::Obj;
      ++i;
      if (peek() == '}') { ++i; --depth; return j; }
      while (true) {
        std::string k = string();
        expect(':');
        j.obj.emplace_back(std::move(k), value());
        if (peek() == ',') { ++i; continue; }
        expect('}');
        break;
      }
    } else if (c == '[') {
      j.kind = Json::Arr;
      ++i;
      if (peek() == ']') { ++i; --depth; return j; }
      while (true) {
        j.arr.push_back(value());
        if (peek() == ',') { ++i; continue; }
        expect(']');
        break;
      }
    } else if (c == '"') {
      j.kind = Json::Str;
      j.str = string();
    } else if (s.compare(i, 4, "true") == 0) { j.kind = Json::Bool; j.num = 1; i += 4; }
    else if (s.compare(i, 5, "false") == 0) { j.kind = Json::Bool; i += 5; }
    else if (s.compare(i, 4, "null") == 0) { i += 4; }
    else {
      const size_t b = i;
      while (i < s.size() && (std::isdigit((unsigned char)s[i]) || s[i] == '-' || s[i] == '+' || s[i] == '.' || s[i] == 'e' || s[i] == 'E')) ++i;
      if (b == i) bad("unexpected token");
      j.kind = Json::Num;
      j.num = std::strtod(s.substr(b, i - b).c_str(), nullptr);
    }
    --depth;
    return j;
  }
};

std::vector<Tensor> load_safetensors(const std::string& path) {
  const std::string buf = read_file(path);
  if (buf.size() < 8) fail(NRS_ERR_ARG, "load: not a valid safetensors file (shorter than its length field)");
  uint64_t n = 0;
  for (int b = 0; b < 8; ++b) n |= (uint64_t)(unsigned char)buf[b] << (8 * b);
  if (n > buf.size() - 8 || n > (100u << 20)) fail(NRS_ERR_ARG, "load: not a valid safetensors file (header length)");
  const std::string header = buf.substr(8, (size_t)n);
  JsonReader rd(header);
  const Json root = rd.value();
  rd.ws();
  if (root.kind != Json::Obj || rd.i != header.size()) fail(NRS_ERR_ARG, "load: not a valid safetensors file (header is not one object)");
  const size_t data_len = buf.size() - 8 - (size_t)n;
  const char* data = buf.data() + 8 + n;
  std::vector<Tensor> out;
  for (auto& kv : root.obj) {
    if (kv.first == "__metadata__") continue;
    const Json& info = kv.second;
    const Json *dt = info.get("dtype"), *sh = info.get("shape"), *off = info.get("data_offsets");
    if (info.kind != Json::Obj || !dt || !sh || !off || dt->kind != Json::Str || sh->kind != Json::Arr ||
        off->kind != Json::Arr || off->arr.size() != 2)
      fail(NRS_ERR_ARG, "load: not a valid safetensors file (tensor `" + kv.first + "`)");
    if (dt->str != "F32") fail(NRS_ERR_ARG, "load: only F32 tensors are supported (tensor `" + kv.first + "`)");
    Tensor t;
    t.name = kv.first;
    size_t count = 1;
    for (const Json& d : sh->arr) {
      if (d.kind != Json::Num || d.num < 0 || d.num != std::floor(d.num)) fail(NRS_ERR_ARG, "load: bad shape (tensor `" + kv.first + "`)");
      t.shape.push_back((int64_t)d.num);
      count *= (size_t)d.num;
    }
    const double b0 = off->arr[0].num, b1 = off->arr[1].num;
    if (off->arr[0].kind != Json::Num || off->arr[1].kind != Json::Num || b0 < 0 || b1 < b0 || b1 > (double)data_len ||
        (size_t)(b1 - b0) != count * 4)
      fail(NRS_ERR_ARG, "load: data offsets do not match the shape (tensor `" + kv.first + "`)");
    t.data.resize(count);
    if (count) std::memcpy(t.data.data(), data + (size_t)b0, count * 4);
    out.push_back(std::move(t));
  }
  std::sort(out.begin(), out.end(), [](const Tensor& a, const Tensor& b) { return a.name < b.name; });   // :235
  return out;
}

}  // namespace

std::string format_f32(float v) {
  if (std::isnan(v)) return "NaN";
  if (std::isinf(v)) return v < 0 ? "-inf" : "inf";
  // Rust's Display: the shortest digit string that reads back to the same f32, laid out positionally
  // (zeros fill up to the decimal point: 6.400897e9 prints as 6400897000, not as its exact integer value).
  char buf[64];
  const auto r = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::scientific);   // [-]d[.ddd]e[+-]XX, shortest
  std::string sci(buf, r.ptr);
  std::string out;
  size_t i = 0;
  if (sci[0] == '-') { out = "-"; i = 1; }
  const size_t e = sci.find('e');
  std::string digits;
  for (size_t k = i; k < e; ++k)
    if (sci[k] != '.') digits += sci[k];
  const int exp10 = std::atoi(sci.c_str() + e + 1);   // value = d.ddd * 10^exp10
  const int point = exp10 + 1;                        // digits before the decimal point
  if (digits == "0") return out + "0";
  if (point <= 0) {
    out += "0.";
    out.append((size_t)(-point), '0');
    out += digits;
  } else if ((size_t)point >= digits.size()) {
    out += digits;
    out.append((size_t)point - digits.size(), '0');
  } else {
    out += digits.substr(0, (size_t)point) + "." + digits.substr((size_t)point);
  }
  return out;
}

void save(const std::vector<Tensor>& tensors, const std::string& path) {
  atomic_write(path, ends_with(path, ".safetensors") ? safetensors_bytes(tensors) : text_bytes(tensors));
}

std::vector<Tensor> load(const std::string& path) {
  return ends_with(path, ".safetensors") ? load_safetensors(path) : load_text(path);
}

}  // namespace checkpoint
}  // namespace nrs

// ------------------------------------------------------------------ C ABI

struct nrs_checkpoint {
  std::vector<nrs::checkpoint::Tensor> tensors;
};

namespace {
template <class F>
int guarded_io(F&& f) {
  try {
    f();
    return NRS_OK;
  } catch (const nrs::Error& e) {
    return nrs_fail(nullptr, e.code, "%s", e.what());
  } catch (const std::exception& e) {
    return nrs_fail(nullptr, NRS_ERR_ARG, "%s", e.what());
  }
}
bool index_ok(const nrs_checkpoint* ck, int i) { return ck && i >= 0 && i < (int)ck->tensors.size(); }
}  // namespace

extern "C" {

int nrs_save(const nrs_named_tensor* tensors, int count, const char* path) {
  if (count < 0 || (count > 0 && !tensors) || !path) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_save: bad arguments");
  return guarded_io([&] {
    std::vector<nrs::checkpoint::Tensor> v;
    for (int i = 0; i < count; ++i) {
      const nrs_named_tensor& s = tensors[i];
      if (!s.name || s.ndim < 0 || (s.ndim > 0 && !s.shape)) throw nrs::Error(NRS_ERR_ARG, "nrs_save: tensor without a name or shape");
      nrs::checkpoint::Tensor t;
      t.name = s.name;
      t.shape.assign(s.shape, s.shape + s.ndim);
      size_t n = 1;
      for (int64_t d : t.shape) {
        if (d < 0) throw nrs::Error(NRS_ERR_SHAPE, "nrs_save: negative extent");
        n *= (size_t)d;
      }
      if (n && !s.data) throw nrs::Error(NRS_ERR_ARG, "nrs_save: tensor without data");
      t.data.assign(s.data, s.data + n);
      v.push_back(std::move(t));
    }
    nrs::checkpoint::save(v, path);
  });
}

int nrs_load(const char* path, nrs_checkpoint** out) {
  if (!path || !out) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_load: bad arguments");
  *out = nullptr;
  return guarded_io([&] {
    auto* ck = new nrs_checkpoint();
    try {
      ck->tensors = nrs::checkpoint::load(path);
    } catch (...) {
      delete ck;
      throw;
    }
    *out = ck;
  });
}

int nrs_checkpoint_count(const nrs_checkpoint* ck) { return ck ? (int)ck->tensors.size() : -1; }
const char* nrs_checkpoint_name(const nrs_checkpoint* ck, int i) { return index_ok(ck, i) ? ck->tensors[i].name.c_str() : nullptr; }
int nrs_checkpoint_ndim(const nrs_checkpoint* ck, int i) { return index_ok(ck, i) ? (int)ck->tensors[i].shape.size() : -1; }
int64_t nrs_checkpoint_dim(const nrs_checkpoint* ck, int i, int d) {
  return index_ok(ck, i) && d >= 0 && d < (int)ck->tensors[i].shape.size() ? ck->tensors[i].shape[d] : -1;
}
int64_t nrs_checkpoint_len(const nrs_checkpoint* ck, int i) { return index_ok(ck, i) ? (int64_t)ck->tensors[i].data.size() : -1; }
const float* nrs_checkpoint_data(const nrs_checkpoint* ck, int i) { return index_ok(ck, i) ? ck->tensors[i].data.data() : nullptr; }
int nrs_checkpoint_find(const nrs_checkpoint* ck, const char* name) {
  if (!ck || !name) return -1;
  for (size_t i = 0; i < ck->tensors.size(); ++i)
    if (ck->tensors[i].name == name) return (int)i;
  return -1;
}
void nrs_checkpoint_free(nrs_checkpoint* ck) { delete ck; }

}  // extern "C"
