// Weight sources: validated safetensors files and sharded-model indexes, imported into a backend
// as read-only buffers, plus lookup of MLX affine-quantised triples by checkpoint name.
//
// Behaviour follows crates/forja-host/src/weights.rs (Safetensors::open :175-226, open_all :114-168,
// parse_tensor :402-465, the size caps :17-25) and the checkpoint naming of the quantised engines
// (engines/qwen3-coder/src/lib.rs:174-188: `<prefix>.weight` u32 [out, in * bits / 32],
// `<prefix>.scales` / `<prefix>.biases` [out, in / group]; :430-437 for stacked experts). Host code
// only: nothing here touches the device except fj_safetensors_import, which hands the mapped data
// region to fj_import_readonly.
#include <errno.h>
#include <fcntl.h>
#include <limits.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "forja_cuda.h"

namespace {

constexpr uint64_t kMaxHeaderBytes = 100ull * 1024 * 1024;  // weights.rs:19
constexpr uint64_t kMaxIndexBytes = 100ull * 1024 * 1024;   // weights.rs:22
constexpr size_t kMaxShards = 1024;                          // weights.rs:25
constexpr int kMaxDepth = 128;                               // serde_json's recursion limit

// ---- a small JSON reader (objects keep insertion order; duplicate keys are kept and reported) ----
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool boolean = false;
  bool is_u64 = false;  // a non-negative integer literal without fraction or exponent that fits 64 bits
  uint64_t u64 = 0;
  std::string text;     // String: decoded text
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;
  const Json* get(const char* key) const {
    const Json* found = nullptr;
    for (auto& m : members)
      if (m.first == key) found = &m.second;  // last one wins, like serde_json's Map::insert
    return found;
  }
};

struct Parser {
  const char* p;
  const char* end;
  std::string error;
  bool fail(const char* what) { if (error.empty()) error = what; return false; }
  void skip() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
  static void utf8(std::string& out, uint32_t c) {
    if (c < 0x80) out += static_cast<char>(c);
    else if (c < 0x800) { out += static_cast<char>(0xC0 | (c >> 6)); out += static_cast<char>(0x80 | (c & 0x3F)); }
    else if (c < 0x10000) { out += static_cast<char>(0xE0 | (c >> 12)); out += static_cast<char>(0x80 | ((c >> 6) & 0x3F)); out += static_cast<char>(0x80 | (c & 0x3F)); }
    else { out += static_cast<char>(0xF0 | (c >> 18)); out += static_cast<char>(0x80 | ((c >> 12) & 0x3F)); out += static_cast<char>(0x80 | ((c >> 6) & 0x3F)); out += static_cast<char>(0x80 | (c & 0x3F)); }
  }
  bool hex4(uint32_t* out) {
    if (end - p < 4) return fail("truncated \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else return fail("invalid \\u escape");
    }
    *out = v;
    return true;
  }
  bool string(std::string* out) {
    if (p >= end || *p != '"') return fail("expected a string");
    ++p;
    out->clear();
    while (true) {
      if (p >= end) return fail("unterminated string");
      unsigned char c = static_cast<unsigned char>(*p++);
      if (c == '"') return true;
      if (c < 0x20) return fail("control character in string");
      if (c != '\\') { *out += static_cast<char>(c); continue; }
      if (p >= end) return fail("unterminated escape");
      char e = *p++;
      switch (e) {
        case '"': *out += '"'; break;
        case '\\': *out += '\\'; break;
        case '/': *out += '/'; break;
        case 'b': *out += '\b'; break;
        case 'f': *out += '\f'; break;
        case 'n': *out += '\n'; break;
        case 'r': *out += '\r'; break;
        case 't': *out += '\t'; break;
        case 'u': {
          uint32_t cp = 0;
          if (!hex4(&cp)) return false;
          if (cp >= 0xD800 && cp <= 0xDBFF) {
            uint32_t lo = 0;
            if (end - p < 2 || p[0] != '\\' || p[1] != 'u') return fail("lone surrogate");
            p += 2;
            if (!hex4(&lo)) return false;
            if (lo < 0xDC00 || lo > 0xDFFF) return fail("lone surrogate");
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
            return fail("lone surrogate");
          }
          utf8(*out, cp);
          break;
        }
        default: return fail("invalid escape");
      }
    }
  }
  bool number(Json* out) {
    const char* start = p;
    bool negative = false, integral = true;
    if (p < end && *p == '-') { negative = true; ++p; }
    if (p >= end || *p < '0' || *p > '9') return fail("invalid number");
    if (*p == '0') { ++p; if (p < end && *p >= '0' && *p <= '9') return fail("leading zero"); }
    else while (p < end && *p >= '0' && *p <= '9') ++p;
    if (p < end && *p == '.') {
      integral = false; ++p;
      if (p >= end || *p < '0' || *p > '9') return fail("invalid fraction");
      while (p < end && *p >= '0' && *p <= '9') ++p;
    }
    if (p < end && (*p == 'e' || *p == 'E')) {
      integral = false; ++p;
      if (p < end && (*p == '+' || *p == '-')) ++p;
      if (p >= end || *p < '0' || *p > '9') return fail("invalid exponent");
      while (p < end && *p >= '0' && *p <= '9') ++p;
    }
    out->kind = Json::Number;
    out->is_u64 = false;
    if (integral && !negative) {
      uint64_t v = 0;
      bool fits = true;
      for (const char* q = start; q < p && fits; ++q) {
        if (__builtin_mul_overflow(v, static_cast<uint64_t>(10), &v) || __builtin_add_overflow(v, static_cast<uint64_t>(*q - '0'), &v)) fits = false;
      }
      out->is_u64 = fits;
      out->u64 = fits ? v : 0;
    }
    return true;
  }
  bool value(Json* out, int depth) {
    skip();
    if (p >= end) return fail("unexpected end of input");
    if (*p == '{' || *p == '[') {
      if (depth >= kMaxDepth) return fail("recursion limit exceeded");
      const bool object = *p == '{';
      ++p;
      out->kind = object ? Json::Object : Json::Array;
      skip();
      if (p < end && *p == (object ? '}' : ']')) { ++p; return true; }
      while (true) {
        if (object) {
          skip();
          std::string key;
          if (!string(&key)) return false;
          skip();
          if (p >= end || *p != ':') return fail("expected ':'");
          ++p;
          out->members.emplace_back(std::move(key), Json());
          if (!value(&out->members.back().second, depth + 1)) return false;
        } else {
          out->items.emplace_back();
          if (!value(&out->items.back(), depth + 1)) return false;
        }
        skip();
        if (p >= end) return fail("unexpected end of input");
        if (*p == ',') { ++p; continue; }
        if (*p == (object ? '}' : ']')) { ++p; return true; }
        return fail("expected ',' or a closing bracket");
      }
    }
    if (*p == '"') { out->kind = Json::String; return string(&out->text); }
    if (end - p >= 4 && !memcmp(p, "true", 4)) { p += 4; out->kind = Json::Bool; out->boolean = true; return true; }
    if (end - p >= 5 && !memcmp(p, "false", 5)) { p += 5; out->kind = Json::Bool; out->boolean = false; return true; }
    if (end - p >= 4 && !memcmp(p, "null", 4)) { p += 4; out->kind = Json::Null; return true; }
    return number(out);
  }
  // A whole document: one value, then only whitespace (the header of a safetensors file is padded with spaces).
  bool document(Json* out) {
    if (!value(out, 0)) return false;
    skip();
    if (p != end) return fail("trailing characters");
    return true;
  }
};

bool duplicate_key(const Json& object, std::string* which) {
  std::set<std::string> seen;
  for (auto& m : object.members)
    if (!seen.insert(m.first).second) { *which = m.first; return true; }
  return false;
}

struct Tensor {
  std::string name;
  uint32_t dtype = 0;
  std::vector<uint32_t> shape;
  uint64_t byte_offset = 0, byte_len = 0;
};

}  // namespace

struct fj_safetensors {
  std::string path, shard_name, error;
  uint64_t file_len = 0, data_start = 0;
  std::vector<Tensor> tensors;  // sorted by byte offset (weights.rs:207)
};

namespace {

thread_local std::string g_last_error;

int32_t fail(int32_t status, const std::string& message) {
  g_last_error = message;
  return status;
}

uint64_t dtype_bytes(uint32_t dt) { return dt == FJ_F16 || dt == FJ_BF16 ? 2 : 4; }

// parse_tensor, weights.rs:402-465
int32_t parse_tensor(const std::string& name, const Json& value, uint64_t data_len, Tensor* out) {
  auto invalid = [&](const char* what) { return fail(FJ_WEIGHTS_INVALID_HEADER, "tensor \"" + name + "\": " + what); };
  if (value.kind != Json::Object) return invalid("entry is not an object");
  const Json* dtype = value.get("dtype");
  if (!dtype || dtype->kind != Json::String) return invalid("dtype is missing");
  if (dtype->text == "F32") out->dtype = FJ_F32;
  else if (dtype->text == "F16") out->dtype = FJ_F16;
  else if (dtype->text == "BF16") out->dtype = FJ_BF16;
  else if (dtype->text == "U32") out->dtype = FJ_U32;
  else return fail(FJ_WEIGHTS_UNSUPPORTED_DTYPE, dtype->text);
  const Json* shape = value.get("shape");
  if (!shape || shape->kind != Json::Array) return invalid("shape is missing");
  for (auto& extent : shape->items) {
    if (extent.kind != Json::Number || !extent.is_u64 || extent.u64 > 0xFFFFFFFFull) return invalid("shape extent is not a u32");
    out->shape.push_back(static_cast<uint32_t>(extent.u64));
  }
  const Json* range = value.get("data_offsets");
  if (!range || range->kind != Json::Array || range->items.size() != 2) return invalid("data_offsets must contain two values");
  for (auto& v : range->items)
    if (v.kind != Json::Number || !v.is_u64) return invalid("data offset is not a u64");
  const uint64_t start = range->items[0].u64, stop = range->items[1].u64;
  if (stop < start) return fail(FJ_WEIGHTS_INVALID_RANGE, "invalid safetensors tensor byte range");
  const uint64_t byte_len = stop - start;
  uint64_t expected = 1;
  for (uint32_t extent : out->shape)
    if (__builtin_mul_overflow(expected, static_cast<uint64_t>(extent), &expected)) return fail(FJ_WEIGHTS_INVALID_RANGE, "invalid safetensors tensor byte range");
  if (__builtin_mul_overflow(expected, dtype_bytes(out->dtype), &expected) || expected != byte_len) return fail(FJ_WEIGHTS_INVALID_RANGE, "invalid safetensors tensor byte range");
  uint64_t byte_end = 0;
  if (__builtin_add_overflow(start, byte_len, &byte_end)) return fail(FJ_WEIGHTS_INVALID_RANGE, "invalid safetensors tensor byte range");
  if (byte_end > data_len) return fail(FJ_WEIGHTS_TRUNCATED, "weight file is truncated");
  out->name = name;
  out->byte_offset = start;
  out->byte_len = byte_len;
  return FJ_OK;
}

bool read_exact(int fd, void* dst, size_t len) {
  char* p = static_cast<char*>(dst);
  while (len) {
    ssize_t n = read(fd, p, len);
    if (n < 0 && errno == EINTR) continue;
    if (n <= 0) return false;
    p += n; len -= static_cast<size_t>(n);
  }
  return true;
}

// Safetensors::open, weights.rs:175-226
int32_t open_one(const char* path, std::unique_ptr<fj_safetensors>* out) {
  struct stat st;
  if (lstat(path, &st) != 0) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  if (!S_ISREG(st.st_mode)) return fail(FJ_WEIGHTS_NOT_REGULAR_FILE, std::string("weight source is not a regular file: ") + path);
  int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  struct Closer { int fd; ~Closer() { close(fd); } } closer{fd};
  if (fstat(fd, &st) != 0) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  const uint64_t file_len = static_cast<uint64_t>(st.st_size);
  unsigned char prefix[8];
  if (!read_exact(fd, prefix, 8)) return fail(FJ_WEIGHTS_TRUNCATED, "weight file is truncated");
  uint64_t header_len = 0;
  for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | prefix[i];
  if (header_len > kMaxHeaderBytes) return fail(FJ_WEIGHTS_HEADER_TOO_LARGE, "safetensors header has " + std::to_string(header_len) + " bytes, exceeding the size cap");
  std::string header(static_cast<size_t>(header_len), '\0');
  if (header_len && !read_exact(fd, &header[0], header.size())) return fail(FJ_WEIGHTS_TRUNCATED, "weight file is truncated");
  const uint64_t data_start = 8 + header_len;
  if (file_len < data_start) return fail(FJ_WEIGHTS_TRUNCATED, "weight file is truncated");
  const uint64_t data_len = file_len - data_start;
  Json root;
  Parser parser{header.data(), header.data() + header.size(), {}};
  if (!parser.document(&root)) return fail(FJ_WEIGHTS_INVALID_HEADER, "invalid safetensors header: " + parser.error);
  if (root.kind != Json::Object) return fail(FJ_WEIGHTS_INVALID_HEADER, "invalid safetensors header: expected a safetensors metadata object");
  std::string dup;
  if (duplicate_key(root, &dup)) return fail(FJ_WEIGHTS_INVALID_HEADER, "invalid safetensors header: duplicate safetensors entry \"" + dup + "\"");
  auto result = std::make_unique<fj_safetensors>();
  for (auto& member : root.members) {
    if (member.first == "__metadata__") continue;
    Tensor t;
    int32_t status = parse_tensor(member.first, member.second, data_len, &t);
    if (status != FJ_OK) return status;
    result->tensors.push_back(std::move(t));
  }
  std::stable_sort(result->tensors.begin(), result->tensors.end(), [](const Tensor& a, const Tensor& b) { return a.byte_offset < b.byte_offset; });
  for (size_t i = 0; i + 1 < result->tensors.size(); ++i) {
    const Tensor& a = result->tensors[i];
    if (a.byte_offset + a.byte_len > result->tensors[i + 1].byte_offset) return fail(FJ_WEIGHTS_OVERLAPPING_RANGES, "safetensors tensor byte ranges overlap");
  }
  result->path = path;
  result->file_len = file_len;
  result->data_start = data_start;
  *out = std::move(result);
  return FJ_OK;
}

// valid_shard_name, weights.rs:271-276
bool valid_shard_name(const std::string& file) {
  if (file.empty() || file.find('/') != std::string::npos || file.find('\\') != std::string::npos) return false;
  if (file == "." || file == "..") return false;
  const std::string suffix = ".safetensors";
  return file.size() >= suffix.size() && file.compare(file.size() - suffix.size(), suffix.size(), suffix) == 0;
}

bool canonical(const std::string& path, std::string* out) {
  char buffer[PATH_MAX];
  if (!realpath(path.c_str(), buffer)) return false;
  *out = buffer;
  return true;
}

bool starts_with_directory(const std::string& path, const std::string& root) {
  if (root == "/") return !path.empty() && path[0] == '/';
  return path.size() > root.size() && path.compare(0, root.size(), root) == 0 && path[root.size()] == '/';
}

}  // namespace

extern "C" {

const char* fj_weights_last_error(void) { return g_last_error.c_str(); }

int32_t fj_safetensors_open(const char* path, fj_safetensors** out) {
  if (!path || !out) return fail(FJ_INVALID_INPUT, "null argument");
  std::unique_ptr<fj_safetensors> source;
  int32_t status = open_one(path, &source);
  if (status != FJ_OK) return status;
  *out = source.release();
  return FJ_OK;
}

// Safetensors::open_all, weights.rs:114-168
int32_t fj_safetensors_open_all(const char* path, fj_safetensors** out, uint32_t cap, uint32_t* count) {
  if (!path || !count || (cap && !out)) return fail(FJ_INVALID_INPUT, "null argument");
  *count = 0;
  const std::string p = path;
  const size_t slash = p.find_last_of('/');
  const std::string file_name = slash == std::string::npos ? p : p.substr(slash + 1);
  const size_t dot = file_name.find_last_of('.');
  const bool is_index = dot != std::string::npos && dot != 0 && file_name.substr(dot + 1) == "json";
  if (!is_index) {
    if (cap < 1) { *count = 1; return fail(FJ_QUOTA_EXCEEDED, "handle array too small"); }
    int32_t status = fj_safetensors_open(path, out);
    if (status == FJ_OK) *count = 1;
    return status;
  }
  // read_index, weights.rs:246-269
  int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno)); }
  if (static_cast<uint64_t>(st.st_size) > kMaxIndexBytes) { close(fd); return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: index has " + std::to_string(st.st_size) + " bytes, exceeding the size cap"); }
  std::string bytes(static_cast<size_t>(st.st_size), '\0');
  const bool whole = bytes.empty() || read_exact(fd, &bytes[0], bytes.size());
  close(fd);
  if (!whole) return fail(FJ_WEIGHTS_IO, "weight file I/O failed: short read of the index");
  Json root;
  Parser parser{bytes.data(), bytes.data() + bytes.size(), {}};
  if (!parser.document(&root) || root.kind != Json::Object) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: " + (parser.error.empty() ? std::string("expected an object") : parser.error));
  const Json* weight_map = nullptr;
  for (auto& member : root.members) {
    if (member.first != "weight_map") continue;
    if (weight_map) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: duplicate field `weight_map`");
    weight_map = &member.second;
  }
  if (!weight_map) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: missing field `weight_map`");
  if (weight_map->kind != Json::Object) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: expected a safetensors metadata object");
  std::string dup;
  if (duplicate_key(*weight_map, &dup)) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: duplicate safetensors entry \"" + dup + "\"");
  std::map<std::string, std::set<std::string>> shards;  // ordered by shard name, like the reference's BTreeMap
  for (auto& member : weight_map->members) {
    if (member.second.kind != Json::String) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: shard for tensor \"" + member.first + "\" is not a string");
    const std::string& file = member.second.text;
    if (!valid_shard_name(file)) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: invalid shard name \"" + file + "\"");
    if (!shards.count(file) && shards.size() == kMaxShards) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: weight map exceeds the 1024-shard limit");
    shards[file].insert(member.first);
  }
  if (shards.empty()) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: weight map is empty");
  std::string root_dir;
  if (!canonical(slash == std::string::npos ? "." : (slash == 0 ? "/" : p.substr(0, slash)), &root_dir)) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  std::vector<std::unique_ptr<fj_safetensors>> opened;
  for (auto& shard : shards) {
    std::string resolved;
    if (!canonical(root_dir + "/" + shard.first, &resolved)) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
    if (!starts_with_directory(resolved, root_dir)) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: shard \"" + shard.first + "\" resolves outside its model directory");
    std::unique_ptr<fj_safetensors> source;
    int32_t status = open_one(resolved.c_str(), &source);
    if (status != FJ_OK) return status;
    std::set<std::string> actual;
    for (auto& t : source->tensors) actual.insert(t.name);
    if (actual != shard.second) return fail(FJ_WEIGHTS_INVALID_INDEX, "invalid safetensors index: shard \"" + shard.first + "\" does not match its weight map");
    source->shard_name = shard.first;
    opened.push_back(std::move(source));
  }
  *count = static_cast<uint32_t>(opened.size());
  if (opened.size() > cap) return fail(FJ_QUOTA_EXCEEDED, "handle array too small");
  for (size_t i = 0; i < opened.size(); ++i) out[i] = opened[i].release();
  return FJ_OK;
}

void fj_safetensors_close(fj_safetensors* source) { delete source; }

uint32_t fj_safetensors_tensor_count(const fj_safetensors* source) { return source ? static_cast<uint32_t>(source->tensors.size()) : 0; }
const char* fj_safetensors_shard_name(const fj_safetensors* source) { return source && !source->shard_name.empty() ? source->shard_name.c_str() : nullptr; }
uint64_t fj_safetensors_file_len(const fj_safetensors* source) { return source ? source->file_len : 0; }
uint64_t fj_safetensors_data_start(const fj_safetensors* source) { return source ? source->data_start : 0; }

static void describe(const Tensor& t, fj_weight_tensor* out) {
  out->name = t.name.c_str();
  out->dtype = t.dtype;
  out->rank = static_cast<uint32_t>(std::min<size_t>(t.shape.size(), 8));
  for (uint32_t a = 0; a < 8; ++a) out->shape[a] = a < t.shape.size() ? t.shape[a] : 0;
  out->byte_offset = t.byte_offset;
  out->byte_len = t.byte_len;
  out->dtype_aligned = t.byte_offset % dtype_bytes(t.dtype) == 0 ? 1 : 0;  // WeightTensor::is_dtype_aligned
}

int32_t fj_safetensors_tensor(const fj_safetensors* source, uint32_t index, fj_weight_tensor* out) {
  if (!source || !out || index >= source->tensors.size()) return FJ_INVALID_INPUT;
  if (source->tensors[index].shape.size() > 8) return FJ_UNSUPPORTED_OPERATION;
  describe(source->tensors[index], out);
  return FJ_OK;
}

int32_t fj_safetensors_find(const fj_safetensors* source, const char* name, fj_weight_tensor* out) {
  if (!source || !name || !out) return FJ_INVALID_INPUT;
  for (auto& t : source->tensors) {
    if (t.name != name) continue;
    if (t.shape.size() > 8) return FJ_UNSUPPORTED_OPERATION;
    describe(t, out);
    return FJ_OK;
  }
  return FJ_INVALID_INPUT;
}

// WeightSource::mapped_region + Backend::import_readonly (weights.rs:326-333, crates/forja-host/src/lib.rs:5885-5900):
// maps the file again, checks that its length is still the validated one, and imports the data region.
int32_t fj_safetensors_import(fj_backend* be, const fj_safetensors* source, uint64_t* buffer) {
  if (!be || !source || !buffer) return fail(FJ_INVALID_INPUT, "null argument");
  int fd = open(source->path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) return fail(FJ_WEIGHTS_IO, std::string("weight file I/O failed: ") + strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0 || static_cast<uint64_t>(st.st_size) != source->file_len) { close(fd); return fail(FJ_WEIGHTS_MAPPING, "weight file changed after validation"); }
  void* map = source->file_len ? mmap(nullptr, source->file_len, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
  close(fd);
  if (source->file_len && map == MAP_FAILED) return fail(FJ_WEIGHTS_MAPPING, std::string("mapping failed: ") + strerror(errno));
  const int32_t status = fj_import_readonly(be, static_cast<const char*>(map) + source->data_start, source->file_len - source->data_start, buffer);
  if (map) munmap(map, source->file_len);
  return status;
}

// A tensor of an imported source as an fj_tensor over the imported buffer (WeightTensor::layout, weights.rs:76-83).
int32_t fj_safetensors_view(const fj_safetensors* source, const char* name, uint64_t buffer, fj_tensor* out) {
  fj_weight_tensor w;
  int32_t status = fj_safetensors_find(source, name, &w);
  if (status != FJ_OK) return status;
  if (!w.dtype_aligned || !out) return FJ_INVALID_INPUT;
  memset(out, 0, sizeof(*out));
  out->buffer = buffer; out->dtype = w.dtype; out->rank = w.rank;
  out->offset = w.byte_offset / dtype_bytes(w.dtype);
  uint64_t stride = 1;
  for (int a = static_cast<int>(w.rank) - 1; a >= 0; --a) { out->shape[a] = w.shape[a]; out->strides[a] = stride; stride *= w.shape[a]; }
  return FJ_OK;
}

// MLX affine-quantised matrix by checkpoint prefix: `<prefix>.weight` u32 [.., out, in * bits / 32], `<prefix>.scales` and
// `<prefix>.biases` f16/bf16 [.., out, in / group] with equal dtypes and leading extents (engines/qwen3-coder/src/lib.rs:174-188,
// :430-437; QuantizedMatrix::new, crates/forja-core/src/quantized.rs:78-121). in_features comes from the scales' last extent.
int32_t fj_safetensors_quant_views(const fj_safetensors* source, const char* prefix, uint64_t buffer, uint32_t bits, uint32_t group_size,
                                   fj_tensor* packed, fj_tensor* scales, fj_tensor* biases) {
  if (!source || !prefix || !packed || !scales || !biases) return FJ_INVALID_INPUT;
  if ((bits != 4 && bits != 8) || (group_size != 32 && group_size != 64 && group_size != 128)) return FJ_INVALID_INPUT;
  const std::string base = prefix;
  int32_t status = fj_safetensors_view(source, (base + ".weight").c_str(), buffer, packed);
  if (status == FJ_OK) status = fj_safetensors_view(source, (base + ".scales").c_str(), buffer, scales);
  if (status == FJ_OK) status = fj_safetensors_view(source, (base + ".biases").c_str(), buffer, biases);
  if (status != FJ_OK) return status;
  if (packed->dtype != FJ_U32 || (scales->dtype != FJ_F16 && scales->dtype != FJ_BF16) || biases->dtype != scales->dtype) return FJ_INVALID_INPUT;
  if (packed->rank < 2 || scales->rank != packed->rank || biases->rank != packed->rank) return FJ_INVALID_INPUT;
  const uint32_t r = packed->rank;
  for (uint32_t a = 0; a + 1 < r; ++a)
    if (scales->shape[a] != packed->shape[a] || biases->shape[a] != packed->shape[a]) return FJ_INVALID_INPUT;
  if (biases->shape[r - 1] != scales->shape[r - 1]) return FJ_INVALID_INPUT;
  const uint64_t in_features = static_cast<uint64_t>(scales->shape[r - 1]) * group_size;
  if (in_features * bits != static_cast<uint64_t>(packed->shape[r - 1]) * 32) return FJ_INVALID_INPUT;
  return FJ_OK;
}

}  // extern "C"
