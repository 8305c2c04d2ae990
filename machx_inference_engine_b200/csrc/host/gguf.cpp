// GGUF v3 container: zero-copy mmap reader (with split-shard merge) and a streaming writer.
//
// Reference parity: src/loaders/gguf_reader.cpp:193-384 (v3 only, per-shard alignment,
// "-00001-of-0000N.gguf" shards merged with metadata taken from shard 1 and a
// split.count / split.tensors.count cross-check), src/loaders/gguf_writer.cpp
// (accumulate-or-stream emit).  The design differs: the reader hands the whole
// metadata table to the caller as one JSON document and exposes tensor payloads as
// raw pointers into the mapping, so the Python layer needs no per-key FFI calls.
#include "quant.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

enum KvType : uint32_t { KV_U8 = 0, KV_I8, KV_U16, KV_I16, KV_U32, KV_I32, KV_F32, KV_BOOL, KV_STR, KV_ARR, KV_U64, KV_I64, KV_F64 };

struct Mapping {
  std::string path; int fd = -1; const uint8_t* base = nullptr; size_t size = 0;
  void close_() { if (base) munmap((void*)base, size); if (fd >= 0) ::close(fd); base = nullptr; fd = -1; }
};

struct TensorInfo { std::string name; std::vector<uint64_t> dims; int32_t type; uint64_t offset; uint64_t nbytes; int shard; const uint8_t* ptr; };

struct Cursor {
  const uint8_t* p; const uint8_t* end;
  template <class T> T get() { need(sizeof(T)); T v; std::memcpy(&v, p, sizeof(T)); p += sizeof(T); return v; }
  std::string str() { uint64_t n = get<uint64_t>(); need(n); std::string s((const char*)p, n); p += n; return s; }
  void need(uint64_t n) { if ((uint64_t)(end - p) < n) throw std::runtime_error("gguf: truncated file"); }
};

void json_escape(std::string& out, const std::string& s) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break; case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break; case '\r': out += "\\r"; break; case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out.push_back((char)c);
    }
  }
  out.push_back('"');
}

void json_scalar(std::string& out, Cursor& c, uint32_t t) {
  char b[64];
  switch (t) {
    case KV_U8: snprintf(b, sizeof b, "%u", c.get<uint8_t>()); out += b; break;
    case KV_I8: snprintf(b, sizeof b, "%d", c.get<int8_t>()); out += b; break;
    case KV_U16: snprintf(b, sizeof b, "%u", c.get<uint16_t>()); out += b; break;
    case KV_I16: snprintf(b, sizeof b, "%d", c.get<int16_t>()); out += b; break;
    case KV_U32: snprintf(b, sizeof b, "%u", c.get<uint32_t>()); out += b; break;
    case KV_I32: snprintf(b, sizeof b, "%d", c.get<int32_t>()); out += b; break;
    case KV_U64: snprintf(b, sizeof b, "%llu", (unsigned long long)c.get<uint64_t>()); out += b; break;
    case KV_I64: snprintf(b, sizeof b, "%lld", (long long)c.get<int64_t>()); out += b; break;
    case KV_F32: { float f = c.get<float>(); if (std::isfinite(f)) { snprintf(b, sizeof b, "%.9g", f); out += b; } else out += "null"; break; }
    case KV_F64: { double f = c.get<double>(); if (std::isfinite(f)) { snprintf(b, sizeof b, "%.17g", f); out += b; } else out += "null"; break; }
    case KV_BOOL: out += c.get<uint8_t>() ? "true" : "false"; break;
    case KV_STR: json_escape(out, c.str()); break;
    default: throw std::runtime_error("gguf: unknown metadata value type");
  }
}

struct Reader {
  std::vector<Mapping> shards;
  std::vector<TensorInfo> tensors;
  std::string kv_json;     // {"key": value, ...}
  std::string meta_json;   // full document
  uint32_t version = 0;
  uint64_t split_count = 0, split_tensors = 0;

  ~Reader() { for (auto& m : shards) m.close_(); }

  void map_file(const std::string& path) {
    Mapping m; m.path = path;
    m.fd = ::open(path.c_str(), O_RDONLY);
    if (m.fd < 0) throw std::runtime_error("gguf: cannot open " + path);
    struct stat st; if (fstat(m.fd, &st) != 0) { ::close(m.fd); throw std::runtime_error("gguf: stat failed " + path); }
    m.size = (size_t)st.st_size;
    if (m.size < 24) { ::close(m.fd); throw std::runtime_error("gguf: file too small " + path); }
    void* p = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (p == MAP_FAILED) { ::close(m.fd); throw std::runtime_error("gguf: mmap failed " + path); }
    madvise(p, m.size, MADV_RANDOM);
    m.base = (const uint8_t*)p;
    shards.push_back(m);
  }

  // Parses shard `si`; metadata is kept only when keep_kv.
  void parse(int si, bool keep_kv) {
    const Mapping& m = shards[si];
    Cursor c{m.base, m.base + m.size};
    if (std::memcmp(c.p, "GGUF", 4) != 0) throw std::runtime_error("gguf: bad magic in " + m.path);
    c.p += 4;
    uint32_t ver = c.get<uint32_t>();
    if (ver != 3) throw std::runtime_error("gguf: only version 3 is supported (got " + std::to_string(ver) + ")");
    version = ver;
    uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    uint64_t alignment = 32;
    std::string js = "{";
    for (uint64_t i = 0; i < n_kv; ++i) {
      std::string key = c.str();
      uint32_t t = c.get<uint32_t>();
      std::string val;
      if (t == KV_ARR) {
        uint32_t et = c.get<uint32_t>(); uint64_t n = c.get<uint64_t>();
        if (et == KV_ARR) throw std::runtime_error("gguf: nested arrays are not supported");
        val.push_back('[');
        for (uint64_t k = 0; k < n; ++k) { if (k) val.push_back(','); json_scalar(val, c, et); }
        val.push_back(']');
      } else {
        const uint8_t* before = c.p;
        json_scalar(val, c, t);
        if (key == "general.alignment" && t == KV_U32) { uint32_t a; std::memcpy(&a, before, 4); if (a) alignment = a; }
        if (key == "split.count") { Cursor cc{before, c.end}; split_count = (t == KV_U16) ? cc.get<uint16_t>() : (t == KV_U32 ? cc.get<uint32_t>() : (uint64_t)cc.get<int32_t>()); }
        if (key == "split.tensors.count") { Cursor cc{before, c.end}; split_tensors = (t == KV_I32) ? (uint64_t)cc.get<int32_t>() : (t == KV_U64 ? cc.get<uint64_t>() : cc.get<uint32_t>()); }
      }
      if (keep_kv) { if (js.size() > 1) js.push_back(','); json_escape(js, key); js.push_back(':'); js += val; }
    }
    js.push_back('}');
    if (keep_kv) kv_json = js;
    size_t first = tensors.size();
    for (uint64_t i = 0; i < n_tensors; ++i) {
      TensorInfo ti; ti.name = c.str();
      uint32_t nd = c.get<uint32_t>();
      if (nd > 8) throw std::runtime_error("gguf: tensor rank too large");
      uint64_t ne = 1;
      for (uint32_t d = 0; d < nd; ++d) { ti.dims.push_back(c.get<uint64_t>()); ne *= ti.dims.back(); }
      ti.type = (int32_t)c.get<uint32_t>();
      ti.offset = c.get<uint64_t>();
      ti.nbytes = mx::bytes_for(ti.type, ne);
      if (!ti.nbytes && ne) throw std::runtime_error("gguf: tensor '" + ti.name + "' has unsupported type " + std::to_string(ti.type) + " or a ragged block count");
      ti.shard = si; ti.ptr = nullptr;
      tensors.push_back(ti);
    }
    uint64_t data_start = (uint64_t)(c.p - m.base);
    data_start = (data_start + alignment - 1) / alignment * alignment;
    for (size_t i = first; i < tensors.size(); ++i) {
      TensorInfo& ti = tensors[i];
      if (data_start + ti.offset + ti.nbytes > m.size) throw std::runtime_error("gguf: tensor '" + ti.name + "' runs past the end of " + m.path);
      ti.ptr = m.base + data_start + ti.offset;
    }
  }

  void build_json() {
    std::string js = "{\"version\":" + std::to_string(version) + ",\"kv\":" + kv_json + ",\"shards\":[";
    for (size_t i = 0; i < shards.size(); ++i) { if (i) js.push_back(','); json_escape(js, shards[i].path); }
    js += "],\"tensors\":[";
    for (size_t i = 0; i < tensors.size(); ++i) {
      const TensorInfo& t = tensors[i];
      if (i) js.push_back(',');
      js += "{\"name\":"; json_escape(js, t.name);
      js += ",\"dims\":[";
      for (size_t d = 0; d < t.dims.size(); ++d) { if (d) js.push_back(','); js += std::to_string(t.dims[d]); }
      js += "],\"type\":" + std::to_string(t.type) + ",\"nbytes\":" + std::to_string(t.nbytes) + ",\"shard\":" + std::to_string(t.shard) + "}";
    }
    js += "]}";
    meta_json.swap(js);
  }
};

// "<prefix>-00001-of-00003.gguf" -> prefix and count; returns false when the name has no shard suffix.
bool split_name(const std::string& path, std::string& prefix, int& idx, int& count) {
  const size_t L = path.size();
  if (L < 20 || path.compare(L - 5, 5, ".gguf") != 0) return false;
  // layout: -DDDDD-of-DDDDD.gguf  (20 chars)
  size_t s = L - 20;
  if (path[s] != '-' || path.compare(s + 6, 4, "-of-") != 0) return false;
  for (int k = 1; k <= 5; ++k) if (!isdigit((unsigned char)path[s + k]) || !isdigit((unsigned char)path[s + 9 + k])) return false;
  idx = std::stoi(path.substr(s + 1, 5)); count = std::stoi(path.substr(s + 10, 5));
  prefix = path.substr(0, s);
  return true;
}

struct Writer {
  struct KV { std::string key; uint32_t type; std::vector<uint8_t> payload; };
  struct T { std::string name; std::vector<uint64_t> dims; int32_t type; uint64_t nbytes, offset; };
  std::vector<KV> kvs; std::vector<T> tensors;
  FILE* f = nullptr; uint64_t data_start = 0, written = 0; size_t next = 0;
  static constexpr uint64_t kAlign = 32;
  ~Writer() { if (f) fclose(f); }
};

template <class V> void put(std::vector<uint8_t>& b, V v) { const uint8_t* p = (const uint8_t*)&v; b.insert(b.end(), p, p + sizeof(V)); }
void put_str(std::vector<uint8_t>& b, const char* s, uint64_t n) { put<uint64_t>(b, n); b.insert(b.end(), s, s + n); }

thread_local std::string g_err;

}  // namespace

extern "C" {

const char* mx_last_error() { return g_err.c_str(); }

void* mx_gguf_open(const char* path) {
  Reader* r = new Reader();
  try {
    std::string prefix; int idx = 0, count = 0;
    if (split_name(path, prefix, idx, count) && count > 1) {
      for (int i = 1; i <= count; ++i) {
        char suf[32]; snprintf(suf, sizeof suf, "-%05d-of-%05d.gguf", i, count);
        r->map_file(prefix + suf);
      }
      for (int i = 0; i < count; ++i) r->parse(i, i == 0);
      // split.count of shard 1 was overwritten by later shards' own values only if they carry the key; re-check on totals
      if (r->split_tensors && r->split_tensors != r->tensors.size())
        throw std::runtime_error("gguf: split.tensors.count=" + std::to_string(r->split_tensors) + " but shards hold " + std::to_string(r->tensors.size()) + " tensors");
    } else {
      r->map_file(path);
      r->parse(0, true);
      if (r->split_count > 1) throw std::runtime_error("gguf: file declares split.count>1 but its name has no -NNNNN-of-NNNNN suffix");
    }
    r->build_json();
    return r;
  } catch (const std::exception& e) { g_err = e.what(); delete r; return nullptr; }
}
const char* mx_gguf_meta_json(void* h) { return ((Reader*)h)->meta_json.c_str(); }
uint64_t mx_gguf_meta_json_len(void* h) { return ((Reader*)h)->meta_json.size(); }
const void* mx_gguf_tensor_ptr(void* h, int64_t i) { Reader* r = (Reader*)h; return (i < 0 || (size_t)i >= r->tensors.size()) ? nullptr : r->tensors[i].ptr; }
void mx_gguf_close(void* h) { delete (Reader*)h; }

// ---- writer ----
void* mx_ggufw_new() { return new Writer(); }
void mx_ggufw_free(void* w) { delete (Writer*)w; }
static void add_kv(void* w, const char* key, uint32_t type, std::vector<uint8_t>&& payload) { ((Writer*)w)->kvs.push_back({key, type, std::move(payload)}); }
void mx_ggufw_kv_u32(void* w, const char* k, uint32_t v) { std::vector<uint8_t> b; put(b, v); add_kv(w, k, KV_U32, std::move(b)); }
void mx_ggufw_kv_i32(void* w, const char* k, int32_t v) { std::vector<uint8_t> b; put(b, v); add_kv(w, k, KV_I32, std::move(b)); }
void mx_ggufw_kv_u64(void* w, const char* k, uint64_t v) { std::vector<uint8_t> b; put(b, v); add_kv(w, k, KV_U64, std::move(b)); }
void mx_ggufw_kv_f32(void* w, const char* k, float v) { std::vector<uint8_t> b; put(b, v); add_kv(w, k, KV_F32, std::move(b)); }
void mx_ggufw_kv_bool(void* w, const char* k, int v) { std::vector<uint8_t> b; put<uint8_t>(b, v ? 1 : 0); add_kv(w, k, KV_BOOL, std::move(b)); }
void mx_ggufw_kv_str(void* w, const char* k, const char* s, uint64_t n) { std::vector<uint8_t> b; put_str(b, s, n); add_kv(w, k, KV_STR, std::move(b)); }
// strings are passed as one concatenated buffer plus per-string lengths (binary safe)
void mx_ggufw_kv_arr_str(void* w, const char* k, const char* blob, const uint64_t* lens, uint64_t n) {
  std::vector<uint8_t> b; put<uint32_t>(b, KV_STR); put<uint64_t>(b, n);
  for (uint64_t i = 0; i < n; ++i) { put_str(b, blob, lens[i]); blob += lens[i]; }
  add_kv(w, k, KV_ARR, std::move(b));
}
void mx_ggufw_kv_arr_i32(void* w, const char* k, const int32_t* v, uint64_t n) {
  std::vector<uint8_t> b; put<uint32_t>(b, KV_I32); put<uint64_t>(b, n); b.insert(b.end(), (const uint8_t*)v, (const uint8_t*)(v + n)); add_kv(w, k, KV_ARR, std::move(b));
}
void mx_ggufw_kv_arr_f32(void* w, const char* k, const float* v, uint64_t n) {
  std::vector<uint8_t> b; put<uint32_t>(b, KV_F32); put<uint64_t>(b, n); b.insert(b.end(), (const uint8_t*)v, (const uint8_t*)(v + n)); add_kv(w, k, KV_ARR, std::move(b));
}
// Returns the payload size in bytes, or 0 when the type/shape is invalid.
uint64_t mx_ggufw_add_tensor(void* w_, const char* name, int ndim, const uint64_t* dims, int32_t type) {
  Writer* w = (Writer*)w_;
  uint64_t ne = 1; for (int i = 0; i < ndim; ++i) ne *= dims[i];
  mx::TypeTraits tt = mx::type_traits(type);
  if (!tt.block_elems || ndim < 1 || dims[0] % tt.block_elems) { g_err = std::string("ggufw: tensor '") + name + "': row length is not a whole number of blocks"; return 0; }
  uint64_t nb = mx::bytes_for(type, ne);
  w->tensors.push_back({name, std::vector<uint64_t>(dims, dims + ndim), type, nb, 0});
  return nb;
}
// Writes header, metadata and tensor table; payloads follow through mx_ggufw_write in declaration order.
int mx_ggufw_begin(void* w_, const char* path) {
  Writer* w = (Writer*)w_;
  w->f = fopen(path, "wb");
  if (!w->f) { g_err = std::string("ggufw: cannot create ") + path; return -1; }
  std::vector<uint8_t> b;
  b.insert(b.end(), {'G', 'G', 'U', 'F'}); put<uint32_t>(b, 3); put<uint64_t>(b, w->tensors.size()); put<uint64_t>(b, w->kvs.size());
  for (auto& kv : w->kvs) { put_str(b, kv.key.data(), kv.key.size()); put<uint32_t>(b, kv.type); b.insert(b.end(), kv.payload.begin(), kv.payload.end()); }
  uint64_t off = 0;
  for (auto& t : w->tensors) {
    t.offset = off;
    put_str(b, t.name.data(), t.name.size()); put<uint32_t>(b, (uint32_t)t.dims.size());
    for (uint64_t d : t.dims) put<uint64_t>(b, d);
    put<uint32_t>(b, (uint32_t)t.type); put<uint64_t>(b, off);
    off += (t.nbytes + Writer::kAlign - 1) / Writer::kAlign * Writer::kAlign;
  }
  while (b.size() % Writer::kAlign) b.push_back(0);
  w->data_start = b.size();
  if (fwrite(b.data(), 1, b.size(), w->f) != b.size()) { g_err = "ggufw: short write"; return -1; }
  return 0;
}
int mx_ggufw_write(void* w_, const void* data, uint64_t nbytes) {
  Writer* w = (Writer*)w_;
  if (!w->f || w->next >= w->tensors.size()) { g_err = "ggufw: no tensor pending"; return -1; }
  const Writer::T& t = w->tensors[w->next];
  if (nbytes != t.nbytes) { g_err = "ggufw: payload size mismatch for '" + t.name + "'"; return -1; }
  if (nbytes && fwrite(data, 1, nbytes, w->f) != nbytes) { g_err = "ggufw: short write"; return -1; }
  static const uint8_t zeros[Writer::kAlign] = {0};
  uint64_t pad = (Writer::kAlign - nbytes % Writer::kAlign) % Writer::kAlign;
  if (pad && fwrite(zeros, 1, pad, w->f) != pad) { g_err = "ggufw: short write"; return -1; }
  ++w->next;
  return 0;
}
int mx_ggufw_end(void* w_) {
  Writer* w = (Writer*)w_;
  int rc = (w->next == w->tensors.size()) ? 0 : -1;
  if (rc) g_err = "ggufw: not every declared tensor was written";
  if (w->f) { fclose(w->f); w->f = nullptr; }
  return rc;
}

// ---- codecs ----
int mx_dequantize(int32_t type, const void* src, float* dst, uint64_t n) { return mx::dequantize(type, src, dst, n); }
int mx_quantize(int32_t type, const float* src, void* dst, uint64_t nrows, uint64_t ncols, int nthreads) { return mx::quantize(type, src, dst, nrows, ncols, nthreads); }
void mx_quantize_set_kquant_fit(int mode) { mx::set_kquant_fit(mode); }
uint64_t mx_bytes_for(int32_t type, uint64_t n) { return mx::bytes_for(type, n); }
int mx_type_block_elems(int32_t type) { return mx::type_traits(type).block_elems; }
int mx_type_block_bytes(int32_t type) { return mx::type_traits(type).block_bytes; }
const char* mx_type_name(int32_t type) { const char* n = mx::type_traits(type).name; return n ? n : ""; }

}  // extern "C"
