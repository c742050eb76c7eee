// JSON reader and deploy-artifact (.npz) loader. Host code only.
#include "engine_io.h"
#include <exception>
#include <algorithm>
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace mu {

// ---------------------------------------------------------------------------
// JSON (objects, arrays, strings with \ escapes, numbers, true/false/null)
// ---------------------------------------------------------------------------
namespace {
struct JsonReader {
  const std::string &s;
  size_t i = 0;
  std::string err;
  explicit JsonReader(const std::string &t) : s(t) {}
  void ws() {
    while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i])))
      ++i;
  }
  bool fail(const std::string &m) {
    if (err.empty())
      err = m + " at offset " + std::to_string(i);
    return false;
  }
  bool str(std::string *out) {
    if (s[i] != '"')
      return fail("expected string");
    ++i;
    out->clear();
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c == '\\') {
        if (i >= s.size())
          return fail("bad escape");
        char e = s[i++];
        switch (e) {
        case 'n': out->push_back('\n'); break;
        case 't': out->push_back('\t'); break;
        case 'r': out->push_back('\r'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'u': {
          if (i + 4 > s.size())
            return fail("bad \\u escape");
          unsigned cp = static_cast<unsigned>(std::strtoul(s.substr(i, 4).c_str(), nullptr, 16));
          i += 4;
          if (cp < 0x80) out->push_back(static_cast<char>(cp));
          else if (cp < 0x800) {
            out->push_back(static_cast<char>(0xC0 | (cp >> 6)));
            out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          } else {
            out->push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          }
          break;
        }
        default: out->push_back(e);
        }
      } else {
        out->push_back(c);
      }
    }
    if (i >= s.size())
      return fail("unterminated string");
    ++i;
    return true;
  }
  bool value(Json *out, int depth) {
    if (depth > 256)
      return fail("nesting too deep");
    ws();
    if (i >= s.size())
      return fail("unexpected end");
    char c = s[i];
    if (c == '{') {
      out->kind = Json::OBJ;
      ++i;
      ws();
      if (i < s.size() && s[i] == '}') { ++i; return true; }
      while (true) {
        ws();
        std::string k;
        if (i >= s.size() || !str(&k))
          return fail("expected object key");
        ws();
        if (i >= s.size() || s[i] != ':')
          return fail("expected ':'");
        ++i;
        Json v;
        if (!value(&v, depth + 1))
          return false;
        out->obj.emplace_back(std::move(k), std::move(v));
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      out->kind = Json::ARR;
      ++i;
      ws();
      if (i < s.size() && s[i] == ']') { ++i; return true; }
      while (true) {
        Json v;
        if (!value(&v, depth + 1))
          return false;
        out->arr.push_back(std::move(v));
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') {
      out->kind = Json::STR;
      return str(&out->str);
    }
    if (s.compare(i, 4, "true") == 0) { out->kind = Json::BOOL; out->b = true; i += 4; return true; }
    if (s.compare(i, 5, "false") == 0) { out->kind = Json::BOOL; out->b = false; i += 5; return true; }
    if (s.compare(i, 4, "null") == 0) { out->kind = Json::NUL; i += 4; return true; }
    {
      const char *b = s.c_str() + i;
      char *e = nullptr;
      double d = std::strtod(b, &e);
      if (e == b)
        return fail("unexpected character");
      out->kind = Json::NUM;
      out->num = d;
      i += static_cast<size_t>(e - b);
      return true;
    }
  }
};
} // namespace

bool parse_json(const std::string &text, Json *out, std::string *why) {
  JsonReader r(text);
  Json v;
  if (!r.value(&v, 0)) {
    *why = r.err;
    return false;
  }
  r.ws();
  if (r.i != text.size()) {
    *why = "trailing characters after JSON value";
    return false;
  }
  *out = std::move(v);
  return true;
}

// ---------------------------------------------------------------------------
// zip (stored members only) + npy v1/v2/v3
// ---------------------------------------------------------------------------
namespace {

uint16_t rd16(const unsigned char *p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
uint32_t rd32(const unsigned char *p) {
  return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
         (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24);
}
uint64_t rd64(const unsigned char *p) { return rd32(p) | (static_cast<uint64_t>(rd32(p + 4)) << 32); }

struct Member {
  std::string name;
  const unsigned char *data;
  uint64_t size;
};

bool read_zip(const std::vector<unsigned char> &f, std::vector<Member> *out, std::string *why) {
  const size_t n = f.size();
  if (n < 22) { *why = "Serialized artifact is too small to be a zip archive"; return false; }
  // End of central directory: scan back over a possible comment
  size_t eocd = std::string::npos;
  for (size_t i = n - 22;; --i) {
    if (rd32(&f[i]) == 0x06054b50u) { eocd = i; break; }
    if (i == 0 || n - i > 22 + 65535) break;
  }
  if (eocd == std::string::npos) { *why = "Serialized artifact is not a zip archive (no end-of-central-directory record)"; return false; }
  uint64_t count = rd16(&f[eocd + 10]);
  uint64_t cd_size = rd32(&f[eocd + 12]);
  uint64_t cd_off = rd32(&f[eocd + 16]);
  // zip64 (archives of 4 GiB and more; numpy writes these for large models)
  if (count == 0xFFFF || cd_size == 0xFFFFFFFFu || cd_off == 0xFFFFFFFFu) {
    if (eocd < 20 || rd32(&f[eocd - 20]) != 0x07064b50u) { *why = "zip64 locator missing"; return false; }
    const uint64_t z = rd64(&f[eocd - 20 + 8]);
    if (z > n || n - z < 56 || rd32(&f[z]) != 0x06064b50u) { *why = "zip64 end-of-central-directory record missing"; return false; }
    count = rd64(&f[z + 32]);
    cd_size = rd64(&f[z + 40]);
    cd_off = rd64(&f[z + 48]);
  }
  // sizes come from the file (64-bit in zip64): compare by subtraction so that nothing wraps
  if (cd_off > n || cd_size > n - cd_off) { *why = "zip central directory out of bounds"; return false; }
  size_t p = static_cast<size_t>(cd_off);
  for (uint64_t k = 0; k < count; ++k) {
    if (p > n || n - p < 46 || rd32(&f[p]) != 0x02014b50u) { *why = "corrupt zip central directory"; return false; }
    const uint16_t method = rd16(&f[p + 10]);
    uint64_t csize = rd32(&f[p + 20]), usize = rd32(&f[p + 24]);
    const uint16_t nlen = rd16(&f[p + 28]), xlen = rd16(&f[p + 30]), clen = rd16(&f[p + 32]);
    uint64_t lho = rd32(&f[p + 42]);
    if (n - p - 46 < static_cast<size_t>(nlen) + xlen + clen) { *why = "corrupt zip central directory entry"; return false; }
    std::string name(reinterpret_cast<const char *>(&f[p + 46]), nlen);
    // zip64 extra field
    size_t x = p + 46 + nlen, xe = x + xlen;
    while (x + 4 <= xe) {
      const uint16_t id = rd16(&f[x]), sz = rd16(&f[x + 2]);
      if (id == 0x0001) {
        size_t q = x + 4;
        if (usize == 0xFFFFFFFFu && q + 8 <= xe) { usize = rd64(&f[q]); q += 8; }
        if (csize == 0xFFFFFFFFu && q + 8 <= xe) { csize = rd64(&f[q]); q += 8; }
        if (lho == 0xFFFFFFFFu && q + 8 <= xe) { lho = rd64(&f[q]); q += 8; }
      }
      x += 4 + sz;
    }
    if (method != 0) { *why = "Compressed npz entries are not supported: " + name; return false; }
    if (csize != usize) { *why = "zip entry size mismatch: " + name; return false; }
    if (lho > n || n - lho < 30 || rd32(&f[lho]) != 0x04034b50u) { *why = "corrupt zip local header: " + name; return false; }
    const uint16_t ln = rd16(&f[lho + 26]), lx = rd16(&f[lho + 28]);
    const uint64_t start = lho + 30 + ln + lx; // lho <= n and three 16-bit terms: cannot wrap
    if (start > n || usize > n - start) { *why = "zip entry out of bounds: " + name; return false; }
    out->push_back({name, &f[start], usize});
    p += 46 + nlen + xlen + clen;
  }
  return true;
}

struct Npy {
  std::string descr;
  bool fortran = false;
  std::vector<long long> shape;
  const unsigned char *data = nullptr;
  uint64_t bytes = 0;
};

bool parse_npy(const Member &m, Npy *out, std::string *why) {
  const unsigned char *d = m.data;
  if (m.size < 10 || memcmp(d, "\x93NUMPY", 6) != 0) { *why = "Invalid npy magic in entry " + m.name; return false; }
  const int major = d[6];
  size_t hlen, hoff;
  if (major == 1) { hlen = rd16(d + 8); hoff = 10; }
  else if (major == 2 || major == 3) { if (m.size < 12) { *why = "truncated npy header"; return false; } hlen = rd32(d + 8); hoff = 12; }
  else { *why = "Unsupported npy version in entry " + m.name; return false; }
  if (hoff + hlen > m.size) { *why = "truncated npy header in entry " + m.name; return false; }
  const std::string h(reinterpret_cast<const char *>(d + hoff), hlen);
  auto find_val = [&](const char *key) -> size_t {
    size_t k = h.find(std::string("'") + key + "'");
    if (k == std::string::npos) return k;
    k = h.find(':', k);
    return k == std::string::npos ? k : k + 1;
  };
  size_t p = find_val("descr");
  if (p == std::string::npos) { *why = "npy header lacks descr"; return false; }
  const size_t q1 = h.find('\'', p);
  const size_t q2 = q1 == std::string::npos ? q1 : h.find('\'', q1 + 1);
  if (q1 == std::string::npos || q2 == std::string::npos) { *why = "npy header: bad descr"; return false; }
  out->descr = h.substr(q1 + 1, q2 - q1 - 1);
  p = find_val("fortran_order");
  if (p == std::string::npos) { *why = "npy header lacks fortran_order"; return false; }
  const size_t fv = h.find_first_not_of(' ', p);
  if (fv == std::string::npos) { *why = "npy header: bad fortran_order"; return false; }
  out->fortran = h.compare(fv, 4, "True") == 0;
  p = find_val("shape");
  if (p == std::string::npos) { *why = "npy header lacks shape"; return false; }
  const size_t a = h.find('(', p);
  const size_t b = a == std::string::npos ? a : h.find(')', a);
  if (a == std::string::npos || b == std::string::npos) { *why = "npy header: bad shape"; return false; }
  const std::string sh = h.substr(a + 1, b - a - 1);
  size_t i = 0;
  while (i < sh.size()) {
    while (i < sh.size() && !std::isdigit(static_cast<unsigned char>(sh[i]))) ++i;
    if (i >= sh.size()) break;
    long long v = 0;
    while (i < sh.size() && std::isdigit(static_cast<unsigned char>(sh[i]))) v = v * 10 + (sh[i++] - '0');
    out->shape.push_back(v);
  }
  out->data = d + hoff + hlen;
  out->bytes = m.size - hoff - hlen;
  return true;
}

long long numel(const std::vector<long long> &s) {
  long long n = 1;
  for (long long v : s) n *= v;
  return n;
}

// 0-d scalars of the metadata members
bool decode_string(const Npy &a, std::string *out, std::string *why) {
  // '<U<n>' little-endian UCS-4, ASCII only; also accept '|S<n>' byte strings
  if (a.descr.size() >= 3 && (a.descr[1] == 'U')) {
    const long long n = std::atoll(a.descr.c_str() + 2);
    if (numel(a.shape) != 1 || static_cast<uint64_t>(n) * 4 > a.bytes) { *why = "bad unicode scalar"; return false; }
    out->clear();
    for (long long i = 0; i < n; ++i) {
      const uint32_t cp = rd32(a.data + 4 * i);
      if (cp == 0) break;
      if (cp > 127) { *why = "Only ASCII metadata strings are supported in serialized artifacts"; return false; }
      out->push_back(static_cast<char>(cp));
    }
    return true;
  }
  if (a.descr.size() >= 3 && a.descr[1] == 'S') {
    const long long n = std::atoll(a.descr.c_str() + 2);
    out->assign(reinterpret_cast<const char *>(a.data), static_cast<size_t>(std::min<long long>(n, static_cast<long long>(a.bytes))));
    while (!out->empty() && out->back() == '\0') out->pop_back();
    return true;
  }
  *why = "Expected a string scalar, got descr " + a.descr;
  return false;
}

bool decode_int(const Npy &a, long long *out, std::string *why) {
  if (a.descr == "<i8" && a.bytes >= 8) { *out = static_cast<long long>(rd64(a.data)); return true; }
  if (a.descr == "<i4" && a.bytes >= 4) { *out = static_cast<int32_t>(rd32(a.data)); return true; }
  *why = "Expected an integer scalar, got descr " + a.descr;
  return false;
}

const char *kForbidden[] = {"optim", "optimizer", "scheduler", "scaler", "master_weight",
                            "checkpoint", "epoch", "step", "grad"};

} // namespace

static bool load_artifact_impl(const std::string &path, Json *config,
                               std::map<std::string, NamedTensor> *tensors, std::string *why);

// The callers are extern "C" entry points that promise never to throw: anything the parser
// raises on a malformed file (std::out_of_range from a string search, std::bad_alloc from a
// size field that asks for more memory than there is) becomes an ordinary load failure.
bool load_artifact(const std::string &path, Json *config,
                   std::map<std::string, NamedTensor> *tensors, std::string *why) {
  try {
    return load_artifact_impl(path, config, tensors, why);
  } catch (const std::exception &e) {
    *why = std::string("Malformed serialized artifact: ") + e.what();
  } catch (...) {
    *why = "Malformed serialized artifact";
  }
  tensors->clear();
  return false;
}

static bool load_artifact_impl(const std::string &path, Json *config,
                               std::map<std::string, NamedTensor> *tensors, std::string *why) {
  FILE *fp = fopen(path.c_str(), "rb");
  if (!fp) { *why = "Unable to open serialized artifact: " + path; return false; }
  fseek(fp, 0, SEEK_END);
  const long long sz = ftell(fp);
  fseek(fp, 0, SEEK_SET);
  std::vector<unsigned char> file(static_cast<size_t>(std::max<long long>(sz, 0)));
  if (sz > 0 && fread(file.data(), 1, file.size(), fp) != file.size()) {
    fclose(fp);
    *why = "Unable to read serialized artifact: " + path;
    return false;
  }
  fclose(fp);
  std::vector<Member> members;
  if (!read_zip(file, &members, why)) return false;

  std::string format_name, legacy_tag, producer, kind, scope, load_mode, loader, policy, config_json, manifest_json;
  long long revision = -1;
  bool training_state = false, have_manifest = false;
  std::vector<std::string> payload;
  tensors->clear();
  for (const Member &m : members) {
    std::string name = m.name;
    if (name.size() > 4 && name.compare(name.size() - 4, 4, ".npy") == 0) name.resize(name.size() - 4);
    Npy a;
    if (!parse_npy(m, &a, why)) return false;
    if (name.rfind("__", 0) == 0) {
      bool ok = true;
      if (name == "__format_name__") ok = decode_string(a, &format_name, why);
      else if (name == "__format_revision__") ok = decode_int(a, &revision, why);
      else if (name == "__format_version__") ok = decode_string(a, &legacy_tag, why);
      else if (name == "__producer__") ok = decode_string(a, &producer, why);
      else if (name == "__artifact_kind__") ok = decode_string(a, &kind, why);
      else if (name == "__artifact_scope__") ok = decode_string(a, &scope, why);
      else if (name == "__default_load_mode__") ok = decode_string(a, &load_mode, why);
      else if (name == "__contains_training_state__") {
        if (a.descr != "|b1" || a.bytes < 1) { *why = "Expected a bool scalar for __contains_training_state__"; return false; }
        training_state = a.data[0] != 0;
      } else if (name == "__recommended_loader__") ok = decode_string(a, &loader, why);
      else if (name == "__compile_contract_policy__") ok = decode_string(a, &policy, why);
      else if (name == "__config__") ok = decode_string(a, &config_json, why);
      else if (name == "__tensor_names__") { ok = decode_string(a, &manifest_json, why); have_manifest = true; }
      if (!ok) return false;
      continue;
    }
    std::string lowered = name;
    std::transform(lowered.begin(), lowered.end(), lowered.begin(),
                   [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
    for (const char *tok : kForbidden)
      if (lowered.find(tok) != std::string::npos) {
        *why = "Unsupported training/checkpoint payload key in deploy artifact: " + name;
        return false;
      }
    NamedTensor t;
    if (a.descr == "<f4") t.dtype = 0;
    else if (a.descr == "<f2") t.dtype = 1;
    else if (a.descr == "<i4") t.dtype = 3;
    else { *why = "Unsupported npy dtype descriptor: " + a.descr; return false; }
    if (a.fortran) { *why = "Fortran-order npy arrays are not supported: " + name; return false; }
    t.shape = a.shape;
    // the extents come from the file: their product must not wrap before it is compared
    uint64_t count = 1;
    for (long long ext : a.shape) {
      if (ext < 0 || (ext > 0 && count > (a.bytes + 1) / static_cast<uint64_t>(ext))) {
        *why = "npy payload shorter than its shape: " + name;
        return false;
      }
      count *= static_cast<uint64_t>(ext);
    }
    const uint64_t need = count * (t.dtype == 1 ? 2 : 4);
    if (need > a.bytes) { *why = "npy payload shorter than its shape: " + name; return false; }
    t.owned.assign(a.data, a.data + need);
    t.data = t.owned.data();
    payload.push_back(name);
    (*tensors)[name] = std::move(t);
    (*tensors)[name].data = (*tensors)[name].owned.data();
  }
  std::sort(payload.begin(), payload.end());
  if (have_manifest) {
    Json mj;
    std::string jerr;
    if (!parse_json(manifest_json, &mj, &jerr) || !mj.is_array()) { *why = "Serialized tensor manifest is not a JSON array"; return false; }
    std::vector<std::string> names;
    for (auto &v : mj.arr) {
      if (!v.is_string()) { *why = "Serialized tensor manifest must hold strings"; return false; }
      names.push_back(v.str);
    }
    if (!names.empty() && names != payload) { *why = "Serialized tensor manifest does not match payload keys"; return false; }
  }
  if (format_name != "munet_model") { *why = "Unsupported serialization format name: " + format_name; return false; }
  if (revision != 1) { *why = "Unsupported serialization format revision: " + std::to_string(revision); return false; }
  if (!legacy_tag.empty() && legacy_tag != "munet_model_v1") { *why = "Unsupported legacy serialization tag: " + legacy_tag; return false; }
  // The C++ loader of the reference accepts only "munet" (inference_serialization.cpp:997-1001)
  // while its own Python writer emits "munet_nn" (src/bindings.cpp:2049): both are accepted.
  if (!producer.empty() && producer != "munet" && producer != "munet_nn") { *why = "Unsupported serialization producer: " + producer; return false; }
  if (kind != "deploy_model") { *why = "Unsupported serialization artifact kind: " + kind; return false; }
  if (scope != "runtime_only") { *why = "Unsupported serialization artifact scope: " + scope; return false; }
  if (load_mode != "eval") { *why = "Unsupported deploy load mode: " + load_mode; return false; }
  if (training_state) { *why = "Unsupported serialization payload: deploy artifacts must not contain training-only state"; return false; }
  if (loader != "load_for_inference") { *why = "Unsupported recommended loader: " + loader; return false; }
  if (policy != "external") { *why = "Unsupported compile contract policy: " + policy; return false; }
  if (config_json.empty()) { *why = "Serialized deploy artifact does not contain architecture config required for C++ reconstruction"; return false; }
  std::string jerr;
  if (!parse_json(config_json, config, &jerr)) { *why = "Serialized module config is not valid JSON: " + jerr; return false; }
  return true;
}

} // namespace mu

// ---------------------------------------------------------------------------
// Host-only inspection of a deploy artifact (no device needed): validates it
// exactly like mu_engine_load and returns a JSON summary
//   {"config": <module tree>, "tensors": {"name": {"dtype": d, "shape": [...]}, ...}}
// ---------------------------------------------------------------------------
namespace {
void json_escape(const std::string &in, std::string *out) {
  for (char c : in) {
    if (c == '"' || c == '\\') { out->push_back('\\'); out->push_back(c); }
    else if (c == '\n') *out += "\\n";
    else if (c == '\t') *out += "\\t";
    else if (static_cast<unsigned char>(c) < 0x20) { char b[8]; snprintf(b, sizeof(b), "\\u%04x", c); *out += b; }
    else out->push_back(c);
  }
}
void json_dump(const mu::Json &j, std::string *out) {
  using mu::Json;
  switch (j.kind) {
  case Json::NUL: *out += "null"; break;
  case Json::BOOL: *out += j.b ? "true" : "false"; break;
  case Json::NUM: {
    char b[64];
    if (j.num == static_cast<long long>(j.num)) snprintf(b, sizeof(b), "%lld", static_cast<long long>(j.num));
    else snprintf(b, sizeof(b), "%.17g", j.num);
    *out += b;
    break;
  }
  case Json::STR: out->push_back('"'); json_escape(j.str, out); out->push_back('"'); break;
  case Json::ARR:
    out->push_back('[');
    for (size_t i = 0; i < j.arr.size(); ++i) { if (i) out->push_back(','); json_dump(j.arr[i], out); }
    out->push_back(']');
    break;
  case Json::OBJ:
    out->push_back('{');
    for (size_t i = 0; i < j.obj.size(); ++i) {
      if (i) out->push_back(',');
      out->push_back('"'); json_escape(j.obj[i].first, out); *out += "\":";
      json_dump(j.obj[i].second, out);
    }
    out->push_back('}');
    break;
  }
}
} // namespace

extern "C" int mu_artifact_inspect(const char *path, char *json_out, size_t json_cap, char *err,
                                   size_t err_len) {
  if (err && err_len) err[0] = 0;
  if (!path || !json_out || json_cap == 0) return 1;
  mu::Json config;
  std::map<std::string, mu::NamedTensor> tensors;
  std::string why;
  if (!mu::load_artifact(path, &config, &tensors, &why)) {
    if (err && err_len) snprintf(err, err_len, "%s", why.c_str());
    return 1;
  }
  std::string out = "{\"config\":";
  json_dump(config, &out);
  out += ",\"tensors\":{";
  bool first = true;
  for (auto &kv : tensors) {
    if (!first) out.push_back(',');
    first = false;
    out.push_back('"'); json_escape(kv.first, &out); out += "\":{\"dtype\":" + std::to_string(kv.second.dtype) + ",\"shape\":[";
    for (size_t i = 0; i < kv.second.shape.size(); ++i) { if (i) out.push_back(','); out += std::to_string(kv.second.shape[i]); }
    out += "]}";
  }
  out += "}}";
  if (out.size() + 1 > json_cap) {
    if (err && err_len) snprintf(err, err_len, "summary needs %zu bytes", out.size() + 1);
    return 7;
  }
  memcpy(json_out, out.c_str(), out.size() + 1);
  return 0;
}
