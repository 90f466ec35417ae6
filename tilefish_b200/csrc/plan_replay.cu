// A native replay loop for exported plans: reads plan.json (the reference's plan schema 1) and this backend's manifest.json from a
// directory, verifies the plan's digest against a pin, allocates the arena once, and then enqueues a bucket's steps on a stream with
// no Python between them, or captures them into a CUDA graph. It is the C++ counterpart of the reference's Rust host for this path
// (crates/tilefish/src/plan_run.rs:678 PlanRun, :1944 launch, :2097 capture): instantiate once, every step checked before the first
// launch, nothing allocated after instantiation, a captured graph kept alive together with the arena it points into.
//
// The file has four parts: a strict JSON reader and the canonical writer the digest is defined on (sorted keys, "," and ":"
// separators, ASCII escapes: python/src/tilefish/_manifest.py:85-115), SHA-256, the plan model, and the step executor, which calls
// this library's own entry points (tf_residual_add_rmsnorm, tf_quantize_*, tf_silu_gate, tf_gemm_blockscaled).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"

namespace tf {
namespace {

// ---- JSON ---------------------------------------------------------------------------------------------------------------------------
struct Json {
  enum Kind { Null, Bool, Int, Str, Arr, Obj } kind = Null;
  bool b = false;
  long long i = 0;
  std::string s;
  std::vector<Json> a;
  std::vector<std::pair<std::string, Json>> o;  // insertion order; keys are unique (checked by the reader)

  const Json* get(const std::string& key) const {
    for (const auto& kv : o)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JsonReader {
  const std::string& t;
  size_t p = 0;
  std::string err;
  int depth = 0;
  explicit JsonReader(const std::string& text) : t(text) {}

  void ws() {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
  }
  bool fail(const std::string& m) {
    if (err.empty()) err = m + " at byte " + std::to_string(p);
    return false;
  }
  bool value(Json& out) {
    if (++depth > 64) return fail("nested too deeply");
    ws();
    if (p >= t.size()) return fail("unexpected end");
    bool ok;
    const char c = t[p];
    if (c == '{') ok = object(out);
    else if (c == '[') ok = array(out);
    else if (c == '"') {
      out.kind = Json::Str;
      ok = string(out.s);
    } else if (t.compare(p, 4, "true") == 0) {
      out.kind = Json::Bool, out.b = true, p += 4, ok = true;
    } else if (t.compare(p, 5, "false") == 0) {
      out.kind = Json::Bool, out.b = false, p += 5, ok = true;
    } else if (t.compare(p, 4, "null") == 0) {
      out.kind = Json::Null, p += 4, ok = true;
    } else ok = number(out);
    --depth;
    return ok;
  }
  bool number(Json& out) {
    const size_t start = p;
    if (p < t.size() && t[p] == '-') ++p;
    if (p >= t.size() || t[p] < '0' || t[p] > '9') return fail("not a JSON value");
    while (p < t.size() && t[p] >= '0' && t[p] <= '9') ++p;
    if (p < t.size() && (t[p] == '.' || t[p] == 'e' || t[p] == 'E')) return fail("a plan holds integers only (no fractions or exponents)");
    const std::string digits = t.substr(start, p - start);
    if (digits.size() > 17) return fail("integer beyond 2**53");
    out.kind = Json::Int;
    out.i = std::stoll(digits);
    if (out.i > (1ll << 53) || out.i < -(1ll << 53)) return fail("integer beyond 2**53");
    return true;
  }
  bool string(std::string& out) {
    ++p;  // opening quote
    out.clear();
    while (p < t.size() && t[p] != '"') {
      unsigned char c = (unsigned char)t[p++];
      if (c < 0x20) return fail("control character in a string");
      if (c != '\\') {
        out.push_back((char)c);
        continue;
      }
      if (p >= t.size()) return fail("unexpected end");
      const char e = t[p++];
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          if (p + 4 > t.size()) return fail("short \\u escape");
          unsigned cp = 0;
          for (int k = 0; k < 4; ++k) {
            const char h = t[p++];
            cp <<= 4;
            if (h >= '0' && h <= '9') cp |= h - '0';
            else if (h >= 'a' && h <= 'f') cp |= h - 'a' + 10;
            else if (h >= 'A' && h <= 'F') cp |= h - 'A' + 10;
            else return fail("bad \\u escape");
          }
          if (cp >= 0x80) return fail("non-ASCII text (names in a plan are ASCII identifiers)");
          out.push_back((char)cp);
          break;
        }
        default: return fail("bad escape");
      }
    }
    if (p >= t.size()) return fail("unterminated string");
    ++p;
    return true;
  }
  bool array(Json& out) {
    out.kind = Json::Arr;
    ++p;
    ws();
    if (p < t.size() && t[p] == ']') return ++p, true;
    for (;;) {
      out.a.emplace_back();
      if (!value(out.a.back())) return false;
      ws();
      if (p < t.size() && t[p] == ',') {
        ++p;
        continue;
      }
      if (p < t.size() && t[p] == ']') return ++p, true;
      return fail("expected , or ]");
    }
  }
  bool object(Json& out) {
    out.kind = Json::Obj;
    ++p;
    ws();
    if (p < t.size() && t[p] == '}') return ++p, true;
    for (;;) {
      ws();
      if (p >= t.size() || t[p] != '"') return fail("expected a key");
      std::string key;
      if (!string(key)) return false;
      if (out.get(key)) return fail("duplicate key '" + key + "'");
      ws();
      if (p >= t.size() || t[p] != ':') return fail("expected :");
      ++p;
      out.o.emplace_back(key, Json());
      if (!value(out.o.back().second)) return false;
      ws();
      if (p < t.size() && t[p] == ',') {
        ++p;
        continue;
      }
      if (p < t.size() && t[p] == '}') return ++p, true;
      return fail("expected , or }");
    }
  }
};

void canonical(const Json& v, std::string& out, const char* skip1 = nullptr, const char* skip2 = nullptr) {
  switch (v.kind) {
    case Json::Null: out += "null"; break;
    case Json::Bool: out += v.b ? "true" : "false"; break;
    case Json::Int: out += std::to_string(v.i); break;
    case Json::Str: {
      out.push_back('"');
      for (unsigned char c : v.s) {
        if (c == '"') out += "\\\"";
        else if (c == '\\') out += "\\\\";
        else if (c == '\n') out += "\\n";
        else if (c == '\r') out += "\\r";
        else if (c == '\t') out += "\\t";
        else if (c == '\b') out += "\\b";
        else if (c == '\f') out += "\\f";
        else if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else out.push_back((char)c);
      }
      out.push_back('"');
      break;
    }
    case Json::Arr: {
      out.push_back('[');
      for (size_t k = 0; k < v.a.size(); ++k) {
        if (k) out.push_back(',');
        canonical(v.a[k], out);
      }
      out.push_back(']');
      break;
    }
    case Json::Obj: {
      std::vector<const std::pair<std::string, Json>*> items;
      for (const auto& kv : v.o)
        if (!(skip1 && kv.first == skip1) && !(skip2 && kv.first == skip2)) items.push_back(&kv);
      std::sort(items.begin(), items.end(), [](auto* x, auto* y) { return x->first < y->first; });
      out.push_back('{');
      for (size_t k = 0; k < items.size(); ++k) {
        if (k) out.push_back(',');
        Json key;
        key.kind = Json::Str;
        key.s = items[k]->first;
        canonical(key, out);
        out.push_back(':');
        canonical(items[k]->second, out);
      }
      out.push_back('}');
      break;
    }
  }
}

// ---- SHA-256 ------------------------------------------------------------------------------------------------------------------------
std::string sha256_hex(const std::string& data) {
  static const uint32_t K[64] = {
      0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74,
      0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d,
      0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e,
      0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5,
      0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  std::string m = data;
  const uint64_t bits = (uint64_t)data.size() * 8;
  m.push_back((char)0x80);
  while (m.size() % 64 != 56) m.push_back(0);
  for (int k = 7; k >= 0; --k) m.push_back((char)(bits >> (8 * k)));
  auto rotr = [](uint32_t x, int n) { return (x >> n) | (x << (32 - n)); };
  for (size_t off = 0; off < m.size(); off += 64) {
    uint32_t w[64];
    for (int k = 0; k < 16; ++k)
      w[k] = ((uint32_t)(unsigned char)m[off + 4 * k] << 24) | ((uint32_t)(unsigned char)m[off + 4 * k + 1] << 16) | ((uint32_t)(unsigned char)m[off + 4 * k + 2] << 8) |
             (uint32_t)(unsigned char)m[off + 4 * k + 3];
    for (int k = 16; k < 64; ++k) {
      const uint32_t s0 = rotr(w[k - 15], 7) ^ rotr(w[k - 15], 18) ^ (w[k - 15] >> 3), s1 = rotr(w[k - 2], 17) ^ rotr(w[k - 2], 19) ^ (w[k - 2] >> 10);
      w[k] = w[k - 16] + s0 + w[k - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int k = 0; k < 64; ++k) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g), t1 = hh + S1 + ch + K[k] + w[k];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c), t2 = S0 + mj;
      hh = g, g = f, f = e, e = d + t1, d = c, c = b, b = a, a = t1 + t2;
    }
    h[0] += a, h[1] += b, h[2] += c, h[3] += d, h[4] += e, h[5] += f, h[6] += g, h[7] += hh;
  }
  char out[65];
  for (int k = 0; k < 8; ++k) snprintf(out + 8 * k, 9, "%08x", h[k]);
  return std::string(out, 64);
}

// ---- the plan model -----------------------------------------------------------------------------------------------------------------
int itemsize(const std::string& dtype) {
  if (dtype == "bf16" || dtype == "f16") return 2;
  if (dtype == "f32" || dtype == "i32") return 4;
  if (dtype == "i64") return 8;
  if (dtype == "u8" || dtype == "e4m3" || dtype == "e5m2") return 1;
  return 0;
}

struct Buffer {
  std::string name, role, dtype;
  std::vector<Json> shape;  // integers or affine expressions over the dimensions
  long long offset = -1;    // arena offset, -1 for an external
  long long bytes = 0;
};

struct Arg {
  std::string name, binding;
  bool has_view = false;
  std::vector<long long> vshape, vstrides;
  long long voffset = 0;
};

struct Step {
  std::string entry, kind, workspace;
  std::vector<Arg> args;
};

struct Entry {
  std::string symbol;
  std::string format, epilogue, q_format;
  uint32_t eps_bits = 0;
  long long workspace_bytes = 0;
};

struct Bucket {
  std::map<std::string, long long> values;
  std::vector<Step> steps;
};

// "M", "3*M", "2*M + 3": the affine forms the writer emits.
bool eval_affine(const std::string& text, const std::map<std::string, long long>& values, long long* out) {
  long long total = 0;
  std::string t;
  for (char c : text)
    if (c != ' ') t.push_back(c);
  size_t p = 0;
  while (p < t.size()) {
    long long sign = 1;
    if (t[p] == '+') ++p;
    else if (t[p] == '-') sign = -1, ++p;
    long long coef = 1, dim = 1;
    bool any = false;
    for (;;) {
      size_t q = p;
      while (q < t.size() && (isalnum((unsigned char)t[q]) || t[q] == '_')) ++q;
      if (q == p) return false;
      const std::string f = t.substr(p, q - p);
      if (isdigit((unsigned char)f[0])) coef *= std::stoll(f);
      else {
        auto it = values.find(f);
        if (it == values.end()) return false;
        dim *= it->second;
      }
      any = true;
      p = q;
      if (p < t.size() && t[p] == '*') {
        ++p;
        continue;
      }
      break;
    }
    if (!any) return false;
    total += sign * coef * dim;
  }
  *out = total;
  return true;
}

}  // namespace

struct PlanImpl {
  std::string graph, digest;
  long long arena_bytes = 0;
  std::vector<Buffer> buffers;
  std::map<std::string, int> buffer_index;
  std::vector<std::string> dim_names;
  std::vector<Bucket> buckets;
  std::map<std::string, Entry> kernels, library;
  // instantiation
  void* arena = nullptr;
  bool owns_arena = false;
  std::map<std::string, void*> bound;
  std::vector<cudaGraphExec_t> graphs;
};

namespace {

tf_status read_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_load: cannot read %s", path.c_str());
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  if (out->size() > (256u << 20)) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_load: %s is larger than 256 MiB", path.c_str());
  return TF_OK;
}

#define TF_PLAN_REQUIRE(cond, ...) \
  do {                             \
    if (!(cond)) return fail(TF_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

const Json* field(const Json& o, const char* key, Json::Kind kind) {
  const Json* v = o.get(key);
  return (v && v->kind == kind) ? v : nullptr;
}

tf_status parse_entries(const Json& section, std::map<std::string, Entry>* out, const char* what) {
  for (const auto& kv : section.o) {
    const Json& e = kv.second;
    Entry en;
    const Json* sym = field(e, "symbol", Json::Str);
    const Json* attrs = field(e, "attrs", Json::Obj);
    TF_PLAN_REQUIRE(sym && attrs, "tf_plan_load: manifest %s entry '%s' lacks symbol / attrs", what, kv.first.c_str());
    en.symbol = sym->s;
    if (const Json* v = field(*attrs, "format", Json::Str)) en.format = v->s;
    if (const Json* v = field(*attrs, "epilogue", Json::Str)) en.epilogue = v->s;
    if (const Json* v = field(*attrs, "q_format", Json::Str)) en.q_format = v->s;
    if (const Json* v = field(*attrs, "eps_bits", Json::Int)) en.eps_bits = (uint32_t)v->i;
    if (const Json* v = field(e, "workspace_bytes", Json::Int)) en.workspace_bytes = v->i;
    (*out)[kv.first] = en;
  }
  return TF_OK;
}

int format_id(const std::string& f) { return f == "mxfp8" ? TF_FMT_MXFP8 : f == "mxfp4" ? TF_FMT_MXFP4 : f == "nvfp4" ? TF_FMT_NVFP4 : -1; }
int epilogue_id(const std::string& e) { return e == "silu_gate" ? TF_EPI_SILU_GATE : e == "residual" ? TF_EPI_RESIDUAL : TF_EPI_NONE; }

struct BoundArg {
  void* ptr = nullptr;
  std::vector<long long> shape, strides;
  long long nbytes = 0;
  bool present = false;
};

}  // namespace
}  // namespace tf

using namespace tf;

struct tf_plan {
  PlanImpl impl;
};

extern "C" {

tf_status tf_plan_load(const char* directory, const char* pin, tf_plan** out) {
  clear_error();
  TF_CHECK_ARG(directory && out, "%s: null pointer", __func__);
  *out = nullptr;
  std::string text, mtext;
  tf_status st = read_file(std::string(directory) + "/plan.json", &text);
  if (st != TF_OK) return st;
  st = read_file(std::string(directory) + "/manifest.json", &mtext);
  if (st != TF_OK) return st;
  Json doc, man;
  JsonReader r(text);
  if (!r.value(doc) || (r.ws(), r.p != text.size()) || doc.kind != Json::Obj)
    return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_load: plan.json is not strict JSON: %s", r.err.empty() ? "trailing data" : r.err.c_str());
  const Json* schema = field(doc, "schema", Json::Str);
  TF_PLAN_REQUIRE(schema && schema->s == "tilefish.plan.v1", "tf_plan_load: not a tilefish plan of schema 'tilefish.plan.v1'");
  // the digest: sha256("tilefish.plan-digest.v1\0" + canonical JSON of the document without plan_digest and tilefish)
  std::string body("tilefish.plan-digest.v1");
  body.push_back('\0');
  canonical(doc, body, "plan_digest", "tilefish");
  const std::string got = sha256_hex(body);
  const Json* stated = field(doc, "plan_digest", Json::Str);
  if (pin && got != pin) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_load: plan.json has digest %s, but the pin is %s", got.c_str(), pin);
  TF_PLAN_REQUIRE(stated && stated->s == got, "tf_plan_load: plan.json was edited: its plan_digest says %s, its content %s", stated ? stated->s.c_str() : "(none)", got.c_str());
  {
    // the manifest holds no number but integers either, so the same reader and writer give its digest
    JsonReader mr(mtext);
    if (!mr.value(man) || man.kind != Json::Obj) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_load: manifest.json is not strict JSON: %s", mr.err.c_str());
    std::string mbody("tilefish.manifest-digest.v1");
    mbody.push_back('\0');
    canonical(man, mbody, "manifest_digest");
    const Json* md = field(man, "manifest_digest", Json::Str);
    const Json* pmd = field(doc, "manifest_digest", Json::Str);
    TF_PLAN_REQUIRE(md && sha256_hex(mbody) == md->s, "tf_plan_load: manifest.json does not match its own digest");
    TF_PLAN_REQUIRE(pmd && pmd->s == md->s, "tf_plan_load: plan.json was built against another manifest");
  }
  std::unique_ptr<tf_plan> plan(new tf_plan());
  PlanImpl& P = plan->impl;
  P.digest = got;
  const Json* graph = field(doc, "graph", Json::Str);
  const Json* arena = field(doc, "arena_bytes", Json::Int);
  const Json* dims = field(doc, "dims", Json::Obj);
  const Json* buffers = field(doc, "buffers", Json::Arr);
  const Json* buckets = field(doc, "buckets", Json::Arr);
  TF_PLAN_REQUIRE(graph && arena && dims && buffers && buckets, "tf_plan_load: plan.json lacks graph / arena_bytes / dims / buffers / buckets");
  P.graph = graph->s;
  P.arena_bytes = arena->i;
  for (const auto& kv : dims->o) P.dim_names.push_back(kv.first);
  for (const Json& b : buffers->a) {
    Buffer buf;
    const Json *name = field(b, "name", Json::Str), *role = field(b, "role", Json::Str), *dtype = field(b, "dtype", Json::Str), *shape = field(b, "shape", Json::Arr),
               *bytes = field(b, "bytes", Json::Int);
    TF_PLAN_REQUIRE(name && role && dtype && shape && bytes && itemsize(dtype->s) > 0, "tf_plan_load: a buffer lacks name / role / dtype / shape / bytes");
    buf.name = name->s, buf.role = role->s, buf.dtype = dtype->s, buf.shape = shape->a, buf.bytes = bytes->i;
    if (const Json* off = field(b, "offset", Json::Int)) {
      buf.offset = off->i;
      TF_PLAN_REQUIRE(buf.offset % 256 == 0 && buf.offset + buf.bytes <= P.arena_bytes, "tf_plan_load: buffer '%s' does not lie inside the arena", buf.name.c_str());
    }
    TF_PLAN_REQUIRE(!P.buffer_index.count(buf.name), "tf_plan_load: buffer name '%s' is used twice", buf.name.c_str());
    P.buffer_index[buf.name] = (int)P.buffers.size();
    P.buffers.push_back(buf);
  }
  for (const Json& b : buckets->a) {
    Bucket bk;
    const Json *values = field(b, "values", Json::Obj), *steps = field(b, "steps", Json::Arr);
    TF_PLAN_REQUIRE(values && steps, "tf_plan_load: a bucket lacks values / steps");
    for (const auto& kv : values->o) {
      TF_PLAN_REQUIRE(kv.second.kind == Json::Int, "tf_plan_load: a bucket value is not an integer");
      bk.values[kv.first] = kv.second.i;
    }
    for (const Json& s : steps->a) {
      Step stp;
      const Json *kind = field(s, "kind", Json::Str), *args = field(s, "args", Json::Arr);
      TF_PLAN_REQUIRE(kind && args, "tf_plan_load: a step lacks kind / args");
      stp.kind = kind->s;
      if (const Json* e = field(s, "entry", Json::Str)) stp.entry = e->s;
      if (const Json* w = field(s, "workspace", Json::Str)) stp.workspace = w->s;
      for (const Json& a : args->a) {
        Arg arg;
        const Json *name = field(a, "name", Json::Str), *binding = field(a, "binding", Json::Str);
        TF_PLAN_REQUIRE(name && binding && P.buffer_index.count(binding->s), "tf_plan_load: step '%s' binds an unknown buffer", stp.entry.c_str());
        arg.name = name->s, arg.binding = binding->s;
        if (const Json* v = field(a, "view", Json::Obj)) {
          const Json *vs = field(*v, "shape", Json::Arr), *vt = field(*v, "strides", Json::Arr), *vo = field(*v, "offset", Json::Int);
          TF_PLAN_REQUIRE(vs && vt && vo && vs->a.size() == vt->a.size(), "tf_plan_load: a malformed view in step '%s'", stp.entry.c_str());
          arg.has_view = true;
          for (const Json& x : vs->a) arg.vshape.push_back(x.i);
          for (const Json& x : vt->a) arg.vstrides.push_back(x.i);
          arg.voffset = vo->i;
        }
        stp.args.push_back(arg);
      }
      bk.steps.push_back(stp);
    }
    P.buckets.push_back(bk);
  }
  if (const Json* k = field(man, "kernels", Json::Obj)) {
    st = parse_entries(*k, &P.kernels, "kernels");
    if (st != TF_OK) return st;
  }
  if (const Json* l = field(man, "library", Json::Obj)) {
    st = parse_entries(*l, &P.library, "library");
    if (st != TF_OK) return st;
  }
  for (const Bucket& bk : P.buckets)
    for (const Step& s : bk.steps) {
      if (s.kind == "memset" || s.kind == "copy") continue;
      const auto& sec = s.kind == "library" ? P.library : P.kernels;
      TF_PLAN_REQUIRE(s.kind == "kernel" || s.kind == "library", "tf_plan_load: unknown step kind '%s'", s.kind.c_str());
      TF_PLAN_REQUIRE(sec.count(s.entry), "tf_plan_load: step '%s' is not an entry of the manifest's %s section", s.entry.c_str(), s.kind.c_str());
      if (s.kind == "library") TF_PLAN_REQUIRE(P.buffer_index.count(s.workspace), "tf_plan_load: library step '%s' names no workspace buffer", s.entry.c_str());
    }
  *out = plan.release();
  return TF_OK;
}

void tf_plan_free(tf_plan* plan) {
  if (!plan) return;
  for (cudaGraphExec_t g : plan->impl.graphs) cudaGraphExecDestroy(g);
  if (plan->impl.owns_arena && plan->impl.arena) cudaFree(plan->impl.arena);
  delete plan;
}

const char* tf_plan_digest(const tf_plan* plan) { return plan ? plan->impl.digest.c_str() : ""; }
int64_t tf_plan_arena_bytes(const tf_plan* plan) { return plan ? plan->impl.arena_bytes : -1; }
int32_t tf_plan_step_count(const tf_plan* plan, int32_t bucket) {
  if (!plan || bucket < 0 || bucket >= (int32_t)plan->impl.buckets.size()) return -1;
  return (int32_t)plan->impl.buckets[bucket].steps.size();
}

int32_t tf_plan_find_bucket(const tf_plan* plan, const char* const* dim_names, const int64_t* values, int32_t n) {
  if (!plan || n < 0 || (n > 0 && (!dim_names || !values))) return -1;
  const PlanImpl& P = plan->impl;
  for (size_t b = 0; b < P.buckets.size(); ++b) {
    if ((int32_t)P.buckets[b].values.size() != n) continue;
    bool ok = true;
    for (int32_t k = 0; k < n && ok; ++k) {
      auto it = P.buckets[b].values.find(dim_names[k]);
      ok = it != P.buckets[b].values.end() && it->second == values[k];
    }
    if (ok) return (int32_t)b;
  }
  return -1;
}

tf_status tf_plan_instantiate(tf_plan* plan, void* arena, int64_t arena_bytes) {
  clear_error();
  TF_CHECK_ARG(plan, "%s: null plan", __func__);
  PlanImpl& P = plan->impl;
  TF_CHECK_ARG(!P.arena, "%s: the plan is already instantiated", __func__);
  if (arena) {
    TF_CHECK_ARG(arena_bytes >= P.arena_bytes, "%s: the arena holds %lld bytes, the plan needs %lld", __func__, (long long)arena_bytes, (long long)P.arena_bytes);
    TF_CHECK_ALIGNED(arena, 256, "arena");
    P.arena = arena;
    return TF_OK;
  }
  void* p = nullptr;
  TF_CUDA(cudaMalloc(&p, (size_t)std::max<long long>(P.arena_bytes, 256)));
  P.arena = p;
  P.owns_arena = true;
  return TF_OK;
}

tf_status tf_plan_bind(tf_plan* plan, const char* buffer, void* device_ptr) {
  clear_error();
  TF_CHECK_ARG(plan && buffer, "%s: null pointer", __func__);
  PlanImpl& P = plan->impl;
  auto it = P.buffer_index.find(buffer);
  TF_CHECK_ARG(it != P.buffer_index.end(), "%s: the plan has no buffer '%s'", __func__, buffer);
  TF_CHECK_ARG(P.buffers[it->second].offset < 0, "%s: buffer '%s' lives in the arena; only the caller's tensors are bound", __func__, buffer);
  P.bound[buffer] = device_ptr;
  return TF_OK;
}

static tf_status run_bucket(PlanImpl& P, int bucket, cudaStream_t stream, bool dry) {
  const Bucket& bk = P.buckets[bucket];
  // shapes of every buffer at this bucket
  std::map<std::string, std::vector<long long>> shapes;
  for (const Buffer& b : P.buffers) {
    std::vector<long long> s;
    for (const Json& e : b.shape) {
      long long v = 0;
      if (e.kind == Json::Int) v = e.i;
      else if (e.kind != Json::Str || !eval_affine(e.s, bk.values, &v)) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: shape of '%s' cannot be evaluated", b.name.c_str());
      s.push_back(v);
    }
    shapes[b.name] = s;
  }
  auto address = [&](const std::string& name, void** out) -> tf_status {
    const Buffer& b = P.buffers[P.buffer_index[name]];
    if (b.offset >= 0) {
      *out = static_cast<char*>(P.arena) + b.offset;
      return TF_OK;
    }
    auto it = P.bound.find(name);
    if (it == P.bound.end() || !it->second) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: no tensor is bound to buffer '%s'", name.c_str());
    *out = it->second;
    return TF_OK;
  };
  for (const Step& s : bk.steps) {
    std::map<std::string, BoundArg> a;
    for (const Arg& arg : s.args) {
      const Buffer& b = P.buffers[P.buffer_index[arg.binding]];
      BoundArg ba;
      void* base = nullptr;
      tf_status st = address(arg.binding, &base);
      if (st != TF_OK) return st;
      const int isz = itemsize(b.dtype);
      if (arg.has_view) {
        ba.shape = arg.vshape, ba.strides = arg.vstrides;
        ba.ptr = static_cast<char*>(base) + arg.voffset * isz;
      } else {
        ba.shape = shapes[arg.binding];
        ba.strides.assign(ba.shape.size(), 1);
        for (int k = (int)ba.shape.size() - 2; k >= 0; --k) ba.strides[k] = ba.strides[k + 1] * ba.shape[k + 1];
        ba.ptr = base;
      }
      long long n = 1;
      for (long long x : ba.shape) n *= x;
      ba.nbytes = n * isz;
      ba.present = true;
      const uintptr_t align = (n == 1) ? 4 : 16;
      if (reinterpret_cast<uintptr_t>(ba.ptr) % align) return fail(TF_ERR_ALIGNMENT, "tf_plan_launch: step '%s': the pointer of '%s' is not %d-byte aligned", s.entry.c_str(), arg.name.c_str(), (int)align);
      a[arg.name] = ba;
    }
    auto ptr = [&](const char* n) -> void* { auto it = a.find(n); return it == a.end() ? nullptr : it->second.ptr; };
    if (s.kind == "memset") {
      if (!a.count("dst")) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: a memset step has no dst");
      if (!dry) TF_CUDA(cudaMemsetAsync(a["dst"].ptr, 0, (size_t)a["dst"].nbytes, stream));
      continue;
    }
    if (s.kind == "copy") {
      if (!a.count("dst") || !a.count("src") || a["dst"].nbytes != a["src"].nbytes) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: a copy step needs src and dst of one size");
      if (!dry) TF_CUDA(cudaMemcpyAsync(a["dst"].ptr, a["src"].ptr, (size_t)a["src"].nbytes, cudaMemcpyDeviceToDevice, stream));
      continue;
    }
    const Entry& e = (s.kind == "library" ? P.library : P.kernels)[s.entry];
    tf_status st = TF_OK;
    if (s.kind == "library") {
      if (!a.count("a") || !a.count("b")) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: library step '%s' lacks its operands", s.entry.c_str());
      const int fmt = format_id(e.format), epi = epilogue_id(e.epilogue);
      if (fmt < 0) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: step '%s': unknown format '%s'", s.entry.c_str(), e.format.c_str());
      const int epb = fmt == TF_FMT_MXFP8 ? 1 : 2;
      const long long m = a["a"].shape[0], k = a["a"].shape[1] * epb, nrows = a["b"].shape[0], n = epi == TF_EPI_SILU_GATE ? nrows / 2 : nrows;
      const Buffer& ws = P.buffers[P.buffer_index[s.workspace]];
      const long long need = tf_gemm_workspace_bytes(m, n, k, fmt, epi);
      if (need > ws.bytes)
        return fail(TF_ERR_WORKSPACE, "tf_plan_launch: step '%s' needs %lld bytes of workspace on this device, the plan reserved %lld", s.entry.c_str(), need, ws.bytes);
      const long long ldo = (a.count("out") && m > 1) ? a["out"].strides[0] : n;
      if (!dry)
        st = tf_gemm_blockscaled(ptr("a"), ptr("a_scales"), static_cast<const float*>(ptr("a_global")), ptr("b"), ptr("b_scales"), static_cast<const float*>(ptr("b_global")),
                                 ptr("out"), ldo, m, n, k, fmt, epi, ptr("residual"), static_cast<float*>(ptr("amax")), ptr("q"), ptr("q_scales"), 0,
                                 static_cast<char*>(P.arena) + ws.offset, ws.bytes, stream);
    } else if (e.symbol == "tf_residual_add_rmsnorm") {
      if (!a.count("x")) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: step '%s' lacks x", s.entry.c_str());
      float eps;
      memcpy(&eps, &e.eps_bits, sizeof(eps));
      if (!dry)
        st = tf_residual_add_rmsnorm(ptr("x"), ptr("residual"), ptr("w"), ptr("out"), a["x"].shape[0], a["x"].shape[1], eps, e.q_format.empty() ? -1 : format_id(e.q_format), ptr("q"),
                                     ptr("q_scales"), TF_SCALES_SWIZZLED, static_cast<const float*>(ptr("q_global")), static_cast<float*>(ptr("amax")), stream);
    } else if (e.symbol == "tf_silu_gate") {
      if (!a.count("gate") || !a.count("up") || !a.count("out")) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: step '%s' lacks gate / up / out", s.entry.c_str());
      const long long m = a["gate"].shape[0], f = a["gate"].shape[1];
      if (!dry) st = tf_silu_gate(ptr("gate"), ptr("up"), m, f, m > 1 ? a["gate"].strides[0] : f, m > 1 ? a["up"].strides[0] : f, ptr("out"), m > 1 ? a["out"].strides[0] : f, stream);
    } else if (e.symbol == "tf_quantize_mxfp8" || e.symbol == "tf_quantize_mxfp4" || e.symbol == "tf_quantize_nvfp4") {
      if (!a.count("x") || !a.count("q")) return fail(TF_ERR_INVALID_ARGUMENT, "tf_plan_launch: step '%s' lacks x / q", s.entry.c_str());
      const long long m = a["x"].shape[0], k = a["x"].shape[1], ldx = m > 1 ? a["x"].strides[0] : k;
      if (dry) continue;
      if (e.symbol == "tf_quantize_mxfp8") st = tf_quantize_mxfp8(ptr("x"), m, k, ldx, ptr("q"), ptr("q_scales"), TF_SCALES_SWIZZLED, stream);
      else if (e.symbol == "tf_quantize_mxfp4") st = tf_quantize_mxfp4(ptr("x"), m, k, ldx, ptr("q"), ptr("q_scales"), TF_SCALES_SWIZZLED, stream);
      else if (a.count("amax"))
        st = tf_quantize_nvfp4_from_amax(ptr("x"), m, k, ldx, ptr("q"), ptr("q_scales"), TF_SCALES_SWIZZLED, static_cast<const float*>(ptr("amax")), static_cast<float*>(ptr("q_global")), stream);
      else {
        st = tf_nvfp4_global_scale(ptr("x"), m, k, ldx, static_cast<float*>(ptr("q_global")), stream);
        if (st == TF_OK) st = tf_quantize_nvfp4(ptr("x"), m, k, ldx, ptr("q"), ptr("q_scales"), TF_SCALES_SWIZZLED, static_cast<const float*>(ptr("q_global")), stream);
      }
    } else {
      return fail(TF_ERR_UNSUPPORTED, "tf_plan_launch: step '%s': unknown entry point %s", s.entry.c_str(), e.symbol.c_str());
    }
    if (st != TF_OK) return st;
  }
  return TF_OK;
}

tf_status tf_plan_launch(tf_plan* plan, int32_t bucket, void* stream) {
  clear_error();
  TF_CHECK_ARG(plan, "%s: null plan", __func__);
  PlanImpl& P = plan->impl;
  TF_CHECK_ARG(bucket >= 0 && bucket < (int32_t)P.buckets.size(), "%s: the plan has %d buckets, not a bucket %d", __func__, (int)P.buckets.size(), bucket);
  TF_CHECK_ARG(P.arena, "%s: instantiate the plan first (tf_plan_instantiate)", __func__);
  // every step is resolved and checked with the real addresses before the first launch: a refusal launches nothing
  tf_status st = run_bucket(P, bucket, (cudaStream_t)stream, true);
  if (st != TF_OK) return st;
  return run_bucket(P, bucket, (cudaStream_t)stream, false);
}

tf_status tf_plan_capture(tf_plan* plan, int32_t bucket, void* stream_, int32_t* graph_out) {
  clear_error();
  TF_CHECK_ARG(plan && graph_out, "%s: null pointer", __func__);
  PlanImpl& P = plan->impl;
  TF_CHECK_ARG(bucket >= 0 && bucket < (int32_t)P.buckets.size(), "%s: the plan has %d buckets, not a bucket %d", __func__, (int)P.buckets.size(), bucket);
  TF_CHECK_ARG(P.arena, "%s: instantiate the plan first (tf_plan_instantiate)", __func__);
  TF_CHECK_ARG(stream_ != nullptr, "%s: a capture needs a stream of its own, not the legacy default stream", __func__);
  cudaStream_t stream = (cudaStream_t)stream_;
  tf_status st = run_bucket(P, bucket, stream, true);
  if (st != TF_OK) return st;
  TF_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
  st = run_bucket(P, bucket, stream, false);
  cudaGraph_t graph = nullptr;
  const cudaError_t end = cudaStreamEndCapture(stream, &graph);
  if (st != TF_OK) {
    if (graph) cudaGraphDestroy(graph);
    return st;
  }
  if (end != cudaSuccess) return fail(TF_ERR_CUDA, "%s: cudaStreamEndCapture failed: %s", __func__, cudaGetErrorString(end));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (inst != cudaSuccess) return fail(TF_ERR_CUDA, "%s: cudaGraphInstantiate failed: %s", __func__, cudaGetErrorString(inst));
  P.graphs.push_back(exec);
  *graph_out = (int32_t)P.graphs.size() - 1;
  return TF_OK;
}

tf_status tf_plan_replay(tf_plan* plan, int32_t graph, void* stream) {
  clear_error();
  TF_CHECK_ARG(plan, "%s: null plan", __func__);
  PlanImpl& P = plan->impl;
  TF_CHECK_ARG(graph >= 0 && graph < (int32_t)P.graphs.size(), "%s: no captured graph %d", __func__, graph);
  TF_CUDA(cudaGraphLaunch(P.graphs[graph], (cudaStream_t)stream));
  return TF_OK;
}

}  // extern "C"
