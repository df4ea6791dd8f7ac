// Host side of the training driver that sits next to the hot path: checkpoint files, the learning-rate
// schedule and the metrics file, in the formats of the reference so that files move between the two.
//
//  * Checkpoint::save / ::load (cpp/src/Checkpoint.cpp:721-1040, 1045-1116): a pair of safetensors files in
//    the reference's "Python/MLX compatible" naming -- every projection stored transposed ([out, in]), Wq|Wk|Wv
//    fused into attention.wqkv.weight, gate|up into feed_forward.w12.weight, fp32 payloads, header padded
//    with spaces to 8 bytes; "<name>.opt.safetensors" holds a U64 "step" and <tensor>.m / <tensor>.v AdamW
//    moments (zeros for the norm weights, which the reference does not train).  Loading also accepts BF16 / F16
//    payloads (cpp/src/Checkpoint.cpp:409-466).
//  * Trainer::get_scheduled_lr (cpp/src/Trainer.cpp:40-51): linear warm-up, cosine decay to lr_min.
//  * metrics.csv (cpp/src/Trainer.cpp:136-170, 247-255, 347-365): header, resume truncation, one row per step.
//
// Everything here works on flat host arrays in the reference's per-tensor order (the order of
// b200_model_load_params); the b200_model_* forms move the data to and from the device-resident engine.
#include "../../include/b200_bridge.h"
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

namespace {

struct Part { size_t ref_off, rows, cols; };          // a [rows(in), cols(out)] matrix of the flat layout
struct Spec {
  std::string name;
  std::vector<size_t> shape;
  std::vector<Part> parts;                            // one part; several when fused along the output dimension
  bool transpose = false;                             // stored as [out, in]
  bool norm = false;                                  // not trained: zero moments
  size_t elems() const { size_t n = 1; for (size_t d : shape) n *= d; return n; }
};

struct Dims { size_t V, H, I, L, Q, KV, lp, total; };
Dims dims(const b200_model_config *c) {
  Dims d;
  d.V = c->vocab_size; d.H = c->hidden_dim; d.I = c->intermediate_dim; d.L = c->n_layers;
  d.Q = c->n_heads * c->head_dim; d.KV = c->n_kv_heads * c->head_dim;
  d.lp = 2 * d.H + d.H * (d.Q + 2 * d.KV) + d.Q * d.H + 3 * d.H * d.I;
  d.total = 2 * d.V * d.H + d.L * d.lp + d.H;
  return d;
}

// Tensors of the model file in file order (cpp/src/Checkpoint.cpp:725-830).
std::vector<Spec> model_specs(const Dims &d) {
  std::vector<Spec> v;
  const size_t H = d.H, I = d.I, Q = d.Q, KV = d.KV;
  const size_t off_final = d.V * H + d.L * d.lp, off_out = off_final + H;
  v.push_back({"tok_embeddings.weight", {d.V, H}, {{0, d.V, H}}, false, false});
  v.push_back({"output.weight", {d.V, H}, {{off_out, H, d.V}}, true, false});
  v.push_back({"norm.weight", {H}, {{off_final, 1, H}}, false, true});
  for (size_t l = 0; l < d.L; ++l) {
    const std::string p = "layers." + std::to_string(l) + ".";
    size_t o = d.V * H + l * d.lp;
    const size_t attn_norm = o; o += H;
    const size_t wq = o; o += H * Q;
    const size_t wk = o; o += H * KV;
    const size_t wv = o; o += H * KV;
    const size_t wo = o; o += Q * H;
    const size_t ffn_norm = o; o += H;
    const size_t gate = o; o += H * I;
    const size_t up = o; o += H * I;
    const size_t down = o;
    v.push_back({p + "attention_norm.weight", {H}, {{attn_norm, 1, H}}, false, true});
    v.push_back({p + "ffn_norm.weight", {H}, {{ffn_norm, 1, H}}, false, true});
    v.push_back({p + "attention.wo.weight", {H, Q}, {{wo, Q, H}}, true, false});
    v.push_back({p + "feed_forward.w3.weight", {H, I}, {{down, I, H}}, true, false});
    v.push_back({p + "attention.wqkv.weight", {Q + 2 * KV, H}, {{wq, H, Q}, {wk, H, KV}, {wv, H, KV}}, true, false});
    v.push_back({p + "feed_forward.w12.weight", {2 * I, H}, {{gate, H, I}, {up, H, I}}, true, false});
  }
  return v;
}
// Order of the moments in the optimizer file (cpp/src/Checkpoint.cpp:860-1036): per layer the two norms come
// first and in the opposite order, then w3, wo, wqkv, w12.
std::vector<Spec> opt_specs(const Dims &d) {
  std::vector<Spec> m = model_specs(d), v;
  v.push_back(m[0]); v.push_back(m[1]); v.push_back(m[2]);
  for (size_t l = 0; l < d.L; ++l) {
    const Spec *s = &m[3 + l * 6];
    v.push_back(s[1]); v.push_back(s[0]); v.push_back(s[3]); v.push_back(s[2]); v.push_back(s[4]); v.push_back(s[5]);
  }
  return v;
}

void transpose_into(const float *src, size_t rows, size_t cols, float *dst) {     // dst[c][r] = src[r][c]
  constexpr size_t T = 32;
#pragma omp parallel for collapse(2) schedule(static)
  for (size_t r0 = 0; r0 < rows; r0 += T)
    for (size_t c0 = 0; c0 < cols; c0 += T) {
      const size_t r1 = r0 + T < rows ? r0 + T : rows, c1 = c0 + T < cols ? c0 + T : cols;
      for (size_t r = r0; r < r1; ++r)
        for (size_t c = c0; c < c1; ++c) dst[c * rows + r] = src[r * cols + c];
    }
}

// flat -> file bytes of one tensor
void pack(const Spec &s, const float *flat, std::vector<float> &out) {
  out.resize(s.elems());
  float *dst = out.data();
  for (const Part &p : s.parts) {
    if (s.transpose) transpose_into(flat + p.ref_off, p.rows, p.cols, dst);
    else memcpy(dst, flat + p.ref_off, p.rows * p.cols * sizeof(float));
    dst += p.rows * p.cols;
  }
}
// file floats of one tensor -> flat
void unpack(const Spec &s, const float *src, float *flat) {
  for (const Part &p : s.parts) {
    if (s.transpose) transpose_into(src, p.cols, p.rows, flat + p.ref_off);        // file holds [cols, rows]
    else memcpy(flat + p.ref_off, src, p.rows * p.cols * sizeof(float));
    src += p.rows * p.cols;
  }
}

struct Entry { std::string name, dtype; std::vector<size_t> shape; size_t bytes; };

std::string header_json(const std::vector<Entry> &es) {
  std::string j = "{\"__metadata__\":{\"format\":\"pt\"}";
  size_t off = 0;
  for (const Entry &e : es) {
    j += ",\"" + e.name + "\":{\"dtype\":\"" + e.dtype + "\",\"shape\":[";
    for (size_t i = 0; i < e.shape.size(); ++i) { j += std::to_string(e.shape[i]); if (i + 1 < e.shape.size()) j += ","; }
    j += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + e.bytes) + "]}";
    off += e.bytes;
  }
  j += "}";
  j.append((8 - j.size() % 8) % 8, ' ');
  return j;
}

bool write_header(std::ofstream &out, const std::vector<Entry> &es) {
  const std::string j = header_json(es);
  const uint64_t n = j.size();
  out.write(reinterpret_cast<const char *>(&n), 8);
  out.write(j.data(), (std::streamsize)j.size());
  return out.good();
}

std::string opt_path_of(const std::string &path) {
  std::string p = path;
  const size_t pos = p.find(".safetensors");
  if (pos != std::string::npos) p.replace(pos, 12, ".opt.safetensors"); else p += ".opt.safetensors";
  return p;
}

// ---- reading ---------------------------------------------------------------------------------
struct Found { size_t start = 0, end = 0; std::string dtype = "F32"; std::vector<size_t> shape; };

bool read_header(std::ifstream &in, std::string &json, size_t &payload) {
  uint64_t n = 0;
  in.read(reinterpret_cast<char *>(&n), 8);
  if (!in.good() || n == 0 || n > (1ull << 30)) return false;
  json.resize(n);
  in.read(&json[0], (std::streamsize)n);
  payload = 8 + n;
  return in.good();
}
// Same tolerant lookup as the reference (cpp/src/Checkpoint.cpp:229-298): locate "name", then the next dtype / shape /
// data_offsets fields after it.
bool find_tensor(const std::string &json, const std::string &name, Found &f) {
  const size_t at = json.find("\"" + name + "\"");
  if (at == std::string::npos) return false;
  size_t p = json.find("\"dtype\"", at);
  if (p != std::string::npos) {
    const size_t q0 = json.find('"', json.find(':', p)), q1 = json.find('"', q0 + 1);
    if (q0 != std::string::npos && q1 != std::string::npos) f.dtype = json.substr(q0 + 1, q1 - q0 - 1);
  }
  p = json.find("\"shape\"", at);
  if (p != std::string::npos) {
    const size_t b0 = json.find('[', p), b1 = json.find(']', p);
    f.shape.clear();
    if (b0 != std::string::npos && b1 != std::string::npos && b0 < b1) {
      const std::string s = json.substr(b0 + 1, b1 - b0 - 1);
      size_t i = 0;
      while (i < s.size()) {
        size_t c = s.find(',', i);
        const std::string tok = s.substr(i, c == std::string::npos ? std::string::npos : c - i);
        if (tok.find_first_of("0123456789") != std::string::npos) f.shape.push_back(std::stoull(tok));
        if (c == std::string::npos) break;
        i = c + 1;
      }
    }
  }
  p = json.find("\"data_offsets\"", at);
  if (p == std::string::npos) return false;
  const size_t b0 = json.find('[', p), b1 = json.find(']', p);
  if (b0 == std::string::npos || b1 == std::string::npos || b0 > b1) return false;
  const std::string s = json.substr(b0 + 1, b1 - b0 - 1);
  const size_t c = s.find(',');
  if (c == std::string::npos) return false;
  f.start = std::stoull(s.substr(0, c)); f.end = std::stoull(s.substr(c + 1));
  return f.end >= f.start;
}

float bf16_to_f32(uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; }
float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else { int e = -1; do { ++e; man <<= 1; } while (!(man & 0x400)); u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13); }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f; memcpy(&f, &u, 4); return f;
}

// Reads tensor `s` (any of F32 / BF16 / F16) into `vals` as floats; checks the element count.
bool read_tensor(std::ifstream &in, size_t payload, const std::string &json, const std::string &name, size_t elems,
                 std::vector<float> &vals, std::string &err) {
  Found f;
  if (!find_tensor(json, name, f)) { err = "tensor '" + name + "' not found in the header"; return false; }
  const size_t bytes = f.end - f.start, es = (f.dtype == "BF16" || f.dtype == "F16") ? 2 : 4;
  if (f.dtype != "F32" && f.dtype != "BF16" && f.dtype != "F16") { err = "tensor '" + name + "' has unsupported dtype " + f.dtype; return false; }
  if (bytes != elems * es) { err = "tensor '" + name + "' has " + std::to_string(bytes / es) + " elements, expected " + std::to_string(elems); return false; }
  in.clear();
  in.seekg((std::streamoff)(payload + f.start));
  vals.resize(elems);
  if (es == 4) in.read(reinterpret_cast<char *>(vals.data()), (std::streamsize)bytes);
  else {
    std::vector<uint16_t> raw(elems);
    in.read(reinterpret_cast<char *>(raw.data()), (std::streamsize)bytes);
    const bool bf = f.dtype == "BF16";
    for (size_t i = 0; i < elems; ++i) vals[i] = bf ? bf16_to_f32(raw[i]) : f16_to_f32(raw[i]);
  }
  if (!in.good()) { err = "short read of tensor '" + name + "'"; return false; }
  return true;
}

thread_local std::string g_err;
int fail(const std::string &e) { g_err = e; return B200_ERR_INVALID; }

}  // namespace

extern "C" const char *b200_checkpoint_last_error(void) { return g_err.c_str(); }

extern "C" size_t b200_checkpoint_param_count(const b200_model_config *cfg) { return cfg ? dims(cfg).total : 0; }

extern "C" int b200_checkpoint_write_flat(const b200_model_config *cfg, const float *params, const float *adam_m,
                                          const float *adam_v, uint64_t step, const char *path) {
  if (!cfg || !params || !path) return fail("checkpoint_write: null argument");
  const Dims d = dims(cfg);
  {
    const std::vector<Spec> specs = model_specs(d);
    std::vector<Entry> es;
    for (const Spec &s : specs) es.push_back({s.name, "F32", s.shape, s.elems() * 4});
    std::ofstream out(path, std::ios::binary);
    if (!out.is_open() || !write_header(out, es)) return fail(std::string("cannot write ") + path);
    std::vector<float> buf;
    for (const Spec &s : specs) { pack(s, params, buf); out.write(reinterpret_cast<const char *>(buf.data()), (std::streamsize)(buf.size() * 4)); }
    if (!out.good()) return fail(std::string("write failed: ") + path);
  }
  if (adam_m && adam_v) {
    const std::vector<Spec> specs = opt_specs(d);
    std::vector<Entry> es;
    es.push_back({"step", "U64", {}, 8});
    for (const Spec &s : specs) { es.push_back({s.name + ".m", "F32", s.shape, s.elems() * 4}); es.push_back({s.name + ".v", "F32", s.shape, s.elems() * 4}); }
    const std::string op = opt_path_of(path);
    std::ofstream out(op, std::ios::binary);
    if (!out.is_open() || !write_header(out, es)) return fail("cannot write " + op);
    out.write(reinterpret_cast<const char *>(&step), 8);
    std::vector<float> buf;
    for (const Spec &s : specs) {
      for (const float *src : {adam_m, adam_v}) {
        if (s.norm) buf.assign(s.elems(), 0.0f); else pack(s, src, buf);
        out.write(reinterpret_cast<const char *>(buf.data()), (std::streamsize)(buf.size() * 4));
      }
    }
    if (!out.good()) return fail("write failed: " + op);
  }
  return B200_OK;
}

extern "C" int b200_checkpoint_read_flat(const b200_model_config *cfg, const char *path, float *params, float *adam_m,
                                         float *adam_v, uint64_t *step, int *has_opt_state) {
  if (!cfg || !params || !path) return fail("checkpoint_read: null argument");
  const Dims d = dims(cfg);
  std::string err;
  {
    std::ifstream in(path, std::ios::binary);
    std::string json; size_t payload = 0;
    if (!in.is_open() || !read_header(in, json, payload)) return fail(std::string("cannot read ") + path);
    if (json.find("\"tok_embeddings.weight\"") == std::string::npos)
      return fail("not a checkpoint in the Python/MLX tensor naming (tok_embeddings.weight missing)");
    std::vector<float> vals;
    for (const Spec &s : model_specs(d)) {
      if (!read_tensor(in, payload, json, s.name, s.elems(), vals, err)) return fail(err);
      unpack(s, vals.data(), params);
    }
  }
  if (has_opt_state) *has_opt_state = 0;
  if (step) *step = 0;
  if (adam_m && adam_v) {
    // a missing or unreadable optimizer file is not an error: moments restart from zero (cpp/src/Checkpoint.cpp:1076-1112)
    memset(adam_m, 0, d.total * 4); memset(adam_v, 0, d.total * 4);
    std::ifstream in(opt_path_of(path), std::ios::binary);
    std::string json; size_t payload = 0;
    if (in.is_open() && read_header(in, json, payload)) {
      bool ok = true;
      uint64_t st = 0;
      Found f;
      if (find_tensor(json, "step", f) && f.end - f.start == 8) {
        in.seekg((std::streamoff)(payload + f.start));
        in.read(reinterpret_cast<char *>(&st), 8);
        ok = in.good();
      }
      std::vector<float> vals;
      for (const Spec &s : opt_specs(d)) {
        if (!ok) break;
        if (s.norm) continue;
        ok = read_tensor(in, payload, json, s.name + ".m", s.elems(), vals, err);
        if (ok) { unpack(s, vals.data(), adam_m); ok = read_tensor(in, payload, json, s.name + ".v", s.elems(), vals, err); }
        if (ok) unpack(s, vals.data(), adam_v);
      }
      if (ok) { if (step) *step = st; if (has_opt_state) *has_opt_state = 1; }
      else { memset(adam_m, 0, d.total * 4); memset(adam_v, 0, d.total * 4); g_err = err; }
    }
  }
  return B200_OK;
}

extern "C" int b200_model_get_config(const b200_model *m, b200_model_config *out);   // model.cu

extern "C" int b200_checkpoint_save(b200_model *m, const char *path, uint64_t step_override, int with_optimizer) {
  b200_model_config cfg;
  if (!m || !path || b200_model_get_config(m, &cfg) != B200_OK) return fail("checkpoint_save: null argument");
  const size_t n = dims(&cfg).total;
  std::vector<float> p(n), mm, vv;
  int rc = b200_model_read_params(m, p.data());
  if (rc) return rc;
  uint64_t step = step_override;
  if (with_optimizer) {
    mm.resize(n); vv.resize(n);
    uint64_t st = 0;
    rc = b200_model_read_opt_state(m, mm.data(), vv.data(), &st);
    if (rc) return rc;
    if (step_override == (uint64_t)-1) step = st;
  }
  return b200_checkpoint_write_flat(&cfg, p.data(), with_optimizer ? mm.data() : nullptr, with_optimizer ? vv.data() : nullptr, step, path);
}

extern "C" int b200_checkpoint_load(b200_model *m, const char *path, int with_optimizer, uint64_t *step) {
  b200_model_config cfg;
  if (!m || !path || b200_model_get_config(m, &cfg) != B200_OK) return fail("checkpoint_load: null argument");
  const size_t n = dims(&cfg).total;
  std::vector<float> p(n), mm, vv;
  if (with_optimizer) { mm.resize(n); vv.resize(n); }
  uint64_t st = 0; int has = 0;
  int rc = b200_checkpoint_read_flat(&cfg, path, p.data(), with_optimizer ? mm.data() : nullptr, with_optimizer ? vv.data() : nullptr, &st, &has);
  if (rc) return rc;
  rc = b200_model_load_params(m, p.data());
  if (rc) return rc;
  if (with_optimizer) {
    rc = b200_model_load_opt_state(m, mm.data(), vv.data(), has ? st : 0);
    if (rc) return rc;
  }
  if (step) *step = has ? st : 0;
  return B200_OK;
}

// ---- learning-rate schedule (cpp/src/Trainer.cpp:40-51) ---------------------------------------------
extern "C" float b200_scheduled_lr(size_t step, size_t warmup_steps, size_t max_steps, float lr_max, float lr_min) {
  if (step < warmup_steps) return lr_max * static_cast<float>(step) / static_cast<float>(warmup_steps);
  if (step >= max_steps) return lr_min;
  const float ratio = static_cast<float>(step - warmup_steps) / static_cast<float>(max_steps - warmup_steps);
  const float cos_decay = 0.5f * (1.0f + std::cos(3.1415926535f * ratio));
  return lr_min + cos_decay * (lr_max - lr_min);
}

// ---- metrics.csv ------------------------------------------------------------------------------------
static const char *METRICS_HEADER =
    "step,train_loss,tokens_per_sec,learning_rate,vram_usage_gb,mfu_pct,step_time_ms,gpu_calls,gpu_time_ms,cpu_calls,"
    "cpu_time_ms,gpu_active_pct";

// Fresh file with the header when start_step == 0 or the file is missing; otherwise rows with step >= start_step
// are dropped (resume, cpp/src/Trainer.cpp:136-170, 247-255).
extern "C" int b200_metrics_begin(const char *path, size_t start_step) {
  if (!path) return fail("metrics_begin: null path");
  std::vector<std::string> keep;
  bool existed = false;
  {
    std::ifstream in(path);
    if (in.is_open()) {
      existed = true;
      std::string line;
      if (std::getline(in, line)) keep.push_back(line);
      while (std::getline(in, line)) {
        if (line.empty()) continue;
        const size_t c = line.find(',');
        if (c == std::string::npos || c == 0 || line.substr(0, c).find_first_not_of("0123456789") != std::string::npos) continue;
        if (std::stoull(line.substr(0, c)) < start_step) keep.push_back(line);
      }
    }
  }
  std::ofstream out(path);
  if (!out.is_open()) return fail(std::string("cannot write ") + path);
  if (start_step == 0 || !existed || keep.empty()) out << METRICS_HEADER << "\n";
  else for (const std::string &l : keep) out << l << "\n";
  return out.good() ? B200_OK : fail(std::string("write failed: ") + path);
}

extern "C" int b200_metrics_append(const char *path, size_t step, double train_loss, double tokens_per_sec,
                                   double learning_rate, double vram_usage_gb, double mfu_pct, double step_time_ms,
                                   uint64_t gpu_calls, double gpu_time_ms, uint64_t cpu_calls, double cpu_time_ms,
                                   double gpu_active_pct) {
  if (!path) return fail("metrics_append: null path");
  std::ofstream out(path, std::ios::app);
  if (!out.is_open()) return fail(std::string("cannot append to ") + path);
  // default ostream formatting of the reference: %g with 6 significant digits
  out << step << "," << train_loss << "," << tokens_per_sec << "," << learning_rate << "," << vram_usage_gb << ","
      << mfu_pct << "," << step_time_ms << "," << gpu_calls << "," << gpu_time_ms << "," << cpu_calls << ","
      << cpu_time_ms << "," << gpu_active_pct << "\n";
  return out.good() ? B200_OK : fail(std::string("write failed: ") + path);
}
