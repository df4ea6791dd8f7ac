// Drop-in implementation of the reference engine's backend interface (`namespace metal_bridge`,
// cpp/include/gpu_kernel/MetalBridge.hpp:14-147) on top of the B200 C ABI (include/b200_bridge.h).
// Build it INSTEAD of cpp/src/gpu_kernel/MetalBridge.mm and link libb200bridge.so; the reference's
// Tensor / Attention / Transformer / Loss / Optimizer sources then run on the CUDA kernels unchanged.
//
// Calling convention kept from the reference (cpp/src/gpu_kernel/MetalBridge.mm:778-833, 2176-2225):
//   - every pointer is a HOST pointer owned by the caller;
//   - inside begin_scope()/end_scope() ops are only enqueued; a buffer produced by one op and
//     consumed by the next stays on the device; end_scope() copies results back and waits once;
//   - outside a scope each op copies back and waits before returning;
//   - failures are reported on std::cerr and the call returns (outputs untouched), as the
//     reference does; the last status is also kept in metal_bridge_b200_last_status().
// Element type: the engine's CPU-visible tensors are fp32.  By default device mirrors are fp32 too (CUDA-core kernels,
// 1e-4 against the CPU ops).  Compiled with -DB200_ADAPTOR_BF16 the mirrors of tensor data are bf16, which is what the
// Metal shaders read (cpp/src/gpu_kernel/MetalBridge.mm:841-843, 1353-1355) and what reaches the tcgen05 kernels:
// uploads go host fp32 -> staging -> bf16 mirror, results come back bf16 mirror -> staging -> host fp32.  Token ids,
// rotary tables, the loss scalar, norm-weight gradients and the AdamW arrays stay 4-byte ("raw") in both builds.
// Profiling externs (MetalBridge.hpp:141-145): every sync point adds the DEVICE time of the work enqueued since the
// previous one to accum_gpu_time_ms and counts one GPU call, as end_scope does in the reference (MetalBridge.mm:2195-2207).
#include "gpu_kernel/MetalBridge.hpp"

#include "b200_bridge.h"

#include <cstdio>
#include <cstring>
#include <iostream>
#include <map>
#include <vector>

namespace metal_bridge {
double accum_gpu_time_ms = 0, accum_cpu_time_ms = 0;
size_t count_gpu_calls = 0, count_cpu_calls = 0;
}

namespace {
#ifdef B200_ADAPTOR_BF16
constexpr b200_dtype DT = B200_BF16;
constexpr bool NARROW = true;
#else
constexpr b200_dtype DT = B200_F32;
constexpr bool NARROW = false;
#endif

b200_ctx *g_ctx = nullptr;
bool g_tried = false, g_scope = false, g_timing = false;
int g_status = 0;
float g_last_loss = 0.f;
const float *g_loss_host = nullptr;                 // where the last cross_entropy call will deliver its loss

// device mirror of a host buffer: `narrow` mirrors hold bf16 for an fp32 host array of `elems` elements
struct Mirror { void *dev = nullptr; size_t bytes = 0, elems = 0; bool device_newer = false, narrow = false; };
std::map<const void *, Mirror> g_mirrors;           // host pointer -> device mirror
std::vector<const void *> g_dirty;                  // outputs to copy back at the next sync point
void *g_stage = nullptr; size_t g_stage_bytes = 0;  // fp32 staging for narrow mirrors (all work is on one stream)

bool fail(const char *what, int rc) {
  g_status = rc;
  std::cerr << "[b200 bridge] " << what << " failed (" << rc << "): " << (g_ctx ? b200_last_error(g_ctx) : "no context") << std::endl;
  return false;
}
void begin_work() {                                    // first enqueue after a sync point starts the device timer
  if (!g_timing && b200_batch_timer_begin(g_ctx) == B200_OK) g_timing = true;
}
void *stage(size_t bytes) {
  if (g_stage_bytes < bytes) {
    if (g_stage) b200_free(g_ctx, g_stage);        // waits for the stream first
    g_stage = nullptr; g_stage_bytes = 0;
    if (b200_malloc(g_ctx, bytes, &g_stage) != B200_OK) { fail("b200_malloc(staging)", B200_ERR_NOMEM); return nullptr; }
    g_stage_bytes = bytes;
  }
  return g_stage;
}
void copy_back(const void *host, Mirror &m) {
  if (!m.dev || !m.device_newer) return;
  if (m.narrow) {
    void *st = stage(m.elems * 4);
    if (st && b200_convert(g_ctx, m.dev, B200_BF16, st, B200_F32, m.elems) == B200_OK)
      b200_memcpy_d2h(g_ctx, const_cast<void *>(host), st, m.elems * 4);
  } else {
    b200_memcpy_d2h(g_ctx, const_cast<void *>(host), m.dev, m.bytes);
  }
}
// The mirror of `host` in the wanted form and size; a mirror of the other form, or a smaller one, is written back
// (if it holds newer data) and replaced.
Mirror *mirror(const void *host, size_t elems, bool narrow) {
  Mirror &m = g_mirrors[host];
  const size_t bytes = elems * (narrow ? 2 : 4);
  if (m.dev && (m.narrow != narrow || m.bytes < bytes)) {
    if (m.device_newer) { copy_back(host, m); b200_sync(g_ctx); }
    b200_free(g_ctx, m.dev);
    m = Mirror();
  }
  if (!m.dev) {
    if (b200_malloc(g_ctx, bytes, &m.dev) != B200_OK) { fail("b200_malloc", B200_ERR_NOMEM); g_mirrors.erase(host); return nullptr; }
    m.bytes = bytes; m.elems = elems; m.narrow = narrow;
  }
  return &m;
}
void *upload(const void *host, size_t elems, bool narrow) {
  if (!host) return nullptr;
  begin_work();
  Mirror *m = mirror(host, elems, narrow);
  if (!m) return nullptr;
  if (!m->device_newer) {
    int rc;
    if (narrow) {
      void *st = stage(elems * 4);
      if (!st) return nullptr;
      rc = b200_memcpy_h2d(g_ctx, st, host, elems * 4);
      if (rc == B200_OK) rc = b200_convert(g_ctx, st, B200_F32, m->dev, B200_BF16, elems);
    } else {
      rc = b200_memcpy_h2d(g_ctx, m->dev, host, elems * 4);
    }
    if (rc != B200_OK) { fail("upload", rc); return nullptr; }
  }
  return m->dev;
}
void *result(void *host, size_t elems, bool narrow, bool keep) {
  if (!host) return nullptr;
  begin_work();
  void *d = nullptr;
  if (keep) d = upload(host, elems, narrow);
  else if (Mirror *m = mirror(host, elems, narrow)) d = m->dev;
  if (d) { g_mirrors[host].device_newer = true; g_dirty.push_back(host); }
  return d;
}
// tensor data (fp32 on the host; bf16 on the device in the bf16 build)
void *in(const void *host, size_t elems) { return upload(host, elems, NARROW); }
void *out(void *host, size_t elems, bool keep = false) { return result(host, elems, NARROW, keep); }
// 4-byte data that is never narrowed
void *in_raw(const void *host, size_t elems) { return upload(host, elems, false); }
void *out_raw(void *host, size_t elems, bool keep = false) { return result(host, elems, false, keep); }

void flush() {                                         // copy results back, wait, account the device time
  for (const void *h : g_dirty) {
    auto it = g_mirrors.find(h);
    if (it != g_mirrors.end()) copy_back(h, it->second);
  }
  if (g_timing) {
    float ms = 0.f;
    if (b200_batch_timer_end(g_ctx, &ms) == B200_OK) { metal_bridge::accum_gpu_time_ms += ms; metal_bridge::count_gpu_calls++; }
    g_timing = false;
  }
  int rc = b200_sync(g_ctx);
  if (rc != B200_OK) fail("b200_sync", rc);
  for (auto &kv : g_mirrors) kv.second.device_newer = false;
  g_dirty.clear();
  if (g_loss_host) { g_last_loss = *g_loss_host; g_loss_host = nullptr; }   // the loss scalar is host-visible now
}
void done(const char *what, int rc) {
  if (rc != B200_OK) fail(what, rc);
  if (!g_scope) flush();
}
}  // namespace

extern "C" int metal_bridge_b200_last_status() { return g_status; }

namespace metal_bridge {
void reset_profile_stats() { accum_gpu_time_ms = accum_cpu_time_ms = 0; count_gpu_calls = count_cpu_calls = 0; }

void initialize() {
  if (g_tried) return;
  g_tried = true;
  int rc = b200_init(0, &g_ctx);
  if (rc != B200_OK) { g_ctx = nullptr; std::cerr << "[b200 bridge] no sm_100 device (b200_init = " << rc << ")" << std::endl; }
}
bool is_available() { initialize(); return g_ctx != nullptr; }
void begin_scope() { if (is_available()) g_scope = true; }
void end_scope() { if (g_ctx) { flush(); g_scope = false; } }
void register_gpu_wrapper(const float *, void **slot) { if (slot) *slot = nullptr; }   // mirrors are keyed by pointer
void unregister_gpu_wrapper(const float *ptr) {
  auto it = g_mirrors.find(ptr);
  if (it == g_mirrors.end() || !g_ctx) return;
  if (it->second.dev) b200_free(g_ctx, it->second.dev);
  g_mirrors.erase(it);
}
void reconcile_buffers() { if (g_ctx) flush(); }
void clear_step_cache() {
  if (!g_ctx) return;
  flush();
  for (auto &kv : g_mirrors) if (kv.second.dev) b200_free(g_ctx, kv.second.dev);
  g_mirrors.clear();
}
float get_last_loss() { return g_last_loss; }
void execute_in_autoreleasepool(std::function<void()> f) { f(); }
void start_step_trace() {}    // Xcode GPU capture: no counterpart on CUDA (use ncu)
void stop_step_trace() {}

void fill_zero_async(float *data, size_t bytes) {      // `bytes` of the fp32 host array
  if (!is_available()) return;
  const size_t n = bytes / 4;
  void *d = out(data, n);
  done("fill_zero", d ? b200_fill_zero(g_ctx, d, n * (NARROW ? 2 : 4)) : B200_ERR_NOMEM);
}
void copy_buffer_async(float *dst, size_t dst_bytes, const float *src, size_t src_bytes) {
  if (!is_available()) return;
  const size_t n = (dst_bytes < src_bytes ? dst_bytes : src_bytes) / 4;
  void *s = in(src, n), *d = out(dst, n);
  done("copy", (s && d) ? b200_copy(g_ctx, d, s, n * (NARROW ? 2 : 4)) : B200_ERR_NOMEM);
}

void gemm_bf16(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, bool transA, bool transB, bool) {
  if (!is_available()) return;
  void *a = in(A, M * K), *b = in(B, K * N), *c = out(C, M * N);
  done("gemm", (a && b && c) ? b200_gemm(g_ctx, a, b, c, M, N, K, transA, transB, 0, DT, DT) : B200_ERR_NOMEM);
}
void gemm_proj(const float *a, const float *b, float *c, size_t M, size_t N, size_t K) { gemm_bf16(a, b, c, M, N, K, false, false, true); }
void gemm_proj_trans_b(const float *a, const float *bt, float *c, size_t M, size_t N, size_t K) { gemm_bf16(a, bt, c, M, N, K, false, true, false); }
void gemm_backward(const float *at, const float *b, float *c, size_t M, size_t N, size_t K) { gemm_bf16(at, b, c, M, N, K, true, false, false); }
void fused_swiglu_gemm(const void *gate, const void *up, const void *B, void *C, size_t M, size_t N, size_t K) {
  if (!is_available()) return;
  void *g = in(gate, M * K), *u = in(up, M * K), *b = in(B, K * N), *c = out(C, M * N), *scr = nullptr;
  int rc = (g && u && b && c) ? b200_malloc(g_ctx, M * K * (NARROW ? 2 : 4), &scr) : B200_ERR_NOMEM;
  if (rc == B200_OK) rc = b200_fused_swiglu_gemm(g_ctx, g, u, b, c, scr, M, N, K, DT);
  if (scr) b200_free(g_ctx, scr);
  done("fused_swiglu_gemm", rc);
}
void gemm_ffn(const float *a, const float *bg, const float *bu, float *c, size_t M, size_t N, size_t K) {
  // c = silu(a*bg) * (a*bu)  (cpp/src/gpu_kernel/gemm_ffn.metal:44-183)
  if (!is_available()) return;
  void *da = in(a, M * K), *g = in(bg, K * N), *u = in(bu, K * N), *dc = out(c, M * N), *t1 = nullptr, *t2 = nullptr;
  int rc = (da && g && u && dc) ? b200_malloc(g_ctx, M * N * (NARROW ? 2 : 4), &t1) : B200_ERR_NOMEM;
  if (rc == B200_OK) rc = b200_malloc(g_ctx, M * N * (NARROW ? 2 : 4), &t2);
  if (rc == B200_OK) rc = b200_gemm(g_ctx, da, g, t1, M, N, K, 0, 0, 0, DT, DT);
  if (rc == B200_OK) rc = b200_gemm(g_ctx, da, u, t2, M, N, K, 0, 0, 0, DT, DT);
  if (rc == B200_OK) rc = b200_swiglu_forward(g_ctx, t1, t2, dc, M * N, DT);
  if (t1) b200_free(g_ctx, t1);
  if (t2) b200_free(g_ctx, t2);
  done("gemm_ffn", rc);
}

void flash_attn_fwd(const void *Q, const void *K, const void *V, void *O, size_t B, size_t nH, size_t nKV, size_t S, size_t hd) {
  if (!is_available()) return;
  void *q = in(Q, B * nH * S * hd), *k = in(K, B * nKV * S * hd), *v = in(V, B * nKV * S * hd), *o = out(O, B * S * nH * hd);
  done("flash_attn_fwd", (q && k && v && o) ? b200_flash_attn_fwd(g_ctx, q, k, v, o, nullptr, B, nH, nKV, S, hd, DT) : B200_ERR_NOMEM);
}
void gemm_gqa(const GQAParams &p, const float *q, const float *k, const float *v, float *o, float *L) {
  if (!is_available()) return;
  size_t B = p.batch, nH = p.n_q_heads, nKV = p.n_kv_heads, S = p.seq_len, hd = p.head_dim;
  void *dq = in(q, B * nH * S * hd), *dk = in(k, B * nKV * S * hd), *dv = in(v, B * nKV * S * hd), *d_o = out(o, B * S * nH * hd);
  float *dl = L ? (float *)out_raw(L, B * nH * S) : nullptr;
  done("gemm_gqa", (dq && dk && dv && d_o) ? b200_flash_attn_fwd(g_ctx, dq, dk, dv, d_o, dl, B, nH, nKV, S, hd, DT) : B200_ERR_NOMEM);
}
void fused_attn_bwd(const void *Q, const void *K, const void *V, const void *dO, void *dQ, void *dK, void *dV, size_t B,
                    size_t nH, size_t nKV, size_t S, size_t hd) {
  if (!is_available()) return;
  size_t qn = B * nH * S * hd, kn = B * nKV * S * hd;
  void *q = in(Q, qn), *k = in(K, kn), *v = in(V, kn), *g = in(dO, qn), *dq = out(dQ, qn), *dk = out(dK, kn), *dv = out(dV, kn);
  done("fused_attn_bwd", (q && k && v && g && dq && dk && dv) ? b200_fused_attn_bwd(g_ctx, q, k, v, g, dq, dk, dv, B, nH, nKV, S, hd, DT) : B200_ERR_NOMEM);
}
void gqa_backward(const GQABackwardParams &p, const float *Q, const float *K, const float *V, const float *dO, float *dQ,
                  float *dK, float *dV, const float *) {
  fused_attn_bwd(Q, K, V, dO, dQ, dK, dV, p.batch, p.n_q_heads, p.n_kv_heads, p.seq_len, p.head_dim);
}
// The unfused score / softmax / dS pieces were retired by the reference itself (no pipeline states are
// created for them, cpp/src/gpu_kernel/MetalBridge.mm:389, 528-532); they report and return.
void gqa_scores(const float *, const float *, float *, size_t, size_t, size_t, size_t, size_t) { fail("gqa_scores (retired op)", B200_ERR_UNSUPPORTED); }
void attn_softmax(const float *, float *, size_t, size_t, size_t) { fail("attn_softmax (retired op)", B200_ERR_UNSUPPORTED); }
void attn_ds(const float *, const float *, float *, size_t, size_t, size_t) { fail("attn_ds (retired op)", B200_ERR_UNSUPPORTED); }

void rms_norm_forward(const float *x, float *y, const float *w, float eps, size_t rows, size_t D) {
  if (!is_available()) return;
  void *dx = in(x, rows * D), *dw = in(w, D), *dy = out(y, rows * D);
  done("rms_norm_forward", (dx && dw && dy) ? b200_rms_norm_forward(g_ctx, dx, dy, dw, nullptr, eps, rows, D, DT) : B200_ERR_NOMEM);
}
void rms_norm_backward(const float *g, const float *x, const float *w, float *gx, float *gw, float eps, size_t rows, size_t D) {
  if (!is_available()) return;
  void *dg = in(g, rows * D), *dx = in(x, rows * D), *dw = in(w, D), *dgx = out(gx, rows * D);
  float *dgw = gw ? (float *)out_raw(gw, D, true) : nullptr;
  done("rms_norm_backward", (dg && dx && dw && dgx) ? b200_rms_norm_backward(g_ctx, dg, dx, dw, dgx, dgw, eps, rows, D, DT) : B200_ERR_NOMEM);
}
void fused_add_norm(float *xr, const float *r, const float *w, float *o, size_t rows, size_t D, float eps) {
  if (!is_available()) return;
  void *dr = in(r, rows * D), *dw = in(w, D), *dx = out(xr, rows * D, true), *d_o = out(o, rows * D);
  done("fused_add_norm", (dr && dw && dx && d_o) ? b200_fused_add_norm(g_ctx, dx, dr, dw, d_o, rows, D, eps, DT) : B200_ERR_NOMEM);
}
void fused_backward_add_norm(const void *g, const void *x, const void *w, const void *rg, void *gx, size_t rows, size_t D, float eps) {
  if (!is_available()) return;
  void *dg = in(g, rows * D), *dx = in(x, rows * D), *dw = in(w, D), *drg = in(rg, rows * D), *dgx = out(gx, rows * D);
  done("fused_backward_add_norm", (dg && dx && dw && drg && dgx) ? b200_fused_backward_add_norm(g_ctx, dg, dx, dw, drg, dgx, rows, D, eps, DT) : B200_ERR_NOMEM);
}
void swiglu_forward(const float *gate, const float *up, float *o, size_t n) {
  if (!is_available()) return;
  void *g = in(gate, n), *u = in(up, n), *d = out(o, n);
  done("swiglu_forward", (g && u && d) ? b200_swiglu_forward(g_ctx, g, u, d, n, DT) : B200_ERR_NOMEM);
}
void swiglu_backward(const float *dy, const float *gate, const float *up, float *dg, float *du, size_t n) {
  if (!is_available()) return;
  void *y = in(dy, n), *g = in(gate, n), *u = in(up, n), *a = out(dg, n), *b = out(du, n);
  done("swiglu_backward", (y && g && u && a && b) ? b200_swiglu_backward(g_ctx, y, g, u, a, b, n, DT) : B200_ERR_NOMEM);
}
void rope_forward(float *q, float *k, const float *c, const float *s, size_t B, size_t qh, size_t kvh, size_t S, size_t hd) {
  if (!is_available()) return;
  void *dc = in_raw(c, S * (hd / 2)), *ds = in_raw(s, S * (hd / 2)), *dq = out(q, B * qh * S * hd, true), *dk = out(k, B * kvh * S * hd, true);
  done("rope_forward", (dc && ds && dq && dk) ? b200_rope_forward(g_ctx, dq, dk, (const float *)dc, (const float *)ds, B, qh, kvh, S, hd, DT) : B200_ERR_NOMEM);
}
void rope_backward(float *g, const float *c, const float *s, size_t B, size_t heads, size_t S, size_t hd) {
  if (!is_available()) return;
  void *dc = in_raw(c, S * (hd / 2)), *ds = in_raw(s, S * (hd / 2)), *dg = out(g, B * heads * S * hd, true);
  done("rope_backward", (dc && ds && dg) ? b200_rope_backward(g_ctx, dg, (const float *)dc, (const float *)ds, B, heads, S, hd, DT) : B200_ERR_NOMEM);
}
void residual_add(float *a, const float *b, size_t n) {
  if (!is_available()) return;
  void *db = in(b, n), *da = out(a, n, true);
  done("residual_add", (da && db) ? b200_residual_add(g_ctx, da, db, n, DT) : B200_ERR_NOMEM);
}
void reshape_to_4d(const float *src, float *dst, size_t B, size_t n, size_t S, size_t hd) {
  if (!is_available()) return;
  void *s = in(src, B * n * S * hd), *d = out(dst, B * n * S * hd);
  done("reshape_to_4d", (s && d) ? b200_reshape_to_4d(g_ctx, s, d, B, n, S, hd, DT) : B200_ERR_NOMEM);
}
void reshape_to_3d(const float *src, float *dst, size_t B, size_t n, size_t S, size_t hd) {
  if (!is_available()) return;
  void *s = in(src, B * n * S * hd), *d = out(dst, B * n * S * hd);
  done("reshape_to_3d", (s && d) ? b200_reshape_to_3d(g_ctx, s, d, B, n, S, hd, DT) : B200_ERR_NOMEM);
}
void embedding_forward(const uint32_t *ids, const float *table, float *o, size_t tokens, size_t H, size_t V) {
  if (!is_available()) return;
  void *di = in_raw(ids, tokens), *dt = in(table, V * H), *d = out(o, tokens * H);
  done("embedding_forward", (di && dt && d) ? b200_embedding_forward(g_ctx, (const uint32_t *)di, dt, d, tokens, H, V, DT) : B200_ERR_NOMEM);
}
void cross_entropy(const void *logits, const uint32_t *targets, float *loss_out, float *grad, size_t tokens, size_t V) {
  if (!is_available()) return;
  void *dl = in(logits, tokens * V), *dt = in_raw(targets, tokens), *lo = out_raw(loss_out, 1), *dg = grad ? out(grad, tokens * V) : nullptr;
  int rc = (dl && dt && lo) ? b200_cross_entropy(g_ctx, dl, (const uint32_t *)dt, (float *)lo, dg, tokens, V, DT) : B200_ERR_NOMEM;
  g_loss_host = loss_out;          // read at the next sync point: now, or at end_scope (cpp/src/gpu_kernel/MetalBridge.mm:2211-2215)
  done("cross_entropy", rc);
}
void adamw_step(float *param, const float *grad, float *m, float *v, const AdamWStepParams &p) {
  if (!is_available()) return;
  size_t n = p.n;
  b200_adamw_params a{p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, p.bias_correction1, p.bias_correction2};
  void *dg = in_raw(grad, n), *dp = out_raw(param, n, true), *dm = out_raw(m, n, true), *dv = out_raw(v, n, true);
  done("adamw_step", (dg && dp && dm && dv) ? b200_adamw_step(g_ctx, (float *)dp, (const float *)dg, (float *)dm, (float *)dv, nullptr, n, &a) : B200_ERR_NOMEM);
}
}  // namespace metal_bridge
