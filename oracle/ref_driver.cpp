// ref_driver.cpp -- C entry points over the REFERENCE's own C++ CPU ops
// (Tensor, RMSNorm, RoPE, activatations::swiglu, Attention, TransformerLayer,
// Transformer, CrossEntropyLoss, AdamWOptimizer), compiled from the reference
// checkout by build_ref.sh into _ref/libref_oracle.so.  TEST INFRASTRUCTURE
// ONLY: it exists to validate block_oracle.c, to generate the golden fixtures
// under tests/golden/, and to serve as the "reference" CPU baseline.
//
// The symbols mirror block_oracle.c's orc_* call surface with a ref_ prefix.
// Two orc_* functions have no counterpart because the reference exposes no
// such standalone function: the bare attention core (it is a lambda inside
// Attention::forward, cpp/src/Attention.cpp:236-280, and a file-static helper
// :292-348) -- covered through ref_attention_layer instead.
#include "Activations.hpp"
#include "Attention.hpp"
#include "Loss.hpp"
#include "Optimizer.hpp"
#include "Positional.hpp"
#include "RMSNorm.hpp"
#include "Tensor.hpp"
#include "Transformer.hpp"
#include <cmath>
#include <cstdint>
#include <cstring>
#include <iostream>
#include <sstream>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
struct Cfg { size_t B, S, H, I, nH, nKV, hd, V, L; float eps, rope_base; };

Tensor from(const float *p, std::initializer_list<size_t> shape) {
  Tensor t{Shape(shape)};
  std::memcpy(t.data(), p, t.size() * sizeof(float));
  return t;
}
void to(const Tensor &t, float *p) { std::memcpy(p, t.data(), t.size() * sizeof(float)); }
void load(Tensor &t, const float *p) { std::memcpy(t.data(), p, t.size() * sizeof(float)); }

ModelConfig mc(const Cfg *c) {
  ModelConfig m{};
  m.vocab_size = c->V; m.hidden_dim = c->H; m.intermediate_dim = c->I; m.n_layers = c->L;
  m.n_heads = c->nH; m.n_kv_heads = c->nKV; m.head_dim = c->hd; m.max_seq_len = c->S;
  m.rope_base = c->rope_base; m.rms_norm_eps = c->eps;
  return m;
}

// The reference prints progress lines from backward; keep test output clean.
struct Quiet {
  std::streambuf *o, *e; std::ostringstream sink;
  Quiet() : o(std::cout.rdbuf(sink.rdbuf())), e(std::cerr.rdbuf(sink.rdbuf())) {}
  ~Quiet() { std::cout.rdbuf(o); std::cerr.rdbuf(e); }
};

size_t layer_params(const Cfg *c) {
  size_t q = c->nH * c->hd, kv = c->nKV * c->hd;
  return c->H + c->H * q + 2 * c->H * kv + q * c->H + c->H + 3 * c->H * c->I;
}
// Flat layer block: attn_norm_w, Wq, Wk, Wv, Wo, ffn_norm_w, w_gate, w_up, w_down.
void load_layer(TransformerLayer &l, const float *p) {
  load(l.attn_norm.weight(), p); p += l.attn_norm.weight().size();
  load(l.attn.Wq(), p); p += l.attn.Wq().size();
  load(l.attn.Wk(), p); p += l.attn.Wk().size();
  load(l.attn.Wv(), p); p += l.attn.Wv().size();
  load(l.attn.Wo(), p); p += l.attn.Wo().size();
  load(l.ffn_norm.weight(), p); p += l.ffn_norm.weight().size();
  load(l.w_gate, p); p += l.w_gate.size();
  load(l.w_up, p); p += l.w_up.size();
  load(l.w_down, p);
}
struct LayerGrads {
  Tensor gate, up, down, q, k, v, o;
  explicit LayerGrads(const TransformerLayer &l)
      : gate(l.w_gate.shape(), 0.0f), up(l.w_up.shape(), 0.0f), down(l.w_down.shape(), 0.0f),
        q(l.attn.Wq().shape(), 0.0f), k(l.attn.Wk().shape(), 0.0f), v(l.attn.Wv().shape(), 0.0f),
        o(l.attn.Wo().shape(), 0.0f) {}
  void load_from(const Cfg *c, const float *g) {
    size_t H = c->H;
    g += H; load(q, g); g += q.size(); load(k, g); g += k.size(); load(v, g); g += v.size();
    load(o, g); g += o.size(); g += H; load(gate, g); g += gate.size(); load(up, g); g += up.size();
    load(down, g);
  }
  void store(const Cfg *c, float *g) const {   // norm-weight slots are left untouched
    size_t H = c->H;
    g += H; to(q, g); g += q.size(); to(k, g); g += k.size(); to(v, g); g += v.size();
    to(o, g); g += o.size(); g += H; to(gate, g); g += gate.size(); to(up, g); g += up.size();
    to(down, g);
  }
};
}  // namespace

REF_API void ref_gemm(const float *A, const float *B, float *C, size_t M, size_t N, size_t K,
                      int transA, int transB, int accumulate) {
  // The reference's CPU branches spell transposed products as
  // x.transpose().matmul(y) and x.matmul(w.transpose()) (cpp/src/Attention.cpp:483,498).
  Tensor a = transA ? from(A, {K, M}).transpose() : from(A, {M, K});
  Tensor b = transB ? from(B, {N, K}).transpose() : from(B, {K, N});
  Tensor c = a.matmul(b);
  if (accumulate) { Tensor acc = from(C, {M, N}); acc.add_(c); to(acc, C); } else to(c, C);
}
REF_API void ref_rms_norm_forward(const float *x, float *y, const float *w, float eps, size_t rows, size_t D) {
  RMSNorm n(D, eps); load(n.weight(), w);
  to(n.forward(from(x, {rows, D})), y);
}
REF_API void ref_rms_norm_backward(const float *g, const float *x, const float *w, float *dx, float *dw,
                                   float eps, size_t rows, size_t D) {
  RMSNorm n(D, eps); load(n.weight(), w);
  Tensor gw({D}, 0.0f);
  if (dw) load(gw, dw);
  to(n.backward(from(g, {rows, D}), from(x, {rows, D}), gw), dx);
  if (dw) to(gw, dw);
}
REF_API void ref_rope_tables(float *cos_t, float *sin_t, size_t max_seq, size_t hd, float base) {
  RoPE r(hd, max_seq, base);
  auto c = r.cos_table(), s = r.sin_table();
  for (size_t p = 0; p < max_seq; ++p)
    for (size_t i = 0; i < hd / 2; ++i) { cos_t[p * (hd / 2) + i] = c[p][i]; sin_t[p * (hd / 2) + i] = s[p][i]; }
}
REF_API void ref_rope_apply(float *t, const float *, const float *, size_t B, size_t heads, size_t S, size_t hd,
                            int backward) {
  RoPE r(hd, S, 10000.0f);   // tables are rebuilt by the reference class itself
  Tensor q = from(t, {B, heads, S, hd});
  Tensor k({B, 1, S, hd}, 0.0f);
  if (backward) r.backward(q, k); else r.forward(q, k);
  to(q, t);
}
REF_API void ref_swiglu_forward(const float *gate, const float *up, float *out, size_t n) {
  to(activatations::swiglu(from(gate, {n}), from(up, {n})), out);
}
REF_API void ref_swiglu_backward(const float *dy, const float *gate, const float *up, float *dg, float *du, size_t n) {
  Tensor g({n}, 0.0f), u({n}, 0.0f);
  activatations::swiglu_backward(from(dy, {n}), from(gate, {n}), from(up, {n}), g, u);
  to(g, dg); to(u, du);
}
REF_API void ref_attention_forward(...) {}    // no standalone counterpart (see header comment)
REF_API void ref_attention_backward(...) {}
REF_API float ref_cross_entropy(const float *logits, const int32_t *targets, float *dlogits, size_t tokens, size_t V) {
  Tensor lg = from(logits, {1, tokens, V});
  Tensor tg({1, tokens}, 0.0f);
  for (size_t i = 0; i < tokens; ++i) tg.data()[i] = (float)targets[i];   // ids travel as floats (cpp/src/Trainer.cpp:56-65)
  CrossEntropyLoss ce;
  float loss = ce.forward(lg, tg);
  if (dlogits) to(ce.backward(tg), dlogits);
  return loss;
}
REF_API void ref_adamw_step(float *p, const float *g, float *m, float *v, size_t n, float lr, float beta1,
                            float beta2, float eps, float wd, float bc1, float bc2) {
  // AdamWOptimizer::step computes the bias corrections itself from its step
  // counter (cpp/src/Optimizer.cpp:139-149); recover the step from bc1.
  Quiet q;
  Tensor P = from(p, {n}), G = from(g, {n});
  AdamWOptimizer opt(beta1, beta2, eps, wd);
  opt.register_parameter(&P, &G);
  load(opt.m_states()[0], m); load(opt.v_states()[0], v);
  size_t step = 1;
  for (; step < 100000; ++step)
    if (std::fabs((1.0f - std::pow(beta1, (float)step)) - bc1) <= 1e-6f * std::fabs(bc1)) break;
  (void)bc2;
  opt.step_count() = step - 1;
  opt.step(lr);
  to(P, p); to(opt.m_states()[0], m); to(opt.v_states()[0], v);
}
REF_API void ref_attention_layer(const Cfg *c, const float *x, const float *Wq, const float *Wk, const float *Wv,
                                 const float *Wo, float *out, const float *gout, float *gx, float *gWq,
                                 float *gWk, float *gWv, float *gWo) {
  Quiet quiet;
  ModelConfig m = mc(c);
  Attention a(m);
  load(a.Wq(), Wq); load(a.Wk(), Wk); load(a.Wv(), Wv); load(a.Wo(), Wo);
  RoPE rope(c->hd, c->S, c->rope_base);
  Tensor X = from(x, {c->B, c->S, c->H});
  to(a.forward(X, rope), out);
  if (gout) {
    Tensor gq(a.Wq().shape(), 0.0f), gk(a.Wk().shape(), 0.0f), gv(a.Wv().shape(), 0.0f), go(a.Wo().shape(), 0.0f);
    to(a.backward(from(gout, {c->B, c->S, c->H}), X, rope, gq, gk, gv, go), gx);
    to(gq, gWq); to(gk, gWk); to(gv, gWv); to(go, gWo);
  }
}
REF_API void ref_layer_forward(const Cfg *c, const float *h_in, const float *params, float *h_out) {
  // The reference has no standalone layer forward; this is the body of the
  // per-layer loop's CPU branch (cpp/src/Transformer.cpp:147-148,178-183)
  // spelled with the reference's own ops.
  Quiet quiet;
  ModelConfig m = mc(c);
  TransformerLayer layer(m);
  load_layer(layer, params);
  RoPE rope(c->hd, c->S, c->rope_base);
  Tensor h = from(h_in, {c->B, c->S, c->H});
  Tensor attn_in = layer.attn_norm.forward(h);
  Tensor attn_out = layer.attn.forward(attn_in, rope);
  h.add_(attn_out);
  Tensor ffn_in = layer.ffn_norm.forward(h);
  Tensor activated = activatations::swiglu(ffn_in.matmul(layer.w_gate), ffn_in.matmul(layer.w_up));
  Tensor ffn_out = activated.matmul(layer.w_down);
  h.add_(ffn_out);
  to(h, h_out);
}
REF_API void ref_layer_backward(const Cfg *c, const float *grad_out, const float *h_in, const float *params,
                                float *grads, float *grad_h_in) {
  Quiet quiet;
  ModelConfig m = mc(c);
  TransformerLayer layer(m);
  load_layer(layer, params);
  RoPE rope(c->hd, c->S, c->rope_base);
  LayerGrads g(layer);
  g.load_from(c, grads);
  Tensor gh = layer.backward(from(grad_out, {c->B, c->S, c->H}), from(h_in, {c->B, c->S, c->H}), g.gate, g.up,
                             g.down, g.q, g.k, g.v, g.o, rope);
  to(gh, grad_h_in);
  g.store(c, grads);
}
REF_API float ref_model_loss_and_grads(const Cfg *c, const int32_t *tokens, const int32_t *targets,
                                       const float *params, float *grads, float *logits_out) {
  Quiet quiet;
  ModelConfig m = mc(c);
  Transformer model(m);
  size_t lp = layer_params(c), V = c->V, H = c->H, L = c->L, M = c->B * c->S;
  load(model.token_embeddings(), params);
  for (size_t l = 0; l < L; ++l) load_layer(model.layers()[l], params + V * H + l * lp);
  load(model.final_norm().weight(), params + V * H + L * lp);
  load(model.output_projection(), params + V * H + L * lp + H);
  Tensor tok({c->B, c->S}, 0.0f), tgt({c->B, c->S}, 0.0f);
  for (size_t i = 0; i < M; ++i) { tok.data()[i] = (float)tokens[i]; tgt.data()[i] = (float)targets[i]; }
  Tensor logits = model.forward(tok);
  if (logits_out) to(logits, logits_out);
  CrossEntropyLoss ce;
  float loss = ce.forward(logits, tgt);
  if (grads) {
    Tensor dlogits = ce.backward(tgt);
    std::vector<Tensor> gg, gu, gd, gq, gk, gv, go;
    for (size_t l = 0; l < L; ++l) {
      LayerGrads g(model.layers()[l]);
      gg.push_back(g.gate); gu.push_back(g.up); gd.push_back(g.down); gq.push_back(g.q); gk.push_back(g.k);
      gv.push_back(g.v); go.push_back(g.o);
    }
    Tensor gemb(model.token_embeddings().shape(), 0.0f), gout(model.output_projection().shape(), 0.0f);
    RoPE rope(c->hd, c->S, c->rope_base);
    model.backward(dlogits, tok, gg, gu, gd, gq, gk, gv, go, gemb, gout, rope);
    to(gemb, grads);
    for (size_t l = 0; l < L; ++l) {
      float *g = grads + V * H + l * lp;
      g += H; to(gq[l], g); g += gq[l].size(); to(gk[l], g); g += gk[l].size(); to(gv[l], g); g += gv[l].size();
      to(go[l], g); g += go[l].size(); g += H; to(gg[l], g); g += gg[l].size(); to(gu[l], g); g += gu[l].size();
      to(gd[l], g);
    }
    to(gout, grads + V * H + L * lp + H);
  }
  return loss;
}

// ---- the backend interface's profiling externs and loss read-back (cpp/include/gpu_kernel/MetalBridge.hpp:136-145),
// as Trainer::train consumes them (cpp/src/Trainer.cpp:347-366): exercised by the drop-in test of a GPU backend; with the
// CPU stub they stay zero.
#include "gpu_kernel/MetalBridge.hpp"
REF_API void ref_backend_stats(double *gpu_ms, uint64_t *gpu_calls, float *last_loss) {
  *gpu_ms = metal_bridge::accum_gpu_time_ms;
  *gpu_calls = (uint64_t)metal_bridge::count_gpu_calls;
  *last_loss = metal_bridge::get_last_loss();
}
REF_API void ref_backend_reset_stats() { metal_bridge::reset_profile_stats(); }
// CrossEntropyLoss inside one begin_scope()/end_scope() pair, the way the trainer's step issues it: the loss scalar is
// only host-visible after end_scope, and get_last_loss() must return it then.
REF_API float ref_scoped_cross_entropy(const float *logits, const int32_t *targets, size_t tokens, size_t V) {
  Quiet q;
  Tensor lg = from(logits, {1, tokens, V});
  Tensor tg({1, tokens}, 0.0f);
  for (size_t i = 0; i < tokens; ++i) tg.data()[i] = (float)targets[i];
  CrossEntropyLoss ce;
  metal_bridge::begin_scope();
  ce.forward(lg, tg);
  metal_bridge::end_scope();
  return metal_bridge::get_last_loss();
}

// ---- training-driver files: the reference's own Checkpoint::save / ::load and LR schedule ------------------
#include "Checkpoint.hpp"
#include "Trainer.hpp"
namespace {
// Registers the parameters in the order Trainer::train does (cpp/src/Trainer.cpp:188-198) so that the moment
// vectors line up with what Checkpoint expects; grads are dummies of the right shape.
struct OptHarness {
  Transformer model;
  AdamWOptimizer opt;
  std::vector<Tensor> grads;
  explicit OptHarness(const Cfg *c) : model(mc(c)), opt(0.9f, 0.95f, 1e-8f, 0.1f) {
    std::vector<Tensor *> ps{&model.token_embeddings(), &model.output_projection()};
    for (auto &l : model.layers()) {
      ps.push_back(&l.w_gate); ps.push_back(&l.w_up); ps.push_back(&l.w_down);
      ps.push_back(&l.attn.Wq()); ps.push_back(&l.attn.Wk()); ps.push_back(&l.attn.Wv()); ps.push_back(&l.attn.Wo());
    }
    grads.reserve(ps.size());
    for (Tensor *p : ps) { grads.emplace_back(p->shape(), 0.0f); opt.register_parameter(p, &grads.back()); }
  }
  // flat (per-tensor order of ref_model_loss_and_grads) <-> the optimizer's registration order
  template <class F> void each_state(const Cfg *c, std::vector<Tensor> &st, float *flat, F f) {
    const size_t V = c->V, H = c->H, L = c->L, lp = layer_params(c);
    f(st[0], flat);
    f(st[1], flat + V * H + L * lp + H);
    for (size_t l = 0; l < L; ++l) {
      float *p = flat + V * H + l * lp;
      const size_t i0 = 2 + l * 7;
      p += H; f(st[i0 + 3], p); p += st[i0 + 3].size(); f(st[i0 + 4], p); p += st[i0 + 4].size();
      f(st[i0 + 5], p); p += st[i0 + 5].size(); f(st[i0 + 6], p); p += st[i0 + 6].size();
      p += H; f(st[i0 + 0], p); p += st[i0 + 0].size(); f(st[i0 + 1], p); p += st[i0 + 1].size(); f(st[i0 + 2], p);
    }
  }
  void load_model(const Cfg *c, const float *params) {
    const size_t V = c->V, H = c->H, L = c->L, lp = layer_params(c);
    load(model.token_embeddings(), params);
    for (size_t l = 0; l < L; ++l) load_layer(model.layers()[l], params + V * H + l * lp);
    load(model.final_norm().weight(), params + V * H + L * lp);
    load(model.output_projection(), params + V * H + L * lp + H);
  }
  void store_model(const Cfg *c, float *params) {
    const size_t V = c->V, H = c->H, L = c->L, lp = layer_params(c);
    to(model.token_embeddings(), params);
    for (size_t l = 0; l < L; ++l) {
      float *p = params + V * H + l * lp;
      TransformerLayer &y = model.layers()[l];
      to(y.attn_norm.weight(), p); p += H; to(y.attn.Wq(), p); p += y.attn.Wq().size(); to(y.attn.Wk(), p); p += y.attn.Wk().size();
      to(y.attn.Wv(), p); p += y.attn.Wv().size(); to(y.attn.Wo(), p); p += y.attn.Wo().size(); to(y.ffn_norm.weight(), p); p += H;
      to(y.w_gate, p); p += y.w_gate.size(); to(y.w_up, p); p += y.w_up.size(); to(y.w_down, p);
    }
    to(model.final_norm().weight(), params + V * H + L * lp);
    to(model.output_projection(), params + V * H + L * lp + H);
  }
};
}  // namespace

REF_API int ref_checkpoint_save(const Cfg *c, const float *params, const float *m, const float *v, uint64_t step, const char *path) {
  Quiet q;
  OptHarness h(c);
  h.load_model(c, params);
  h.each_state(c, h.opt.m_states(), const_cast<float *>(m), [](Tensor &t, float *p) { load(t, p); });
  h.each_state(c, h.opt.v_states(), const_cast<float *>(v), [](Tensor &t, float *p) { load(t, p); });
  h.opt.step_count() = (size_t)step;
  return Checkpoint::save(path, h.model, h.opt, (size_t)step) ? 0 : 1;
}
REF_API int ref_checkpoint_load(const Cfg *c, const char *path, float *params, float *m, float *v, uint64_t *step) {
  Quiet q;
  OptHarness h(c);
  size_t st = 0;
  if (!Checkpoint::load(path, h.model, h.opt, st)) return 1;
  h.store_model(c, params);
  std::memset(m, 0, (2 * c->V * c->H + c->L * layer_params(c) + c->H) * sizeof(float));
  std::memset(v, 0, (2 * c->V * c->H + c->L * layer_params(c) + c->H) * sizeof(float));
  h.each_state(c, h.opt.m_states(), m, [](Tensor &t, float *p) { to(t, p); });
  h.each_state(c, h.opt.v_states(), v, [](Tensor &t, float *p) { to(t, p); });
  *step = st;
  return 0;
}
// Trainer::get_scheduled_lr reads nothing but its config; the model / optimizer / data-loader references the
// constructor wants are never touched, so a small real model and an unconstructed loader slot are enough.
REF_API float ref_scheduled_lr(size_t step, size_t warmup, size_t max_steps, float lr_max, float lr_min) {
  Quiet q;
  Cfg c{1, 4, 8, 8, 2, 1, 4, 8, 1, 1e-5f, 10000.0f};
  OptHarness h(&c);
  RoPE rope(4, 4, 10000.0f);
  alignas(DataIngestion) static unsigned char slot[sizeof(DataIngestion)];
  TrainerConfig tc;
  tc.warmup_steps = warmup; tc.max_steps = max_steps; tc.lr_max = lr_max; tc.lr_min = lr_min;
  Trainer t(tc, h.model, h.opt, *reinterpret_cast<DataIngestion *>(slot), rope);
  return t.get_scheduled_lr(step);
}
