/*
 * block_oracle.c -- CPU restatement of the reference training engine's
 * decoder-block hot path.  TEST INFRASTRUCTURE ONLY: it is the checker that
 * the CUDA kernels are compared against and the "port" CPU baseline that the
 * benchmark times; no product code path may call into it.
 *
 * Every function restates, in plain fp32 C, what the reference's C++ CPU
 * branch computes (file:line citations are paths inside the reference
 * project).  Where the reference has no CPU branch (GEMM, RMSNorm forward,
 * AdamW) the maths of the corresponding shader is restated instead.
 *
 * Parity pin: the functions here are checked (tests/test_oracle.py) against
 *   - the scalar golden values the reference's own unit tests hold
 *     (cpp/tests/test_rmsnorm.cpp:75-78, test_rope.cpp:87-136,
 *      test_activations.cpp:48-75, test_loss.cpp:56-101,
 *      test_math_ops.cpp:167-188), and
 *   - fixtures under tests/golden/ produced by the reference's own C++ CPU
 *     ops compiled from its sources (oracle/build_ref.sh, alias-fixed build).
 *
 * Two deliberate departures from the reference as written, both because the
 * reference's Tensor copy is shallow (cpp/include/Tensor.hpp:237):
 *   - swiglu() in the reference overwrites its gate argument
 *     (cpp/src/Activations.cpp:71-73) and the layer backward then differentiates
 *     with the clobbered gate (cpp/src/Transformer.cpp:377-379,411);
 *   - h_cache_.push_back(h) aliases all cached hidden states
 *     (cpp/src/Transformer.cpp:142,187).
 * This file implements the mathematically intended (deep-copy) behaviour.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ GEMM */
/* C[M,N] (+)= op(A)[M,K] * op(B)[K,N], row-major, fp32.
 * Follows metal_bridge::gemm_bf16's contract (cpp/include/gpu_kernel/MetalBridge.hpp:39-42,
 * index maths cpp/src/gpu_kernel/gemm_bf16.metal:45,63): transA means A is
 * stored [K,M]; transB means B is stored [N,K].  Accumulation order over k is
 * ascending, as in the shader's tile loop. */
ORC_API void orc_gemm(const float *A, const float *B, float *C, size_t M,
                      size_t N, size_t K, int transA, int transB,
                      int accumulate) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)M; ++i) {
    float *crow = C + (size_t)i * N;
    if (!accumulate) memset(crow, 0, N * sizeof(float));
    if (!transB) {
      for (size_t k = 0; k < K; ++k) {
        float a = transA ? A[k * M + i] : A[(size_t)i * K + k];
        const float *brow = B + k * N;
        for (size_t j = 0; j < N; ++j) crow[j] += a * brow[j];
      }
    } else {
      for (size_t j = 0; j < N; ++j) {
        const float *brow = B + j * K;
        float acc = 0.f;
        if (!transA) {
          const float *arow = A + (size_t)i * K;
          for (size_t k = 0; k < K; ++k) acc += arow[k] * brow[k];
        } else {
          for (size_t k = 0; k < K; ++k) acc += A[k * M + i] * brow[k];
        }
        crow[j] += acc;
      }
    }
  }
}

/* --------------------------------------------------------------- RMSNorm */
/* y = x * rsqrt(mean(x^2) + eps) * w   (cpp/src/RMSNorm.cpp:49-76 calls the
 * bridge unconditionally; maths from cpp/src/gpu_kernel/rms_norm_forward.metal:29-60). */
ORC_API void orc_rms_norm_forward(const float *x, float *y, const float *w,
                                  float eps, size_t rows, size_t D) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
    const float *xr = x + (size_t)r * D;
    float *yr = y + (size_t)r * D;
    float ss = 0.f;
    for (size_t c = 0; c < D; ++c) ss += xr[c] * xr[c];
    float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (size_t c = 0; c < D; ++c) yr[c] = xr[c] * inv * w[c];
  }
}

/* dx = (1/rms) * (g*w - xhat * mean(g*w*xhat)); dw += sum_rows g*xhat
 * (cpp/src/RMSNorm.cpp:126-160). dw may be NULL (the reference's callers
 * discard it: cpp/src/Transformer.cpp:450-451,468-469,631-633). */
ORC_API void orc_rms_norm_backward(const float *g, const float *x,
                                   const float *w, float *dx, float *dw,
                                   float eps, size_t rows, size_t D) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
    const float *xr = x + (size_t)r * D;
    const float *gr = g + (size_t)r * D;
    float *dr = dx + (size_t)r * D;
    float ss = 0.f;
    for (size_t c = 0; c < D; ++c) ss += xr[c] * xr[c];
    float rms = sqrtf(ss / (float)D + eps);
    float s = 0.f;
    for (size_t c = 0; c < D; ++c) s += gr[c] * w[c] * (xr[c] / rms);
    s /= (float)D;
    for (size_t c = 0; c < D; ++c) {
      float xhat = xr[c] / rms;
      dr[c] = (1.0f / rms) * (gr[c] * w[c] - xhat * s);
    }
  }
  if (dw) {
    for (size_t r = 0; r < rows; ++r) {
      const float *xr = x + r * D;
      const float *gr = g + r * D;
      float ss = 0.f;
      for (size_t c = 0; c < D; ++c) ss += xr[c] * xr[c];
      float rms = sqrtf(ss / (float)D + eps);
      for (size_t c = 0; c < D; ++c) dw[c] += gr[c] * (xr[c] / rms);
    }
  }
}

/* ------------------------------------------------------------------ RoPE */
/* theta_i = base^(-2i/hd); tables [max_seq, hd/2] (cpp/src/Positional.cpp:48-68). */
ORC_API void orc_rope_tables(float *cos_t, float *sin_t, size_t max_seq,
                             size_t hd, float base) {
  size_t half = hd / 2;
  for (size_t i = 0; i < half; ++i) {
    float exponent = (2.0f * (float)i) / (float)hd;
    float theta = 1.0f / powf(base, exponent);
    for (size_t pos = 0; pos < max_seq; ++pos) {
      cos_t[pos * half + i] = cosf((float)pos * theta);
      sin_t[pos * half + i] = sinf((float)pos * theta);
    }
  }
}

/* In-place rotation of interleaved pairs (2i,2i+1) of t[B,heads,S,hd];
 * forward cpp/src/Positional.cpp:120-147, backward (inverse rotation) :207-231. */
ORC_API void orc_rope_apply(float *t, const float *cos_t, const float *sin_t,
                            size_t B, size_t heads, size_t S, size_t hd,
                            int backward) {
  size_t half = hd / 2;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t bh = 0; bh < (ptrdiff_t)(B * heads); ++bh) {
    for (size_t s = 0; s < S; ++s) {
      float *row = t + ((size_t)bh * S + s) * hd;
      for (size_t i = 0; i < half; ++i) {
        float x0 = row[2 * i], x1 = row[2 * i + 1];
        float c = cos_t[s * half + i], sn = sin_t[s * half + i];
        if (!backward) {
          row[2 * i] = x0 * c - x1 * sn;
          row[2 * i + 1] = x0 * sn + x1 * c;
        } else {
          row[2 * i] = x0 * c + x1 * sn;
          row[2 * i + 1] = -x0 * sn + x1 * c;
        }
      }
    }
  }
}

/* ---------------------------------------------------------------- SwiGLU */
/* out = gate * sigmoid(gate) * up  (cpp/src/Activations.cpp:31-75). */
ORC_API void orc_swiglu_forward(const float *gate, const float *up, float *out,
                                size_t n) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) {
    float sig = 1.0f / (1.0f + expf(-gate[i]));
    out[i] = gate[i] * sig * up[i];
  }
}

/* d_up = dy*silu(g); d_gate = dy*up*sig*(1+g*(1-sig)) (cpp/src/Activations.cpp:119-167). */
ORC_API void orc_swiglu_backward(const float *dy, const float *gate,
                                 const float *up, float *dgate, float *dup,
                                 size_t n) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) {
    float sig = 1.0f / (1.0f + expf(-gate[i]));
    float silu = gate[i] * sig;
    float dsilu = sig * (1.0f + gate[i] * (1.0f - sig));
    dup[i] = dy[i] * silu;
    dgate[i] = dy[i] * up[i] * dsilu;
  }
}

/* ------------------------------------------------------------- reshapes */
/* [B,S,n*hd] -> [B,n,S,hd]  (cpp/src/Attention.cpp:68-98) and back (:118-152). */
ORC_API void orc_reshape_to_4d(const float *src, float *dst, size_t B,
                               size_t n, size_t S, size_t hd) {
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < n; ++h)
      for (size_t s = 0; s < S; ++s)
        memcpy(dst + ((b * n + h) * S + s) * hd,
               src + (b * S + s) * (n * hd) + h * hd, hd * sizeof(float));
}
ORC_API void orc_reshape_to_3d(const float *src, float *dst, size_t B,
                               size_t n, size_t S, size_t hd) {
  for (size_t b = 0; b < B; ++b)
    for (size_t h = 0; h < n; ++h)
      for (size_t s = 0; s < S; ++s)
        memcpy(dst + (b * S + s) * (n * hd) + h * hd,
               src + ((b * n + h) * S + s) * hd, hd * sizeof(float));
}

/* ------------------------------------------------------ causal GQA core */
/* q4 [B,nH,S,hd], k4/v4 [B,nKV,S,hd] -> out [B,S,nH*hd]; two-pass softmax,
 * kv head = h / (nH/nKV)  (cpp/src/Attention.cpp:236-280). */
ORC_API void orc_attention_forward(const float *q4, const float *k4,
                                   const float *v4, float *out, size_t B,
                                   size_t nH, size_t nKV, size_t S,
                                   size_t hd) {
  size_t G = nH / nKV;
  float scale = 1.0f / sqrtf((float)hd);
  memset(out, 0, B * S * nH * hd * sizeof(float));
#pragma omp parallel for schedule(dynamic)
  for (ptrdiff_t bh = 0; bh < (ptrdiff_t)(B * nH); ++bh) {
    size_t b = (size_t)bh / nH, h = (size_t)bh % nH, kvh = h / G;
    float *scores = (float *)malloc(S * sizeof(float));
    for (size_t sq = 0; sq < S; ++sq) {
      const float *qr = q4 + ((b * nH + h) * S + sq) * hd;
      float mx = -INFINITY;
      for (size_t sk = 0; sk <= sq; ++sk) {
        const float *kr = k4 + ((b * nKV + kvh) * S + sk) * hd;
        float dot = 0.f;
        for (size_t d = 0; d < hd; ++d) dot += qr[d] * kr[d];
        scores[sk] = dot * scale;
        if (scores[sk] > mx) mx = scores[sk];
      }
      float sum = 0.f;
      for (size_t sk = 0; sk <= sq; ++sk) {
        scores[sk] = expf(scores[sk] - mx);
        sum += scores[sk];
      }
      float *orow = out + (b * S + sq) * (nH * hd) + h * hd;
      for (size_t sk = 0; sk <= sq; ++sk) {
        float p = scores[sk] / sum;
        const float *vr = v4 + ((b * nKV + kvh) * S + sk) * hd;
        for (size_t d = 0; d < hd; ++d) orow[d] += p * vr[d];
      }
    }
    free(scores);
  }
}

/* Per query token: recompute P; dV += P^T dO; dP = dO V^T;
 * dS = P*(dP - sum(P*dP)); dQ += dS*scale*K; dK += dS*scale*Q
 * (cpp/src/Attention.cpp:292-348, driver loop :531-540).
 * dO is [B,S,nH*hd]; dq4 [B,nH,S,hd]; dk4/dv4 [B,nKV,S,hd] (zeroed here). */
ORC_API void orc_attention_backward(const float *q4, const float *k4,
                                    const float *v4, const float *dO,
                                    float *dq4, float *dk4, float *dv4,
                                    size_t B, size_t nH, size_t nKV, size_t S,
                                    size_t hd) {
  size_t G = nH / nKV;
  float scale = 1.0f / sqrtf((float)hd);
  memset(dq4, 0, B * nH * S * hd * sizeof(float));
  memset(dk4, 0, B * nKV * S * hd * sizeof(float));
  memset(dv4, 0, B * nKV * S * hd * sizeof(float));
  /* parallel over (b, kv head): the G query heads of one kv head are handled
   * by one thread in ascending h order, like the reference's serial loop. */
#pragma omp parallel for schedule(dynamic)
  for (ptrdiff_t bk = 0; bk < (ptrdiff_t)(B * nKV); ++bk) {
    size_t b = (size_t)bk / nKV, kvh = (size_t)bk % nKV;
    float *raw = (float *)malloc(3 * S * sizeof(float));
    float *prob = raw + S, *dP = raw + 2 * S;
    for (size_t h = kvh * G; h < (kvh + 1) * G; ++h) {
      for (size_t sq = 0; sq < S; ++sq) {
        const float *qr = q4 + ((b * nH + h) * S + sq) * hd;
        const float *gr = dO + (b * S + sq) * (nH * hd) + h * hd;
        float *dqr = dq4 + ((b * nH + h) * S + sq) * hd;
        float mx = -INFINITY;
        for (size_t sk = 0; sk <= sq; ++sk) {
          const float *kr = k4 + ((b * nKV + kvh) * S + sk) * hd;
          float dot = 0.f;
          for (size_t d = 0; d < hd; ++d) dot += qr[d] * kr[d];
          raw[sk] = dot * scale;
          if (raw[sk] > mx) mx = raw[sk];
        }
        float sum = 0.f;
        for (size_t sk = 0; sk <= sq; ++sk) sum += expf(raw[sk] - mx);
        for (size_t sk = 0; sk <= sq; ++sk) prob[sk] = expf(raw[sk] - mx) / sum;
        float sdp = 0.f;
        for (size_t sk = 0; sk <= sq; ++sk) {
          const float *vr = v4 + ((b * nKV + kvh) * S + sk) * hd;
          float *dvr = dv4 + ((b * nKV + kvh) * S + sk) * hd;
          float dot = 0.f;
          for (size_t d = 0; d < hd; ++d) {
            dot += gr[d] * vr[d];
            dvr[d] += prob[sk] * gr[d];
          }
          dP[sk] = dot;
          sdp += dP[sk] * prob[sk];
        }
        for (size_t sk = 0; sk <= sq; ++sk) {
          float dS = prob[sk] * (dP[sk] - sdp) * scale;
          const float *kr = k4 + ((b * nKV + kvh) * S + sk) * hd;
          float *dkr = dk4 + ((b * nKV + kvh) * S + sk) * hd;
          for (size_t d = 0; d < hd; ++d) {
            dqr[d] += dS * kr[d];
            dkr[d] += dS * qr[d];
          }
        }
      }
    }
    free(raw);
  }
}

/* --------------------------------------------------------- cross-entropy */
/* mean over tokens of -log(max(p_target,1e-15)); optional probs out and
 * dlogits = (p - onehot)/tokens  (cpp/src/Loss.cpp:77-134, 163-194).
 * Per-token losses are summed in token order (the reference sums per-thread
 * partials; the difference is below fp32 rounding of the mean). */
ORC_API float orc_cross_entropy(const float *logits, const int32_t *targets,
                                float *dlogits, size_t tokens, size_t V) {
  double total = 0.0;
  float inv = 1.0f / (float)tokens;
  float *tok_loss = (float *)malloc(tokens * sizeof(float));
#pragma omp parallel for schedule(static)
  for (ptrdiff_t t = 0; t < (ptrdiff_t)tokens; ++t) {
    const float *lr = logits + (size_t)t * V;
    float mx = -INFINITY;
    for (size_t v = 0; v < V; ++v)
      if (lr[v] > mx) mx = lr[v];
    float sum = 0.f;
    for (size_t v = 0; v < V; ++v) sum += expf(lr[v] - mx);
    size_t tgt = (size_t)targets[t];
    float pt = expf(lr[tgt] - mx) / sum;
    tok_loss[t] = -logf(fmaxf(pt, 1e-15f));
    if (dlogits) {
      float *dr = dlogits + (size_t)t * V;
      for (size_t v = 0; v < V; ++v) {
        float p = expf(lr[v] - mx) / sum;
        dr[v] = (v == tgt) ? (p - 1.0f) * inv : p * inv;
      }
    }
  }
  float acc = 0.f;
  for (size_t t = 0; t < tokens; ++t) acc += tok_loss[t];
  total = acc;
  free(tok_loss);
  return (float)(total / (double)tokens);
}

/* ------------------------------------------------------------------ AdamW */
/* m,v EMA; decoupled decay p -= lr*wd*p; p -= lr*mhat/(sqrt(vhat)+eps)
 * (cpp/src/gpu_kernel/adamw_step.metal:49-68; host wrapper
 * cpp/src/Optimizer.cpp:139-149 supplies bc1 = 1-beta1^t, bc2 = 1-beta2^t). */
ORC_API void orc_adamw_step(float *p, const float *g, float *m, float *v,
                            size_t n, float lr, float beta1, float beta2,
                            float eps, float wd, float bc1, float bc2) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) {
    float gi = g[i];
    m[i] = beta1 * m[i] + (1.0f - beta1) * gi;
    v[i] = beta2 * v[i] + (1.0f - beta2) * gi * gi;
    float pi = p[i];
    if (wd > 0.0f) pi = pi - lr * wd * pi;
    float mh = m[i] / bc1, vh = v[i] / bc2;
    p[i] = pi - lr * mh / (sqrtf(vh) + eps);
  }
}

/* ----------------------------------------------------------- embeddings */
/* h[t,:] = table[id[t],:]  (cpp/src/Transformer.cpp:124-135);
 * scatter-add of grads (cpp/src/Transformer.cpp:524-537). */
ORC_API void orc_embedding_forward(const int32_t *ids, const float *table,
                                   float *h, size_t tokens, size_t H) {
  for (size_t t = 0; t < tokens; ++t)
    memcpy(h + t * H, table + (size_t)ids[t] * H, H * sizeof(float));
}
ORC_API void orc_embedding_backward(const int32_t *ids, const float *gh,
                                    float *gtable, size_t tokens, size_t H,
                                    size_t V) {
  memset(gtable, 0, V * H * sizeof(float));
  for (size_t t = 0; t < tokens; ++t) {
    float *row = gtable + (size_t)ids[t] * H;
    for (size_t d = 0; d < H; ++d) row[d] += gh[t * H + d];
  }
}

/* ======================================================= compositions === */

typedef struct {
  size_t B, S, H, I, nH, nKV, hd, V, L;
  float eps, rope_base;
} orc_cfg;

/* Per-layer parameter block, in this order, all row-major [in,out]
 * (cpp/src/Attention.cpp:40-43, cpp/src/Transformer.cpp:29-31):
 *   attn_norm_w[H], Wq[H,nH*hd], Wk[H,nKV*hd], Wv[H,nKV*hd], Wo[nH*hd,H],
 *   ffn_norm_w[H], w_gate[H,I], w_up[H,I], w_down[I,H]                    */
ORC_API size_t orc_layer_param_count(const orc_cfg *c) {
  size_t q = c->nH * c->hd, kv = c->nKV * c->hd;
  return c->H + c->H * q + 2 * c->H * kv + q * c->H + c->H + 2 * c->H * c->I +
         c->I * c->H;
}
/* Whole model: embedding[V,H], L layer blocks, final_norm_w[H], out_proj[H,V]
 * (cpp/src/Transformer.cpp:76-88). */
ORC_API size_t orc_model_param_count(const orc_cfg *c) {
  return c->V * c->H + c->L * orc_layer_param_count(c) + c->H + c->H * c->V;
}

typedef struct {
  const float *attn_norm_w, *Wq, *Wk, *Wv, *Wo, *ffn_norm_w, *w_gate, *w_up,
      *w_down;
} layer_w;
typedef struct {
  float *attn_norm_w, *Wq, *Wk, *Wv, *Wo, *ffn_norm_w, *w_gate, *w_up, *w_down;
} layer_g;

static void split_layer(const orc_cfg *c, const float *p, layer_w *w) {
  size_t q = c->nH * c->hd, kv = c->nKV * c->hd, H = c->H, I = c->I;
  w->attn_norm_w = p; p += H;
  w->Wq = p; p += H * q;
  w->Wk = p; p += H * kv;
  w->Wv = p; p += H * kv;
  w->Wo = p; p += q * H;
  w->ffn_norm_w = p; p += H;
  w->w_gate = p; p += H * I;
  w->w_up = p; p += H * I;
  w->w_down = p;
}

static float *falloc(size_t n) {
  float *p = (float *)malloc((n ? n : 1) * sizeof(float));
  if (!p) abort();
  return p;
}

/* State kept by the attention sub-layer forward for its backward. */
typedef struct {
  float *x_norm, *q4, *k4, *v4, *attn_output;
} attn_state;

/* Attention::forward (cpp/src/Attention.cpp:171-284): inner unit-weight
 * RMSNorm, Q/K/V projections, head split, RoPE, causal GQA core, Wo. */
static void attention_layer_forward(const orc_cfg *c, const float *x,
                                    const layer_w *w, const float *cos_t,
                                    const float *sin_t, float *out,
                                    attn_state *st) {
  size_t M = c->B * c->S, H = c->H, q = c->nH * c->hd, kv = c->nKV * c->hd;
  float *ones = falloc(H);
  for (size_t i = 0; i < H; ++i) ones[i] = 1.0f;
  st->x_norm = falloc(M * H);
  orc_rms_norm_forward(x, st->x_norm, ones, c->eps, M, H);
  float *tmp = falloc(M * q);
  st->q4 = falloc(M * q); st->k4 = falloc(M * kv); st->v4 = falloc(M * kv);
  orc_gemm(st->x_norm, w->Wq, tmp, M, q, H, 0, 0, 0);
  orc_reshape_to_4d(tmp, st->q4, c->B, c->nH, c->S, c->hd);
  orc_gemm(st->x_norm, w->Wk, tmp, M, kv, H, 0, 0, 0);
  orc_reshape_to_4d(tmp, st->k4, c->B, c->nKV, c->S, c->hd);
  orc_gemm(st->x_norm, w->Wv, tmp, M, kv, H, 0, 0, 0);
  orc_reshape_to_4d(tmp, st->v4, c->B, c->nKV, c->S, c->hd);
  orc_rope_apply(st->q4, cos_t, sin_t, c->B, c->nH, c->S, c->hd, 0);
  orc_rope_apply(st->k4, cos_t, sin_t, c->B, c->nKV, c->S, c->hd, 0);
  st->attn_output = falloc(M * q);
  orc_attention_forward(st->q4, st->k4, st->v4, st->attn_output, c->B, c->nH,
                        c->nKV, c->S, c->hd);
  orc_gemm(st->attn_output, w->Wo, out, M, H, q, 0, 0, 0);
  free(tmp); free(ones);
}
static void attn_state_free(attn_state *st) {
  free(st->x_norm); free(st->q4); free(st->k4); free(st->v4);
  free(st->attn_output);
}

/* Attention::backward (cpp/src/Attention.cpp:365-597).  Weight grads are
 * ASSIGNED (:483,:558-566), not accumulated. Returns grad wrt x. */
static void attention_layer_backward(const orc_cfg *c, const float *gout,
                                     const float *x, const layer_w *w,
                                     const float *cos_t, const float *sin_t,
                                     const attn_state *st, float *gx,
                                     layer_g *g) {
  size_t M = c->B * c->S, H = c->H, q = c->nH * c->hd, kv = c->nKV * c->hd;
  orc_gemm(st->attn_output, gout, g->Wo, q, H, M, 1, 0, 0);       /* :472-484 */
  float *g_attn = falloc(M * q);
  orc_gemm(gout, w->Wo, g_attn, M, q, H, 0, 1, 0);                /* :487-499 */
  float *dq4 = falloc(M * q), *dk4 = falloc(M * kv), *dv4 = falloc(M * kv);
  orc_attention_backward(st->q4, st->k4, st->v4, g_attn, dq4, dk4, dv4, c->B,
                         c->nH, c->nKV, c->S, c->hd);
  orc_rope_apply(dq4, cos_t, sin_t, c->B, c->nH, c->S, c->hd, 1); /* :544 */
  orc_rope_apply(dk4, cos_t, sin_t, c->B, c->nKV, c->S, c->hd, 1);
  float *dq = falloc(M * q), *dk = falloc(M * kv), *dv = falloc(M * kv);
  orc_reshape_to_3d(dq4, dq, c->B, c->nH, c->S, c->hd);           /* :547-549 */
  orc_reshape_to_3d(dk4, dk, c->B, c->nKV, c->S, c->hd);
  orc_reshape_to_3d(dv4, dv, c->B, c->nKV, c->S, c->hd);
  orc_gemm(st->x_norm, dq, g->Wq, H, q, M, 1, 0, 0);              /* :552-566 */
  orc_gemm(st->x_norm, dk, g->Wk, H, kv, M, 1, 0, 0);
  orc_gemm(st->x_norm, dv, g->Wv, H, kv, M, 1, 0, 0);
  float *g_xn = falloc(M * H);
  orc_gemm(dq, w->Wq, g_xn, M, H, q, 0, 1, 0);                    /* :569-590 */
  orc_gemm(dk, w->Wk, g_xn, M, H, kv, 0, 1, 1);
  orc_gemm(dv, w->Wv, g_xn, M, H, kv, 0, 1, 1);
  float *ones = falloc(H);
  for (size_t i = 0; i < H; ++i) ones[i] = 1.0f;
  orc_rms_norm_backward(g_xn, x, ones, gx, NULL, c->eps, M, H);   /* :593-594 */
  free(ones); free(g_xn); free(dq); free(dk); free(dv);
  free(dq4); free(dk4); free(dv4); free(g_attn);
}

/* Exported: Attention::forward / ::backward on host arrays. */
ORC_API void orc_attention_layer(const orc_cfg *c, const float *x,
                                 const float *Wq, const float *Wk,
                                 const float *Wv, const float *Wo,
                                 float *out, const float *gout, float *gx,
                                 float *gWq, float *gWk, float *gWv,
                                 float *gWo) {
  size_t half = c->hd / 2;
  float *cos_t = falloc(c->S * half), *sin_t = falloc(c->S * half);
  orc_rope_tables(cos_t, sin_t, c->S, c->hd, c->rope_base);
  layer_w w = {0}; w.Wq = Wq; w.Wk = Wk; w.Wv = Wv; w.Wo = Wo;
  attn_state st;
  attention_layer_forward(c, x, &w, cos_t, sin_t, out, &st);
  if (gout) {
    layer_g g = {0}; g.Wq = gWq; g.Wk = gWk; g.Wv = gWv; g.Wo = gWo;
    attention_layer_backward(c, gout, x, &w, cos_t, sin_t, &st, gx, &g);
  }
  attn_state_free(&st);
  free(cos_t); free(sin_t);
}

/* One decoder layer forward, CPU branch of the per-layer loop
 * (cpp/src/Transformer.cpp:145-188): h += attn(attn_norm(h));
 * h += swiglu(ffn_norm(h) Wg, ffn_norm(h) Wu) Wd. */
ORC_API void orc_layer_forward(const orc_cfg *c, const float *h_in,
                               const float *params, float *h_out) {
  size_t M = c->B * c->S, H = c->H, I = c->I, half = c->hd / 2;
  layer_w w; split_layer(c, params, &w);
  float *cos_t = falloc(c->S * half), *sin_t = falloc(c->S * half);
  orc_rope_tables(cos_t, sin_t, c->S, c->hd, c->rope_base);
  float *attn_in = falloc(M * H), *attn_out = falloc(M * H);
  orc_rms_norm_forward(h_in, attn_in, w.attn_norm_w, c->eps, M, H);
  attn_state st;
  attention_layer_forward(c, attn_in, &w, cos_t, sin_t, attn_out, &st);
  attn_state_free(&st);
  for (size_t i = 0; i < M * H; ++i) h_out[i] = h_in[i] + attn_out[i];
  float *ffn_in = falloc(M * H), *gate = falloc(M * I), *up = falloc(M * I),
        *act = falloc(M * I), *ffn_out = falloc(M * H);
  orc_rms_norm_forward(h_out, ffn_in, w.ffn_norm_w, c->eps, M, H);
  orc_gemm(ffn_in, w.w_gate, gate, M, I, H, 0, 0, 0);
  orc_gemm(ffn_in, w.w_up, up, M, I, H, 0, 0, 0);
  orc_swiglu_forward(gate, up, act, M * I);
  orc_gemm(act, w.w_down, ffn_out, M, H, I, 0, 0, 0);
  for (size_t i = 0; i < M * H; ++i) h_out[i] += ffn_out[i];
  free(cos_t); free(sin_t); free(attn_in); free(attn_out); free(ffn_in);
  free(gate); free(up); free(act); free(ffn_out);
}

/* TransformerLayer::backward (cpp/src/Transformer.cpp:322-474): recompute the
 * layer forward from h_in, then back-propagate.  FFN weight grads are
 * ACCUMULATED into the given buffers (:236,:288-289; pinned by the
 * reference's test_transformer TC-28); attention weight grads are assigned.
 * Norm-weight grads are written to grads when the slots exist (the
 * reference computes and discards them). */
ORC_API void orc_layer_backward(const orc_cfg *c, const float *grad_out,
                                const float *h_in, const float *params,
                                float *grads, float *grad_h_in) {
  size_t M = c->B * c->S, H = c->H, I = c->I, half = c->hd / 2;
  size_t q = c->nH * c->hd, kv = c->nKV * c->hd;
  layer_w w; split_layer(c, params, &w);
  layer_w gw_c; split_layer(c, grads, &gw_c);
  layer_g g;
  g.attn_norm_w = (float *)gw_c.attn_norm_w; g.Wq = (float *)gw_c.Wq;
  g.Wk = (float *)gw_c.Wk; g.Wv = (float *)gw_c.Wv; g.Wo = (float *)gw_c.Wo;
  g.ffn_norm_w = (float *)gw_c.ffn_norm_w; g.w_gate = (float *)gw_c.w_gate;
  g.w_up = (float *)gw_c.w_up; g.w_down = (float *)gw_c.w_down;
  (void)q; (void)kv;
  float *cos_t = falloc(c->S * half), *sin_t = falloc(c->S * half);
  orc_rope_tables(cos_t, sin_t, c->S, c->hd, c->rope_base);
  /* A. recompute (:372-379) */
  float *attn_in = falloc(M * H), *attn_out = falloc(M * H),
        *h_mid = falloc(M * H);
  orc_rms_norm_forward(h_in, attn_in, w.attn_norm_w, c->eps, M, H);
  attn_state st;
  attention_layer_forward(c, attn_in, &w, cos_t, sin_t, attn_out, &st);
  for (size_t i = 0; i < M * H; ++i) h_mid[i] = h_in[i] + attn_out[i];
  float *ffn_in = falloc(M * H), *gate = falloc(M * I), *up = falloc(M * I),
        *act = falloc(M * I);
  orc_rms_norm_forward(h_mid, ffn_in, w.ffn_norm_w, c->eps, M, H);
  orc_gemm(ffn_in, w.w_gate, gate, M, I, H, 0, 0, 0);
  orc_gemm(ffn_in, w.w_up, up, M, I, H, 0, 0, 0);
  orc_swiglu_forward(gate, up, act, M * I);
  /* B. down projection (:382-401) */
  orc_gemm(act, grad_out, g.w_down, I, H, M, 1, 0, 1);
  float *g_act = falloc(M * I);
  orc_gemm(grad_out, w.w_down, g_act, M, I, H, 0, 1, 0);
  /* C. SwiGLU + gate/up (:405-439) */
  float *g_gate = falloc(M * I), *g_up = falloc(M * I);
  orc_swiglu_backward(g_act, gate, up, g_gate, g_up, M * I);
  orc_gemm(ffn_in, g_gate, g.w_gate, H, I, M, 1, 0, 1);
  orc_gemm(ffn_in, g_up, g.w_up, H, I, M, 1, 0, 1);
  float *g_ffn_in = falloc(M * H);
  orc_gemm(g_gate, w.w_gate, g_ffn_in, M, H, I, 0, 1, 0);
  orc_gemm(g_up, w.w_up, g_ffn_in, M, H, I, 0, 1, 1);
  /* D. ffn norm + residual (:442-453) */
  float *g_h_mid = falloc(M * H);
  memset(g.ffn_norm_w, 0, H * sizeof(float));
  orc_rms_norm_backward(g_ffn_in, h_mid, w.ffn_norm_w, g_h_mid, g.ffn_norm_w,
                        c->eps, M, H);
  for (size_t i = 0; i < M * H; ++i) g_h_mid[i] += grad_out[i];
  /* E. attention (:456) */
  float *g_attn_in = falloc(M * H);
  attention_layer_backward(c, g_h_mid, attn_in, &w, cos_t, sin_t, &st,
                           g_attn_in, &g);
  /* F. attn norm + residual (:460-471) */
  memset(g.attn_norm_w, 0, H * sizeof(float));
  orc_rms_norm_backward(g_attn_in, h_in, w.attn_norm_w, grad_h_in,
                        g.attn_norm_w, c->eps, M, H);
  for (size_t i = 0; i < M * H; ++i) grad_h_in[i] += g_h_mid[i];
  attn_state_free(&st);
  free(cos_t); free(sin_t); free(attn_in); free(attn_out); free(h_mid);
  free(ffn_in); free(gate); free(up); free(act); free(g_act); free(g_gate);
  free(g_up); free(g_ffn_in); free(g_h_mid); free(g_attn_in);
}

/* Whole model: Transformer::forward (cpp/src/Transformer.cpp:90-197) ->
 * CrossEntropyLoss (cpp/src/Loss.cpp) -> Transformer::backward (:571-657).
 * params/grads use the flat layout of orc_model_param_count.  grads must be
 * zero-filled by the caller (the trainer does so each step,
 * cpp/src/Trainer.cpp:305-315).  logits_out (optional) is [B*S,V].
 * Returns the mean loss; when grads is NULL only the forward runs. */
ORC_API float orc_model_loss_and_grads(const orc_cfg *c, const int32_t *tokens,
                                       const int32_t *targets,
                                       const float *params, float *grads,
                                       float *logits_out) {
  size_t M = c->B * c->S, H = c->H, V = c->V, L = c->L;
  size_t lp = orc_layer_param_count(c);
  const float *emb = params, *layers = params + V * H;
  const float *final_w = layers + L * lp, *outp = final_w + H;
  float **hs = (float **)malloc((L + 1) * sizeof(float *));
  for (size_t l = 0; l <= L; ++l) hs[l] = falloc(M * H);
  orc_embedding_forward(tokens, emb, hs[0], M, H);
  for (size_t l = 0; l < L; ++l)
    orc_layer_forward(c, hs[l], layers + l * lp, hs[l + 1]);
  float *final_h = falloc(M * H);
  orc_rms_norm_forward(hs[L], final_h, final_w, c->eps, M, H);
  float *logits = logits_out ? logits_out : falloc(M * V);
  orc_gemm(final_h, outp, logits, M, V, H, 0, 0, 0);
  float *dlogits = grads ? falloc(M * V) : NULL;
  float loss = orc_cross_entropy(logits, targets, dlogits, M, V);
  if (grads) {
    float *g_emb = grads, *g_layers = grads + V * H;
    float *g_final_w = g_layers + L * lp, *g_outp = g_final_w + H;
    orc_gemm(final_h, dlogits, g_outp, H, V, M, 1, 0, 0);        /* :515-521 */
    float *g_final_h = falloc(M * H), *g_h = falloc(M * H),
          *g_prev = falloc(M * H);
    orc_gemm(dlogits, outp, g_final_h, M, H, V, 0, 1, 0);        /* :607-627 */
    memset(g_final_w, 0, H * sizeof(float));
    orc_rms_norm_backward(g_final_h, hs[L], final_w, g_h, g_final_w, c->eps, M,
                          H);                                    /* :632 */
    for (size_t l = L; l-- > 0;) {                               /* :638-642 */
      orc_layer_backward(c, g_h, hs[l], layers + l * lp, g_layers + l * lp,
                         g_prev);
      float *t = g_h; g_h = g_prev; g_prev = t;
    }
    orc_embedding_backward(tokens, g_h, g_emb, M, H, V);         /* :649 */
    free(g_final_h); free(g_h); free(g_prev); free(dlogits);
  }
  if (!logits_out) free(logits);
  free(final_h);
  for (size_t l = 0; l <= L; ++l) free(hs[l]);
  free(hs);
  return loss;
}
