// Bandwidth-bound kernels of the decoder block: RMSNorm (+residual fusions),
// RoPE, SwiGLU, residual add, head split/merge, embedding gather/scatter,
// cross-entropy, AdamW, dtype conversion, seeded fill.
// All are 16-byte vectorised, coalesced, warp-shuffle reduced; maths in fp32.
#include "common.cuh"

// =========================================================== RMSNorm =====
// One CTA per row (grid-stride over rows).  The row is held in registers
// (up to VPT 16-byte vectors per thread) so x is read from HBM exactly once.
//   forward : [h += r;]  y = h * rstd * w          (rstd optionally saved)
//   backward: dx = rstd*(g*w - xhat*mean(g*w*xhat)) [+ residual_grad]; dw += sum_rows g*xhat
// Reference: cpp/src/gpu_kernel/rms_norm_forward.metal:29-60, fused_add_norm.metal:25-72,
// cpp/src/RMSNorm.cpp:126-160, fused_backward_add_norm.metal:19-84.
constexpr int NORM_THREADS = 256;
constexpr int NORM_VPT = 4;  // register-cached vectors per thread

template <class T, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_fwd_kernel(const T *x, T *h_out, const T *__restrict__ r,
                    const T *__restrict__ w, T *__restrict__ y, float *__restrict__ rstd_out, float eps,
                    size_t rows, int D) {
  constexpr int N = Vec16<T>::N;
  __shared__ float red[32];
  const int nvec = D / N;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *xr = x + row * (size_t)D;
    float vals[NORM_VPT][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        Vec16<T> a; a.load(xr + v * N); a.unpack(vals[i]);
        if (ADD) {
          Vec16<T> b; float rb[N]; b.load(r + row * (size_t)D + v * N); b.unpack(rb);
#pragma unroll
          for (int j = 0; j < N; ++j) vals[i][j] += rb[j];
          // the stored residual stream is the rounded value; normalise what is stored
          Vec16<T> o; o.pack(vals[i]); o.store(h_out + row * (size_t)D + v * N); o.unpack(vals[i]);
        }
#pragma unroll
        for (int j = 0; j < N; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    // columns beyond the register cache (very wide rows): re-read
    for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
      Vec16<T> a; float f[N]; a.load(xr + v * N); a.unpack(f);
      if (ADD) {
        Vec16<T> b; float rb[N]; b.load(r + row * (size_t)D + v * N); b.unpack(rb);
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] += rb[j];
        Vec16<T> o; o.pack(f); o.store(h_out + row * (size_t)D + v * N); o.unpack(f);
      }
#pragma unroll
      for (int j = 0; j < N; ++j) ss += f[j] * f[j];
    }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / (float)D + eps);
    if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
    T *yr = y + row * (size_t)D;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        Vec16<T> wv; float wf[N], o[N]; wv.load(w + v * N); wv.unpack(wf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = vals[i][j] * rstd * wf[j];
        Vec16<T> ov; ov.pack(o); ov.store(yr + v * N);
      }
    }
    for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
      const T *src = (ADD ? (const T *)h_out : x) + row * (size_t)D;
      Vec16<T> a, wv; float f[N], wf[N], o[N];
      a.load(src + v * N); a.unpack(f); wv.load(w + v * N); wv.unpack(wf);
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = f[j] * rstd * wf[j];
      Vec16<T> ov; ov.pack(o); ov.store(yr + v * N);
    }
  }
}

// Scalar variant for row widths that are not a multiple of the vector width.
template <class T, bool ADD>
__global__ void rms_norm_fwd_scalar_kernel(const T *x, T *h_out, const T *r, const T *w, T *y, float *rstd_out,
                                           float eps, size_t rows, int D) {
  __shared__ float red[32];
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float v;
      if (ADD) {
        v = to_f(x[row * D + c]) + to_f(r[row * D + c]);
        T s = from_f<T>(v); h_out[row * D + c] = s; v = to_f(s);
      } else v = to_f(x[row * D + c]);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / (float)D + eps);
    if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
    const T *src = ADD ? (const T *)h_out : x;
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      y[row * D + c] = from_f<T>(to_f(src[row * D + c]) * rstd * to_f(w[c]));
  }
}

template <class T, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_bwd_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ w,
                    const T *__restrict__ res_grad, T *__restrict__ dx, float *__restrict__ dw, float eps,
                    size_t rows, int D) {
  constexpr int N = Vec16<T>::N;
  __shared__ float red[32];
  const int nvec = D / N;
  float dw_acc[NORM_VPT][N];
#pragma unroll
  for (int i = 0; i < NORM_VPT; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) dw_acc[i][j] = 0.f;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float xv[NORM_VPT][N], gv[NORM_VPT][N], wv[NORM_VPT][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        Vec16<T> a, b, c;
        a.load(x + row * (size_t)D + v * N); a.unpack(xv[i]);
        b.load(g + row * (size_t)D + v * N); b.unpack(gv[i]);
        c.load(w + v * N); c.unpack(wv[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) ss += xv[i][j] * xv[i][j];
      }
    }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / (float)D + eps);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) s += gv[i][j] * wv[i][j] * (xv[i][j] * rstd);
      }
    }
    s = block_sum(s, red) / (float)D;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float o[N];
        if (ADD) { Vec16<T> rg; rg.load(res_grad + row * (size_t)D + v * N); rg.unpack(o); }
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xhat = xv[i][j] * rstd;
          float d = rstd * (gv[i][j] * wv[i][j] - xhat * s);
          o[j] = ADD ? o[j] + d : d;
          dw_acc[i][j] += gv[i][j] * xhat;
        }
        Vec16<T> ov; ov.pack(o); ov.store(dx + row * (size_t)D + v * N);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec)
#pragma unroll
        for (int j = 0; j < N; ++j) atomicAdd(dw + v * N + j, dw_acc[i][j]);
    }
  }
}

// Generic (any D) backward: values re-read instead of cached.
template <class T, bool ADD>
__global__ void rms_norm_bwd_scalar_kernel(const T *g, const T *x, const T *w, const T *res_grad, T *dx, float *dw,
                                           float eps, size_t rows, int D) {
  __shared__ float red[32];
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) { float v = to_f(x[row * D + c]); ss += v * v; }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / (float)D + eps);
    float s = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      s += to_f(g[row * D + c]) * to_f(w[c]) * (to_f(x[row * D + c]) * rstd);
    s = block_sum(s, red) / (float)D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float xhat = to_f(x[row * D + c]) * rstd, gg = to_f(g[row * D + c]);
      float d = rstd * (gg * to_f(w[c]) - xhat * s);
      if (ADD) d += to_f(res_grad[row * D + c]);
      dx[row * D + c] = from_f<T>(d);
      if (dw) atomicAdd(dw + c, gg * xhat);
    }
  }
}

static int norm_grid(b200_ctx *ctx, size_t rows) {
  size_t cap = (size_t)ctx->sm_count * 8;
  return (int)(rows < cap ? (rows ? rows : 1) : cap);
}

// warp-per-row kernels (norm_warp.cu): 1 = launched, 0 = shape does not fit, < 0 = error
template <class T>
int rms_fwd_warp(b200_ctx *, const void *, void *, const void *, const void *, void *, float *, float, size_t, size_t, bool,
                 const void *w2 = nullptr, void *y2 = nullptr);
template <class T>
int rms_bwd_warp(b200_ctx *, const void *, const void *, const void *, const void *, void *, float *, float, size_t, size_t, bool);

template <class T>
static int rms_fwd_t(b200_ctx *ctx, const void *x, void *h, const void *r, const void *w, void *y, float *rstd,
                     float eps, size_t rows, size_t D, bool add) {   // h: where x + r is stored (may be x itself)
  constexpr int N = Vec16<T>::N;
  if (int rc = rms_fwd_warp<T>(ctx, x, h, r, w, y, rstd, eps, rows, D, add)) return rc < 0 ? rc : B200_OK;
  int grid = norm_grid(ctx, rows);
  bool vec = (D % N == 0) && (((uintptr_t)x | (uintptr_t)h | (uintptr_t)r | (uintptr_t)w | (uintptr_t)y) % 16 == 0);
  if (vec) {
    if (add) rms_norm_fwd_kernel<T, true><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, rows, (int)D);
    else rms_norm_fwd_kernel<T, false><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, rows, (int)D);
  } else {
    if (add) rms_norm_fwd_scalar_kernel<T, true><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, rows, (int)D);
    else rms_norm_fwd_scalar_kernel<T, false><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, rows, (int)D);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}

template <class T>
static int rms_bwd_t(b200_ctx *ctx, const void *g, const void *x, const void *w, const void *rg, void *dx, float *dw,
                     float eps, size_t rows, size_t D, bool add) {
  constexpr int N = Vec16<T>::N;
  if (int rc = rms_bwd_warp<T>(ctx, g, x, w, rg, dx, dw, eps, rows, D, add)) return rc < 0 ? rc : B200_OK;
  int grid = norm_grid(ctx, rows);
  bool vec = (D % N == 0) && (D / N <= (size_t)NORM_VPT * NORM_THREADS) &&
             (((uintptr_t)g | (uintptr_t)x | (uintptr_t)w | (uintptr_t)rg | (uintptr_t)dx) % 16 == 0);
  if (vec) {
    if (add) rms_norm_bwd_kernel<T, true><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)g, (const T *)x, (const T *)w, (const T *)rg, (T *)dx, dw, eps, rows, (int)D);
    else rms_norm_bwd_kernel<T, false><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)g, (const T *)x, (const T *)w, (const T *)rg, (T *)dx, dw, eps, rows, (int)D);
  } else {
    if (add) rms_norm_bwd_scalar_kernel<T, true><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)g, (const T *)x, (const T *)w, (const T *)rg, (T *)dx, dw, eps, rows, (int)D);
    else rms_norm_bwd_scalar_kernel<T, false><<<grid, NORM_THREADS, 0, ctx->stream>>>((const T *)g, (const T *)x, (const T *)w, (const T *)rg, (T *)dx, dw, eps, rows, (int)D);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}

extern "C" int b200_rms_norm_forward(b200_ctx *ctx, const void *x, void *y, const void *w, float *rstd, float eps,
                                     size_t rows, size_t D, b200_dtype dt) {
  B200_REQUIRE(ctx, x && y && w && D > 0, "rms_norm_forward: null pointer or empty row");
  if (rows == 0) return B200_OK;
  return dt == B200_BF16 ? rms_fwd_t<bf16>(ctx, x, nullptr, nullptr, w, y, rstd, eps, rows, D, false)
                         : rms_fwd_t<float>(ctx, x, nullptr, nullptr, w, y, rstd, eps, rows, D, false);
}
extern "C" int b200_fused_add_norm(b200_ctx *ctx, void *h, const void *r, const void *w, void *out, size_t rows,
                                   size_t D, float eps, b200_dtype dt) {
  B200_REQUIRE(ctx, h && r && w && out && D > 0, "fused_add_norm: null pointer or empty row");
  if (rows == 0) return B200_OK;
  return dt == B200_BF16 ? rms_fwd_t<bf16>(ctx, h, h, r, w, out, nullptr, eps, rows, D, true)
                         : rms_fwd_t<float>(ctx, h, h, r, w, out, nullptr, eps, rows, D, true);
}
// Out-of-place form used by the engine: h_out = x + r; y = rmsnorm(h_out) * w.
int add_norm_oop(b200_ctx *ctx, const void *x, const void *r, void *h_out, const void *w, void *y, size_t rows,
                 size_t D, float eps, b200_dtype dt) {
  if (rows == 0) return B200_OK;
  return dt == B200_BF16 ? rms_fwd_t<bf16>(ctx, x, h_out, r, w, y, nullptr, eps, rows, D, true)
                         : rms_fwd_t<float>(ctx, x, h_out, r, w, y, nullptr, eps, rows, D, true);
}
// Engine form of the block entry: h_out = x (+ r); y = rmsnorm(h_out) * w; y2 = rmsnorm(y) * w2, one pass when the
// row fits the warp kernel.  r may be null (no add; h_out unused); y may be null when only y2 is wanted.
int add_norm_norm_oop(b200_ctx *ctx, const void *x, const void *r, void *h_out, const void *w, void *y, const void *w2,
                      void *y2, void *y_scratch, size_t rows, size_t D, float eps, b200_dtype dt) {
  if (rows == 0) return B200_OK;
  const bool add = r != nullptr;
  const int rc = dt == B200_BF16 ? rms_fwd_warp<bf16>(ctx, x, h_out, r, w, y, nullptr, eps, rows, D, add, w2, y2)
                                 : rms_fwd_warp<float>(ctx, x, h_out, r, w, y, nullptr, eps, rows, D, add, w2, y2);
  if (rc) return rc < 0 ? rc : B200_OK;
  void *y1 = y ? y : y_scratch;                    // two passes for shapes the warp kernel does not take
  B200_REQUIRE(ctx, y1, "add_norm_norm: no buffer for the first norm's output");
  const int r1 = dt == B200_BF16 ? rms_fwd_t<bf16>(ctx, x, h_out, r, w, y1, nullptr, eps, rows, D, add)
                                 : rms_fwd_t<float>(ctx, x, h_out, r, w, y1, nullptr, eps, rows, D, add);
  if (r1) return r1;
  return b200_rms_norm_forward(ctx, y1, y2, w2, nullptr, eps, rows, D, dt);
}
template <class T>
int rms_bwd2_warp(b200_ctx *, const void *, const void *, const void *, const void *, void *, float, size_t, size_t);
// Engine form: backward of y2 = rmsnorm(rmsnorm(h) * w) (second norm with unit weight) plus the residual gradient in
// one pass, without the first norm's output.  Returns 1 when done, 0 when the row shape needs the two-pass route.
int norm_norm_backward_fused(b200_ctx *ctx, const void *g, const void *h, const void *w, const void *res_grad, void *dx,
                             size_t rows, size_t D, float eps, b200_dtype dt) {
  if (rows == 0) return 1;
  return dt == B200_BF16 ? rms_bwd2_warp<bf16>(ctx, g, h, w, res_grad, dx, eps, rows, D)
                         : rms_bwd2_warp<float>(ctx, g, h, w, res_grad, dx, eps, rows, D);
}
extern "C" int b200_rms_norm_backward(b200_ctx *ctx, const void *g, const void *x, const void *w, void *dx,
                                      float *dw, float eps, size_t rows, size_t D, b200_dtype dt) {
  B200_REQUIRE(ctx, g && x && w && dx && D > 0, "rms_norm_backward: null pointer or empty row");
  if (rows == 0) return B200_OK;
  return dt == B200_BF16 ? rms_bwd_t<bf16>(ctx, g, x, w, nullptr, dx, dw, eps, rows, D, false)
                         : rms_bwd_t<float>(ctx, g, x, w, nullptr, dx, dw, eps, rows, D, false);
}
extern "C" int b200_fused_backward_add_norm(b200_ctx *ctx, const void *g, const void *x, const void *w,
                                            const void *rg, void *dx, size_t rows, size_t D, float eps,
                                            b200_dtype dt) {
  B200_REQUIRE(ctx, g && x && w && rg && dx && D > 0, "fused_backward_add_norm: null pointer or empty row");
  if (rows == 0) return B200_OK;
  return dt == B200_BF16 ? rms_bwd_t<bf16>(ctx, g, x, w, rg, dx, nullptr, eps, rows, D, true)
                         : rms_bwd_t<float>(ctx, g, x, w, rg, dx, nullptr, eps, rows, D, true);
}

// ============================================================== RoPE =====
// Interleaved pairs (2i, 2i+1) rotated by (cos,sin)[s,i]; backward is the
// inverse rotation (cpp/src/Positional.cpp:120-147, 207-231).  The tensor is
// addressed as base + b*sb + h*sh + s*ss + d so that both the reference's
// [B,heads,S,hd] layout and the engine's token-major fused QKV rows are served.
__global__ void rope_tables_kernel(float *cos_t, float *sin_t, int max_seq, int hd, float base) {
  int half = hd / 2;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= max_seq * half) return;
  int pos = idx / half, i = idx % half;
  // theta = 1 / base^(2i/hd), evaluated in fp32 like the reference (Positional.cpp:57-60)
  float exponent = (2.0f * (float)i) / (float)hd;
  float theta = 1.0f / powf(base, exponent);
  float a = (float)pos * theta;
  cos_t[idx] = cosf(a);
  sin_t[idx] = sinf(a);
}

template <class T, bool BWD>
__global__ void rope_kernel(T *__restrict__ t, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                            int heads, int S, int hd, long long sb, long long sh, long long ss, size_t total_pairs4) {
  // each thread rotates 4 consecutive pairs (8 elements) when hd % 8 == 0, else 1 pair
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_pairs4) return;
  int quads = hd / 8;
  int qd = (int)(idx % quads);
  size_t r = idx / quads;
  int s = (int)(r % S); r /= S;
  int h = (int)(r % heads);
  size_t b = r / heads;
  T *p = t + b * sb + h * sh + (long long)s * ss + qd * 8;
  const float *c = cos_t + (size_t)s * (hd / 2) + qd * 4;
  const float *sn = sin_t + (size_t)s * (hd / 2) + qd * 4;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = to_f(p[j]);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float x0 = v[2 * j], x1 = v[2 * j + 1], cc = c[j], s_ = sn[j];
    if (!BWD) { v[2 * j] = x0 * cc - x1 * s_; v[2 * j + 1] = x0 * s_ + x1 * cc; }
    else      { v[2 * j] = x0 * cc + x1 * s_; v[2 * j + 1] = -x0 * s_ + x1 * cc; }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) p[j] = from_f<T>(v[j]);
}
template <class T, bool BWD>
__global__ void rope_pair_kernel(T *t, const float *cos_t, const float *sin_t, int heads, int S, int hd,
                                 long long sb, long long sh, long long ss, size_t total_pairs) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_pairs) return;
  int half = hd / 2;
  int i = (int)(idx % half);
  size_t r = idx / half;
  int s = (int)(r % S); r /= S;
  int h = (int)(r % heads);
  size_t b = r / heads;
  T *p = t + b * sb + h * sh + (long long)s * ss + 2 * i;
  float x0 = to_f(p[0]), x1 = to_f(p[1]), cc = cos_t[(size_t)s * half + i], s_ = sin_t[(size_t)s * half + i];
  if (!BWD) { p[0] = from_f<T>(x0 * cc - x1 * s_); p[1] = from_f<T>(x0 * s_ + x1 * cc); }
  else      { p[0] = from_f<T>(x0 * cc + x1 * s_); p[1] = from_f<T>(-x0 * s_ + x1 * cc); }
}

int rope_strided(b200_ctx *ctx, void *t, const float *cos_t, const float *sin_t, size_t B, size_t heads, size_t S,
                 size_t hd, long long sb, long long sh, long long ss, b200_dtype dt, bool bwd) {
  B200_REQUIRE(ctx, t && cos_t && sin_t && hd % 2 == 0, "rope: null pointer or odd head_dim");
  if (B * heads * S == 0) return B200_OK;
  if (hd % 8 == 0) {
    size_t total = B * heads * S * (hd / 8);
    int grid = (int)((total + 255) / 256);
#define RL(T_, BW) rope_kernel<T_, BW><<<grid, 256, 0, ctx->stream>>>((T_ *)t, cos_t, sin_t, (int)heads, (int)S, (int)hd, sb, sh, ss, total)
    if (dt == B200_BF16) { if (bwd) RL(bf16, true); else RL(bf16, false); }
    else { if (bwd) RL(float, true); else RL(float, false); }
#undef RL
  } else {
    size_t total = B * heads * S * (hd / 2);
    int grid = (int)((total + 255) / 256);
#define RL(T_, BW) rope_pair_kernel<T_, BW><<<grid, 256, 0, ctx->stream>>>((T_ *)t, cos_t, sin_t, (int)heads, (int)S, (int)hd, sb, sh, ss, total)
    if (dt == B200_BF16) { if (bwd) RL(bf16, true); else RL(bf16, false); }
    else { if (bwd) RL(float, true); else RL(float, false); }
#undef RL
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}

extern "C" int b200_rope_tables(b200_ctx *ctx, float *cos_t, float *sin_t, size_t max_seq, size_t hd, float base) {
  B200_REQUIRE(ctx, cos_t && sin_t && hd % 2 == 0 && hd > 0, "rope_tables: bad arguments");
  size_t n = max_seq * (hd / 2);
  if (!n) return B200_OK;
  rope_tables_kernel<<<(int)((n + 255) / 256), 256, 0, ctx->stream>>>(cos_t, sin_t, (int)max_seq, (int)hd, base);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
extern "C" int b200_rope_forward(b200_ctx *ctx, void *q, void *k, const float *cos_t, const float *sin_t, size_t B,
                                 size_t qh, size_t kvh, size_t S, size_t hd, b200_dtype dt) {
  int rc = rope_strided(ctx, q, cos_t, sin_t, B, qh, S, hd, (long long)(qh * S * hd), (long long)(S * hd), (long long)hd, dt, false);
  if (rc) return rc;
  return rope_strided(ctx, k, cos_t, sin_t, B, kvh, S, hd, (long long)(kvh * S * hd), (long long)(S * hd), (long long)hd, dt, false);
}
extern "C" int b200_rope_backward(b200_ctx *ctx, void *g, const float *cos_t, const float *sin_t, size_t B,
                                  size_t heads, size_t S, size_t hd, b200_dtype dt) {
  return rope_strided(ctx, g, cos_t, sin_t, B, heads, S, hd, (long long)(heads * S * hd), (long long)(S * hd), (long long)hd, dt, true);
}

// ============================================================ SwiGLU =====
// out = g*sigmoid(g)*u ; d_up = dy*silu(g) ; d_gate = dy*u*sig*(1+g*(1-sig))
// (cpp/src/Activations.cpp:31-75, 119-167).  Row-strided so the engine can
// read gate|up from one fused [rows, 2*cols] buffer.
template <class T>
__global__ void swiglu_fwd_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out,
                                  size_t rows, size_t cols, size_t ld_in, size_t ld_out) {
  constexpr int N = Vec16<T>::N;
  size_t vec_per_row = cols / N, total = rows * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t r = idx / vec_per_row, c = (idx % vec_per_row) * N;
    Vec16<T> a, b; float g[N], u[N], o[N];
    a.load(gate + r * ld_in + c); a.unpack(g);
    b.load(up + r * ld_in + c); b.unpack(u);
#pragma unroll
    for (int j = 0; j < N; ++j) { float sig = 1.0f / (1.0f + __expf(-g[j])); o[j] = g[j] * sig * u[j]; }
    Vec16<T> ov; ov.pack(o); ov.store(out + r * ld_out + c);
  }
}
template <class T>
__global__ void swiglu_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ gate, const T *__restrict__ up,
                                  T *__restrict__ dgate, T *__restrict__ dup, size_t rows, size_t cols, size_t ld_dy,
                                  size_t ld_in, size_t ld_out) {
  constexpr int N = Vec16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  size_t vec_per_row = cols / N, total = rows * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t r = idx / vec_per_row, c = (idx % vec_per_row) * N;
    Vec16<T> a, b, d; float g[N], u[N], y[N], og[N], ou[N];
    a.load(gate + r * ld_in + c); a.unpack(g);
    b.load(up + r * ld_in + c); b.unpack(u);
    d.load(dy + r * ld_dy + c); d.unpack(y);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float sig = 1.0f / (1.0f + __expf(-g[j]));
      ou[j] = y[j] * g[j] * sig;
      og[j] = y[j] * u[j] * sig * (1.0f + g[j] * (1.0f - sig));
    }
    Vec16<T> v1, v2; v1.pack(og); v1.store(dgate + r * ld_out + c); v2.pack(ou); v2.store(dup + r * ld_out + c);
  }
}
template <class T>
__global__ void swiglu_fwd_scalar(const T *gate, const T *up, T *out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float g = to_f(gate[i]), sig = 1.0f / (1.0f + __expf(-g));
    out[i] = from_f<T>(g * sig * to_f(up[i]));
  }
}
template <class T>
__global__ void swiglu_bwd_scalar(const T *dy, const T *gate, const T *up, T *dgate, T *dup, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float g = to_f(gate[i]), u = to_f(up[i]), y = to_f(dy[i]), sig = 1.0f / (1.0f + __expf(-g));
    dup[i] = from_f<T>(y * g * sig);
    dgate[i] = from_f<T>(y * u * sig * (1.0f + g * (1.0f - sig)));
  }
}
static int ew_grid(b200_ctx *ctx, size_t work_items) {
  size_t blocks = (work_items + 255) / 256, cap = (size_t)ctx->sm_count * 16;
  return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}
int swiglu_fwd_strided(b200_ctx *ctx, const void *gate, const void *up, void *out, size_t rows, size_t cols,
                       size_t ld_in, size_t ld_out, b200_dtype dt) {
  if (rows * cols == 0) return B200_OK;
  size_t N = 16 / dtype_size(dt);
  bool vec = cols % N == 0 && ld_in % N == 0 && ld_out % N == 0 && (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) % 16 == 0);
  if (vec) {
    int grid = ew_grid(ctx, rows * cols / N);
    if (dt == B200_BF16) swiglu_fwd_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)gate, (const bf16 *)up, (bf16 *)out, rows, cols, ld_in, ld_out);
    else swiglu_fwd_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)gate, (const float *)up, (float *)out, rows, cols, ld_in, ld_out);
  } else {
    B200_REQUIRE(ctx, ld_in == cols && ld_out == cols, "swiglu: unaligned strided form unsupported");
    int grid = ew_grid(ctx, rows * cols);
    if (dt == B200_BF16) swiglu_fwd_scalar<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)gate, (const bf16 *)up, (bf16 *)out, rows * cols);
    else swiglu_fwd_scalar<float><<<grid, 256, 0, ctx->stream>>>((const float *)gate, (const float *)up, (float *)out, rows * cols);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}
int swiglu_bwd_strided(b200_ctx *ctx, const void *dy, const void *gate, const void *up, void *dgate, void *dup,
                       size_t rows, size_t cols, size_t ld_dy, size_t ld_in, size_t ld_out, b200_dtype dt) {
  if (rows * cols == 0) return B200_OK;
  size_t N = 16 / dtype_size(dt);
  bool vec = cols % N == 0 && ld_in % N == 0 && ld_out % N == 0 && ld_dy % N == 0 &&
             (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)dy | (uintptr_t)dgate | (uintptr_t)dup) % 16 == 0);
  if (vec) {
    int grid = ew_grid(ctx, rows * cols / N);
    if (dt == B200_BF16) launch_k(ctx, swiglu_bwd_kernel<bf16>, dim3(grid), dim3(256), 0, 0, (const bf16 *)dy, (const bf16 *)gate, (const bf16 *)up, (bf16 *)dgate, (bf16 *)dup, rows, cols, ld_dy, ld_in, ld_out);
    else launch_k(ctx, swiglu_bwd_kernel<float>, dim3(grid), dim3(256), 0, 0, (const float *)dy, (const float *)gate, (const float *)up, (float *)dgate, (float *)dup, rows, cols, ld_dy, ld_in, ld_out);
  } else {
    B200_REQUIRE(ctx, ld_in == cols && ld_out == cols && ld_dy == cols, "swiglu: unaligned strided form unsupported");
    int grid = ew_grid(ctx, rows * cols);
    if (dt == B200_BF16) swiglu_bwd_scalar<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)dy, (const bf16 *)gate, (const bf16 *)up, (bf16 *)dgate, (bf16 *)dup, rows * cols);
    else swiglu_bwd_scalar<float><<<grid, 256, 0, ctx->stream>>>((const float *)dy, (const float *)gate, (const float *)up, (float *)dgate, (float *)dup, rows * cols);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}
extern "C" int b200_swiglu_forward(b200_ctx *ctx, const void *gate, const void *up, void *out, size_t n, b200_dtype dt) {
  B200_REQUIRE(ctx, gate && up && out, "swiglu_forward: null pointer");
  return swiglu_fwd_strided(ctx, gate, up, out, 1, n, n, n, dt);
}
extern "C" int b200_swiglu_backward(b200_ctx *ctx, const void *dy, const void *gate, const void *up, void *dgate,
                                    void *dup, size_t n, b200_dtype dt) {
  B200_REQUIRE(ctx, dy && gate && up && dgate && dup, "swiglu_backward: null pointer");
  return swiglu_bwd_strided(ctx, dy, gate, up, dgate, dup, 1, n, n, n, n, dt);
}

// ===================================================== residual add etc. ==
template <class T>
__global__ void add_kernel(T *__restrict__ a, const T *__restrict__ b, size_t n) {
  constexpr int N = Vec16<T>::N;
  size_t nv = n / N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Vec16<T> x, y; float fx[N], fy[N];
    x.load(a + i * N); x.unpack(fx); y.load(b + i * N); y.unpack(fy);
#pragma unroll
    for (int j = 0; j < N; ++j) fx[j] += fy[j];
    x.pack(fx); x.store(a + i * N);
  }
  for (size_t i = nv * N + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    a[i] = from_f<T>(to_f(a[i]) + to_f(b[i]));
}
template <class T>
__global__ void add_scalar_kernel(T *a, const T *b, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    a[i] = from_f<T>(to_f(a[i]) + to_f(b[i]));
}
extern "C" int b200_residual_add(b200_ctx *ctx, void *a, const void *b, size_t n, b200_dtype dt) {
  B200_REQUIRE(ctx, a && b, "residual_add: null pointer");
  if (!n) return B200_OK;
  bool al = (((uintptr_t)a | (uintptr_t)b) % 16) == 0;
  int grid = ew_grid(ctx, al ? n / (16 / dtype_size(dt)) + 1 : n);
  if (dt == B200_BF16) { if (al) add_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((bf16 *)a, (const bf16 *)b, n); else add_scalar_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((bf16 *)a, (const bf16 *)b, n); }
  else { if (al) add_kernel<float><<<grid, 256, 0, ctx->stream>>>((float *)a, (const float *)b, n); else add_scalar_kernel<float><<<grid, 256, 0, ctx->stream>>>((float *)a, (const float *)b, n); }
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// [B,S,n*hd] <-> [B,n,S,hd]  (cpp/src/Attention.cpp:68-152).  The engine never
// needs these (its attention kernels read the token-major layout directly);
// they exist for callers that keep the reference's 4-D layout.
template <class T, bool TO4D>
__global__ void reshape_heads_kernel(const T *__restrict__ src, T *__restrict__ dst, size_t B, size_t n, size_t S,
                                     size_t hd) {
  size_t total = B * n * S * hd;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t d = i % hd, r = i / hd;
    size_t s = r % S; r /= S;
    size_t h = r % n, b = r / n;
    size_t i3 = (b * S + s) * (n * hd) + h * hd + d;   // i is the 4-D index
    if (TO4D) dst[i] = src[i3]; else dst[i3] = src[i];
  }
}
extern "C" int b200_reshape_to_4d(b200_ctx *ctx, const void *src, void *dst, size_t B, size_t n, size_t S, size_t hd,
                                  b200_dtype dt) {
  B200_REQUIRE(ctx, src && dst, "reshape_to_4d: null pointer");
  size_t total = B * n * S * hd;
  if (!total) return B200_OK;
  int grid = ew_grid(ctx, total);
  if (dt == B200_BF16) reshape_heads_kernel<bf16, true><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, B, n, S, hd);
  else reshape_heads_kernel<float, true><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, B, n, S, hd);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
extern "C" int b200_reshape_to_3d(b200_ctx *ctx, const void *src, void *dst, size_t B, size_t n, size_t S, size_t hd,
                                  b200_dtype dt) {
  B200_REQUIRE(ctx, src && dst, "reshape_to_3d: null pointer");
  size_t total = B * n * S * hd;
  if (!total) return B200_OK;
  int grid = ew_grid(ctx, total);
  if (dt == B200_BF16) reshape_heads_kernel<bf16, false><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, B, n, S, hd);
  else reshape_heads_kernel<float, false><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, B, n, S, hd);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// =========================================================== embedding ====
template <class T>
__global__ void embedding_fwd_kernel(const uint32_t *__restrict__ ids, const T *__restrict__ table,
                                     T *__restrict__ out, size_t tokens, size_t H, size_t V, int *status) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    uint32_t id = ids[t];
    if (id >= V) { if (threadIdx.x == 0) atomicExch(status, 2); id = (uint32_t)(V - 1); }  // reference throws (Transformer.cpp:127-129)
    for (size_t c = threadIdx.x; c < H; c += blockDim.x) out[t * H + c] = table[(size_t)id * H + c];
  }
}
template <class T>
__global__ void embedding_bwd_kernel(const uint32_t *__restrict__ ids, const T *__restrict__ gh,
                                     float *__restrict__ gtable, size_t tokens, size_t H, size_t V) {
  for (size_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    uint32_t id = ids[t];
    if (id >= V) continue;
    for (size_t c = threadIdx.x; c < H; c += blockDim.x) atomicAdd(gtable + (size_t)id * H + c, to_f(gh[t * H + c]));
  }
}
// Bit-reproducible form: one thread per column walks the tokens in order.
template <class T>
__global__ void embedding_bwd_ordered_kernel(const uint32_t *__restrict__ ids, const T *__restrict__ gh,
                                             float *gtable, size_t tokens, size_t H, size_t V) {
  const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  for (size_t t = 0; t < tokens; ++t) {
    const uint32_t id = ids[t];
    if (id < V) gtable[(size_t)id * H + c] += to_f(gh[t * H + c]);
  }
}
extern "C" int b200_embedding_forward(b200_ctx *ctx, const uint32_t *ids, const void *table, void *out,
                                      size_t tokens, size_t H, size_t V, b200_dtype dt) {
  B200_REQUIRE(ctx, ids && table && out && H && V, "embedding_forward: bad arguments");
  if (!tokens) return B200_OK;
  int grid = (int)(tokens < (size_t)ctx->sm_count * 16 ? tokens : (size_t)ctx->sm_count * 16);
  if (dt == B200_BF16) B200_CUDA(ctx, launch_k(ctx, embedding_fwd_kernel<bf16>, dim3(grid), dim3(256), 0, 0, ids, (const bf16 *)table, (bf16 *)out, tokens, H, V, ctx->dev_status));
  else B200_CUDA(ctx, launch_k(ctx, embedding_fwd_kernel<float>, dim3(grid), dim3(256), 0, 0, ids, (const float *)table, (float *)out, tokens, H, V, ctx->dev_status));
  B200_LAUNCHED(ctx);
  return B200_OK;
}
extern "C" int b200_embedding_backward(b200_ctx *ctx, const uint32_t *ids, const void *gh, float *gtable,
                                       size_t tokens, size_t H, size_t V, b200_dtype dt) {
  B200_REQUIRE(ctx, ids && gh && gtable && H && V, "embedding_backward: bad arguments");
  B200_CUDA(ctx, cudaMemsetAsync(gtable, 0, V * H * sizeof(float), ctx->stream));   // reference zero-fills first (Transformer.cpp:528)
  if (!tokens) return B200_OK;
  if (ctx->deterministic) {
    const unsigned blocks = (unsigned)((H + 63) / 64);
    if (dt == B200_BF16) embedding_bwd_ordered_kernel<bf16><<<blocks, 64, 0, ctx->stream>>>(ids, (const bf16 *)gh, gtable, tokens, H, V);
    else embedding_bwd_ordered_kernel<float><<<blocks, 64, 0, ctx->stream>>>(ids, (const float *)gh, gtable, tokens, H, V);
    B200_LAUNCHED(ctx);
    return B200_OK;
  }
  int grid = (int)(tokens < (size_t)ctx->sm_count * 16 ? tokens : (size_t)ctx->sm_count * 16);
  if (dt == B200_BF16) embedding_bwd_kernel<bf16><<<grid, 256, 0, ctx->stream>>>(ids, (const bf16 *)gh, gtable, tokens, H, V);
  else embedding_bwd_kernel<float><<<grid, 256, 0, ctx->stream>>>(ids, (const float *)gh, gtable, tokens, H, V);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// ======================================================= cross-entropy ====
// One CTA per token: max, sum-exp, then (softmax - onehot)/tokens; per-token
// loss = -log(max(p_target, 1e-15)) (cpp/src/Loss.cpp:84-119, 163-194).  The
// mean is a second, deterministic single-CTA reduction (no float atomics).
// grad may be the same array as logits (neither pointer is __restrict__): a thread overwrites only
// elements it has read itself in the same pass, and the target logit is read before the first
// block-wide barrier, i.e. before any thread can have reached the gradient pass of this row.
template <class T>
__global__ void __launch_bounds__(512)
ce_token_kernel(const T *logits, const uint32_t *__restrict__ targets, float *__restrict__ tok_loss,
                T *grad, size_t tokens, size_t V) {
  __shared__ float red[32];
  constexpr int N = Vec16<T>::N;
  const bool vec = (V % N == 0) && ((uintptr_t)logits % 16 == 0) && (!grad || (uintptr_t)grad % 16 == 0);
  const float inv_tokens = 1.0f / (float)tokens;
  for (size_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    const T *lr = logits + t * V;
    const uint32_t tgt = targets[t];
    float tgt_logit = 0.f;
    if (threadIdx.x == 0 && tgt < V) tgt_logit = to_f(lr[tgt]);
    float mx = -INFINITY;
    if (vec) {
      for (size_t v = threadIdx.x; v < V / N; v += blockDim.x) {
        Vec16<T> a; float f[N]; a.load(lr + v * N); a.unpack(f);
#pragma unroll
        for (int j = 0; j < N; ++j) mx = fmaxf(mx, f[j]);
      }
    } else for (size_t v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, to_f(lr[v]));
    mx = block_max(mx, red);
    float sum = 0.f;
    if (vec) {
      for (size_t v = threadIdx.x; v < V / N; v += blockDim.x) {
        Vec16<T> a; float f[N]; a.load(lr + v * N); a.unpack(f);
#pragma unroll
        for (int j = 0; j < N; ++j) sum += __expf(f[j] - mx);
      }
    } else for (size_t v = threadIdx.x; v < V; v += blockDim.x) sum += __expf(to_f(lr[v]) - mx);
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) {
      float pt = (tgt < V) ? __expf(tgt_logit - mx) / sum : 0.f;
      tok_loss[t] = -logf(fmaxf(pt, 1e-15f));
    }
    if (grad) {
      T *gr = grad + t * V;
      float inv_sum = 1.0f / sum;
      if (vec) {
        for (size_t v = threadIdx.x; v < V / N; v += blockDim.x) {
          Vec16<T> a; float f[N]; a.load(lr + v * N); a.unpack(f);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            float p = __expf(f[j] - mx) * inv_sum;
            f[j] = ((v * N + j == tgt) ? p - 1.0f : p) * inv_tokens;
          }
          a.pack(f); a.store(gr + v * N);
        }
      } else {
        for (size_t v = threadIdx.x; v < V; v += blockDim.x) {
          float p = __expf(to_f(lr[v]) - mx) * inv_sum;
          gr[v] = from_f<T>(((v == tgt) ? p - 1.0f : p) * inv_tokens);
        }
      }
    }
  }
}
__global__ void mean_kernel(const float *__restrict__ v, float *__restrict__ out, size_t n) {
  __shared__ float red[32];
  float s = 0.f;
  for (size_t i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out = s / (float)n;
}
// Deterministic mean of n floats into *out (one CTA, fixed summation order).
int mean_launch(b200_ctx *ctx, const float *v, float *out, size_t n) {
  mean_kernel<<<1, 1024, 0, ctx->stream>>>(v, out, n);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
extern "C" int b200_cross_entropy(b200_ctx *ctx, const void *logits, const uint32_t *targets, float *loss_out,
                                  void *grad, size_t tokens, size_t V, b200_dtype dt) {
  B200_REQUIRE(ctx, logits && targets && loss_out && V > 0, "cross_entropy: bad arguments");
  if (!tokens) return B200_OK;
  float *tok_loss = (float *)b200_scratch(ctx, tokens * sizeof(float));
  if (!tok_loss) return B200_ERR_NOMEM;
  int grid = (int)(tokens < (size_t)ctx->sm_count * 4 ? tokens : (size_t)ctx->sm_count * 4);
  if (dt == B200_BF16) ce_token_kernel<bf16><<<grid, 512, 0, ctx->stream>>>((const bf16 *)logits, targets, tok_loss, (bf16 *)grad, tokens, V);
  else ce_token_kernel<float><<<grid, 512, 0, ctx->stream>>>((const float *)logits, targets, tok_loss, (float *)grad, tokens, V);
  B200_LAUNCHED(ctx);
  mean_kernel<<<1, 1024, 0, ctx->stream>>>(tok_loss, loss_out, tokens);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// =============================================================== AdamW ====
// m,v EMA -> decoupled decay -> bias-corrected step with eps outside the sqrt
// (cpp/src/gpu_kernel/adamw_step.metal:49-68).  fp32 master, optional bf16 shadow.
__device__ __forceinline__ float4 load4(const float *g, size_t i) { return reinterpret_cast<const float4 *>(g)[i]; }
__device__ __forceinline__ float4 load4(const bf16 *g, size_t i) {
  const uint2 r = reinterpret_cast<const uint2 *>(g)[i];
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
// G: element type of the gradient (fp32, or bf16 when the data-parallel exchange ran in bf16)
// gscale (optional, device): every gradient is multiplied by *gscale first (global-norm clipping).
template <class G>
__global__ void adamw_kernel(float *__restrict__ p, const G *__restrict__ g, float *__restrict__ m,
                             float *__restrict__ v, bf16 *__restrict__ shadow, size_t n, b200_adamw_params a,
                             const float *__restrict__ gscale) {
  pdl_launch_dependents();
  pdl_wait();
  const float gs = gscale ? *gscale : 1.0f;
  size_t nv = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4 *>(p)[i], gg = load4(g, i);
    float4 mm = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
    float *pf = &pp.x, *gf = &gg.x, *mf = &mm.x, *vf = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gf[j] *= gs;
      mf[j] = a.beta1 * mf[j] + (1.0f - a.beta1) * gf[j];
      vf[j] = a.beta2 * vf[j] + (1.0f - a.beta2) * gf[j] * gf[j];
      float x = pf[j];
      if (a.weight_decay > 0.0f) x = x - a.lr * a.weight_decay * x;
      float mh = mf[j] / a.bias_correction1, vh = vf[j] / a.bias_correction2;
      pf[j] = x - a.lr * mh / (sqrtf(vh) + a.eps);
    }
    reinterpret_cast<float4 *>(p)[i] = pp;
    reinterpret_cast<float4 *>(m)[i] = mm;
    reinterpret_cast<float4 *>(v)[i] = vv;
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pf[0], pf[1]), hi = __floats2bfloat162_rn(pf[2], pf[3]);
      uint2 pk; pk.x = *reinterpret_cast<uint32_t *>(&lo); pk.y = *reinterpret_cast<uint32_t *>(&hi);
      reinterpret_cast<uint2 *>(shadow)[i] = pk;
    }
  }
  for (size_t i = nv * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float gi = to_f(g[i]) * gs;
    float mi = a.beta1 * m[i] + (1.0f - a.beta1) * gi, vi = a.beta2 * v[i] + (1.0f - a.beta2) * gi * gi;
    float x = p[i];
    if (a.weight_decay > 0.0f) x = x - a.lr * a.weight_decay * x;
    x = x - a.lr * (mi / a.bias_correction1) / (sqrtf(vi / a.bias_correction2) + a.eps);
    p[i] = x; m[i] = mi; v[i] = vi;
    if (shadow) shadow[i] = __float2bfloat16_rn(x);
  }
}
extern "C" int b200_adamw_step(b200_ctx *ctx, float *p, const float *g, float *m, float *v, void *shadow, size_t n,
                               const b200_adamw_params *a) {
  B200_REQUIRE(ctx, p && g && m && v && a, "adamw_step: null pointer");
  B200_REQUIRE(ctx, (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) % 16 == 0) && ((uintptr_t)shadow % 8 == 0),
               "adamw_step: arrays must be 16-byte aligned");
  if (!n) return B200_OK;
  launch_k(ctx, adamw_kernel<float>, dim3(ew_grid(ctx, n / 4 + 1)), dim3(256), 0, 0, p, g, m, v, (bf16 *)shadow, n, *a, (const float *)nullptr);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
// AdamW with every gradient multiplied by the device scalar *gscale (the clip factor of clip_scale_launch).
int adamw_step_scaled(b200_ctx *ctx, float *p, const float *g, float *m, float *v, void *shadow, size_t n,
                      const b200_adamw_params *a, const float *gscale) {
  B200_REQUIRE(ctx, p && g && m && v && a && gscale, "adamw_step: null pointer");
  B200_REQUIRE(ctx, (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) % 16 == 0) && ((uintptr_t)shadow % 8 == 0),
               "adamw_step: arrays must be 16-byte aligned");
  if (!n) return B200_OK;
  launch_k(ctx, adamw_kernel<float>, dim3(ew_grid(ctx, n / 4 + 1)), dim3(256), 0, 0, p, g, m, v, (bf16 *)shadow, n, *a, gscale);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
// Global gradient norm and clip factor (python/apple-silicon/src/pre-training/train.py:858-867 of the reference's MLX
// trainer): out[0] = ||g||_2 over n floats, out[1] = norm > max_norm ? max_norm / (norm + 1e-6) : 1.  Fixed summation
// order (1024 partial sums in fp64, then one thread), so replicas holding the same gradients get the same factor.
namespace {
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const float *__restrict__ g, size_t n, double *__restrict__ part) {
  __shared__ double sh[256];
  double a = 0.0;
  const size_t nv = n / 4;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < nv; i += (size_t)gridDim.x * 256) {
    const float4 x = reinterpret_cast<const float4 *>(g)[i];
    a += (double)x.x * x.x + (double)x.y * x.y + (double)x.z * x.z + (double)x.w * x.w;
  }
  if (blockIdx.x == 0) for (size_t i = nv * 4 + threadIdx.x; i < n; i += 256) a += (double)g[i] * g[i];
  sh[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o]; __syncthreads(); }
  if (threadIdx.x == 0) part[blockIdx.x] = sh[0];
}
__global__ void clip_scale_kernel(const double *__restrict__ part, int blocks, float max_norm, float *__restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double a = 0.0;
    for (int i = 0; i < blocks; ++i) a += part[i];
    const float norm = (float)sqrt(a);
    out[0] = norm;
    out[1] = norm > max_norm ? max_norm / (norm + 1e-6f) : 1.0f;
  }
}
}  // namespace
int clip_scale_launch(b200_ctx *ctx, const float *g, size_t n, float max_norm, double *part1024, float *out2) {
  B200_REQUIRE(ctx, g && part1024 && out2 && (uintptr_t)g % 16 == 0, "clip_scale: bad arguments");
  sumsq_partial_kernel<<<1024, 256, 0, ctx->stream>>>(g, n, part1024);
  B200_LAUNCHED(ctx);
  clip_scale_kernel<<<1, 32, 0, ctx->stream>>>(part1024, 1024, max_norm, out2);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
// The same step with the gradient held in bf16 (8-byte aligned).
int adamw_step_bf16_grad(b200_ctx *ctx, float *p, const void *g_bf16, float *m, float *v, void *shadow, size_t n,
                         const b200_adamw_params *a) {
  B200_REQUIRE(ctx, p && g_bf16 && m && v && a, "adamw_step: null pointer");
  B200_REQUIRE(ctx, (((uintptr_t)p | (uintptr_t)m | (uintptr_t)v) % 16 == 0) && ((uintptr_t)shadow % 8 == 0) && ((uintptr_t)g_bf16 % 8 == 0),
               "adamw_step: arrays must be 16-byte aligned (bf16 arrays 8-byte)");
  if (!n) return B200_OK;
  launch_k(ctx, adamw_kernel<bf16>, dim3(ew_grid(ctx, n / 4 + 1)), dim3(256), 0, 0, p, (const bf16 *)g_bf16, m, v, (bf16 *)shadow, n, *a, (const float *)nullptr);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// ============================================== conversion / seeded fill ===
template <class S, class D>
__global__ void convert_kernel(const S *__restrict__ s, D *__restrict__ d, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    d[i] = from_f<D>(to_f(s[i]));
}
extern "C" int b200_convert(b200_ctx *ctx, const void *src, b200_dtype sd, void *dst, b200_dtype dd, size_t n) {
  B200_REQUIRE(ctx, src && dst, "convert: null pointer");
  if (!n) return B200_OK;
  int grid = ew_grid(ctx, n);
  if (sd == B200_F32 && dd == B200_BF16) convert_kernel<float, bf16><<<grid, 256, 0, ctx->stream>>>((const float *)src, (bf16 *)dst, n);
  else if (sd == B200_BF16 && dd == B200_F32) convert_kernel<bf16, float><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (float *)dst, n);
  else if (sd == B200_F32) convert_kernel<float, float><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, n);
  else convert_kernel<bf16, bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, n);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
// Strided 2-D copy with conversion: dst[r*ldd + c] = src[r*lds + c] (used to pack/unpack fused weights).
template <class S, class D>
__global__ void convert2d_kernel(const S *__restrict__ s, D *__restrict__ d, size_t rows, size_t cols, size_t lds,
                                 size_t ldd) {
  size_t total = rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / cols, c = i % cols;
    d[r * ldd + c] = from_f<D>(to_f(s[r * lds + c]));
  }
}
int convert2d(b200_ctx *ctx, const void *src, b200_dtype sd, void *dst, b200_dtype dd, size_t rows, size_t cols,
              size_t lds, size_t ldd) {
  if (rows * cols == 0) return B200_OK;
  int grid = ew_grid(ctx, rows * cols);
  if (sd == B200_F32 && dd == B200_BF16) convert2d_kernel<float, bf16><<<grid, 256, 0, ctx->stream>>>((const float *)src, (bf16 *)dst, rows, cols, lds, ldd);
  else if (sd == B200_BF16 && dd == B200_F32) convert2d_kernel<bf16, float><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (float *)dst, rows, cols, lds, ldd);
  else if (sd == B200_F32) convert2d_kernel<float, float><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, rows, cols, lds, ldd);
  else convert2d_kernel<bf16, bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, rows, cols, lds, ldd);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
template <class T>
__global__ void fill_normal_kernel(T *d, size_t n, uint64_t key, float std) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint64_t a = splitmix64(key + 2 * i), b = splitmix64(key + 2 * i + 1);
    float u1 = ((float)(a >> 40) + 0.5f) * (1.0f / 16777216.0f), u2 = ((float)(b >> 40) + 0.5f) * (1.0f / 16777216.0f);
    d[i] = from_f<T>(sqrtf(-2.0f * __logf(u1)) * __cosf(6.283185307f * u2) * std);
  }
}
extern "C" int b200_fill_normal(b200_ctx *ctx, void *d, b200_dtype dt, size_t n, uint64_t seed, float std) {
  B200_REQUIRE(ctx, d, "fill_normal: null pointer");
  if (!n) return B200_OK;
  int grid = ew_grid(ctx, n);
  if (dt == B200_BF16) fill_normal_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((bf16 *)d, n, seed * 0x9E3779B97F4A7C15ull, std);
  else fill_normal_kernel<float><<<grid, 256, 0, ctx->stream>>>((float *)d, n, seed * 0x9E3779B97F4A7C15ull, std);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
template <class T>
__global__ void fill_const_kernel(T *d, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) d[i] = from_f<T>(v);
}
int fill_const(b200_ctx *ctx, void *d, b200_dtype dt, size_t n, float v) {
  if (!n) return B200_OK;
  int grid = ew_grid(ctx, n);
  if (dt == B200_BF16) fill_const_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((bf16 *)d, n, v);
  else fill_const_kernel<float><<<grid, 256, 0, ctx->stream>>>((float *)d, n, v);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// ============================== cross-entropy for callers that must not allocate ==========
// Some hosts of this library cannot call cudaMalloc at the point where they need the loss: code
// running inside a fixed-memory budget that was carved up at start-up, plugins whose embedding
// application forbids device allocation after initialisation, and callers on a real-time path where
// the implicit device synchronisation of an allocation is not acceptable.  The regular
// b200_cross_entropy() keeps its per-token losses in the context's grow-on-demand scratch block,
// which may allocate.  This variant keeps them in a fixed array that is part of the library image
// instead: every GPU that loads the library holds the 256 KiB until the process exits, and in
// exchange the call performs no cudaMalloc / cudaFree and uses no allocating library routine.
//
// Limits and rules:
//   - at most B200_CE_NOALLOC_MAX_TOKENS (65536) tokens per call; larger inputs are rejected with
//     B200_ERR_INVALID and a message, nothing is launched;
//   - the first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current); make that first call before starting any stream capture;
//   - all calls share the one array.  It still holds the previous call's per-token losses; nothing
//     in it has to start at zero because each call overwrites entries [0, tokens) before the
//     reduction reads exactly those entries.  Two calls that overlap on the GPU (different streams,
//     or different contexts on the same device) race on the array: serialise them.
constexpr size_t B200_CE_NOALLOC_MAX_TOKENS = 65536;
static __device__ __align__(256) float g_ce_noalloc_token_loss[B200_CE_NOALLOC_MAX_TOKENS];
static float *g_ce_noalloc_dev_ptr[64] = {nullptr};   // device address of the array, per device ordinal

extern "C" int b200_cross_entropy_noalloc(b200_ctx *ctx, const void *logits, const uint32_t *targets,
                                          float *loss_out, void *grad, size_t tokens, size_t V, b200_dtype dt) {
  B200_REQUIRE(ctx, logits && targets && loss_out && V > 0, "cross_entropy_noalloc: bad arguments");
  if (tokens > B200_CE_NOALLOC_MAX_TOKENS)
    return b200_fail(ctx, B200_ERR_INVALID, "cross_entropy_noalloc: %zu tokens exceed the fixed scratch of %zu tokens; "
                     "split the batch or use b200_cross_entropy", tokens, B200_CE_NOALLOC_MAX_TOKENS);
  if (!tokens) return B200_OK;
  B200_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "cross_entropy_noalloc: device ordinal out of range");
  if (!g_ce_noalloc_dev_ptr[ctx->device]) {
    // The array's name is only a host-side handle here; kernels need its device address.  The lookup
    // answers for the CURRENT device, so the context's device is made current for it and the
    // caller's own choice of device is put back afterwards.
    int prev = -1;
    B200_CUDA(ctx, cudaGetDevice(&prev));
    if (prev != ctx->device) B200_CUDA(ctx, cudaSetDevice(ctx->device));
    float *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_ce_noalloc_token_loss);
    if (prev != ctx->device) cudaSetDevice(prev);
    if (e != cudaSuccess || !p)
      return b200_fail(ctx, B200_ERR_CUDA, "cross_entropy_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_ce_noalloc_dev_ptr[ctx->device] = p;
  }
  float *tok_loss = g_ce_noalloc_dev_ptr[ctx->device];
  int grid = (int)(tokens < (size_t)ctx->sm_count * 4 ? tokens : (size_t)ctx->sm_count * 4);
  if (dt == B200_BF16) ce_token_kernel<bf16><<<grid, 512, 0, ctx->stream>>>((const bf16 *)logits, targets, tok_loss, (bf16 *)grad, tokens, V);
  else ce_token_kernel<float><<<grid, 512, 0, ctx->stream>>>((const float *)logits, targets, tok_loss, (float *)grad, tokens, V);
  B200_LAUNCHED(ctx);
  mean_kernel<<<1, 1024, 0, ctx->stream>>>(tok_loss, loss_out, tokens);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
