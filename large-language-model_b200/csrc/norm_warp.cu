// RMSNorm forward / backward, one WARP per row: the row lives in registers (VPL 16-byte vectors per
// lane), reductions are warp shuffles only (no block barriers), and every lane keeps VPL independent
// 16-byte loads per tensor in flight, which is what saturates HBM for the 2048-wide rows of the
// 1.6B configuration.  Same maths as the block-per-row kernels in elementwise.cu
// (cpp/src/gpu_kernel/rms_norm_forward.metal:29-60, fused_add_norm.metal:25-72,
//  cpp/src/RMSNorm.cpp:126-160, fused_backward_add_norm.metal:19-84).
#include "common.cuh"

namespace {
constexpr int WARPS_PER_CTA = 8;
constexpr int ROW_THREADS = 256;                    // CTA-per-row kernel for few rows

template <class T, int VPL, bool ADD>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
rms_fwd_warp_kernel(const T *x, T *h_out, const T *__restrict__ r, const T *__restrict__ w, T *__restrict__ y,
                    float *__restrict__ rstd_out, float eps, size_t rows, int D, const T *__restrict__ w2,
                    T *__restrict__ y2) {
  constexpr int N = Vec16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t warp_global = (size_t)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const size_t n_warps = (size_t)gridDim.x * WARPS_PER_CTA;
  for (size_t row = warp_global; row < rows; row += n_warps) {
    const size_t base = row * (size_t)D;
    float v[VPL][N];
    Vec16<T> a[VPL], b[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) a[i].load(x + base + (lane + 32 * i) * N);
    if (ADD) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) b[i].load(r + base + (lane + 32 * i) * N);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      a[i].unpack(v[i]);
      if (ADD) {
        float rb[N];
        b[i].unpack(rb);
#pragma unroll
        for (int j = 0; j < N; ++j) v[i][j] += rb[j];
        Vec16<T> o; o.pack(v[i]); o.store(h_out + base + (lane + 32 * i) * N); o.unpack(v[i]);   // normalise what is stored
      }
#pragma unroll
      for (int j = 0; j < N; ++j) ss += v[i][j] * v[i][j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (rstd_out && lane == 0) rstd_out[row] = rstd;
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      Vec16<T> wv; float wf[N], o[N];
      wv.load(w + (lane + 32 * i) * N); wv.unpack(wf);
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = v[i][j] * rstd * wf[j];
      Vec16<T> ov; ov.pack(o);
      if (y) ov.store(y + base + (lane + 32 * i) * N);
      if (y2) {                                   // second norm reads the first one's output as stored
        ov.unpack(v[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) ss2 += v[i][j] * v[i][j];
      }
    }
    if (y2) {
      // y2 = rmsnorm(y) * w2 in the same pass (the reference's attention re-normalises its already normalised
      // input, cpp/src/Attention.cpp:171-190)
      ss2 = warp_sum(ss2);
      const float rstd2 = rsqrtf(ss2 / (float)D + eps);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        Vec16<T> wv; float wf[N], o[N];
        wv.load(w2 + (lane + 32 * i) * N); wv.unpack(wf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = v[i][j] * rstd2 * wf[j];
        Vec16<T> ov; ov.pack(o); ov.store(y2 + base + (lane + 32 * i) * N);
      }
    }
  }
}

// Few rows (a decode step normalises one row per sequence): one CTA per row, one 16-byte vector per thread and chunk,
// every load of the row in flight at once and the weights requested before the wait on the previous kernel, so that the
// kernel is one memory round trip plus two block reductions instead of a chain of dependent loads in a single warp.
template <class T, int CH, bool ADD>
__global__ void __launch_bounds__(ROW_THREADS)
rms_fwd_row_kernel(const T *x, T *h_out, const T *__restrict__ r, const T *__restrict__ w, T *__restrict__ y,
                   float *__restrict__ rstd_out, float eps, int D, const T *__restrict__ w2, T *__restrict__ y2) {
  constexpr int N = Vec16<T>::N;
  __shared__ float red[2][ROW_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  Vec16<T> wv[CH], w2v[CH];                          // parameters: no kernel of the stream writes them
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    wv[i].load(w + (tid + ROW_THREADS * i) * N);
    if (y2) w2v[i].load(w2 + (tid + ROW_THREADS * i) * N);
  }
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * (size_t)D;
  Vec16<T> a[CH], b[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) a[i].load(x + base + (tid + ROW_THREADS * i) * N);
  if (ADD) {
#pragma unroll
    for (int i = 0; i < CH; ++i) b[i].load(r + base + (tid + ROW_THREADS * i) * N);
  }
  float v[CH][N], ss = 0.f;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    a[i].unpack(v[i]);
    if (ADD) {
      float rb[N];
      b[i].unpack(rb);
#pragma unroll
      for (int j = 0; j < N; ++j) v[i][j] += rb[j];
      Vec16<T> o; o.pack(v[i]); o.store(h_out + base + (tid + ROW_THREADS * i) * N); o.unpack(v[i]);   // normalise what is stored
    }
#pragma unroll
    for (int j = 0; j < N; ++j) ss += v[i][j] * v[i][j];
  }
  auto block_sum = [&](float t, float *buf) {
    t = warp_sum(t);
    if (lane == 0) buf[warp] = t;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ROW_THREADS / 32; ++k) s += buf[k];
    return s;
  };
  const float rstd = rsqrtf(block_sum(ss, red[0]) / (float)D + eps);
  if (rstd_out && tid == 0) rstd_out[blockIdx.x] = rstd;
  float ss2 = 0.f;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    float wf[N], o[N];
    wv[i].unpack(wf);
#pragma unroll
    for (int j = 0; j < N; ++j) o[j] = v[i][j] * rstd * wf[j];
    Vec16<T> ov; ov.pack(o);
    if (y) ov.store(y + base + (tid + ROW_THREADS * i) * N);
    if (y2) {                                       // the second norm reads the first one's output as stored
      ov.unpack(v[i]);
#pragma unroll
      for (int j = 0; j < N; ++j) ss2 += v[i][j] * v[i][j];
    }
  }
  if (y2) {
    const float rstd2 = rsqrtf(block_sum(ss2, red[1]) / (float)D + eps);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float wf[N], o[N];
      w2v[i].unpack(wf);
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = v[i][j] * rstd2 * wf[j];
      Vec16<T> ov; ov.pack(o); ov.store(y2 + base + (tid + ROW_THREADS * i) * N);
    }
  }
}

template <class T, int VPL, bool ADD, bool DW>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
rms_bwd_warp_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ w,
                    const T *__restrict__ res_grad, T *__restrict__ dx, float *__restrict__ dw, float eps,
                    size_t rows, int D) {
  constexpr int N = Vec16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t warp_global = (size_t)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const size_t n_warps = (size_t)gridDim.x * WARPS_PER_CTA;
  float dw_acc[DW ? VPL : 1][N];
  if (DW) {
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int j = 0; j < N; ++j) dw_acc[i][j] = 0.f;
  }
  for (size_t row = warp_global; row < rows; row += n_warps) {
    const size_t base = row * (size_t)D;
    Vec16<T> xa[VPL], ga[VPL], ra[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) { xa[i].load(x + base + (lane + 32 * i) * N); ga[i].load(g + base + (lane + 32 * i) * N); }
    if (ADD) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) ra[i].load(res_grad + base + (lane + 32 * i) * N);
    }
    float xv[VPL][N], gw[VPL][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      xa[i].unpack(xv[i]);
#pragma unroll
      for (int j = 0; j < N; ++j) ss += xv[i][j] * xv[i][j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      Vec16<T> wv; float wf[N], gf[N];
      wv.load(w + (lane + 32 * i) * N); wv.unpack(wf);
      ga[i].unpack(gf);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float xhat = xv[i][j] * rstd;
        if (DW) dw_acc[i][j] += gf[j] * xhat;
        gw[i][j] = gf[j] * wf[j];
        s += gw[i][j] * xhat;
      }
    }
    s = warp_sum(s) / (float)D;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float o[N];
      if (ADD) ra[i].unpack(o);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float d = rstd * (gw[i][j] - xv[i][j] * rstd * s);
        o[j] = ADD ? o[j] + d : d;
      }
      Vec16<T> ov; ov.pack(o); ov.store(dx + base + (lane + 32 * i) * N);
    }
  }
  if (DW) {
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int j = 0; j < N; ++j) atomicAdd(dw + (lane + 32 * i) * N + j, dw_acc[i][j]);
  }
}

// Backward of the pair "a1 = rmsnorm(h) * w; a2 = rmsnorm(a1)" (the layer's norm followed by the attention's own
// unit-weight norm, cpp/src/Transformer.cpp:147 + cpp/src/Attention.cpp:192-194) plus the residual gradient, in ONE
// pass: dx = d(a2)/d(h)^T g + res_grad.  a1 is not read: it is recomputed from h exactly as the forward kernel stored
// it (same arithmetic, rounded to T), so the forward need not keep it.  Reads g, h, res_grad; writes dx.
// WPR warps share a row (a 2048-wide bf16 row held by one warp, widened to floats, does not fit in the register file);
// their partial sums meet in shared memory behind a named barrier of the row's WPR*32 threads.
template <class T, int VPL, int WPR>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32, VPL <= 2 ? 2 : 1)
rms_bwd2_warp_kernel(const T *__restrict__ g, const T *__restrict__ h, const T *__restrict__ w,
                     const T *__restrict__ res_grad, T *__restrict__ dx, float eps, size_t rows, int D) {
  constexpr int N = Vec16<T>::N, ROWS_PER_CTA = WARPS_PER_CTA / WPR;
  __shared__ float part[4][ROWS_PER_CTA][WPR];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, slot = warp / WPR, sub = warp % WPR;
  const float inv_d = 1.0f / (float)D;
  auto row_sum = [&](float v, int which) -> float {
    v = warp_sum(v);
    if (WPR == 1) return v;
    if (lane == 0) part[which][slot][sub] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "n"(WPR * 32) : "memory");
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) t += part[which][slot][k];
    return t;
  };
  const size_t n_slots = (size_t)gridDim.x * ROWS_PER_CTA;
  // every warp of a row group runs the same number of iterations (the barrier counts on it)
  auto at = [&](int i) { return (size_t)((i * WPR + sub) * 32 + lane) * N; };
  size_t row = (size_t)blockIdx.x * ROWS_PER_CTA + slot;
  Vec16<T> ha[VPL], ga[VPL], ra[VPL];
  if (row < rows) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) { ha[i].load(h + row * (size_t)D + at(i)); ga[i].load(g + row * (size_t)D + at(i)); ra[i].load(res_grad + row * (size_t)D + at(i)); }
  }
  for (; row < rows; row += n_slots) {
    const size_t base = row * (size_t)D;
    float hv[VPL][N], gv[VPL][N], a1[VPL][N], rv[VPL][N];
    float ss1 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      ha[i].unpack(hv[i]); ga[i].unpack(gv[i]); ra[i].unpack(rv[i]);
#pragma unroll
      for (int j = 0; j < N; ++j) ss1 += hv[i][j] * hv[i][j];
    }
    // the next row of this group is requested now: its latency hides behind the four reductions of the current row
    if (row + n_slots < rows) {
      const size_t nb = (row + n_slots) * (size_t)D;
#pragma unroll
      for (int i = 0; i < VPL; ++i) { ha[i].load(h + nb + at(i)); ga[i].load(g + nb + at(i)); ra[i].load(res_grad + nb + at(i)); }
    }
    const float rstd1 = rsqrtf(row_sum(ss1, 0) * inv_d + eps);
    // a1 as the forward stored it, and the statistics of the second norm
    float ss2 = 0.f, dot2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      Vec16<T> wv; float wf[N];
      wv.load(w + at(i)); wv.unpack(wf);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        a1[i][j] = to_f(from_f<T>(hv[i][j] * rstd1 * wf[j]));
        ss2 += a1[i][j] * a1[i][j]; dot2 += gv[i][j] * a1[i][j];
      }
    }
    const float rstd2 = rsqrtf(row_sum(ss2, 1) * inv_d + eps);
    const float s2 = row_sum(dot2, 2) * rstd2 * inv_d;          // mean(g * a1_hat)
    // g1 = d/d(a1) through the unit-weight norm, times w; the first norm's statistic mean(g1 * w * h_hat)
    float dot1 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      Vec16<T> wv; float wf[N];
      wv.load(w + at(i)); wv.unpack(wf);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        gv[i][j] = rstd2 * (gv[i][j] - a1[i][j] * rstd2 * s2) * wf[j];
        dot1 += gv[i][j] * hv[i][j];
      }
    }
    const float s1 = row_sum(dot1, 3) * rstd1 * inv_d;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float o[N];
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = rv[i][j] + rstd1 * (gv[i][j] - hv[i][j] * rstd1 * s1);
      Vec16<T> ov; ov.pack(o); ov.store(dx + base + at(i));
    }
  }
}

int warp_grid(b200_ctx *ctx, size_t rows) {
  size_t blocks = (rows + WARPS_PER_CTA - 1) / WARPS_PER_CTA, cap = (size_t)ctx->sm_count * 4;
  return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}
bool aligned16(std::initializer_list<const void *> ps) {
  for (auto p : ps) if ((uintptr_t)p % 16) return false;
  return true;
}
}  // namespace

// Returns 1 when the warp-per-row kernel was launched, 0 when the shape does not fit it, <0 on error.
template <class T>
int rms_fwd_warp(b200_ctx *ctx, const void *x, void *h, const void *r, const void *w, void *y, float *rstd, float eps,
                 size_t rows, size_t D, bool add, const void *w2, void *y2) {
  constexpr int N = Vec16<T>::N;
  if (D % (32 * N) || !aligned16({x, h, r, w, y, w2, y2})) return 0;
  if (rows <= (size_t)ctx->sm_count && D % (ROW_THREADS * N) == 0 && D / (ROW_THREADS * N) <= 2) {
    // fewer rows than SMs: a CTA per row
#define FR(C, A) launch_k(ctx, rms_fwd_row_kernel<T, C, A>, dim3((unsigned)rows), dim3(ROW_THREADS), 0, 0, (const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, (int)D, (const T *)w2, (T *)y2)
    if (D / (ROW_THREADS * N) == 1) { if (add) FR(1, true); else FR(1, false); }
    else { if (add) FR(2, true); else FR(2, false); }
#undef FR
    ctx->launches++;
    if (ctx->trace_on) b200_trace_mark(ctx, __FILE__, __LINE__);
    if (cudaGetLastError() != cudaSuccess) return b200_fail(ctx, B200_ERR_CUDA, "rms_norm forward launch failed");
    return 1;
  }
  const int vpl = (int)(D / (32 * N));
  const int grid = warp_grid(ctx, rows);
#define FW(V, A) launch_k(ctx, rms_fwd_warp_kernel<T, V, A>, dim3(grid), dim3(WARPS_PER_CTA * 32), 0, 0, (const T *)x, (T *)h, (const T *)r, (const T *)w, (T *)y, rstd, eps, rows, (int)D, (const T *)w2, (T *)y2)
  switch (vpl) {
    case 1: if (add) FW(1, true); else FW(1, false); break;
    case 2: if (add) FW(2, true); else FW(2, false); break;
    case 4: if (add) FW(4, true); else FW(4, false); break;
    case 8: if (add) FW(8, true); else FW(8, false); break;
    default: return 0;
  }
#undef FW
  ctx->launches++;
  if (ctx->trace_on) b200_trace_mark(ctx, __FILE__, __LINE__);
  if (cudaGetLastError() != cudaSuccess) return b200_fail(ctx, B200_ERR_CUDA, "rms_norm forward launch failed");
  return 1;
}
template <class T>
int rms_bwd_warp(b200_ctx *ctx, const void *g, const void *x, const void *w, const void *rg, void *dx, float *dw,
                 float eps, size_t rows, size_t D, bool add) {
  constexpr int N = Vec16<T>::N;
  if (D % (32 * N) || !aligned16({g, x, w, rg, dx})) return 0;
  const int vpl = (int)(D / (32 * N));
  const int grid = warp_grid(ctx, rows);
#define BW(V, A, W_) launch_k(ctx, rms_bwd_warp_kernel<T, V, A, W_>, dim3(grid), dim3(WARPS_PER_CTA * 32), 0, 0, (const T *)g, (const T *)x, (const T *)w, (const T *)rg, (T *)dx, dw, eps, rows, (int)D)
#define BWV(V) do { if (add) { if (dw) BW(V, true, true); else BW(V, true, false); } else { if (dw) BW(V, false, true); else BW(V, false, false); } } while (0)
  switch (vpl) {
    case 1: BWV(1); break;
    case 2: BWV(2); break;
    case 4: BWV(4); break;
    case 8: BWV(8); break;
    default: return 0;
  }
#undef BWV
#undef BW
  ctx->launches++;
  if (ctx->trace_on) b200_trace_mark(ctx, __FILE__, __LINE__);
  if (cudaGetLastError() != cudaSuccess) return b200_fail(ctx, B200_ERR_CUDA, "rms_norm backward launch failed");
  return 1;
}
// Returns 1 when launched, 0 when the shape does not fit (the caller then runs the two separate backward passes).
template <class T>
int rms_bwd2_warp(b200_ctx *ctx, const void *g, const void *h, const void *w, const void *rg, void *dx, float eps,
                  size_t rows, size_t D) {
  constexpr int N = Vec16<T>::N;
  if (D % (32 * N) || !aligned16({g, h, w, rg, dx})) return 0;
  const int vecs = (int)(D / (32 * N));               // 16-byte vectors per lane if one warp took the row
#define B2(V, W_) do { const size_t per = WARPS_PER_CTA / W_; size_t blocks = (rows + per - 1) / per; const size_t cap = (size_t)ctx->sm_count * 4; \
    if (blocks > cap) blocks = cap; if (!blocks) blocks = 1; \
    launch_k(ctx, rms_bwd2_warp_kernel<T, V, W_>, dim3((unsigned)blocks), dim3(WARPS_PER_CTA * 32), 0, 0, (const T *)g, (const T *)h, (const T *)w, (const T *)rg, (T *)dx, eps, rows, (int)D); } while (0)
  switch (vecs) {
    case 1: B2(1, 1); break;
    case 2: B2(2, 1); break;
    case 4: B2(4, 1); break;
    // wide rows: several warps per row, few enough vectors per lane that two CTAs fit the register file of an SM
    case 8: if (sizeof(T) == 2) B2(2, 4); else B2(4, 2); break;
    case 16: if (sizeof(T) == 2) B2(2, 8); else B2(4, 4); break;
    default: return 0;
  }
#undef B2
  ctx->launches++;
  if (ctx->trace_on) b200_trace_mark(ctx, __FILE__, __LINE__);
  if (cudaGetLastError() != cudaSuccess) return b200_fail(ctx, B200_ERR_CUDA, "double rms_norm backward launch failed");
  return 1;
}
template int rms_bwd2_warp<float>(b200_ctx *, const void *, const void *, const void *, const void *, void *, float, size_t, size_t);
template int rms_bwd2_warp<bf16>(b200_ctx *, const void *, const void *, const void *, const void *, void *, float, size_t, size_t);
template int rms_fwd_warp<float>(b200_ctx *, const void *, void *, const void *, const void *, void *, float *, float, size_t, size_t, bool, const void *, void *);
template int rms_fwd_warp<bf16>(b200_ctx *, const void *, void *, const void *, const void *, void *, float *, float, size_t, size_t, bool, const void *, void *);
template int rms_bwd_warp<float>(b200_ctx *, const void *, const void *, const void *, const void *, void *, float *, float, size_t, size_t, bool);
template int rms_bwd_warp<bf16>(b200_ctx *, const void *, const void *, const void *, const void *, void *, float *, float, size_t, size_t, bool);
