// C-ABI plumbing: context, device memory, op dispatch between the tensor-core and
// CUDA-core kernels, and the host-pointer calls that follow the reference backend's
// calling convention (host buffers in, results visible on return).
#include "common.cuh"
#include <cstdarg>
#include <cstdlib>
#include <vector>

int attn_fwd_simt_launch(b200_ctx *, const void *, const void *, const void *, void *, float *, size_t, size_t, size_t,
                         size_t, size_t, const AttnStrides &, b200_dtype);
int attn_bwd_simt_launch(b200_ctx *, const void *, const void *, const void *, const void *, const void *,
                         const float *, void *, void *, void *, float *, size_t, size_t, size_t, size_t, size_t,
                         const AttnStrides &, const AttnStrides &, b200_dtype);
bool attn_tc_supported(size_t B, size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt,
                       const void *Q, const void *K, const void *V, const void *O);
int attn_fwd_tc_launch(b200_ctx *, const void *, const void *, const void *, void *, float *, size_t, size_t, size_t,
                       size_t, size_t, const AttnStrides &);
int attn_fwd2_tc_launch(b200_ctx *, const void *, const void *, const void *, void *, float *, size_t, size_t, size_t,
                        size_t, size_t, const AttnStrides &);
int attn_bwd_tc_launch(b200_ctx *, const void *, const void *, const void *, const void *, const void *,
                       const float *, void *, void *, void *, size_t, size_t, size_t, size_t, size_t,
                       const AttnStrides &, const AttnStrides &, const float *, const float *);
int swiglu_fwd_strided(b200_ctx *, const void *, const void *, void *, size_t, size_t, size_t, size_t, b200_dtype);

int b200_fail(b200_ctx *ctx, int code, const char *fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

void *b200_scratch(b200_ctx *ctx, size_t bytes) {
  if (bytes <= ctx->scratch_bytes) return ctx->scratch;
  // growing: earlier kernels may still be using the old block
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  ctx->scratch = nullptr; ctx->scratch_bytes = 0;
  size_t want = bytes + bytes / 4;
  if (cudaMalloc(&ctx->scratch, want) != cudaSuccess) {
    b200_fail(ctx, B200_ERR_NOMEM, "scratch allocation of %zu bytes failed", want);
    ctx->scratch = nullptr;
    return nullptr;
  }
  ctx->scratch_bytes = want;
  return ctx->scratch;
}

extern "C" int b200_is_available(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return 0;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, 0) != cudaSuccess) return 0;
  return p.major == 10 ? 1 : 0;
}

extern "C" int b200_init(int device, b200_ctx **out) {
  if (!out) return B200_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return B200_ERR_CUDA;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return B200_ERR_CUDA;
  if (p.major != 10) return B200_ERR_UNSUPPORTED;   // sm_100a code only: fail loudly elsewhere
  if (cudaSetDevice(device) != cudaSuccess) return B200_ERR_CUDA;
  b200_ctx *ctx = new b200_ctx();
  ctx->device = device;
  ctx->sm_count = p.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&ctx->dev_status, sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->host_status, sizeof(int)) != cudaSuccess) {
    delete ctx;
    return B200_ERR_CUDA;
  }
  ctx->stream = ctx->own_stream;
  if (const char *e = getenv("B200_ATTN_FWD2")) ctx->attn_fwd2 = e[0] != '0';     // A/B switch for measurements
  if (const char *e = getenv("B200_ATTN_BWD2")) ctx->attn_bwd2 = e[0] != '0';
  if (const char *e = getenv("B200_DECODE_ATTN_TC")) ctx->attn_decode_tc = e[0] != '0';
  // B200_PDL=1: programmatic dependent launch for every kernel that supports it (each waits before its first dependent
  // access), so that a kernel's launch and set-up overlap the tail of the one before.  The decode step always uses it
  // (it is a chain of microsecond kernels); for training steps it measured no gain on a power-capped B200
  // (152.5 vs 152.7 ms per step, same GPU), so plain stream order is the default there.
  ctx->pdl = getenv("B200_PDL") && getenv("B200_PDL")[0] == '1';
  ctx->deterministic = getenv("B200_DETERMINISTIC") && getenv("B200_DETERMINISTIC")[0] == '1';
  cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  *out = ctx;
  return B200_OK;
}

extern "C" int b200_destroy(b200_ctx *ctx) {
  if (!ctx) return B200_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  for (auto &t : ctx->timed) { cudaEventDestroy(t.start); cudaEventDestroy(t.stop); }
  for (auto e : ctx->event_pool) cudaEventDestroy(e);
  if (ctx->batch_t0) { cudaEventDestroy(ctx->batch_t0); cudaEventDestroy(ctx->batch_t1); }
  cudaFree(ctx->dev_status);
  cudaFreeHost(ctx->host_status);
  cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return B200_OK;
}

extern "C" const char *b200_last_error(const b200_ctx *ctx) { return ctx ? ctx->err : "null context"; }
extern "C" void *b200_stream(b200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" int b200_set_stream(b200_ctx *ctx, void *s) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->stream = s ? (cudaStream_t)s : ctx->own_stream;
  return B200_OK;
}
extern "C" uint64_t b200_launch_count(const b200_ctx *ctx) { return ctx ? ctx->launches : 0; }

extern "C" int b200_sync(b200_ctx *ctx) {
  if (!ctx) return B200_ERR_INVALID;
  B200_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  int st = *ctx->host_status;
  if (st != 0) {
    cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream);
    if (st == 2) return b200_fail(ctx, B200_ERR_INVALID, "token id out of range in embedding lookup");
    return b200_fail(ctx, B200_ERR_DEVICE_WAIT, "a device-side wait gave up (code %d)", st);
  }
  return B200_OK;
}

// Bring-up / A-B hook (not part of the public header): 0 forces the single-CTA tensor-core GEMM.
extern "C" int b200_internal_set_gemm_2cta(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->gemm_2cta = enable != 0;
  return B200_OK;
}
// Same kind of hook: 0 selects the one-query-tile forward attention kernel.
extern "C" int b200_internal_set_attn_decode_tc(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->attn_decode_tc = enable != 0;
  return B200_OK;
}
extern "C" int b200_internal_set_attn_bwd2(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->attn_bwd2 = enable != 0;
  return B200_OK;
}
extern "C" int b200_internal_set_attn_fwd2(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->attn_fwd2 = enable != 0;
  return B200_OK;
}
// Test hook: bit-reproducible gradient paths on or off (B200_DETERMINISTIC sets the initial value).
extern "C" int b200_internal_set_deterministic(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->deterministic = enable != 0;
  return B200_OK;
}
// Same kind of hook: 0 sends few-row GEMMs through the general tile kernel instead of the weight-streaming one.
extern "C" int b200_internal_set_gemm_skinny(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->gemm_skinny = enable != 0;
  return B200_OK;
}
// Test hook for the epilogues of the few-row GEMM that only the decode step uses (bf16; null pointers switch a part off):
//   producer half: C = residual + A W, xw_out = C * next_norm_w, stat_acc[row * 2 + {0, 1}] += the row's sums of squares (2^-32 fixed point);
//   consumer half: C = rstd(row_acc) * (A W), optionally through the SwiGLU or the rotary epilogue (table row `pos`).
extern "C" int b200_internal_few_row_gemm(b200_ctx *ctx, const void *A, const void *W, void *C, size_t M, size_t N, size_t K,
                                          const void *residual, const void *next_norm_w, void *xw_out, unsigned long long *stat_acc,
                                          const unsigned long long *row_acc, int norm_double, float eps,
                                          int swiglu_I, const float *cos_t, const float *sin_t, int hd, int rope_cols, int pos) {
  if (!ctx) return B200_ERR_INVALID;
  GemmEpilogue epi;
  epi.residual = residual; epi.ld_res = N;
  epi.next_norm_w = next_norm_w; epi.xw_out = xw_out; epi.ld_xw = N; epi.stat_acc = stat_acc;
  epi.row_acc = row_acc; epi.norm_double = norm_double; epi.norm_eps = eps;
  epi.swiglu_I = swiglu_I;
  if (cos_t) { epi.cos_t = cos_t + (size_t)pos * (hd / 2); epi.sin_t = sin_t + (size_t)pos * (hd / 2); epi.S = 1; epi.hd = hd; epi.cols = rope_cols; }
  return b200_gemm_ld(ctx, A, W, C, M, N, K, 0, 0, 0, B200_BF16, B200_BF16, K, N, swiglu_I > 0 ? (size_t)swiglu_I : N, &epi);
}
extern "C" int b200_profile_gemm(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  ctx->time_gemm = enable != 0;
  return B200_OK;
}
extern "C" int b200_profile_gemm_read(b200_ctx *ctx, double *total_ms, double *total_flops, uint64_t *launches) {
  if (!ctx || !total_ms || !total_flops || !launches) return B200_ERR_INVALID;
  B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *total_ms = 0; *total_flops = 0; *launches = ctx->timed.size();
  for (auto &t : ctx->timed) {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t.start, t.stop);
    *total_ms += ms; *total_flops += t.flops;
    ctx->event_pool.push_back(t.start); ctx->event_pool.push_back(t.stop);
  }
  ctx->timed.clear();
  return B200_OK;
}

// ---- launch trace (development hook, not part of the public header) ------------------------------------------------
// With the trace on, an event is recorded on the stream after every kernel launch of this library.  The dump attributes the
// time between consecutive events to the source line of the later launch (the kernel's own time plus the gap in front of
// it: everything runs on one stream) and writes one line per launch site, largest first.
void b200_trace_mark(b200_ctx *ctx, const char *file, int line) {
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, ctx->stream);
  ctx->marks.push_back({e, file, line});
}
extern "C" int b200_internal_trace(b200_ctx *ctx, int enable) {
  if (!ctx) return B200_ERR_INVALID;
  if (enable && !ctx->trace_on) b200_trace_mark(ctx, "start", 0);
  ctx->trace_on = enable != 0;
  return B200_OK;
}
extern "C" int b200_internal_trace_dump(b200_ctx *ctx, const char *path) {
  if (!ctx || !path) return B200_ERR_INVALID;
  B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  struct Site { std::string key; double ms = 0; size_t n = 0; };
  std::vector<Site> sites;
  double total = 0;
  for (size_t i = 1; i < ctx->marks.size(); ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ctx->marks[i - 1].ev, ctx->marks[i].ev) != cudaSuccess) { cudaGetLastError(); continue; }
    const char *f = strrchr(ctx->marks[i].file, '/');
    std::string key = std::string(f ? f + 1 : ctx->marks[i].file) + ":" + std::to_string(ctx->marks[i].line);
    size_t k = 0;
    while (k < sites.size() && sites[k].key != key) ++k;
    if (k == sites.size()) { sites.push_back(Site()); sites[k].key = key; }
    sites[k].ms += ms; sites[k].n++; total += ms;
  }
  for (auto &m : ctx->marks) cudaEventDestroy(m.ev);
  ctx->marks.clear();
  FILE *fp = fopen(path, "w");
  if (!fp) return b200_fail(ctx, B200_ERR_INVALID, "trace_dump: cannot open %s", path);
  fprintf(fp, "total_ms %.3f\n", total);
  for (size_t a = 0; a < sites.size(); ++a) {      // selection sort, largest first
    size_t best = a;
    for (size_t b = a + 1; b < sites.size(); ++b) if (sites[b].ms > sites[best].ms) best = b;
    std::swap(sites[a], sites[best]);
    fprintf(fp, "%-28s launches %6zu  total_ms %9.3f  avg_us %9.2f  share %5.1f%%\n", sites[a].key.c_str(), sites[a].n, sites[a].ms,
            1000.0 * sites[a].ms / (double)sites[a].n, 100.0 * sites[a].ms / total);
  }
  fclose(fp);
  return B200_OK;
}

extern "C" int b200_batch_timer_begin(b200_ctx *ctx) {
  if (!ctx) return B200_ERR_INVALID;
  if (!ctx->batch_t0) { B200_CUDA(ctx, cudaEventCreate(&ctx->batch_t0)); B200_CUDA(ctx, cudaEventCreate(&ctx->batch_t1)); }
  B200_CUDA(ctx, cudaEventRecord(ctx->batch_t0, ctx->stream));
  ctx->batch_timing = true;
  return B200_OK;
}
extern "C" int b200_batch_timer_end(b200_ctx *ctx, float *elapsed_ms) {
  if (!ctx) return B200_ERR_INVALID;
  B200_REQUIRE(ctx, elapsed_ms && ctx->batch_timing, "batch_timer_end: no timer running");
  ctx->batch_timing = false;
  B200_CUDA(ctx, cudaEventRecord(ctx->batch_t1, ctx->stream));
  B200_CUDA(ctx, cudaEventSynchronize(ctx->batch_t1));
  B200_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, ctx->batch_t0, ctx->batch_t1));
  return B200_OK;
}

extern "C" int b200_malloc(b200_ctx *ctx, size_t bytes, void **d) {
  if (!ctx || !d) return B200_ERR_INVALID;
  if (cudaMalloc(d, bytes ? bytes : 16) != cudaSuccess) {
    cudaGetLastError();
    return b200_fail(ctx, B200_ERR_NOMEM, "cudaMalloc of %zu bytes failed", bytes);
  }
  return B200_OK;
}
extern "C" int b200_free(b200_ctx *ctx, void *d) {
  if (!ctx) return B200_ERR_INVALID;
  if (d) { cudaStreamSynchronize(ctx->stream); cudaFree(d); }
  return B200_OK;
}
extern "C" int b200_memcpy_h2d(b200_ctx *ctx, void *d, const void *h, size_t n) {
  B200_REQUIRE(ctx, d && h, "memcpy_h2d: null pointer");
  B200_CUDA(ctx, cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, ctx->stream));
  return B200_OK;
}
extern "C" int b200_memcpy_d2h(b200_ctx *ctx, void *h, const void *d, size_t n) {
  B200_REQUIRE(ctx, d && h, "memcpy_d2h: null pointer");
  B200_CUDA(ctx, cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, ctx->stream));
  return B200_OK;
}
extern "C" int b200_fill_zero(b200_ctx *ctx, void *d, size_t n) {
  B200_REQUIRE(ctx, d, "fill_zero: null pointer");
  B200_CUDA(ctx, cudaMemsetAsync(d, 0, n, ctx->stream));
  return B200_OK;
}
extern "C" int b200_copy(b200_ctx *ctx, void *dst, const void *src, size_t n) {
  B200_REQUIRE(ctx, dst && src, "copy: null pointer");
  B200_CUDA(ctx, cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, ctx->stream));
  return B200_OK;
}

// ------------------------------------------------------------------ GEMM --
int b200_gemm_ld(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                 int acc, b200_dtype in_dt, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc,
                 const GemmEpilogue *epi) {
  B200_REQUIRE(ctx, A && B && C, "gemm: null pointer");
  B200_REQUIRE(ctx, !epi || (in_dt == B200_BF16 && out_dt == B200_BF16 && !acc && K > 0 &&
                             gemm_tc_supported(A, B, C, M, N, K, lda, ldb, ldc, out_dt)),
               "gemm: a fused epilogue needs the tensor-core path");
  const bool few_rows = K > 0 && ctx->gemm_skinny && gemm_skinny_supported(M, ta, tb, acc);
  B200_REQUIRE(ctx, !(epi && (epi->pos_dev || epi->row_acc || epi->next_norm_w || epi->residual)) || few_rows,
               "gemm: device-side positions, the folded normalisation and the residual epilogue exist only in the few-row kernel");
  B200_REQUIRE(ctx, !(epi && epi->swiglu_I) || few_rows || (epi->act_out && K > 0 && gemm_tc2_swiglu_eligible(ctx, M, (size_t)epi->swiglu_I)),
               "gemm: no kernel with a SwiGLU epilogue takes this shape");
  if (M == 0 || N == 0) return B200_OK;
  if (K == 0) {
    if (!acc) {
      B200_REQUIRE(ctx, ldc == N, "gemm: K == 0 with a strided C is unsupported");
      return b200_fill_zero(ctx, C, M * N * dtype_size(out_dt));
    }
    return B200_OK;
  }
  if (in_dt == B200_BF16 && !(acc && out_dt == B200_BF16) && gemm_tc_supported(A, B, C, M, N, K, lda, ldb, ldc, out_dt))
  {
    // a handful of rows against a stored [K,N] weight: bound by streaming the weight, own kernel
    if (ctx->gemm_skinny && gemm_skinny_supported(M, ta, tb, acc))
      return gemm_skinny_launch(ctx, A, B, C, M, N, K, out_dt, lda, ldb, ldc, epi);
    // two-CTA kernel when there are enough 256x256 tile pairs to fill the SM pairs; else 128x256 tiles
    const size_t pairs = ((M + 255) / 256) * ((N + 255) / 256);
    if ((epi && epi->swiglu_I) || (ctx->gemm_2cta && pairs >= (size_t)ctx->sm_count / 4))
      return gemm_tc2_launch(ctx, A, B, C, M, N, K, ta, tb, acc, out_dt, lda, ldb, ldc, epi);
    return gemm_tc_launch(ctx, A, B, C, M, N, K, ta, tb, acc, out_dt, lda, ldb, ldc, epi);
  }
  return gemm_simt_launch(ctx, A, B, C, M, N, K, ta, tb, acc, in_dt, out_dt, lda, ldb, ldc);
}

extern "C" int b200_gemm(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta,
                         int tb, int acc, b200_dtype in_dt, b200_dtype out_dt) {
  if (!ctx) return B200_ERR_INVALID;
  return b200_gemm_ld(ctx, A, B, C, M, N, K, ta, tb, acc, in_dt, out_dt, ta ? M : K, tb ? K : N, N);
}

extern "C" int b200_fused_swiglu_gemm(b200_ctx *ctx, const void *gate, const void *up, const void *B, void *C,
                                      void *scratch, size_t M, size_t N, size_t K, b200_dtype dt) {
  B200_REQUIRE(ctx, gate && up && B && C && scratch, "fused_swiglu_gemm: null pointer");
  int rc = swiglu_fwd_strided(ctx, gate, up, scratch, 1, M * K, M * K, M * K, dt);
  if (rc) return rc;
  return b200_gemm(ctx, scratch, B, C, M, N, K, 0, 0, 0, dt, dt);
}

// metal_bridge::gemm_ffn (MetalBridge.hpp:119-120, gemm_ffn.metal:44-183): c = silu(a*W_gate) * (a*W_up), with the two
// weights stored side by side as W = [gate | up] ([K, 2N], the engine's layout).  gate_up_out (optional, [M, 2N])
// receives the two products, which the backward pass needs.  bf16: one GEMM whose epilogue applies the activation
// (two-CTA kernel for large M, few-row kernel for M <= 64 when gate_up_out is not wanted); otherwise GEMM + SwiGLU.
extern "C" int b200_gemm_ffn(b200_ctx *ctx, const void *a, const void *w_gate_up, void *gate_up_out, void *c, size_t M,
                             size_t N, size_t K, b200_dtype dt) {
  B200_REQUIRE(ctx, a && w_gate_up && c, "gemm_ffn: null pointer");
  if (M == 0 || N == 0) return B200_OK;
  const size_t es = dtype_size(dt);
  if (dt == B200_BF16 && K > 0 && gemm_tc_supported(a, w_gate_up, c, M, 2 * N, K, K, 2 * N, N, dt) && N % 8 == 0) {
    GemmEpilogue epi;
    epi.swiglu_I = (int)N;
    if (!gate_up_out && ctx->gemm_skinny && gemm_skinny_supported(M, 0, 0, 0))
      return b200_gemm_ld(ctx, a, w_gate_up, c, M, 2 * N, K, 0, 0, 0, dt, dt, K, 2 * N, N, &epi);
    if (!(ctx->gemm_skinny && gemm_skinny_supported(M, 0, 0, 0)) && gemm_tc2_swiglu_eligible(ctx, M, N)) {
      void *gu = gate_up_out ? gate_up_out : b200_scratch(ctx, M * 2 * N * es);
      if (!gu) return B200_ERR_NOMEM;
      epi.act_out = c; epi.ld_act = N;
      return b200_gemm_ld(ctx, a, w_gate_up, gu, M, 2 * N, K, 0, 0, 0, dt, dt, K, 2 * N, 2 * N, &epi);
    }
  }
  void *gu = gate_up_out ? gate_up_out : b200_scratch(ctx, M * 2 * N * es);
  if (!gu) return B200_ERR_NOMEM;
  int rc = b200_gemm_ld(ctx, a, w_gate_up, gu, M, 2 * N, K, 0, 0, 0, dt, dt, K, 2 * N, 2 * N);
  if (rc) return rc;
  return swiglu_fwd_strided(ctx, gu, (const char *)gu + N * es, c, M, N, 2 * N, N, dt);
}

// ------------------------------------------------------------- attention --
int attn_fwd_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                    size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt) {
  B200_REQUIRE(ctx, Q && K && V && O, "attention forward: null pointer");
  B200_REQUIRE(ctx, nKV > 0 && nH % nKV == 0, "attention: n_heads must be a multiple of n_kv (cpp/src/Attention.cpp:48-50)");
  if (attn_tc_supported(B, nH, nKV, S, hd, st, dt, Q, K, V, O))
    return ctx->attn_fwd2 ? attn_fwd2_tc_launch(ctx, Q, K, V, O, lse, B, nH, nKV, S, hd, st)
                          : attn_fwd_tc_launch(ctx, Q, K, V, O, lse, B, nH, nKV, S, hd, st);
  return attn_fwd_simt_launch(ctx, Q, K, V, O, lse, B, nH, nKV, S, hd, st, dt);
}
int attn_bwd_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                    const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                    size_t hd, const AttnStrides &st, const AttnStrides &gst, b200_dtype dt, const float *rope_cos,
                    const float *rope_sin) {
  B200_REQUIRE(ctx, Q && K && V && O && dO && lse && dQ && dK && dV, "attention backward: null pointer");
  B200_REQUIRE(ctx, nKV > 0 && nH % nKV == 0, "attention: n_heads must be a multiple of n_kv");
  if (attn_tc_supported(B, nH, nKV, S, hd, st, dt, Q, K, V, O) &&
      attn_tc_supported(B, nH, nKV, S, hd, gst, dt, dQ, dK, dV, dO))
    return attn_bwd_tc_launch(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, hd, st, gst, rope_cos, rope_sin);
  B200_REQUIRE(ctx, !rope_cos && !rope_sin, "attention backward: fused rotary gradient needs the tensor-core path");
  float *scr = (float *)b200_scratch(ctx, 2 * B * nKV * S * hd * sizeof(float));
  if (!scr) return B200_ERR_NOMEM;
  return attn_bwd_simt_launch(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, scr, B, nH, nKV, S, hd, st, gst, dt);
}

bool attn_bwd_fuses_rope(size_t B, size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st,
                         const AttnStrides &gst, b200_dtype dt, const void *Q, const void *K, const void *V,
                         const void *O, const void *dO, const void *dQ, const void *dK, const void *dV) {
  return attn_tc_supported(B, nH, nKV, S, hd, st, dt, Q, K, V, O) && attn_tc_supported(B, nH, nKV, S, hd, gst, dt, dQ, dK, dV, dO);
}

static AttnStrides ref_layout(size_t nH, size_t nKV, size_t S, size_t hd) {
  // Q [B,nH,S,hd], K/V [B,nKV,S,hd], O [B,S,nH*hd]
  AttnStrides st;
  st.q_b = (long long)(nH * S * hd); st.q_h = (long long)(S * hd); st.q_s = (long long)hd;
  st.k_b = st.v_b = (long long)(nKV * S * hd); st.k_h = st.v_h = (long long)(S * hd); st.k_s = st.v_s = (long long)hd;
  st.o_b = (long long)(S * nH * hd); st.o_h = (long long)hd; st.o_s = (long long)(nH * hd);
  return st;
}

extern "C" int b200_flash_attn_fwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse,
                                   size_t B, size_t nH, size_t nKV, size_t S, size_t hd, b200_dtype dt) {
  if (!ctx) return B200_ERR_INVALID;
  return attn_fwd_launch(ctx, Q, K, V, O, lse, B, nH, nKV, S, hd, ref_layout(nH, nKV, S, hd), dt);
}

extern "C" int b200_fused_attn_bwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *dO,
                                   void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S, size_t hd,
                                   b200_dtype dt) {
  if (!ctx) return B200_ERR_INVALID;
  // The reference call carries neither the forward output nor its softmax statistics
  // (its shader recomputes them, cpp/src/gpu_kernel/fused_attn_bwd.metal:26-254): recompute
  // O and the log-sum-exp into temporaries, then run the backward proper.
  size_t o_bytes = B * S * nH * hd * dtype_size(dt), lse_bytes = B * nH * S * sizeof(float);
  void *tmpO = nullptr; float *tmpL = nullptr;
  int rc = b200_malloc(ctx, o_bytes, &tmpO);
  if (rc) return rc;
  rc = b200_malloc(ctx, lse_bytes, (void **)&tmpL);
  if (rc) { b200_free(ctx, tmpO); return rc; }
  AttnStrides st = ref_layout(nH, nKV, S, hd);
  rc = attn_fwd_launch(ctx, Q, K, V, tmpO, tmpL, B, nH, nKV, S, hd, st, dt);
  if (!rc) rc = attn_bwd_launch(ctx, Q, K, V, tmpO, dO, tmpL, dQ, dK, dV, B, nH, nKV, S, hd, st, st, dt);
  b200_free(ctx, tmpO);   // synchronises the stream first
  b200_free(ctx, tmpL);
  return rc;
}

// Backward from what the forward call left behind (its output and log-sum-exp): what a training engine calls,
// no recomputation and no temporaries.
extern "C" int b200_flash_attn_bwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                                   const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV,
                                   size_t S, size_t hd, b200_dtype dt) {
  if (!ctx) return B200_ERR_INVALID;
  AttnStrides st = ref_layout(nH, nKV, S, hd);
  return attn_bwd_launch(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, hd, st, st, dt);
}

// --------------------------------------------------- host-pointer calls --
namespace {
struct DevBuf {
  b200_ctx *ctx; void *p = nullptr;
  DevBuf(b200_ctx *c, size_t bytes) : ctx(c) { if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) { cudaGetLastError(); p = nullptr; } }
  ~DevBuf() { if (p) cudaFree(p); }
};
#define HOST_REQUIRE_ALLOC(ctx, b) do { if (!(b).p) return b200_fail(ctx, B200_ERR_NOMEM, "device staging allocation failed"); } while (0)
}  // namespace

extern "C" int b200_host_gemm(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                              int ta, int tb, b200_dtype dt) {
  B200_REQUIRE(ctx, A && B && C, "host_gemm: null pointer");
  size_t es = dtype_size(dt);
  DevBuf a(ctx, M * K * es), b(ctx, K * N * es), c(ctx, M * N * es);
  HOST_REQUIRE_ALLOC(ctx, a); HOST_REQUIRE_ALLOC(ctx, b); HOST_REQUIRE_ALLOC(ctx, c);
  int rc = b200_memcpy_h2d(ctx, a.p, A, M * K * es);
  if (!rc) rc = b200_memcpy_h2d(ctx, b.p, B, K * N * es);
  if (!rc) rc = b200_gemm(ctx, a.p, b.p, c.p, M, N, K, ta, tb, 0, dt, dt);
  if (!rc) rc = b200_memcpy_d2h(ctx, C, c.p, M * N * es);
  int rs = b200_sync(ctx);
  return rc ? rc : rs;
}
extern "C" int b200_host_rms_norm_forward(b200_ctx *ctx, const float *x, float *y, const float *w, float eps,
                                          size_t rows, size_t D) {
  B200_REQUIRE(ctx, x && y && w, "host_rms_norm_forward: null pointer");
  DevBuf dx(ctx, rows * D * 4), dy(ctx, rows * D * 4), dw(ctx, D * 4);
  HOST_REQUIRE_ALLOC(ctx, dx); HOST_REQUIRE_ALLOC(ctx, dy); HOST_REQUIRE_ALLOC(ctx, dw);
  int rc = b200_memcpy_h2d(ctx, dx.p, x, rows * D * 4);
  if (!rc) rc = b200_memcpy_h2d(ctx, dw.p, w, D * 4);
  if (!rc) rc = b200_rms_norm_forward(ctx, dx.p, dy.p, dw.p, nullptr, eps, rows, D, B200_F32);
  if (!rc) rc = b200_memcpy_d2h(ctx, y, dy.p, rows * D * 4);
  int rs = b200_sync(ctx);
  return rc ? rc : rs;
}
extern "C" int b200_host_flash_attn_fwd(b200_ctx *ctx, const float *Q, const float *K, const float *V, float *O,
                                        size_t B, size_t nH, size_t nKV, size_t S, size_t hd) {
  B200_REQUIRE(ctx, Q && K && V && O, "host_flash_attn_fwd: null pointer");
  size_t qn = B * nH * S * hd * 4, kn = B * nKV * S * hd * 4;
  DevBuf q(ctx, qn), k(ctx, kn), v(ctx, kn), o(ctx, qn);
  HOST_REQUIRE_ALLOC(ctx, q); HOST_REQUIRE_ALLOC(ctx, k); HOST_REQUIRE_ALLOC(ctx, v); HOST_REQUIRE_ALLOC(ctx, o);
  int rc = b200_memcpy_h2d(ctx, q.p, Q, qn);
  if (!rc) rc = b200_memcpy_h2d(ctx, k.p, K, kn);
  if (!rc) rc = b200_memcpy_h2d(ctx, v.p, V, kn);
  if (!rc) rc = b200_flash_attn_fwd(ctx, q.p, k.p, v.p, o.p, nullptr, B, nH, nKV, S, hd, B200_F32);
  if (!rc) rc = b200_memcpy_d2h(ctx, O, o.p, qn);
  int rs = b200_sync(ctx);
  return rc ? rc : rs;
}
extern "C" int b200_host_fused_attn_bwd(b200_ctx *ctx, const float *Q, const float *K, const float *V, const float *dO,
                                        float *dQ, float *dK, float *dV, size_t B, size_t nH, size_t nKV, size_t S,
                                        size_t hd) {
  B200_REQUIRE(ctx, Q && K && V && dO && dQ && dK && dV, "host_fused_attn_bwd: null pointer");
  size_t qn = B * nH * S * hd * 4, kn = B * nKV * S * hd * 4;
  DevBuf q(ctx, qn), k(ctx, kn), v(ctx, kn), g(ctx, qn), dq(ctx, qn), dk(ctx, kn), dv(ctx, kn);
  HOST_REQUIRE_ALLOC(ctx, q); HOST_REQUIRE_ALLOC(ctx, k); HOST_REQUIRE_ALLOC(ctx, v); HOST_REQUIRE_ALLOC(ctx, g);
  HOST_REQUIRE_ALLOC(ctx, dq); HOST_REQUIRE_ALLOC(ctx, dk); HOST_REQUIRE_ALLOC(ctx, dv);
  int rc = b200_memcpy_h2d(ctx, q.p, Q, qn);
  if (!rc) rc = b200_memcpy_h2d(ctx, k.p, K, kn);
  if (!rc) rc = b200_memcpy_h2d(ctx, v.p, V, kn);
  if (!rc) rc = b200_memcpy_h2d(ctx, g.p, dO, qn);
  if (!rc) rc = b200_fused_attn_bwd(ctx, q.p, k.p, v.p, g.p, dq.p, dk.p, dv.p, B, nH, nKV, S, hd, B200_F32);
  if (!rc) rc = b200_memcpy_d2h(ctx, dQ, dq.p, qn);
  if (!rc) rc = b200_memcpy_d2h(ctx, dK, dk.p, kn);
  if (!rc) rc = b200_memcpy_d2h(ctx, dV, dv.p, kn);
  int rs = b200_sync(ctx);
  return rc ? rc : rs;
}
extern "C" int b200_host_cross_entropy(b200_ctx *ctx, const float *logits, const uint32_t *targets, float *loss_out,
                                       float *grad, size_t tokens, size_t V) {
  B200_REQUIRE(ctx, logits && targets && loss_out, "host_cross_entropy: null pointer");
  DevBuf l(ctx, tokens * V * 4), t(ctx, tokens * 4), lo(ctx, 4), g(ctx, grad ? tokens * V * 4 : 16);
  HOST_REQUIRE_ALLOC(ctx, l); HOST_REQUIRE_ALLOC(ctx, t); HOST_REQUIRE_ALLOC(ctx, lo); HOST_REQUIRE_ALLOC(ctx, g);
  int rc = b200_memcpy_h2d(ctx, l.p, logits, tokens * V * 4);
  if (!rc) rc = b200_memcpy_h2d(ctx, t.p, targets, tokens * 4);
  if (!rc) rc = b200_cross_entropy(ctx, l.p, (const uint32_t *)t.p, (float *)lo.p, grad ? g.p : nullptr, tokens, V, B200_F32);
  if (!rc) rc = b200_memcpy_d2h(ctx, loss_out, lo.p, 4);
  if (!rc && grad) rc = b200_memcpy_d2h(ctx, grad, g.p, tokens * V * 4);
  int rs = b200_sync(ctx);
  return rc ? rc : rs;
}
