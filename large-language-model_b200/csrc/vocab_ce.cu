// Vocabulary projection fused with the cross-entropy loss: the B200 form of the tail of
// Transformer::forward (logits = final_h * W_out, cpp/src/Transformer.cpp:190-196), CrossEntropyLoss
// (cpp/src/Loss.cpp:43-135, 147-197; cpp/src/gpu_kernel/cross_entropy.metal:47-92) and the output-projection
// gradients (cpp/src/Transformer.cpp:515-521, 607-627).
//
// The reference materialises logits [tokens, V], runs a three-pass kernel over them (max, sum-exp, gradient) and keeps
// probabilities and gradient as further [tokens, V] tensors.  Here, on the bf16 tensor-core path:
//   forward   one GEMM whose epilogue reduces every 256-column tile of a row to (max, sum-exp) straight from the fp32
//             accumulators in tensor memory and picks out the target logit; the logits are never stored.  A small
//             kernel merges the tiles of a row into its log-sum-exp and loss; the mean is a fixed-order reduction.
//   backward  the same GEMM again with an epilogue that turns the accumulators into (softmax - onehot)/tokens and
//             stores that as bf16 -- the one [tokens, V] tensor that has to exist, because it is an operand of the
//             two gradient GEMMs (a [256, V] or [H, 256] accumulator block does not fit in tensor memory, so neither
//             product can consume the tile while it is still on chip).
//   Alternatively the forward GEMM also stores bf16 logits (statistics from the rounded values) and the backward is
//   one in-place pass logits -> gradient: one GEMM fewer, one more [tokens, V] write; the engine picks by measurement.
// fp32 (and shapes the tensor-core kernel does not take): CUDA-core GEMM into the workspace, per-row statistics,
// the same in-place gradient pass.
#include "common.cuh"

int mean_launch(b200_ctx *ctx, const float *v, float *out, size_t n);

namespace {
constexpr float LN2 = 0.6931471805599453f, LOG2E = 1.4426950408889634f;
constexpr float LOSS_CLAMP = 34.538776394910684f;   // -log(1e-15): the reference clamps the target probability (cpp/src/Loss.cpp:113-117)

// lse[r] = log sum_j exp(x[r,j]) from the per-tile (max, sum) pairs (base-2 units); loss[r] = lse - x[r, target].
// A CTA handles 32 rows; its 8 warps take every 8th tile (loads coalesced over the rows) and meet in shared memory.
__global__ void __launch_bounds__(256)
ce_merge_kernel(const float *__restrict__ pmax, const float *__restrict__ psum, const float *__restrict__ tgt_logit,
                const uint32_t *__restrict__ targets, float *__restrict__ lse, float *__restrict__ tok_loss, size_t M,
                int tiles, size_t V) {
  __shared__ float sm[8][32], ss[8][32];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const size_t r = (size_t)blockIdx.x * 32 + lane;
  float m = -1e30f, s = 0.f;
  if (r < M) {
    for (int t = g; t < tiles; t += 8) {
      const float pm = pmax[(size_t)t * M + r], ps = psum[(size_t)t * M + r];
      const float mn = fmaxf(m, pm);
      s = s * exp2f(m - mn) + ps * exp2f(pm - mn);
      m = mn;
    }
  }
  sm[g][lane] = m; ss[g][lane] = s;
  __syncthreads();
  if (g == 0 && r < M) {
    float mm = sm[0][lane];
#pragma unroll
    for (int i = 1; i < 8; ++i) mm = fmaxf(mm, sm[i][lane]);
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += ss[i][lane] * exp2f(sm[i][lane] - mm);      // fixed order: deterministic
    const float l = (mm + log2f(tot)) * LN2;
    lse[r] = l;
    const uint32_t tgt = targets[r];
    tok_loss[r] = tgt < V ? fminf(l - tgt_logit[r], LOSS_CLAMP) : LOSS_CLAMP;
  }
}

// One CTA per row of stored logits: log-sum-exp and loss (the path without the fused epilogue).
template <class T>
__global__ void __launch_bounds__(256)
ce_row_stats_kernel(const T *__restrict__ logits, const uint32_t *__restrict__ targets, float *__restrict__ lse,
                    float *__restrict__ tok_loss, size_t tokens, size_t V) {
  __shared__ float red[32];
  for (size_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    const T *lr = logits + t * V;
    float mx = -1e30f;
    for (size_t v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, to_f(lr[v]));
    mx = block_max(mx, red);
    float sum = 0.f;
    for (size_t v = threadIdx.x; v < V; v += blockDim.x) sum += __expf(to_f(lr[v]) - mx);
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) {
      const float l = mx + logf(sum);
      const uint32_t tgt = targets[t];
      lse[t] = l;
      tok_loss[t] = tgt < V ? fminf(l - to_f(lr[tgt]), LOSS_CLAMP) : LOSS_CLAMP;
    }
    __syncthreads();
  }
}

// In place: x[r, j] <- (exp(x[r, j] - lse[r]) - [j == target[r]]) * scale.  One read and one write of the array.
template <class T>
__global__ void __launch_bounds__(256)
ce_apply_kernel(T *x, const uint32_t *__restrict__ targets, const float *__restrict__ lse, float scale, size_t tokens, size_t V) {
  constexpr int N = Vec16<T>::N;
  const bool vec = (V % N == 0) && ((uintptr_t)x % 16 == 0);
  for (size_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    T *xr = x + t * V;
    const float l2 = lse[t] * LOG2E;
    const uint32_t tgt = targets[t];
    if (vec) {
      for (size_t v = threadIdx.x; v < V / N; v += blockDim.x) {
        Vec16<T> a; float f[N]; a.load(xr + v * N); a.unpack(f);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float p = exp2f(fmaf(f[j], LOG2E, -l2));
          f[j] = ((uint32_t)(v * N + j) == tgt ? p - 1.0f : p) * scale;
        }
        a.pack(f); a.store(xr + v * N);
      }
    } else {
      for (size_t v = threadIdx.x; v < V; v += blockDim.x) {
        const float p = exp2f(fmaf(to_f(xr[v]), LOG2E, -l2));
        xr[v] = from_f<T>(((uint32_t)v == tgt ? p - 1.0f : p) * scale);
      }
    }
  }
}

bool fused_ok(const void *x, const void *w, const void *c, size_t M, size_t V, size_t H, b200_dtype dt) {
  return dt == B200_BF16 && gemm_tc_supported(x, w, c ? c : x, M, V, H, H, V, V, B200_BF16);
}
int row_grid(const b200_ctx *ctx, size_t tokens) { return (int)(tokens < (size_t)ctx->sm_count * 8 ? tokens : (size_t)ctx->sm_count * 8); }
}  // namespace

extern "C" int b200_vocab_ce_forward(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, float *loss_out,
                                     float *lse_out, void *logits_out, size_t tokens, size_t V, size_t H, b200_dtype dt) {
  if (!ctx) return B200_ERR_INVALID;
  B200_REQUIRE(ctx, x && w && targets && loss_out && lse_out && V > 0 && H > 0, "vocab_ce_forward: bad arguments");
  if (!tokens) return B200_OK;
  if (fused_ok(x, w, logits_out, tokens, V, H, dt)) {
    const size_t tiles = gemm_tc2_ce_tiles(V);
    float *ws = (float *)b200_scratch(ctx, (2 * tiles + 2) * tokens * sizeof(float));
    if (!ws) return B200_ERR_NOMEM;
    float *pmax = ws, *psum = ws + tiles * tokens, *tl = ws + 2 * tiles * tokens, *tok_loss = tl + tokens;
    GemmEpilogue epi;
    epi.ce_mode = logits_out ? 2 : 1; epi.ce_targets = targets; epi.ce_part_max = pmax; epi.ce_part_sum = psum; epi.ce_tgt_logit = tl;
    int rc = gemm_tc2_launch(ctx, x, w, logits_out, tokens, V, H, 0, 0, 0, B200_BF16, H, V, V, &epi);
    if (rc) return rc;
    ce_merge_kernel<<<(unsigned)((tokens + 31) / 32), 256, 0, ctx->stream>>>(pmax, psum, tl, targets, lse_out, tok_loss, tokens, (int)tiles, V);
    B200_LAUNCHED(ctx);
    return mean_launch(ctx, tok_loss, loss_out, tokens);
  }
  // CUDA-core / unfused path: logits into the caller's array or the context workspace
  const size_t es = dtype_size(dt);
  char *ws = (char *)b200_scratch(ctx, tokens * sizeof(float) + (logits_out ? 0 : tokens * V * es + 16));
  if (!ws) return B200_ERR_NOMEM;
  float *tok_loss = (float *)ws;
  void *lg = logits_out ? logits_out : (void *)(ws + ((tokens * sizeof(float) + 15) & ~(size_t)15));
  int rc = b200_gemm_ld(ctx, x, w, lg, tokens, V, H, 0, 0, 0, dt, dt, H, V, V);
  if (rc) return rc;
  if (dt == B200_BF16) ce_row_stats_kernel<bf16><<<row_grid(ctx, tokens), 256, 0, ctx->stream>>>((const bf16 *)lg, targets, lse_out, tok_loss, tokens, V);
  else ce_row_stats_kernel<float><<<row_grid(ctx, tokens), 256, 0, ctx->stream>>>((const float *)lg, targets, lse_out, tok_loss, tokens, V);
  B200_LAUNCHED(ctx);
  return mean_launch(ctx, tok_loss, loss_out, tokens);
}

// true when the forward call takes its statistics in the GEMM epilogue (no logits needed afterwards)
bool vocab_ce_is_fused(const void *x, const void *w, size_t tokens, size_t V, size_t H, b200_dtype dt) {
  return fused_ok(x, w, nullptr, tokens, V, H, dt);
}

// d(mean loss)/d(logits) into `dlogits` [tokens, V]: from the logits already stored there (in_place) or by running the
// projection again with the gradient epilogue.
int vocab_ce_dlogits(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, const float *lse, void *dlogits,
                     int in_place, size_t tokens, size_t V, size_t H, b200_dtype dt) {
  const float scale = 1.0f / (float)tokens;
  if (!in_place && fused_ok(x, w, dlogits, tokens, V, H, dt)) {
    GemmEpilogue epi;
    epi.ce_mode = 3; epi.ce_targets = targets; epi.ce_lse = lse; epi.ce_scale = scale;
    return gemm_tc2_launch(ctx, x, w, dlogits, tokens, V, H, 0, 0, 0, B200_BF16, H, V, V, &epi);
  }
  if (!in_place) {
    int rc = b200_gemm_ld(ctx, x, w, dlogits, tokens, V, H, 0, 0, 0, dt, dt, H, V, V);
    if (rc) return rc;
  }
  if (dt == B200_BF16) ce_apply_kernel<bf16><<<row_grid(ctx, tokens), 256, 0, ctx->stream>>>((bf16 *)dlogits, targets, lse, scale, tokens, V);
  else ce_apply_kernel<float><<<row_grid(ctx, tokens), 256, 0, ctx->stream>>>((float *)dlogits, targets, lse, scale, tokens, V);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

extern "C" int b200_vocab_ce_backward(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, const float *lse,
                                      void *dlogits, int logits_in_place, float *grad_w, void *grad_x, size_t tokens,
                                      size_t V, size_t H, b200_dtype dt) {
  if (!ctx) return B200_ERR_INVALID;
  B200_REQUIRE(ctx, x && w && targets && lse && dlogits && V > 0 && H > 0, "vocab_ce_backward: bad arguments");
  if (!tokens) return B200_OK;
  int rc = vocab_ce_dlogits(ctx, x, w, targets, lse, dlogits, logits_in_place, tokens, V, H, dt);
  if (rc) return rc;
  // dW = x^T * dlogits (cpp/src/Transformer.cpp:515-521), dx = dlogits * W^T (:607-627)
  if (grad_w) rc = b200_gemm_ld(ctx, x, dlogits, grad_w, H, V, tokens, 1, 0, 0, dt, B200_F32, H, V, V);
  if (!rc && grad_x) rc = b200_gemm_ld(ctx, dlogits, w, grad_x, tokens, H, V, 0, 1, 0, dt, dt, V, V, H);
  return rc;
}
