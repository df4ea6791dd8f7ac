// CPU bodies for the backend interface (namespace metal_bridge) so that the
// reference's C++ CPU ops link on Linux as a test oracle.  is_available() is
// false, so every op takes its CPU branch; the three ops the reference has no
// CPU branch for are restated from their shader sources:
//   gemm_bf16          cpp/src/gpu_kernel/gemm_bf16.metal:45,63 (fp32 here)
//   rms_norm_forward   cpp/src/gpu_kernel/rms_norm_forward.metal:29-60
//   adamw_step         cpp/src/gpu_kernel/adamw_step.metal:49-68
// plus residual_add (cpp/src/gpu_kernel/residual_add.metal:15-28).
#include "gpu_kernel/MetalBridge.hpp"
#include <cmath>
#include <cstring>

namespace metal_bridge {
double accum_gpu_time_ms = 0, accum_cpu_time_ms = 0;
size_t count_gpu_calls = 0, count_cpu_calls = 0;
void reset_profile_stats() { accum_gpu_time_ms = accum_cpu_time_ms = 0; count_gpu_calls = count_cpu_calls = 0; }
void initialize() {}
bool is_available() { return false; }
void begin_scope() {}
void end_scope() {}
void register_gpu_wrapper(const float *, void **) {}
void unregister_gpu_wrapper(const float *) {}
void fill_zero_async(float *d, size_t bytes) { std::memset(d, 0, bytes); }
void copy_buffer_async(float *dst, size_t db, const float *src, size_t sb) { std::memcpy(dst, src, db < sb ? db : sb); }
void reconcile_buffers() {}
void clear_step_cache() {}
float get_last_loss() { return 0.f; }
void execute_in_autoreleasepool(std::function<void()> f) { f(); }
void start_step_trace() {}
void stop_step_trace() {}

void gemm_bf16(const void *Av, const void *Bv, void *Cv, size_t M, size_t N, size_t K,
               bool transA, bool transB, bool) {
  const float *A = (const float *)Av, *B = (const float *)Bv;
  float *C = (float *)Cv;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)M; ++i) {
    float *crow = C + (size_t)i * N;
    std::memset(crow, 0, N * sizeof(float));
    if (!transB) {
      for (size_t k = 0; k < K; ++k) {
        float a = transA ? A[k * M + i] : A[(size_t)i * K + k];
        const float *brow = B + k * N;
        for (size_t j = 0; j < N; ++j) crow[j] += a * brow[j];
      }
    } else {
      for (size_t j = 0; j < N; ++j) {
        float acc = 0.f;
        for (size_t k = 0; k < K; ++k)
          acc += (transA ? A[k * M + i] : A[(size_t)i * K + k]) * B[j * K + k];
        crow[j] = acc;
      }
    }
  }
}
void rms_norm_forward(const float *x, float *y, const float *w, float eps, size_t rows, size_t D) {
  for (size_t r = 0; r < rows; ++r) {
    float ss = 0.f;
    for (size_t c = 0; c < D; ++c) ss += x[r * D + c] * x[r * D + c];
    float inv = 1.0f / std::sqrt(ss / (float)D + eps);
    for (size_t c = 0; c < D; ++c) y[r * D + c] = x[r * D + c] * inv * w[c];
  }
}
void adamw_step(float *p, const float *g, float *m, float *v, const AdamWStepParams &a) {
  for (uint32_t i = 0; i < a.n; ++i) {
    m[i] = a.beta1 * m[i] + (1.0f - a.beta1) * g[i];
    v[i] = a.beta2 * v[i] + (1.0f - a.beta2) * g[i] * g[i];
    if (a.weight_decay > 0.0f) p[i] = p[i] - a.lr * a.weight_decay * p[i];
    float mh = m[i] / a.bias_correction1, vh = v[i] / a.bias_correction2;
    p[i] = p[i] - a.lr * mh / (std::sqrt(vh) + a.eps);
  }
}
void residual_add(float *a, const float *b, size_t n) { for (size_t i = 0; i < n; ++i) a[i] += b[i]; }

// Never reached while is_available() is false; present so the link succeeds.
#define UNREACHED {}
void fused_swiglu_gemm(const void *, const void *, const void *, void *, size_t, size_t, size_t) UNREACHED
void flash_attn_fwd(const void *, const void *, const void *, void *, size_t, size_t, size_t, size_t, size_t) UNREACHED
void fused_attn_bwd(const void *, const void *, const void *, const void *, void *, void *, void *, size_t, size_t, size_t, size_t, size_t) UNREACHED
void rms_norm_backward(const float *, const float *, const float *, float *, float *, float, size_t, size_t) UNREACHED
void swiglu_backward(const float *, const float *, const float *, float *, float *, size_t) UNREACHED
void swiglu_forward(const float *, const float *, float *, size_t) UNREACHED
void rope_backward(float *, const float *, const float *, size_t, size_t, size_t, size_t) UNREACHED
void fused_add_norm(float *, const float *, const float *, float *, size_t, size_t, float) UNREACHED
void fused_backward_add_norm(const void *, const void *, const void *, const void *, void *, size_t, size_t, float) UNREACHED
void embedding_forward(const uint32_t *, const float *, float *, size_t, size_t, size_t) UNREACHED
void cross_entropy(const void *, const uint32_t *, float *, float *, size_t, size_t) UNREACHED
void attn_softmax(const float *, float *, size_t, size_t, size_t) UNREACHED
void attn_ds(const float *, const float *, float *, size_t, size_t, size_t) UNREACHED
void gemm_gqa(const GQAParams &, const float *, const float *, const float *, float *, float *) UNREACHED
void gqa_backward(const GQABackwardParams &, const float *, const float *, const float *, const float *, float *, float *, float *, const float *) UNREACHED
void gqa_scores(const float *, const float *, float *, size_t, size_t, size_t, size_t, size_t) UNREACHED
void gemm_ffn(const float *, const float *, const float *, float *, size_t, size_t, size_t) UNREACHED
void gemm_proj(const float *, const float *, float *, size_t, size_t, size_t) UNREACHED
void gemm_backward(const float *, const float *, float *, size_t, size_t, size_t) UNREACHED
void gemm_proj_trans_b(const float *, const float *, float *, size_t, size_t, size_t) UNREACHED
void reshape_to_4d(const float *, float *, size_t, size_t, size_t, size_t) UNREACHED
void reshape_to_3d(const float *, float *, size_t, size_t, size_t, size_t) UNREACHED
void rope_forward(float *, float *, const float *, const float *, size_t, size_t, size_t, size_t, size_t) UNREACHED
}  // namespace metal_bridge
