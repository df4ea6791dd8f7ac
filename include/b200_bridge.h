/*
 * b200_bridge.h -- C ABI of the B200 (sm_100a) backend for the decoder-block
 * hot path of the reference C++ training engine.
 *
 * The reference talks to its GPU backend through the free functions of
 * `namespace metal_bridge` (cpp/include/gpu_kernel/MetalBridge.hpp:14-147).
 * Every compute entry point below replaces one of those functions; the
 * citation beside each declaration names the interface it stands in for.
 * Differences that are deliberate:
 *   - every call returns a status code (the reference prints and returns void);
 *   - the element type is an explicit argument (the reference's pointers are
 *     nominally float* while its shaders read bf16);
 *   - pointers are DEVICE pointers and work is enqueued on the context's
 *     stream; the host-pointer behaviour of the reference interface (caller
 *     passes host buffers, results are visible after end_scope) is provided by
 *     the b200_host_* calls at the end and by the C++ `namespace metal_bridge`
 *     adaptor (large-language-model_b200/adaptor/metal_bridge_b200.cpp).
 *
 * All matrices are row-major.  Plain C: no C++ or torch types cross this
 * boundary.  Functions are not thread-safe per context (the reference
 * backend is single-threaded with file-static state).
 */
#ifndef B200_BRIDGE_H
#define B200_BRIDGE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_ctx b200_ctx;
typedef struct b200_model b200_model;

typedef enum { B200_F32 = 0, B200_BF16 = 1 } b200_dtype;

enum {
  B200_OK = 0,
  B200_ERR_INVALID = -1,     /* bad argument (null pointer, shape, alignment) */
  B200_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
  B200_ERR_UNSUPPORTED = -3, /* shape/dtype combination has no kernel */
  B200_ERR_NOMEM = -4,
  B200_ERR_DEVICE_WAIT = -5, /* a bounded device-side wait gave up */
  B200_ERR_COMM = -6         /* NCCL failure */
};

/* ---- lifecycle (metal_bridge::initialize / is_available, MetalBridge.hpp:20-21) */
int b200_init(int device, b200_ctx **out);
int b200_destroy(b200_ctx *ctx);
int b200_is_available(void);
const char *b200_last_error(const b200_ctx *ctx);
/* cudaStream_t the context enqueues on, as an opaque pointer. */
void *b200_stream(b200_ctx *ctx);
/* Use a caller-owned stream (NULL restores the context's own stream). */
int b200_set_stream(b200_ctx *ctx, void *cuda_stream);
/* One stream synchronise; also surfaces device-side wait failures.
 * (metal_bridge::end_scope, MetalBridge.hpp:29-30) */
int b200_sync(b200_ctx *ctx);
/* Number of kernels this library has launched on the context since creation. */
uint64_t b200_launch_count(const b200_ctx *ctx);

/* Per-launch device timing of the tensor-core GEMM with CUDA events on the launching
 * stream (the reference keeps wall-clock counters accum_gpu_time_ms / count_gpu_calls,
 * MetalBridge.hpp:141-145).  _read synchronises, returns the totals since the last read
 * and clears them. */
int b200_profile_gemm(b200_ctx *ctx, int enable);
int b200_profile_gemm_read(b200_ctx *ctx, double *total_ms, double *total_flops, uint64_t *launches);

/* Device time of a batch of enqueued work: _begin records a CUDA event on the context's stream, _end records a second
 * one, waits for it and returns the milliseconds between them.  This is what the reference accumulates into
 * accum_gpu_time_ms around commit + waitUntilCompleted in end_scope (cpp/src/gpu_kernel/MetalBridge.mm:2195-2207),
 * measured on the device instead of the host clock. */
int b200_batch_timer_begin(b200_ctx *ctx);
int b200_batch_timer_end(b200_ctx *ctx, float *elapsed_ms);

/* ---- device memory (the reference wraps host pages zero-copy; a discrete GPU needs mirrors) */
int b200_malloc(b200_ctx *ctx, size_t bytes, void **dptr);
int b200_free(b200_ctx *ctx, void *dptr);
int b200_memcpy_h2d(b200_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int b200_memcpy_d2h(b200_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
/* metal_bridge::fill_zero_async / copy_buffer_async (MetalBridge.hpp:75-76) */
int b200_fill_zero(b200_ctx *ctx, void *dptr, size_t bytes);
int b200_copy(b200_ctx *ctx, void *dst_dev, const void *src_dev, size_t bytes);
/* dtype conversion between fp32 and bf16 device arrays (n elements). */
int b200_convert(b200_ctx *ctx, const void *src, b200_dtype src_dtype, void *dst, b200_dtype dst_dtype, size_t n);
/* Seeded N(0, std) fill of a device array (synthetic weights for benchmarks). */
int b200_fill_normal(b200_ctx *ctx, void *dptr, b200_dtype dtype, size_t n, uint64_t seed, float std);

/* ---- GEMM: C[M,N] (+)= op(A)[M,K] * op(B)[K,N]
 * metal_bridge::gemm_bf16 (MetalBridge.hpp:39-42); with trans_b also
 * gemm_proj_trans_b (:121-122); with trans_a also gemm_backward (:119-120).
 * trans_a: A is stored [K,M]; trans_b: B is stored [N,K].  in_dtype is the
 * type of A and B, out_dtype of C.  accumulate != 0 adds into C. bf16 inputs
 * run on the tcgen05 tensor-core kernel (fp32 accumulation in tensor memory);
 * fp32 inputs run an fp32 CUDA-core kernel that meets the 1e-4 contract. */
int b200_gemm(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
              int trans_a, int trans_b, int accumulate, b200_dtype in_dtype, b200_dtype out_dtype);

/* ---- RMSNorm
 * metal_bridge::rms_norm_forward (MetalBridge.hpp:60-61). rstd_out (optional,
 * fp32 [rows]) receives 1/sqrt(mean(x^2)+eps) for reuse by the backward. */
int b200_rms_norm_forward(b200_ctx *ctx, const void *x, void *y, const void *weight, float *rstd_out,
                          float eps, size_t rows, size_t dims, b200_dtype dtype);
/* metal_bridge::rms_norm_backward (MetalBridge.hpp:62-64). grad_weight is
 * optional fp32 [dims] and is ACCUMULATED into, as the reference does. */
int b200_rms_norm_backward(b200_ctx *ctx, const void *grad_output, const void *x, const void *weight,
                           void *grad_input, float *grad_weight, float eps, size_t rows, size_t dims,
                           b200_dtype dtype);
/* metal_bridge::fused_add_norm (MetalBridge.hpp:79-81): x_residual += residual; output = rmsnorm(x_residual)*weight */
int b200_fused_add_norm(b200_ctx *ctx, void *x_residual, const void *residual, const void *weight, void *output,
                        size_t rows, size_t dims, float eps, b200_dtype dtype);
/* metal_bridge::fused_backward_add_norm (MetalBridge.hpp:82-85): grad_input = rmsnorm_bwd(grad_output, x, weight) + residual_grad */
int b200_fused_backward_add_norm(b200_ctx *ctx, const void *grad_output, const void *x, const void *weight,
                                 const void *residual_grad, void *grad_input, size_t rows, size_t dims, float eps,
                                 b200_dtype dtype);

/* ---- RoPE on [batch, heads, seq, head_dim], interleaved pairs, in place.
 * Tables are fp32 [seq, head_dim/2].
 * metal_bridge::rope_forward (MetalBridge.hpp:130-133) / rope_backward (:68-69). */
int b200_rope_tables(b200_ctx *ctx, float *cos_table, float *sin_table, size_t max_seq, size_t head_dim, float base);
int b200_rope_forward(b200_ctx *ctx, void *q, void *k, const float *cos_table, const float *sin_table,
                      size_t batch, size_t q_heads, size_t kv_heads, size_t seq_len, size_t head_dim, b200_dtype dtype);
int b200_rope_backward(b200_ctx *ctx, void *grad, const float *cos_table, const float *sin_table, size_t batch,
                       size_t heads, size_t seq_len, size_t head_dim, b200_dtype dtype);

/* ---- SwiGLU: metal_bridge::swiglu_forward / swiglu_backward (MetalBridge.hpp:65-67) */
int b200_swiglu_forward(b200_ctx *ctx, const void *gate, const void *up, void *out, size_t n, b200_dtype dtype);
int b200_swiglu_backward(b200_ctx *ctx, const void *grad_output, const void *gate, const void *up, void *grad_gate,
                         void *grad_up, size_t n, b200_dtype dtype);
/* metal_bridge::fused_swiglu_gemm (MetalBridge.hpp:44-46): C[M,N] = (silu(gate)*up)[M,K] * B[K,N].
 * scratch must hold M*K elements of dtype. */
int b200_fused_swiglu_gemm(b200_ctx *ctx, const void *gate, const void *up, const void *B, void *C, void *scratch,
                           size_t M, size_t N, size_t K, b200_dtype dtype);

/* metal_bridge::gemm_ffn (MetalBridge.hpp:119-120; gemm_ffn.metal:44-183): c[M,N] = silu(a*W_gate) * (a*W_up) with the two
 * weights stored side by side, w_gate_up = [gate | up] of shape [K, 2N].  gate_up_out (optional, [M,2N]) receives the two
 * products (kept for the backward pass).  For bf16 the activation runs in the GEMM epilogue. */
int b200_gemm_ffn(b200_ctx *ctx, const void *a, const void *w_gate_up, void *gate_up_out, void *c, size_t M, size_t N,
                  size_t K, b200_dtype dtype);

/* ---- metal_bridge::residual_add (MetalBridge.hpp:78): a += b */
int b200_residual_add(b200_ctx *ctx, void *a, const void *b, size_t n, b200_dtype dtype);

/* ---- head split / merge: metal_bridge::reshape_to_4d / reshape_to_3d (MetalBridge.hpp:123-129) */
int b200_reshape_to_4d(b200_ctx *ctx, const void *src, void *dst, size_t batch, size_t heads, size_t seq_len,
                       size_t head_dim, b200_dtype dtype);
int b200_reshape_to_3d(b200_ctx *ctx, const void *src, void *dst, size_t batch, size_t heads, size_t seq_len,
                       size_t head_dim, b200_dtype dtype);

/* ---- causal GQA attention
 * metal_bridge::flash_attn_fwd (MetalBridge.hpp:49-51).  Q [B,nH,S,hd], K/V
 * [B,nKV,S,hd], O [B,S,nH*hd] (the caller's contract, cpp/src/Attention.cpp:211,227,282).
 * lse (optional fp32 [B,nH,S]) receives log-sum-exp of the scaled scores. */
int b200_flash_attn_fwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse,
                        size_t batch, size_t n_heads, size_t n_kv, size_t seq_len, size_t head_dim, b200_dtype dtype);
/* metal_bridge::fused_attn_bwd (MetalBridge.hpp:54-57).  dO [B,S,nH*hd]; dQ
 * like Q, dK/dV like K/V (summed over the nH/nKV query heads of each kv head). */
int b200_fused_attn_bwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *dO, void *dQ,
                        void *dK, void *dV, size_t batch, size_t n_heads, size_t n_kv, size_t seq_len,
                        size_t head_dim, b200_dtype dtype);

/* The same backward for callers that kept the forward call's output O and lse (b200_flash_attn_fwd): nothing is
 * recomputed and nothing is allocated.  The reference has no such entry (its shader recomputes the forward,
 * cpp/src/gpu_kernel/fused_attn_bwd.metal:26-254); this is the form the engine and the benchmark use. */
int b200_flash_attn_bwd(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                        const float *lse, void *dQ, void *dK, void *dV, size_t batch, size_t n_heads, size_t n_kv,
                        size_t seq_len, size_t head_dim, b200_dtype dtype);

/* ---- embedding gather: metal_bridge::embedding_forward (MetalBridge.hpp:86-88) */
int b200_embedding_forward(b200_ctx *ctx, const uint32_t *token_ids, const void *table, void *output,
                           size_t total_tokens, size_t hidden_dim, size_t vocab_size, b200_dtype dtype);
/* scatter-add of hidden-state grads into the fp32 table grad (cpp/src/Transformer.cpp:524-537). */
int b200_embedding_backward(b200_ctx *ctx, const uint32_t *token_ids, const void *grad_hidden, float *grad_table,
                            size_t total_tokens, size_t hidden_dim, size_t vocab_size, b200_dtype dtype);

/* ---- metal_bridge::cross_entropy (MetalBridge.hpp:89-91): mean loss into the
 * device float *loss_out and, when grad_logits != NULL, (softmax - onehot)/tokens.
 * grad_logits has dtype `dtype` and may alias logits. */
int b200_cross_entropy(b200_ctx *ctx, const void *logits, const uint32_t *targets, float *loss_out,
                       void *grad_logits, size_t total_tokens, size_t vocab_size, b200_dtype dtype);

/* ---- vocabulary projection fused with cross-entropy: the tail of Transformer::forward (logits = x * W,
 * cpp/src/Transformer.cpp:190-196) + CrossEntropyLoss::forward (cpp/src/Loss.cpp:43-135) in one call.
 * x [tokens, hidden], w [hidden, vocab] ([in,out] like every weight).  loss_out (device float) receives the mean loss,
 * lse_out (device fp32 [tokens]) the log-sum-exp of every row.  bf16: one tensor-core GEMM whose epilogue reduces the
 * fp32 accumulators to per-row softmax statistics; with logits_out == NULL the logits are never written to memory.
 * logits_out (optional, [tokens, vocab], dtype) additionally receives the logits.  fp32 inputs, or shapes the tensor-core
 * kernel does not take (vocab or hidden not a multiple of 8), run GEMM + statistics with the logits in logits_out or in
 * the context workspace. */
int b200_vocab_ce_forward(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, float *loss_out,
                          float *lse_out, void *logits_out, size_t tokens, size_t vocab, size_t hidden, b200_dtype dtype);
/* CrossEntropyLoss::backward + the output-projection gradients (cpp/src/Loss.cpp:147-197,
 * cpp/src/Transformer.cpp:515-521, 607-627).  dlogits [tokens, vocab] (dtype) is a caller-owned work array that
 * receives (softmax - onehot)/tokens: with logits_in_place != 0 it must hold the logits written by the forward call
 * and is converted in one pass; otherwise the projection is run again with the gradient as its epilogue.
 * grad_w (optional, fp32 [hidden, vocab]) = x^T * dlogits; grad_x (optional, dtype, [tokens, hidden]) = dlogits * w^T. */
int b200_vocab_ce_backward(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, const float *lse,
                           void *dlogits, int logits_in_place, float *grad_w, void *grad_x, size_t tokens, size_t vocab,
                           size_t hidden, b200_dtype dtype);

/* ---- cross-entropy for callers that must not allocate device memory.
 * No counterpart in the reference.  Same inputs, outputs and results as b200_cross_entropy, but the
 * per-token losses live in a fixed 256 KiB device array inside the library (held by every GPU that
 * loads it until process exit) instead of the context's grow-on-demand scratch, so the call never
 * reaches cudaMalloc/cudaFree.  For hosts that may not allocate at call time: fixed-budget
 * embedders, plugins whose application forbids allocation after start-up, real-time paths that
 * cannot take an allocation's implicit synchronisation.  At most 65536 tokens per call (larger
 * inputs return B200_ERR_INVALID).  The first call on a device resolves the array's address; make
 * it before any stream capture.  All calls share the array: calls that overlap on the GPU race. */
int b200_cross_entropy_noalloc(b200_ctx *ctx, const void *logits, const uint32_t *targets, float *loss_out,
                               void *grad_logits, size_t total_tokens, size_t vocab_size, b200_dtype dtype);

/* ---- metal_bridge::adamw_step (MetalBridge.hpp:92-98). param/m/v fp32; grad
 * fp32; bf16_shadow (optional) receives the updated parameter rounded to bf16. */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2;
} b200_adamw_params;
int b200_adamw_step(b200_ctx *ctx, float *param, const float *grad, float *m, float *v, void *bf16_shadow,
                    size_t n, const b200_adamw_params *p);

/* ======================= device-resident training engine =======================
 * The reference composes the ops above in Transformer::forward / ::backward
 * (cpp/src/Transformer.cpp:90-197, 571-657) with one h_in kept per layer and
 * everything else recomputed.  The engine keeps activations in HBM instead
 * (no recompute) and uses fused [Wq|Wk|Wv] and [Wgate|Wup] weights; parameter
 * import/export uses the reference's own per-tensor layout:
 *   embedding[V,H]; per layer attn_norm_w[H], Wq[H,nH*hd], Wk[H,nKV*hd],
 *   Wv[H,nKV*hd], Wo[nH*hd,H], ffn_norm_w[H], w_gate[H,I], w_up[H,I],
 *   w_down[I,H]; final_norm_w[H]; output_projection[H,V]   (all [in,out]). */
typedef struct {   /* mirrors ModelConfig, cpp/include/TransformerConfig.hpp:16-98 */
  size_t vocab_size, hidden_dim, intermediate_dim, n_layers, n_heads, n_kv_heads, head_dim, max_seq_len;
  float rope_base, rms_norm_eps;
} b200_model_config;

int b200_model_create(b200_ctx *ctx, const b200_model_config *cfg, b200_dtype compute_dtype, size_t max_batch,
                      int with_optimizer, b200_model **out);
int b200_model_destroy(b200_model *m);
size_t b200_model_param_count(const b200_model *m);
int b200_model_get_config(const b200_model *m, b200_model_config *out);
int b200_model_load_params(b200_model *m, const float *host_flat);
int b200_model_read_params(b200_model *m, float *host_flat);
int b200_model_read_grads(b200_model *m, float *host_flat);
/* AdamW first/second moments in the parameter layout above (norm slots: zero on read, ignored on load) and the
 * optimizer step counter; what Checkpoint::save / ::load put in and take from the ".opt.safetensors" file
 * (cpp/src/Checkpoint.cpp:836-1040, 1066-1110). */
int b200_model_read_opt_state(b200_model *m, float *host_m_flat, float *host_v_flat, uint64_t *step);
int b200_model_load_opt_state(b200_model *m, const float *host_m_flat, const float *host_v_flat, uint64_t step);
int b200_model_init_synthetic(b200_model *m, uint64_t seed, float std);
/* Transformer::forward (cpp/src/Transformer.cpp:90-197): logits_out (optional, device, compute dtype, [B*S,V]). */
int b200_model_forward(b200_model *m, const int32_t *dev_tokens, size_t batch, size_t seq_len, void *logits_out);
/* forward + CrossEntropyLoss + Transformer::backward: all weight grads (fp32) and the mean loss (device float). */
int b200_model_loss_and_grads(b200_model *m, const int32_t *dev_tokens, const int32_t *dev_targets, size_t batch,
                              size_t seq_len, float *dev_loss);
/* AdamWOptimizer::step over every registered parameter (cpp/src/Optimizer.cpp:139-149);
 * norm weights are not trained (cpp/src/Trainer.cpp:195-205). */
int b200_model_adamw_step(b200_model *m, float lr, float beta1, float beta2, float eps, float weight_decay);
/* Global-norm gradient clipping for the optimizer step (the reference's MLX trainer: grad_clip_norm,
 * python/apple-silicon/src/pre-training/train.py:858-867; its C++ trainer has none): when the L2 norm of all trainable
 * gradients exceeds max_norm they are scaled by max_norm / (norm + 1e-6) inside the AdamW kernel.  0 (default) = off.
 * Data-parallel steps with clipping all-reduce the gradients first (the sharded optimizer would update buckets before
 * the norm is known).  _last_grad_norm returns the norm and factor of the last clipped step (host; synchronises). */
int b200_model_set_grad_clip(b200_model *m, float max_norm);
int b200_model_last_grad_norm(b200_model *m, float *norm, float *factor);
/* One whole training step from HOST buffers: copies tokens/targets in, runs
 * forward, loss, backward, (gradient all-reduce when data-parallel), AdamW,
 * copies the loss out and synchronises. (Trainer::train step body, cpp/src/Trainer.cpp:263-378) */
int b200_model_train_step_host(b200_model *m, const int32_t *host_tokens, const int32_t *host_targets, size_t batch,
                               size_t seq_len, float lr, float beta1, float beta2, float eps, float weight_decay,
                               float *host_loss);
/* Same with tokens already on the device; loss stays on the device. */
int b200_model_train_step(b200_model *m, const int32_t *dev_tokens, const int32_t *dev_targets, size_t batch,
                          size_t seq_len, float lr, float beta1, float beta2, float eps, float weight_decay,
                          float *dev_loss);
/* One decoder layer through the engine's fused path, for parity tests:
 * h_out = layer(h_in); and the backward given grad_out (TransformerLayer::backward,
 * cpp/src/Transformer.cpp:322-474).  h_in/h_out/grads in compute dtype, [B*S,H]. */
int b200_model_layer_forward(b200_model *m, size_t layer, const void *h_in, void *h_out, size_t batch, size_t seq_len);
int b200_model_layer_backward(b200_model *m, size_t layer, const void *grad_out, void *grad_h_in, size_t batch,
                              size_t seq_len);

/* ---- autoregressive decode with a KV cache.
 * The reference C++ engine threads a KVCache through its signatures but never uses it
 * (cpp/include/TransformerConfig.hpp:121-124, cpp/src/Attention.cpp:171-284) and generates by re-running
 * the full context per token in Python (python/pipeline/inference/sampler.py:115-148).  Here the
 * prompt is run once (prefill fills per-layer K/V caches), then each step runs one token per sequence.
 * Sampling rules follow sampler.py:43-108 (repetition penalty over the last 128 ids, top-k, top-p,
 * temperature; temperature 0 = greedy argmax, lowest id on ties). */
typedef struct {
  float temperature, top_p, repetition_penalty;
  int top_k;                       /* 0 disables */
  uint64_t seed;                   /* counter-based: token t of sequence b depends only on (seed, t, b) */
  int n_whitespace_ids;            /* ids never penalised (sampler.py:27-28), at most 8 */
  int whitespace_ids[8];
} b200_sampler_config;
/* One sampling step for `batch` rows of device logits [batch, vocab] (any vocabulary size; rows of more than 32768
 * entries are worked on in the context workspace instead of shared memory).  history is a device
 * int32 [batch, hist_ld] array whose first hist_len entries per row are the ids seen so far; with append != 0
 * the drawn id is also stored at history[b, hist_len].  out_threshold / out_kept (optional, device) receive
 * the logit threshold and the number of surviving ids per row, for checking the filters. */
int b200_sample(b200_ctx *ctx, const void *logits, b200_dtype dtype, size_t batch, size_t vocab, int32_t *history,
                size_t hist_len, size_t hist_ld, int append, const b200_sampler_config *cfg, uint64_t step,
                int32_t *out_tokens, float *out_threshold, int32_t *out_kept);
/* Allocates K/V caches for `batch` sequences of up to max_total_len positions (<= max_seq_len of the model).  A later
 * call that asks for more sequences or positions re-allocates (the cached keys/values of the earlier generation are
 * dropped); a call that fits the existing caches keeps them. */
int b200_model_decode_begin(b200_model *m, size_t batch, size_t max_total_len);
/* Runs the prompt [batch, prompt_len] (device ids), fills the caches, writes the logits of the last prompt
 * position to logits_last (device, compute dtype, [batch, vocab]). */
int b200_model_prefill(b200_model *m, const int32_t *dev_tokens, size_t batch, size_t prompt_len, void *logits_last);
/* One token per sequence at position `pos` (= number of positions already in the cache): logits [batch, vocab]. */
int b200_model_decode_step(b200_model *m, const int32_t *dev_tokens, size_t batch, size_t pos, void *logits);
/* Whole generation from HOST buffers: prompt [batch, prompt_len] in, [batch, new_tokens] ids out.
 * decode_ms (optional) receives the device time of the new_tokens-1 decode steps (prefill excluded). */
int b200_model_generate(b200_model *m, const int32_t *host_prompt, size_t batch, size_t prompt_len, size_t new_tokens,
                        const b200_sampler_config *cfg, int32_t *host_out, float *prefill_ms, float *decode_ms);

/* ---- training driver files: checkpoints, learning-rate schedule, metrics (host code, no GPU needed for the
 * *_flat and metrics forms).
 * Checkpoint::save / ::load (cpp/src/Checkpoint.cpp:721-1040, 1045-1116): "<path>" holds the weights and
 * "<path with .safetensors -> .opt.safetensors>" the AdamW moments and a U64 "step", both safetensors files in
 * the reference's Python/MLX tensor naming (projections transposed to [out,in], wqkv and w12 fused, fp32).
 * Flat arrays use the parameter order of b200_model_load_params; loading also accepts BF16 / F16 payloads. */
size_t b200_checkpoint_param_count(const b200_model_config *cfg);
int b200_checkpoint_write_flat(const b200_model_config *cfg, const float *params, const float *adam_m /* optional */,
                               const float *adam_v /* optional */, uint64_t step, const char *path);
/* adam_m / adam_v optional; a missing optimizer file leaves them zero, *step 0 and *has_opt_state 0 (the
 * reference restarts the moments in that case, cpp/src/Checkpoint.cpp:1076-1112). */
int b200_checkpoint_read_flat(const b200_model_config *cfg, const char *path, float *params, float *adam_m, float *adam_v,
                              uint64_t *step, int *has_opt_state);
/* Device-resident engine <-> files.  step_override == UINT64_MAX stores the engine's own optimizer step count. */
int b200_checkpoint_save(b200_model *m, const char *path, uint64_t step_override, int with_optimizer);
int b200_checkpoint_load(b200_model *m, const char *path, int with_optimizer, uint64_t *step);
const char *b200_checkpoint_last_error(void);
/* Trainer::get_scheduled_lr (cpp/src/Trainer.cpp:40-51): linear warm-up then cosine decay to lr_min. */
float b200_scheduled_lr(size_t step, size_t warmup_steps, size_t max_steps, float lr_max, float lr_min);
/* metrics.csv of Trainer::train (cpp/src/Trainer.cpp:136-170, 247-255, 347-365): begin writes the header, or on
 * resume keeps the rows below start_step; append adds one row in the reference's column order and formatting. */
int b200_metrics_begin(const char *path, size_t start_step);
int b200_metrics_append(const char *path, size_t step, double train_loss, double tokens_per_sec, double learning_rate,
                        double vram_usage_gb, double mfu_pct, double step_time_ms, uint64_t gpu_calls,
                        double gpu_time_ms, uint64_t cpu_calls, double cpu_time_ms, double gpu_active_pct);

/* ---- data parallel (no counterpart in the reference, which is single-device):
 * replicas all-reduce (average) fp32 gradient buckets with NCCL on a side
 * stream as soon as each layer's weight gradients are enqueued. */
int b200_dp_unique_id(void *out128);                     /* rank 0: ncclGetUniqueId */
int b200_dp_init(b200_model *m, const void *unique_id128, int rank, int world);
int b200_dp_shutdown(b200_model *m);
/* Order-fixed fp64 sum and sum of squares of the model's fp32 master weights (host outputs; synchronises).  Replicas
 * that hold identical weights return bit-identical values: the check that data-parallel ranks have not drifted. */
int b200_model_param_checksum(b200_model *m, double *sum, double *sum_sq);

/* ======================= host-pointer calls (the reference's calling convention) =========
 * Same semantics as the device calls, but every pointer is a HOST pointer:
 * inputs are copied to the device, the kernel runs, outputs are copied back
 * and the stream is synchronised before returning (the reference's behaviour
 * outside a begin_scope/end_scope pair, cpp/src/gpu_kernel/MetalBridge.mm:1384-1406). */
int b200_host_gemm(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int trans_a,
                   int trans_b, b200_dtype dtype);
int b200_host_rms_norm_forward(b200_ctx *ctx, const float *x, float *y, const float *w, float eps, size_t rows, size_t dims);
int b200_host_flash_attn_fwd(b200_ctx *ctx, const float *Q, const float *K, const float *V, float *O, size_t batch,
                             size_t n_heads, size_t n_kv, size_t seq_len, size_t head_dim);
int b200_host_fused_attn_bwd(b200_ctx *ctx, const float *Q, const float *K, const float *V, const float *dO, float *dQ,
                             float *dK, float *dV, size_t batch, size_t n_heads, size_t n_kv, size_t seq_len,
                             size_t head_dim);
int b200_host_cross_entropy(b200_ctx *ctx, const float *logits, const uint32_t *targets, float *loss_out,
                            float *grad_logits, size_t total_tokens, size_t vocab_size);

#ifdef __cplusplus
}
#endif
#endif /* B200_BRIDGE_H */
