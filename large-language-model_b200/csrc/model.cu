// Device-resident training engine for the decoder-only GQA transformer: the B200
// counterpart of Transformer::forward / ::backward, CrossEntropyLoss and AdamW
// (cpp/src/Transformer.cpp:90-197, 322-474, 571-657; cpp/src/Loss.cpp; cpp/src/Optimizer.cpp).
//
// What is kept from the reference: the maths of every op, the double RMSNorm in front of
// the attention projections (cpp/src/Attention.cpp:192-194), interleaved RoPE, [in,out]
// weights, untied output projection, untrained norm weights (cpp/src/Trainer.cpp:195-205),
// mean cross-entropy.  What is B200-first: activations stay in HBM (the reference keeps
// one tensor per layer and recomputes each layer's forward up to three times in
// backward), Q/K/V and gate/up projections are single GEMMs on fused weights, attention
// reads the token-major QKV rows directly (no head split/merge passes), gradients are
// fp32 and all-reduced per layer on a side stream while backward continues.
#include "common.cuh"
#include <chrono>
#include <cstdlib>
#include <dlfcn.h>
#include <vector>

int rope_strided(b200_ctx *, void *, const float *, const float *, size_t, size_t, size_t, size_t, long long,
                 long long, long long, b200_dtype, bool);
int swiglu_fwd_strided(b200_ctx *, const void *, const void *, void *, size_t, size_t, size_t, size_t, b200_dtype);
int swiglu_bwd_strided(b200_ctx *, const void *, const void *, const void *, void *, void *, size_t, size_t, size_t,
                       size_t, size_t, b200_dtype);
int add_norm_norm_oop(b200_ctx *ctx, const void *x, const void *r, void *h_out, const void *w, void *y, const void *w2,
                      void *y2, void *y_scratch, size_t rows, size_t D, float eps, b200_dtype dt);
int add_norm_oop(b200_ctx *, const void *, const void *, void *, const void *, void *, size_t, size_t, float,
                 b200_dtype);
int convert2d(b200_ctx *, const void *, b200_dtype, void *, b200_dtype, size_t, size_t, size_t, size_t);
int fill_const(b200_ctx *, void *, b200_dtype, size_t, float);
int norm_norm_backward_fused(b200_ctx *ctx, const void *g, const void *h, const void *w, const void *res_grad, void *dx,
                             size_t rows, size_t D, float eps, b200_dtype dt);
int adamw_step_bf16_grad(b200_ctx *ctx, float *p, const void *g_bf16, float *m, float *v, void *shadow, size_t n,
                         const b200_adamw_params *a);
int adamw_step_scaled(b200_ctx *ctx, float *p, const float *g, float *m, float *v, void *shadow, size_t n,
                      const b200_adamw_params *a, const float *gscale);
int clip_scale_launch(b200_ctx *ctx, const float *g, size_t n, float max_norm, double *part1024, float *out2);
bool vocab_ce_is_fused(const void *x, const void *w, size_t tokens, size_t V, size_t H, b200_dtype dt);
int vocab_ce_dlogits(b200_ctx *ctx, const void *x, const void *w, const uint32_t *targets, const float *lse, void *dlogits,
                     int in_place, size_t tokens, size_t V, size_t H, b200_dtype dt);

// ---- NCCL, resolved at run time from the library already in the process (or libnccl.so.2) ----
namespace nccl {
typedef struct ncclComm *comm_t;
typedef struct { char internal[128]; } unique_id;
typedef int (*GetUniqueId_t)(unique_id *);
typedef int (*CommInitRank_t)(comm_t *, int, unique_id, int);
typedef int (*CommDestroy_t)(comm_t);
typedef int (*AllReduce_t)(const void *, void *, size_t, int, int, comm_t, cudaStream_t);
typedef const char *(*GetErrorString_t)(int);
typedef int (*CommGetAsyncError_t)(comm_t, int *);
typedef int (*CommAbort_t)(comm_t);
typedef int (*ReduceScatter_t)(const void *, void *, size_t, int, int, comm_t, cudaStream_t);
typedef int (*AllGather_t)(const void *, void *, size_t, int, comm_t, cudaStream_t);
constexpr int kFloat32 = 7, kBfloat16 = 9, kSum = 0, kAvg = 4;
struct Api {
  void *handle = nullptr;
  GetUniqueId_t GetUniqueId = nullptr; CommInitRank_t CommInitRank = nullptr; CommDestroy_t CommDestroy = nullptr;
  AllReduce_t AllReduce = nullptr; GetErrorString_t GetErrorString = nullptr; CommGetAsyncError_t CommGetAsyncError = nullptr;
  CommAbort_t CommAbort = nullptr;
  ReduceScatter_t ReduceScatter = nullptr; AllGather_t AllGather = nullptr;
  bool ok() const { return GetUniqueId && CommInitRank && CommDestroy && AllReduce; }
};
static Api &api() {
  static Api a;
  if (!a.handle) {
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (a.handle) {
      a.GetUniqueId = (GetUniqueId_t)dlsym(a.handle, "ncclGetUniqueId");
      a.CommInitRank = (CommInitRank_t)dlsym(a.handle, "ncclCommInitRank");
      a.CommDestroy = (CommDestroy_t)dlsym(a.handle, "ncclCommDestroy");
      a.AllReduce = (AllReduce_t)dlsym(a.handle, "ncclAllReduce");
      a.GetErrorString = (GetErrorString_t)dlsym(a.handle, "ncclGetErrorString");
      a.CommGetAsyncError = (CommGetAsyncError_t)dlsym(a.handle, "ncclCommGetAsyncError");
      a.CommAbort = (CommAbort_t)dlsym(a.handle, "ncclCommAbort");
      a.ReduceScatter = (ReduceScatter_t)dlsym(a.handle, "ncclReduceScatter");
      a.AllGather = (AllGather_t)dlsym(a.handle, "ncclAllGather");
    }
  }
  return a;
}
}  // namespace nccl

struct b200_model {
  b200_ctx *ctx = nullptr;
  b200_model_config cfg{};
  b200_dtype dt = B200_F32;
  size_t max_batch = 0;
  bool with_opt = false;
  // sizes
  size_t H = 0, I = 0, L = 0, V = 0, nH = 0, nKV = 0, hd = 0, Q = 0, KV = 0, QKV = 0;
  size_t layer_train = 0;   // trainable elements per layer: w_qkv, w_o, w_gate_up, w_down
  size_t n_train = 0;       // emb + L*layer_train + out_proj
  size_t n_total = 0;       // + norm weights (2 per layer + final)
  // flat parameter storage in ENGINE order:
  //   [emb V*H][layer l: w_qkv H*QKV | w_o Q*H | w_gate_up H*2I | w_down I*H][out_proj H*V][norms: (attn,ffn) per layer, final]
  void *params = nullptr;    // compute dtype
  float *master = nullptr;   // fp32 (aliases params in fp32 mode)
  float *grads = nullptr;    // fp32, same order
  float *adam_m = nullptr, *adam_v = nullptr;
  size_t step_count = 0;
  void *ones = nullptr;      // unit weight of the inner norm
  float *cos_t = nullptr, *sin_t = nullptr;
  // activations kept for backward, per layer (compute dtype)
  std::vector<void *> hs;    // L+1 residual-stream states [M,H]
  struct Act { void *a1, *a2, *qkv, *o, *h_mid, *ffn_in, *gate_up, *act; float *lse; bool a1_valid; };
  std::vector<Act> acts;
  // workspace
  void *tmpH = nullptr, *g_act = nullptr, *g_gate_up = nullptr, *g_ffn_in = nullptr, *g_h_mid = nullptr, *g_o = nullptr,
       *g_qkv = nullptr, *g_a2 = nullptr, *g_a1 = nullptr, *g_ping = nullptr, *g_pong = nullptr, *logits = nullptr,
       *fh = nullptr;
  int32_t *d_tokens = nullptr, *d_targets = nullptr;
  float *d_loss = nullptr;
  float grad_clip = 0.f;          // > 0: gradients are scaled so that their global L2 norm does not exceed it
  double *clip_part = nullptr;    // 1024 partial sums of squares
  float *clip_out = nullptr;      // [0] gradient norm of the last clipped step, [1] the factor applied
  float *ce_lse = nullptr;        // [M] log-sum-exp of every token's logits, kept from the loss for its gradient
  // 1: the loss GEMM stores no logits and the gradient of the logits comes from a second run of the projection;
  // 0: the loss GEMM also stores bf16 logits and one in-place pass turns them into their gradient
  int vocab_ce_recompute = 0;
  int32_t *pin_tokens = nullptr, *pin_targets = nullptr; float *pin_loss = nullptr;
  std::vector<void *> allocs;
  // decode: per-layer K/V caches [cache_batch, cache_len, KV] (keys stored after RoPE), generation buffers
  std::vector<void *> k_cache, v_cache;
  size_t cache_batch = 0, cache_len = 0;
  void *dec_logits = nullptr, *dec_h = nullptr;      // [cache_batch, V], [cache_batch, H]
  int32_t *dec_history = nullptr, *dec_next = nullptr;
  float *dec_attn_ws = nullptr;                      // partial results of the split-key decode attention
  int *dec_attn_tickets = nullptr;                   // [cache_batch, nH], zero between launches
  uint64_t dec_graph_nodes = 0;                      // kernel launches in one captured decode step
  unsigned long long *dec_stats = nullptr;           // [2 L][cache_batch][2] row sums of the normalisations folded into the decode projections
  int *dec_pos = nullptr;                            // device copy of the position being decoded (captured steps read it)
  // data parallel
  nccl::comm_t comm = nullptr;
  int rank = 0, world = 1;
  // Sharded optimizer (data parallel, whole training steps): per bucket reduce-scatter of the gradients, AdamW on this
  // rank's 1/world slice, all-gather of the updated compute-dtype weights -- all on the side stream while backward goes
  // on.  The fp32 master weights and the moments are then current only inside this rank's slices until gathered.
  int dp_sharded = 1;              // 0: every rank all-reduces and runs the full AdamW (B200_DP_MODE=allreduce)
  int dp_grad_bf16 = 0;            // 1: gradients cross NVLink as bf16 (B200_DP_GRAD_DTYPE=bf16)
  bool state_sharded = false;      // masters / moments outside this rank's slices are stale
  void *grad_bf16 = nullptr;       // one bucket of bf16 gradients (largest bucket)
  bool comm_failed = false;        // an NCCL call or the communicator reported an error: shut down with ncclCommAbort
  int inject_comm_error = 0;       // test hook: the next gradient exchange fails with this NCCL result code (host side only)
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_grad_ready = nullptr, ev_comm_done = nullptr;
  // optimizer-in-backward: AdamW of a bucket runs on a side stream as soon as its gradients are final and its
  // weights are no longer read by the rest of the backward pass (HBM-bound work under the tensor-bound GEMMs)
  cudaStream_t opt_stream = nullptr;
  cudaEvent_t ev_bucket = nullptr, ev_opt_done = nullptr;
  const b200_adamw_params *fused_opt = nullptr;

  size_t off_emb() const { return 0; }
  size_t off_layer(size_t l) const { return V * H + l * layer_train; }
  size_t off_qkv(size_t l) const { return off_layer(l); }
  size_t off_o(size_t l) const { return off_layer(l) + H * QKV; }
  size_t off_gate_up(size_t l) const { return off_o(l) + Q * H; }
  size_t off_down(size_t l) const { return off_gate_up(l) + H * 2 * I; }
  size_t off_out() const { return V * H + L * layer_train; }
  size_t off_attn_norm(size_t l) const { return n_train + 2 * l * H; }
  size_t off_ffn_norm(size_t l) const { return n_train + (2 * l + 1) * H; }
  size_t off_final_norm() const { return n_train + 2 * L * H; }
  void *P(size_t off) const { return (char *)params + off * dtype_size(dt); }
  float *G(size_t off) const { return grads + off; }
};

static int gather_sharded_state(b200_model *m);

namespace {
int dalloc(b200_model *m, void **p, size_t bytes) {
  int rc = b200_malloc(m->ctx, bytes, p);
  if (rc == B200_OK) m->allocs.push_back(*p);
  return rc;
}
#define TRY(x) do { int rc_ = (x); if (rc_ != B200_OK) return rc_; } while (0)

AttnStrides token_major(const b200_model *m, size_t S) {
  // fused rows [q (nH*hd) | k (nKV*hd) | v (nKV*hd)] per token; output rows [nH*hd]
  AttnStrides st;
  long long ld = (long long)m->QKV;
  st.q_b = (long long)S * ld; st.q_h = (long long)m->hd; st.q_s = ld;
  st.k_b = st.q_b; st.k_h = (long long)m->hd; st.k_s = ld;
  st.v_b = st.q_b; st.v_h = (long long)m->hd; st.v_s = ld;
  st.o_b = (long long)(S * m->Q); st.o_h = (long long)m->hd; st.o_s = (long long)m->Q;
  return st;
}
}  // namespace

extern "C" int b200_model_create(b200_ctx *ctx, const b200_model_config *cfg, b200_dtype dt, size_t max_batch,
                                 int with_optimizer, b200_model **out) {
  B200_REQUIRE(ctx, cfg && out && max_batch > 0, "model_create: bad arguments");
  B200_REQUIRE(ctx, cfg->n_kv_heads > 0 && cfg->n_kv_heads <= cfg->n_heads && cfg->n_heads % cfg->n_kv_heads == 0,
               "n_heads must be a multiple of n_kv_heads (cpp/src/Attention.cpp:45-50)");
  B200_REQUIRE(ctx, cfg->head_dim % 2 == 0 && cfg->hidden_dim > 0 && cfg->vocab_size > 0 && cfg->max_seq_len > 0,
               "model_create: bad dimensions");
  b200_model *m = new b200_model();
  m->ctx = ctx; m->cfg = *cfg; m->dt = dt; m->max_batch = max_batch; m->with_opt = with_optimizer != 0;
  m->H = cfg->hidden_dim; m->I = cfg->intermediate_dim; m->L = cfg->n_layers; m->V = cfg->vocab_size;
  m->nH = cfg->n_heads; m->nKV = cfg->n_kv_heads; m->hd = cfg->head_dim;
  m->Q = m->nH * m->hd; m->KV = m->nKV * m->hd; m->QKV = m->Q + 2 * m->KV;
  m->layer_train = m->H * m->QKV + m->Q * m->H + m->H * 2 * m->I + m->I * m->H;
  m->n_train = 2 * m->V * m->H + m->L * m->layer_train;
  m->n_total = m->n_train + (2 * m->L + 1) * m->H;
  const size_t es = dtype_size(dt), M = max_batch * cfg->max_seq_len, H = m->H, I = m->I;
  int rc = B200_OK;
  auto A = [&](void **p, size_t bytes) { if (rc == B200_OK) rc = dalloc(m, p, bytes); };
  A(&m->params, m->n_total * es);
  if (dt == B200_BF16 && m->with_opt) A((void **)&m->master, m->n_total * 4);
  A((void **)&m->grads, m->n_total * 4);
  if (m->with_opt) { A((void **)&m->adam_m, m->n_train * 4); A((void **)&m->adam_v, m->n_train * 4); }
  A(&m->ones, H * es);
  A((void **)&m->cos_t, cfg->max_seq_len * (m->hd / 2) * 4);
  A((void **)&m->sin_t, cfg->max_seq_len * (m->hd / 2) * 4);
  m->hs.resize(m->L + 1, nullptr);
  for (auto &p : m->hs) A(&p, M * H * es);
  m->acts.resize(m->L);
  for (auto &a : m->acts) {
    A(&a.a1, M * H * es); A(&a.a2, M * H * es); A(&a.qkv, M * m->QKV * es); A(&a.o, M * m->Q * es);
    A(&a.h_mid, M * H * es); A(&a.ffn_in, M * H * es); A(&a.gate_up, M * 2 * I * es); A(&a.act, M * I * es);
    A((void **)&a.lse, max_batch * m->nH * cfg->max_seq_len * 4);
  }
  A(&m->tmpH, M * H * es); A(&m->g_act, M * I * es); A(&m->g_gate_up, M * 2 * I * es); A(&m->g_ffn_in, M * H * es);
  A(&m->g_h_mid, M * H * es); A(&m->g_o, M * m->Q * es); A(&m->g_qkv, M * m->QKV * es); A(&m->g_a2, M * H * es);
  A(&m->g_a1, M * H * es); A(&m->g_ping, M * H * es); A(&m->g_pong, M * H * es); A(&m->logits, M * m->V * es);
  A(&m->fh, M * H * es);
  A((void **)&m->d_tokens, M * 4); A((void **)&m->d_targets, M * 4); A((void **)&m->d_loss, 4);
  A((void **)&m->ce_lse, M * 4);
  A((void **)&m->clip_part, 1024 * sizeof(double)); A((void **)&m->clip_out, 2 * sizeof(float));
  if (const char *e = getenv("B200_VOCAB_CE")) m->vocab_ce_recompute = (e[0] == 'r' || e[0] == '1');   // "recompute" | "store"
  if (rc == B200_OK && (cudaMallocHost(&m->pin_tokens, M * 4) != cudaSuccess || cudaMallocHost(&m->pin_targets, M * 4) != cudaSuccess ||
                        cudaMallocHost(&m->pin_loss, 4) != cudaSuccess))
    rc = b200_fail(ctx, B200_ERR_NOMEM, "pinned host allocation failed");
  if (rc == B200_OK) rc = fill_const(ctx, m->ones, dt, H, 1.0f);
  if (rc == B200_OK) rc = b200_rope_tables(ctx, m->cos_t, m->sin_t, cfg->max_seq_len, m->hd, cfg->rope_base);
  if (rc == B200_OK) rc = b200_fill_zero(ctx, m->params, m->n_total * es);
  if (rc == B200_OK) rc = b200_fill_zero(ctx, m->grads, m->n_total * 4);
  if (rc == B200_OK && m->with_opt) { rc = b200_fill_zero(ctx, m->adam_m, m->n_train * 4); if (!rc) rc = b200_fill_zero(ctx, m->adam_v, m->n_train * 4); }
  if (rc == B200_OK && !m->master && dt == B200_F32) m->master = (float *)m->params;
  if (rc == B200_OK && m->with_opt &&
      (cudaStreamCreateWithFlags(&m->opt_stream, cudaStreamNonBlocking) != cudaSuccess ||
       cudaEventCreateWithFlags(&m->ev_bucket, cudaEventDisableTiming) != cudaSuccess ||
       cudaEventCreateWithFlags(&m->ev_opt_done, cudaEventDisableTiming) != cudaSuccess))
    rc = b200_fail(ctx, B200_ERR_CUDA, "side stream for the optimizer could not be created");
  if (rc != B200_OK) { b200_model_destroy(m); return rc; }
  *out = m;
  return B200_OK;
}

extern "C" int b200_model_destroy(b200_model *m) {
  if (!m) return B200_OK;
  m->state_sharded = false;            // nobody reads the state again: no collective on the way out
  b200_dp_shutdown(m);
  cudaStreamSynchronize(m->ctx->stream);
  if (m->opt_stream) { cudaStreamSynchronize(m->opt_stream); cudaStreamDestroy(m->opt_stream); }
  if (m->ev_bucket) cudaEventDestroy(m->ev_bucket);
  if (m->ev_opt_done) cudaEventDestroy(m->ev_opt_done);
  for (void *p : m->allocs) cudaFree(p);
  if (m->pin_tokens) cudaFreeHost(m->pin_tokens);
  if (m->pin_targets) cudaFreeHost(m->pin_targets);
  if (m->pin_loss) cudaFreeHost(m->pin_loss);
  delete m;
  return B200_OK;
}

extern "C" size_t b200_model_param_count(const b200_model *m) { return m ? m->n_total : 0; }
extern "C" int b200_model_get_config(const b200_model *m, b200_model_config *out) {
  if (!m || !out) return B200_ERR_INVALID;
  *out = m->cfg;
  return B200_OK;
}

// ---- import / export in the reference's per-tensor order -----------------------------------
namespace {
struct Piece { size_t ref_off, rows, cols, eng_off, eng_ld; };
// Maps every reference tensor onto its (possibly strided) place in the engine's fused storage.
std::vector<Piece> layout_map(const b200_model *m) {
  std::vector<Piece> v;
  size_t r = 0;
  const size_t H = m->H, I = m->I, Q = m->Q, KV = m->KV, QKV = m->QKV;
  v.push_back({r, m->V, H, m->off_emb(), H}); r += m->V * H;
  for (size_t l = 0; l < m->L; ++l) {
    v.push_back({r, 1, H, m->off_attn_norm(l), H}); r += H;
    v.push_back({r, H, Q, m->off_qkv(l), QKV}); r += H * Q;
    v.push_back({r, H, KV, m->off_qkv(l) + Q, QKV}); r += H * KV;
    v.push_back({r, H, KV, m->off_qkv(l) + Q + KV, QKV}); r += H * KV;
    v.push_back({r, Q, H, m->off_o(l), H}); r += Q * H;
    v.push_back({r, 1, H, m->off_ffn_norm(l), H}); r += H;
    v.push_back({r, H, I, m->off_gate_up(l), 2 * I}); r += H * I;
    v.push_back({r, H, I, m->off_gate_up(l) + I, 2 * I}); r += H * I;
    v.push_back({r, I, H, m->off_down(l), H}); r += I * H;
  }
  v.push_back({r, 1, H, m->off_final_norm(), H}); r += H;
  v.push_back({r, H, m->V, m->off_out(), m->V});
  return v;
}
}  // namespace

extern "C" int b200_model_load_params(b200_model *m, const float *host) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(gather_sharded_state(m));        // moments of other ranks' slices must not be lost by overwriting only the weights
  B200_REQUIRE(ctx, host, "model_load_params: null pointer");
  auto map = layout_map(m);
  size_t biggest = 0;
  for (auto &p : map) biggest = p.rows * p.cols > biggest ? p.rows * p.cols : biggest;
  float *stage = nullptr;
  TRY(b200_malloc(ctx, biggest * 4, (void **)&stage));
  int rc = B200_OK;
  for (auto &p : map) {
    rc = b200_memcpy_h2d(ctx, stage, host + p.ref_off, p.rows * p.cols * 4);
    if (!rc) rc = convert2d(ctx, stage, B200_F32, m->P(p.eng_off), m->dt, p.rows, p.cols, p.cols, p.eng_ld);
    if (!rc && m->master && (void *)m->master != m->params)
      rc = convert2d(ctx, stage, B200_F32, m->master + p.eng_off, B200_F32, p.rows, p.cols, p.cols, p.eng_ld);
    if (!rc) rc = b200_sync(ctx);     // stage is reused by the next tensor
    if (rc) break;
  }
  b200_free(ctx, stage);
  return rc;
}

static int export_flat(b200_model *m, const void *src, b200_dtype sdt, float *host) {
  b200_ctx *ctx = m->ctx;
  auto map = layout_map(m);
  size_t biggest = 0;
  for (auto &p : map) biggest = p.rows * p.cols > biggest ? p.rows * p.cols : biggest;
  float *stage = nullptr;
  TRY(b200_malloc(ctx, biggest * 4, (void **)&stage));
  int rc = B200_OK;
  for (auto &p : map) {
    rc = convert2d(ctx, (const char *)src + p.eng_off * dtype_size(sdt), sdt, stage, B200_F32, p.rows, p.cols, p.eng_ld, p.cols);
    if (!rc) rc = b200_memcpy_d2h(ctx, host + p.ref_off, stage, p.rows * p.cols * 4);
    if (!rc) rc = b200_sync(ctx);
    if (rc) break;
  }
  b200_free(ctx, stage);
  return rc;
}
extern "C" int b200_model_read_params(b200_model *m, float *host) {
  if (!m || !host) return B200_ERR_INVALID;
  TRY(gather_sharded_state(m));
  if (m->master) return export_flat(m, m->master, B200_F32, host);
  return export_flat(m, m->params, m->dt, host);
}
extern "C" int b200_model_read_grads(b200_model *m, float *host) {
  if (!m || !host) return B200_ERR_INVALID;
  return export_flat(m, m->grads, B200_F32, host);
}

// AdamW moments in the same per-tensor order as the parameters (norm weights are not trained by the reference,
// cpp/src/Trainer.cpp:188-198: their slots read as zero and are ignored on load) plus the step counter, for
// checkpoints (cpp/src/Checkpoint.cpp:836-1040).
extern "C" int b200_model_read_opt_state(b200_model *m, float *host_m, float *host_v, uint64_t *step) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, m->with_opt && host_m && host_v && step, "read_opt_state: model has no optimizer state or null pointer");
  TRY(gather_sharded_state(m));
  auto map = layout_map(m);
  size_t biggest = 0;
  for (auto &p : map) biggest = p.rows * p.cols > biggest ? p.rows * p.cols : biggest;
  float *stage = nullptr;
  TRY(b200_malloc(ctx, biggest * 4, (void **)&stage));
  int rc = B200_OK;
  for (int which = 0; which < 2 && !rc; ++which) {
    const float *src = which ? m->adam_v : m->adam_m;
    float *host = which ? host_v : host_m;
    for (auto &p : map) {
      if (p.eng_off >= m->n_train) { memset(host + p.ref_off, 0, p.rows * p.cols * 4); continue; }
      rc = convert2d(ctx, src + p.eng_off, B200_F32, stage, B200_F32, p.rows, p.cols, p.eng_ld, p.cols);
      if (!rc) rc = b200_memcpy_d2h(ctx, host + p.ref_off, stage, p.rows * p.cols * 4);
      if (!rc) rc = b200_sync(ctx);
      if (rc) break;
    }
  }
  b200_free(ctx, stage);
  *step = m->step_count;
  return rc;
}
extern "C" int b200_model_load_opt_state(b200_model *m, const float *host_m, const float *host_v, uint64_t step) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, m->with_opt && host_m && host_v, "load_opt_state: model has no optimizer state or null pointer");
  TRY(gather_sharded_state(m));
  auto map = layout_map(m);
  size_t biggest = 0;
  for (auto &p : map) biggest = p.rows * p.cols > biggest ? p.rows * p.cols : biggest;
  float *stage = nullptr;
  TRY(b200_malloc(ctx, biggest * 4, (void **)&stage));
  int rc = B200_OK;
  for (int which = 0; which < 2 && !rc; ++which) {
    float *dst = which ? m->adam_v : m->adam_m;
    const float *host = which ? host_v : host_m;
    for (auto &p : map) {
      if (p.eng_off >= m->n_train) continue;
      rc = b200_memcpy_h2d(ctx, stage, host + p.ref_off, p.rows * p.cols * 4);
      if (!rc) rc = convert2d(ctx, stage, B200_F32, dst + p.eng_off, B200_F32, p.rows, p.cols, p.cols, p.eng_ld);
      if (!rc) rc = b200_sync(ctx);
      if (rc) break;
    }
  }
  b200_free(ctx, stage);
  m->step_count = (size_t)step;
  return rc;
}

extern "C" int b200_model_init_synthetic(b200_model *m, uint64_t seed, float std) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(gather_sharded_state(m));
  // trainable tensors ~ N(0, std); norm weights 1 (cpp/src/RMSNorm.cpp:32)
  if (m->master && (void *)m->master != m->params) {
    TRY(b200_fill_normal(ctx, m->master, B200_F32, m->n_train, seed, std));
    TRY(fill_const(ctx, m->master + m->n_train, B200_F32, m->n_total - m->n_train, 1.0f));
    TRY(b200_convert(ctx, m->master, B200_F32, m->params, m->dt, m->n_total));
  } else {
    TRY(b200_fill_normal(ctx, m->params, m->dt, m->n_train, seed, std));
    TRY(fill_const(ctx, m->P(m->n_train), m->dt, m->n_total - m->n_train, 1.0f));
  }
  return B200_OK;
}

// ---- one decoder layer ------------------------------------------------------------------
// Forward, given the layer input h_in and its first norm output a1 already in acts[l].a1:
// returns h_mid and ffn_out(tmpH) so that the caller fuses "h_out = h_mid + ffn_out" with the next norm.
static int layer_forward_core(b200_model *m, size_t l, const void *h_in, size_t B, size_t S, bool a2_ready = false) {
  b200_ctx *ctx = m->ctx;
  const size_t M = B * S, H = m->H, I = m->I;
  const float eps = m->cfg.rms_norm_eps;
  b200_model::Act &a = m->acts[l];
  const b200_dtype dt = m->dt;
  // inner unit-weight norm (cpp/src/Attention.cpp:192-194), unless the caller produced it with the outer one
  if (!a2_ready) TRY(b200_rms_norm_forward(ctx, a.a1, a.a2, m->ones, nullptr, eps, M, H, dt));
  // Q|K|V in one GEMM on the fused weight
  // RoPE on the q and k column blocks (cpp/src/Attention.cpp:203): in the GEMM epilogue on the tensor-core
  // path (applied to the fp32 accumulators), else as its own in-place pass
  const long long ld = (long long)m->QKV;
  const bool rope_in_gemm = dt == B200_BF16 && m->hd % 32 == 0 &&
                            gemm_tc_supported(a.a2, m->P(m->off_qkv(l)), a.qkv, M, m->QKV, H, H, m->QKV, m->QKV, dt);
  if (rope_in_gemm) {
    GemmEpilogue epi;
    epi.cos_t = m->cos_t; epi.sin_t = m->sin_t; epi.S = (int)S; epi.hd = (int)m->hd; epi.cols = (int)(m->Q + m->KV);
    TRY(b200_gemm_ld(ctx, a.a2, m->P(m->off_qkv(l)), a.qkv, M, m->QKV, H, 0, 0, 0, dt, dt, H, m->QKV, m->QKV, &epi));
  } else {
    TRY(b200_gemm_ld(ctx, a.a2, m->P(m->off_qkv(l)), a.qkv, M, m->QKV, H, 0, 0, 0, dt, dt, H, m->QKV, m->QKV));
    TRY(rope_strided(ctx, a.qkv, m->cos_t, m->sin_t, B, m->nH + m->nKV, S, m->hd, (long long)S * ld, (long long)m->hd, ld, dt, false));
  }
  AttnStrides st = token_major(m, S);
  const char *qkv = (const char *)a.qkv;
  TRY(attn_fwd_launch(ctx, qkv, qkv + m->Q * dtype_size(dt), qkv + (m->Q + m->KV) * dtype_size(dt), a.o, a.lse, B, m->nH,
                      m->nKV, S, m->hd, st, dt));
  TRY(b200_gemm_ld(ctx, a.o, m->P(m->off_o(l)), m->tmpH, M, H, m->Q, 0, 0, 0, dt, dt, m->Q, H, H));
  // h_mid = h_in + attn_out ; ffn_in = rmsnorm(h_mid) * ffn_norm_w   (cpp/src/Transformer.cpp:178-179)
  TRY(add_norm_oop(ctx, h_in, m->tmpH, a.h_mid, m->P(m->off_ffn_norm(l)), a.ffn_in, M, H, eps, dt));
  if (dt == B200_BF16 && !(ctx->gemm_skinny && gemm_skinny_supported(M, 0, 0, 0)) && gemm_tc2_swiglu_eligible(ctx, M, I) &&
      gemm_tc_supported(a.ffn_in, m->P(m->off_gate_up(l)), a.gate_up, M, 2 * I, H, H, 2 * I, 2 * I, dt) && (I * 2) % 16 == 0) {
    // gate and up are stored for the backward pass and silu(gate) * up leaves the same GEMM epilogue
    GemmEpilogue epi;
    epi.swiglu_I = (int)I; epi.act_out = a.act; epi.ld_act = I;
    TRY(b200_gemm_ld(ctx, a.ffn_in, m->P(m->off_gate_up(l)), a.gate_up, M, 2 * I, H, 0, 0, 0, dt, dt, H, 2 * I, 2 * I, &epi));
  } else {
    TRY(b200_gemm_ld(ctx, a.ffn_in, m->P(m->off_gate_up(l)), a.gate_up, M, 2 * I, H, 0, 0, 0, dt, dt, H, 2 * I, 2 * I));
    TRY(swiglu_fwd_strided(ctx, a.gate_up, (char *)a.gate_up + I * dtype_size(dt), a.act, M, I, 2 * I, I, dt));
  }
  TRY(b200_gemm_ld(ctx, a.act, m->P(m->off_down(l)), m->tmpH, M, H, I, 0, 0, 0, dt, dt, I, H, H));
  return B200_OK;
}

// Backward of layer l: g = dL/dh_out -> g_in = dL/dh_in, weight grads into m->grads (overwritten).
static int layer_backward_core(b200_model *m, size_t l, const void *g, void *g_in, size_t B, size_t S) {
  b200_ctx *ctx = m->ctx;
  const size_t M = B * S, H = m->H, I = m->I;
  const float eps = m->cfg.rms_norm_eps;
  b200_model::Act &a = m->acts[l];
  const b200_dtype dt = m->dt;
  const size_t es = dtype_size(dt);
  // B. down projection (cpp/src/Transformer.cpp:382-401)
  TRY(b200_gemm_ld(ctx, a.act, g, m->G(m->off_down(l)), I, H, M, 1, 0, 0, dt, B200_F32, I, H, H));
  TRY(b200_gemm_ld(ctx, g, m->P(m->off_down(l)), m->g_act, M, I, H, 0, 1, 0, dt, dt, H, H, I));
  // C. SwiGLU and gate/up projections (:405-439).  (Turning dY into d_gate | d_up inside that GEMM's epilogue was
  // measured slower, 163.8 vs 161.1 ms per step on the same GPU: the row-scattered gate/up reads stretch the epilogue
  // of a K = 2048 tile past its main loop.)
  TRY(swiglu_bwd_strided(ctx, m->g_act, a.gate_up, (char *)a.gate_up + I * es, m->g_gate_up, (char *)m->g_gate_up + I * es, M, I, I, 2 * I, 2 * I, dt));
  TRY(b200_gemm_ld(ctx, a.ffn_in, m->g_gate_up, m->G(m->off_gate_up(l)), H, 2 * I, M, 1, 0, 0, dt, B200_F32, H, 2 * I, 2 * I));
  TRY(b200_gemm_ld(ctx, m->g_gate_up, m->P(m->off_gate_up(l)), m->g_ffn_in, M, H, 2 * I, 0, 1, 0, dt, dt, 2 * I, 2 * I, H));
  // D. ffn norm + residual (:442-453)
  TRY(b200_fused_backward_add_norm(ctx, m->g_ffn_in, a.h_mid, m->P(m->off_ffn_norm(l)), g, m->g_h_mid, M, H, eps, dt));
  // E. attention (cpp/src/Attention.cpp:472-594)
  TRY(b200_gemm_ld(ctx, a.o, m->g_h_mid, m->G(m->off_o(l)), m->Q, H, M, 1, 0, 0, dt, B200_F32, m->Q, H, H));
  TRY(b200_gemm_ld(ctx, m->g_h_mid, m->P(m->off_o(l)), m->g_o, M, m->Q, H, 0, 1, 0, dt, dt, H, H, m->Q));
  AttnStrides st = token_major(m, S);
  const char *qkv = (const char *)a.qkv; char *gq = (char *)m->g_qkv;
  // the gradient of RoPE (inverse rotation of dQ and dK) is applied inside the tensor-core attention backward
  // where that path runs, else as its own in-place pass (cpp/src/Attention.cpp:544)
  const bool rope_in_attn = attn_bwd_fuses_rope(B, m->nH, m->nKV, S, m->hd, st, st, dt, qkv, qkv + m->Q * es, qkv + (m->Q + m->KV) * es,
                                                a.o, m->g_o, gq, gq + m->Q * es, gq + (m->Q + m->KV) * es);
  TRY(attn_bwd_launch(ctx, qkv, qkv + m->Q * es, qkv + (m->Q + m->KV) * es, a.o, m->g_o, a.lse, gq, gq + m->Q * es,
                      gq + (m->Q + m->KV) * es, B, m->nH, m->nKV, S, m->hd, st, st, dt, rope_in_attn ? m->cos_t : nullptr,
                      rope_in_attn ? m->sin_t : nullptr));
  const long long ld = (long long)m->QKV;
  if (!rope_in_attn)
    TRY(rope_strided(ctx, gq, m->cos_t, m->sin_t, B, m->nH + m->nKV, S, m->hd, (long long)S * ld, (long long)m->hd, ld, dt, true));
  TRY(b200_gemm_ld(ctx, a.a2, m->g_qkv, m->G(m->off_qkv(l)), H, m->QKV, M, 1, 0, 0, dt, B200_F32, H, m->QKV, m->QKV));
  TRY(b200_gemm_ld(ctx, m->g_qkv, m->P(m->off_qkv(l)), m->g_a2, M, H, m->QKV, 0, 1, 0, dt, dt, m->QKV, m->QKV, H));
  // the attention's inner unit-weight norm and F. attn norm + residual (cpp/src/Transformer.cpp:460-471) in one pass
  // that recomputes the first norm's output from the layer input; two passes for row shapes the warp kernel does not take
  static const bool allow_fused = !(getenv("B200_NORM_BWD_FUSED") && getenv("B200_NORM_BWD_FUSED")[0] == '0');   // A/B switch
  const int fused = allow_fused ? norm_norm_backward_fused(ctx, m->g_a2, m->hs[l], m->P(m->off_attn_norm(l)), m->g_h_mid, g_in, M, H, eps, dt) : 0;
  if (fused < 0) return fused;
  if (fused == 0) {
    if (!a.a1_valid) {     // the forward pass skipped the first norm's output: make it now
      TRY(b200_rms_norm_forward(ctx, m->hs[l], a.a1, m->P(m->off_attn_norm(l)), nullptr, eps, M, H, dt));
      a.a1_valid = true;
    }
    TRY(b200_rms_norm_backward(ctx, m->g_a2, a.a1, m->ones, m->g_a1, nullptr, eps, M, H, dt));
    TRY(b200_fused_backward_add_norm(ctx, m->g_a1, m->hs[l], m->P(m->off_attn_norm(l)), m->g_h_mid, g_in, M, H, eps, dt));
  }
  return B200_OK;
}

static int check_shape(b200_model *m, size_t B, size_t S) {
  B200_REQUIRE(m->ctx, B > 0 && B <= m->max_batch && S > 0 && S <= m->cfg.max_seq_len,
               "batch/sequence exceed what the model was created for (cpp/src/Positional.cpp:90-94)");
  return B200_OK;
}

static int forward_all(b200_model *m, const int32_t *tok, size_t B, size_t S) {
  b200_ctx *ctx = m->ctx;
  const size_t M = B * S, H = m->H;
  const float eps = m->cfg.rms_norm_eps;
  const b200_dtype dt = m->dt;
  TRY(b200_embedding_forward(ctx, (const uint32_t *)tok, m->P(m->off_emb()), m->hs[0], M, H, m->V, dt));
  if (m->L == 0) return b200_rms_norm_forward(ctx, m->hs[0], m->fh, m->P(m->off_final_norm()), nullptr, eps, M, H, dt);
  // the layer's outer norm and the attention's inner unit-weight norm are produced in one pass
  // The first norm's output a1 is only an intermediate here: the backward pass recomputes it from the layer input, so it
  // is not written (a1 doubles as the scratch of the two-pass route for row shapes the one-pass kernel does not take).
  TRY(add_norm_norm_oop(ctx, m->hs[0], nullptr, nullptr, m->P(m->off_attn_norm(0)), nullptr, m->ones, m->acts[0].a2, m->acts[0].a1, M, H, eps, dt));
  m->acts[0].a1_valid = false;
  for (size_t l = 0; l < m->L; ++l) {
    TRY(layer_forward_core(m, l, m->hs[l], B, S, true));
    // h_out = h_mid + ffn_out, fused with the norm(s) that consume it next
    if (l + 1 < m->L) {
      TRY(add_norm_norm_oop(ctx, m->acts[l].h_mid, m->tmpH, m->hs[l + 1], m->P(m->off_attn_norm(l + 1)), nullptr, m->ones,
                            m->acts[l + 1].a2, m->acts[l + 1].a1, M, H, eps, dt));
      m->acts[l + 1].a1_valid = false;
    }
    else
      TRY(add_norm_oop(ctx, m->acts[l].h_mid, m->tmpH, m->hs[l + 1], m->P(m->off_final_norm()), m->fh, M, H, eps, dt));
  }
  return B200_OK;
}

extern "C" int b200_model_forward(b200_model *m, const int32_t *tok, size_t B, size_t S, void *logits_out) {
  if (!m) return B200_ERR_INVALID;
  TRY(check_shape(m, B, S));
  B200_REQUIRE(m->ctx, tok, "model_forward: null tokens");
  TRY(forward_all(m, tok, B, S));
  void *lg = logits_out ? logits_out : m->logits;
  return b200_gemm_ld(m->ctx, m->fh, m->P(m->off_out()), lg, B * S, m->V, m->H, 0, 0, 0, m->dt, m->dt, m->H, m->V, m->V);
}

static int allreduce_async(b200_model *m, float *buf, size_t n) {
  if (!m->comm || (m->world <= 1 && !m->inject_comm_error)) return B200_OK;
  b200_ctx *ctx = m->ctx;
  B200_CUDA(ctx, cudaEventRecord(m->ev_grad_ready, ctx->stream));
  B200_CUDA(ctx, cudaStreamWaitEvent(m->comm_stream, m->ev_grad_ready, 0));
  int r;
  if (m->inject_comm_error) { r = m->inject_comm_error; m->inject_comm_error = 0; }     // injected on the host: nothing is launched
  else r = nccl::api().AllReduce(buf, buf, n, nccl::kFloat32, nccl::kAvg, m->comm, m->comm_stream);
  if (r != 0) {
    m->comm_failed = true;
    return b200_fail(ctx, B200_ERR_COMM, "ncclAllReduce failed: %s", nccl::api().GetErrorString ? nccl::api().GetErrorString(r) : "?");
  }
  return B200_OK;
}
static bool dp_shardable(const b200_model *m) {
  // every bucket splits into `world` slices whose offsets keep the 16-byte alignment AdamW and the vector loads want
  const size_t q = (size_t)m->world * 8;
  // (global-norm clipping needs every bucket's gradients before the first update: it runs the all-reduce route)
  return m->world > 1 && m->comm && m->dp_sharded && m->grad_clip <= 0.f && m->with_opt && m->master && nccl::api().ReduceScatter && nccl::api().AllGather &&
         (m->V * m->H) % q == 0 && m->layer_train % q == 0;
}
// Sharded-optimizer exchange of bucket [off, off+n): everything below runs on the side stream, after the work enqueued so
// far on the main stream (the bucket's weight gradients AND the last kernel that reads the bucket's weights).
static int sharded_bucket(b200_model *m, size_t off, size_t n) {
  b200_ctx *ctx = m->ctx;
  const size_t sh = n / (size_t)m->world, mine = off + (size_t)m->rank * sh;
  const size_t es = dtype_size(m->dt);
  B200_CUDA(ctx, cudaEventRecord(m->ev_grad_ready, ctx->stream));
  B200_CUDA(ctx, cudaStreamWaitEvent(m->comm_stream, m->ev_grad_ready, 0));
  cudaStream_t keep = ctx->stream;
  ctx->stream = m->comm_stream;
  int rc = B200_OK, r = 0;
  void *shadow = ((void *)m->master != m->params) ? (void *)((char *)m->params + mine * es) : nullptr;
  if (m->inject_comm_error) { r = m->inject_comm_error; m->inject_comm_error = 0; }
  else if (m->dp_grad_bf16) {
    rc = b200_convert(ctx, m->grads + off, B200_F32, m->grad_bf16, B200_BF16, n);
    if (!rc) r = nccl::api().ReduceScatter(m->grad_bf16, (char *)m->grad_bf16 + (size_t)m->rank * sh * 2, sh, nccl::kBfloat16, nccl::kAvg, m->comm, m->comm_stream);
    if (!rc && !r) rc = adamw_step_bf16_grad(ctx, m->master + mine, (char *)m->grad_bf16 + (size_t)m->rank * sh * 2, m->adam_m + mine, m->adam_v + mine, shadow, sh, m->fused_opt);
  } else {
    r = nccl::api().ReduceScatter(m->grads + off, m->grads + mine, sh, nccl::kFloat32, nccl::kAvg, m->comm, m->comm_stream);
    if (!r) rc = b200_adamw_step(ctx, m->master + mine, m->grads + mine, m->adam_m + mine, m->adam_v + mine, shadow, sh, m->fused_opt);
  }
  if (!rc && !r)
    r = nccl::api().AllGather((char *)m->params + mine * es, (char *)m->params + off * es, sh, m->dt == B200_BF16 ? nccl::kBfloat16 : nccl::kFloat32,
                              m->comm, m->comm_stream);
  ctx->stream = keep;
  if (r != 0) {
    m->comm_failed = true;
    return b200_fail(ctx, B200_ERR_COMM, "NCCL reduce-scatter / all-gather failed: %s", nccl::api().GetErrorString ? nccl::api().GetErrorString(r) : "?");
  }
  m->state_sharded = true;
  return rc;
}
// Brings the fp32 master weights and the AdamW moments of every rank's slices to all ranks (collective: every rank calls).
static int gather_sharded_state(b200_model *m) {
  if (!m->state_sharded || !m->comm || m->world <= 1) return B200_OK;
  b200_ctx *ctx = m->ctx;
  TRY(b200_sync(ctx));
  auto gather = [&](float *base, size_t off, size_t n) -> int {
    if (!base) return 0;
    const size_t sh = n / (size_t)m->world;
    return nccl::api().AllGather(base + off + (size_t)m->rank * sh, base + off, sh, nccl::kFloat32, m->comm, m->comm_stream);
  };
  int r = 0;
  float *arrays[3] = {((void *)m->master != m->params) ? m->master : nullptr, m->adam_m, m->adam_v};   // fp32 models: params were gathered already
  for (float *a : arrays) {
    if (!r) r = gather(a, m->off_emb(), m->V * m->H);
    for (size_t l = 0; l < m->L && !r; ++l) r = gather(a, m->off_layer(l), m->layer_train);
    if (!r) r = gather(a, m->off_out(), m->H * m->V);
  }
  if (r != 0) { m->comm_failed = true; return b200_fail(ctx, B200_ERR_COMM, "ncclAllGather of the optimizer state failed"); }
  B200_CUDA(ctx, cudaStreamSynchronize(m->comm_stream));
  m->state_sharded = false;
  return B200_OK;
}

// AdamW for parameters [off, off+n) on the side stream, ordered after everything enqueued so far on the main stream
// (and, data-parallel, after the bucket's all-reduce, which runs on that same side stream).
static int opt_bucket(b200_model *m, size_t off, size_t n) {
  if (!m->fused_opt || !n) return B200_OK;
  b200_ctx *ctx = m->ctx;
  cudaStream_t side = (m->world > 1 && m->comm) ? m->comm_stream : m->opt_stream;
  B200_CUDA(ctx, cudaEventRecord(m->ev_bucket, ctx->stream));
  B200_CUDA(ctx, cudaStreamWaitEvent(side, m->ev_bucket, 0));
  void *shadow = ((void *)m->master != m->params) ? (void *)((char *)m->params + off * dtype_size(m->dt)) : nullptr;
  cudaStream_t keep = ctx->stream;
  ctx->stream = side;
  const int rc = b200_adamw_step(ctx, m->master + off, m->grads + off, m->adam_m + off, m->adam_v + off, shadow, n, m->fused_opt);
  ctx->stream = keep;
  return rc;
}
static int opt_join(b200_model *m) {
  if (!m->fused_opt || (m->world > 1 && m->comm)) return B200_OK;     // data-parallel: allreduce_join covers the side stream
  b200_ctx *ctx = m->ctx;
  B200_CUDA(ctx, cudaEventRecord(m->ev_opt_done, m->opt_stream));
  B200_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, m->ev_opt_done, 0));
  return B200_OK;
}
static int allreduce_join(b200_model *m) {
  if (m->world <= 1 || !m->comm) return B200_OK;
  b200_ctx *ctx = m->ctx;
  B200_CUDA(ctx, cudaEventRecord(m->ev_comm_done, m->comm_stream));
  B200_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, m->ev_comm_done, 0));
  if (nccl::api().CommGetAsyncError) {
    int aerr = 0;
    if (nccl::api().CommGetAsyncError(m->comm, &aerr) == 0 && aerr != 0) {
      m->comm_failed = true;
      return b200_fail(ctx, B200_ERR_COMM, "NCCL asynchronous error %d", aerr);
    }
  }
  return B200_OK;
}

extern "C" int b200_model_loss_and_grads(b200_model *m, const int32_t *tok, const int32_t *tgt, size_t B, size_t S,
                                         float *dev_loss) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(check_shape(m, B, S));
  B200_REQUIRE(ctx, tok && tgt && dev_loss, "model_loss_and_grads: null pointer");
  const size_t M = B * S, H = m->H, V = m->V;
  const float eps = m->cfg.rms_norm_eps;
  const b200_dtype dt = m->dt;
  TRY(forward_all(m, tok, B, S));
  // vocabulary projection + loss in one GEMM: per-row softmax statistics leave the epilogue (cpp/src/Transformer.cpp:190-196,
  // cpp/src/Loss.cpp:77-134); then d(loss)/d(logits) in m->logits (cpp/src/Loss.cpp:163-194), either from stored logits in
  // one in-place pass or from a second run of the projection with the gradient epilogue
  const bool keep_logits = !m->vocab_ce_recompute || !vocab_ce_is_fused(m->fh, m->P(m->off_out()), M, V, H, dt);
  TRY(b200_vocab_ce_forward(ctx, m->fh, m->P(m->off_out()), (const uint32_t *)tgt, dev_loss, m->ce_lse, keep_logits ? m->logits : nullptr, M, V, H, dt));
  TRY(vocab_ce_dlogits(ctx, m->fh, m->P(m->off_out()), (const uint32_t *)tgt, m->ce_lse, m->logits, keep_logits, M, V, H, dt));
  // output projection (cpp/src/Transformer.cpp:515-521, 607-627) and final norm (:632)
  const bool sharded = m->fused_opt && dp_shardable(m);
  TRY(b200_gemm_ld(ctx, m->fh, m->logits, m->G(m->off_out()), H, V, M, 1, 0, 0, dt, B200_F32, H, V, V));
  if (!sharded) TRY(allreduce_async(m, m->G(m->off_out()), H * V));
  TRY(b200_gemm_ld(ctx, m->logits, m->P(m->off_out()), m->tmpH, M, H, V, 0, 1, 0, dt, dt, V, V, H));
  // after the data-gradient GEMM, the last reader of this weight
  if (sharded) TRY(sharded_bucket(m, m->off_out(), H * V)); else TRY(opt_bucket(m, m->off_out(), H * V));
  void *g = m->g_ping, *g_next = m->g_pong;
  TRY(b200_rms_norm_backward(ctx, m->tmpH, m->hs[m->L], m->P(m->off_final_norm()), g, nullptr, eps, M, H, dt));
  for (size_t l = m->L; l-- > 0;) {
    TRY(layer_backward_core(m, l, g, g_next, B, S));
    if (sharded) TRY(sharded_bucket(m, m->off_layer(l), m->layer_train));
    else { TRY(allreduce_async(m, m->G(m->off_layer(l)), m->layer_train)); TRY(opt_bucket(m, m->off_layer(l), m->layer_train)); }
    void *t = g; g = g_next; g_next = t;
  }
  TRY(b200_embedding_backward(ctx, (const uint32_t *)tok, g, m->G(m->off_emb()), M, H, V, dt));
  if (sharded) TRY(sharded_bucket(m, m->off_emb(), V * H));
  else { TRY(allreduce_async(m, m->G(m->off_emb()), V * H)); TRY(opt_bucket(m, m->off_emb(), V * H)); }
  TRY(opt_join(m));
  return allreduce_join(m);
}

extern "C" int b200_model_adamw_step(b200_model *m, float lr, float beta1, float beta2, float eps, float wd) {
  if (!m) return B200_ERR_INVALID;
  B200_REQUIRE(m->ctx, m->with_opt && m->master, "model was created without optimizer state");
  TRY(gather_sharded_state(m));
  m->step_count++;
  b200_adamw_params p;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = wd;
  p.bias_correction1 = 1.0f - powf(beta1, (float)m->step_count);   // cpp/src/Optimizer.cpp:141-142
  p.bias_correction2 = 1.0f - powf(beta2, (float)m->step_count);
  void *shadow = ((void *)m->master != m->params) ? m->params : nullptr;
  if (m->grad_clip > 0.f) {
    TRY(clip_scale_launch(m->ctx, m->grads, m->n_train, m->grad_clip, m->clip_part, m->clip_out));
    return adamw_step_scaled(m->ctx, m->master, m->grads, m->adam_m, m->adam_v, shadow, m->n_train, &p, m->clip_out + 1);
  }
  return b200_adamw_step(m->ctx, m->master, m->grads, m->adam_m, m->adam_v, shadow, m->n_train, &p);
}
// Optional global-norm gradient clipping of the optimizer step (the MLX trainer's grad_clip_norm,
// python/apple-silicon/src/pre-training/train.py:858-867; the C++ trainer has none): 0 turns it off.
extern "C" int b200_model_set_grad_clip(b200_model *m, float max_norm) {
  if (!m) return B200_ERR_INVALID;
  B200_REQUIRE(m->ctx, max_norm >= 0.f, "set_grad_clip: the norm bound must not be negative");
  m->grad_clip = max_norm;
  return B200_OK;
}
// Norm of the gradients and the factor applied in the last clipped optimizer step (host outputs; synchronises).
extern "C" int b200_model_last_grad_norm(b200_model *m, float *norm, float *factor) {
  if (!m) return B200_ERR_INVALID;
  B200_REQUIRE(m->ctx, norm && factor, "last_grad_norm: null pointer");
  float h[2] = {0.f, 1.f};
  TRY(b200_memcpy_d2h(m->ctx, h, m->clip_out, sizeof(h)));
  TRY(b200_sync(m->ctx));
  *norm = h[0]; *factor = h[1];
  return B200_OK;
}

extern "C" int b200_model_train_step(b200_model *m, const int32_t *tok, const int32_t *tgt, size_t B, size_t S,
                                     float lr, float beta1, float beta2, float eps, float wd, float *dev_loss) {
  if (!m) return B200_ERR_INVALID;
  // Optimizer in backward (opt-in, B200_FUSED_OPT=1): measured no faster on a power-capped B200 -- the GEMMs it runs
  // under lose what the hidden AdamW gains -- so the plain order is the default.  Every bucket offset keeps the
  // 16-byte alignment the AdamW kernel wants.
  // Data parallel: the optimizer is sharded over the ranks and runs bucket by bucket behind the gradient exchange.
  const char *env = getenv("B200_FUSED_OPT");
  const bool fuse = (((env && env[0] == '1') && m->grad_clip <= 0.f) || dp_shardable(m)) && m->with_opt && m->master && m->opt_stream && (m->V * m->H) % 4 == 0 && m->layer_train % 4 == 0;
  if (!fuse) {
    TRY(gather_sharded_state(m));
    TRY(b200_model_loss_and_grads(m, tok, tgt, B, S, dev_loss));
    return b200_model_adamw_step(m, lr, beta1, beta2, eps, wd);
  }
  m->step_count++;
  b200_adamw_params p;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = wd;
  p.bias_correction1 = 1.0f - powf(beta1, (float)m->step_count);   // cpp/src/Optimizer.cpp:141-142
  p.bias_correction2 = 1.0f - powf(beta2, (float)m->step_count);
  m->fused_opt = &p;
  const int rc = b200_model_loss_and_grads(m, tok, tgt, B, S, dev_loss);
  m->fused_opt = nullptr;
  return rc;
}

extern "C" int b200_model_train_step_host(b200_model *m, const int32_t *tok, const int32_t *tgt, size_t B, size_t S,
                                          float lr, float beta1, float beta2, float eps, float wd, float *host_loss) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(check_shape(m, B, S));
  B200_REQUIRE(ctx, tok && tgt && host_loss, "model_train_step_host: null pointer");
  const size_t M = B * S;
  memcpy(m->pin_tokens, tok, M * 4);
  memcpy(m->pin_targets, tgt, M * 4);
  TRY(b200_memcpy_h2d(ctx, m->d_tokens, m->pin_tokens, M * 4));
  TRY(b200_memcpy_h2d(ctx, m->d_targets, m->pin_targets, M * 4));
  TRY(b200_model_train_step(m, m->d_tokens, m->d_targets, B, S, lr, beta1, beta2, eps, wd, m->d_loss));
  TRY(b200_memcpy_d2h(ctx, m->pin_loss, m->d_loss, 4));
  TRY(b200_sync(ctx));
  *host_loss = *m->pin_loss;
  return B200_OK;
}

extern "C" int b200_model_layer_forward(b200_model *m, size_t l, const void *h_in, void *h_out, size_t B, size_t S) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(check_shape(m, B, S));
  B200_REQUIRE(ctx, l < m->L && h_in && h_out, "model_layer_forward: bad arguments");
  const size_t M = B * S, H = m->H;
  TRY(b200_copy(ctx, m->hs[l], h_in, M * H * dtype_size(m->dt)));
  TRY(b200_rms_norm_forward(ctx, m->hs[l], m->acts[l].a1, m->P(m->off_attn_norm(l)), nullptr, m->cfg.rms_norm_eps, M, H, m->dt));
  m->acts[l].a1_valid = true;
  TRY(layer_forward_core(m, l, m->hs[l], B, S));
  TRY(b200_copy(ctx, h_out, m->acts[l].h_mid, M * H * dtype_size(m->dt)));
  return b200_residual_add(ctx, h_out, m->tmpH, M * H, m->dt);
}
extern "C" int b200_model_layer_backward(b200_model *m, size_t l, const void *grad_out, void *grad_h_in, size_t B,
                                         size_t S) {
  if (!m) return B200_ERR_INVALID;
  TRY(check_shape(m, B, S));
  B200_REQUIRE(m->ctx, l < m->L && grad_out && grad_h_in, "model_layer_backward: bad arguments");
  return layer_backward_core(m, l, grad_out, grad_h_in, B, S);
}

// ---- data parallel ------------------------------------------------------------------------
extern "C" int b200_dp_unique_id(void *out128) {
  if (!out128 || !nccl::api().ok()) return B200_ERR_COMM;
  nccl::unique_id id;
  if (nccl::api().GetUniqueId(&id) != 0) return B200_ERR_COMM;
  memcpy(out128, &id, sizeof(id));
  return B200_OK;
}
extern "C" int b200_dp_init(b200_model *m, const void *id128, int rank, int world) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, id128 && world >= 1 && rank >= 0 && rank < world, "dp_init: bad arguments");
  if (!nccl::api().ok()) return b200_fail(ctx, B200_ERR_COMM, "NCCL library not found (libnccl.so.2)");
  nccl::unique_id id;
  memcpy(&id, id128, sizeof(id));
  int r = nccl::api().CommInitRank(&m->comm, world, id, rank);
  if (r != 0) return b200_fail(ctx, B200_ERR_COMM, "ncclCommInitRank failed: %s", nccl::api().GetErrorString ? nccl::api().GetErrorString(r) : "?");
  m->rank = rank; m->world = world;
  if (const char *e = getenv("B200_DP_MODE")) m->dp_sharded = !(e[0] == 'a');             // "allreduce" | "sharded"
  if (const char *e = getenv("B200_DP_GRAD_DTYPE")) m->dp_grad_bf16 = (e[0] == 'b');      // "bf16" | "fp32"
  if (m->dp_grad_bf16 && !m->grad_bf16) {
    const size_t biggest = m->V * m->H > m->layer_train ? m->V * m->H : m->layer_train;
    TRY(dalloc(m, &m->grad_bf16, biggest * 2));
  }
  B200_CUDA(ctx, cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking));
  B200_CUDA(ctx, cudaEventCreateWithFlags(&m->ev_grad_ready, cudaEventDisableTiming));
  B200_CUDA(ctx, cudaEventCreateWithFlags(&m->ev_comm_done, cudaEventDisableTiming));
  return B200_OK;
}
// Order-fixed fp64 sum and sum of squares of the fp32 master weights: replicas that hold the same weights report
// bit-identical numbers, so comparing two doubles per rank shows whether data-parallel replicas have drifted apart.
namespace {
__global__ void __launch_bounds__(256) checksum_partial_kernel(const float *__restrict__ v, size_t n, double *__restrict__ part) {
  __shared__ double s1[256], s2[256];
  double a = 0.0, b = 0.0;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) { const double x = v[i]; a += x; b += x * x; }
  s1[threadIdx.x] = a; s2[threadIdx.x] = b;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) { s1[threadIdx.x] += s1[threadIdx.x + o]; s2[threadIdx.x] += s2[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { part[2 * blockIdx.x] = s1[0]; part[2 * blockIdx.x + 1] = s2[0]; }
}
__global__ void checksum_final_kernel(const double *__restrict__ part, int blocks, double *__restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double a = 0.0, b = 0.0;
    for (int i = 0; i < blocks; ++i) { a += part[2 * i]; b += part[2 * i + 1]; }
    out[0] = a; out[1] = b;
  }
}
}  // namespace
extern "C" int b200_model_param_checksum(b200_model *m, double *sum, double *sum_sq) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, sum && sum_sq, "param_checksum: null pointer");
  TRY(gather_sharded_state(m));
  constexpr int BLOCKS = 1024;
  double *d = (double *)b200_scratch(ctx, (2 * BLOCKS + 2) * sizeof(double));
  if (!d) return B200_ERR_NOMEM;
  double host[2] = {0, 0};
  if (m->master) {
    checksum_partial_kernel<<<BLOCKS, 256, 0, ctx->stream>>>(m->master, m->n_total, d);
  } else {   // model without optimizer state in bf16: widen first
    float *tmp = nullptr;
    TRY(b200_malloc(ctx, m->n_total * 4, (void **)&tmp));
    int rc = b200_convert(ctx, m->params, m->dt, tmp, B200_F32, m->n_total);
    if (!rc) checksum_partial_kernel<<<BLOCKS, 256, 0, ctx->stream>>>(tmp, m->n_total, d);
    b200_free(ctx, tmp);
    if (rc) return rc;
  }
  B200_LAUNCHED(ctx);
  checksum_final_kernel<<<1, 32, 0, ctx->stream>>>(d, BLOCKS, d + 2 * BLOCKS);
  B200_LAUNCHED(ctx);
  TRY(b200_memcpy_d2h(ctx, host, d + 2 * BLOCKS, sizeof(host)));
  TRY(b200_sync(ctx));
  *sum = host[0]; *sum_sq = host[1];
  return B200_OK;
}

// Test hook (not part of the public header): the next gradient exchange reports NCCL result `nccl_result` without
// calling NCCL -- a host-side failure injection; no kernel or collective is disturbed.
extern "C" int b200_internal_dp_inject_failure(b200_model *m, int nccl_result) {
  if (!m) return B200_ERR_INVALID;
  m->inject_comm_error = nccl_result;
  return B200_OK;
}
extern "C" int b200_internal_dp_comm_failed(const b200_model *m) { return m && m->comm_failed ? 1 : 0; }

extern "C" int b200_dp_shutdown(b200_model *m) {
  if (!m || !m->comm) return B200_OK;
  if (!m->comm_failed) gather_sharded_state(m);      // leave every replica with complete masters and moments
  if (m->comm_failed && nccl::api().CommAbort) {
    // after an error the communicator may never complete what is queued on it: ncclCommDestroy would block on that work,
    // ncclCommAbort tears it down; only then is the side stream waited for
    nccl::api().CommAbort(m->comm);
    cudaStreamSynchronize(m->comm_stream);
  } else {
    cudaStreamSynchronize(m->comm_stream);
    nccl::api().CommDestroy(m->comm);
  }
  m->comm_failed = false;
  m->comm = nullptr; m->world = 1;
  cudaEventDestroy(m->ev_grad_ready); cudaEventDestroy(m->ev_comm_done);
  cudaStreamDestroy(m->comm_stream);
  return B200_OK;
}

// ---- autoregressive decode ------------------------------------------------------------------
int kv_append(b200_ctx *, const void *, void *, void *, size_t, size_t, size_t, size_t, size_t, size_t, size_t, b200_dtype);
size_t attn_decode_workspace_floats(size_t B, size_t nH, size_t hd);
int attn_decode(b200_ctx *ctx, const void *q, const void *k_new, const void *v_new, void *kc, void *vc, void *o, size_t B,
                size_t nH, size_t nKV, size_t hd, size_t S_max, size_t t_len, size_t ldq, size_t ldo, float *ws, int *tickets,
                b200_dtype dt, const int *pos_dev = nullptr);
int sample_launch(b200_ctx *ctx, const void *logits, b200_dtype dt, size_t batch, size_t vocab, int32_t *history,
                  size_t hist_len, size_t hist_ld, int append, const b200_sampler_config *cfg, uint64_t step,
                  int32_t *out_tokens, float *out_threshold, int32_t *out_kept, const int *pos_dev);
int advance_pos(b200_ctx *ctx, int *pos);
int gather_rows(b200_ctx *, const void *, void *, size_t, size_t, size_t, size_t, b200_dtype);

extern "C" int b200_model_decode_begin(b200_model *m, size_t batch, size_t max_total_len) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, batch > 0 && batch <= m->max_batch && max_total_len > 0 && max_total_len <= m->cfg.max_seq_len,
               "decode_begin: batch / length exceed what the model was created for");
  if (m->cache_batch >= batch && m->cache_len >= max_total_len) return B200_OK;
  if (!m->k_cache.empty()) {
    // a larger batch or a longer total length than the caches were made for: let the stream drain, drop the old
    // decode buffers and allocate again (their contents belong to a finished generation)
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    auto drop = [&](void *p) {
      if (!p) return;
      for (size_t i = 0; i < m->allocs.size(); ++i) if (m->allocs[i] == p) { m->allocs.erase(m->allocs.begin() + i); break; }
      cudaFree(p);
    };
    for (void *p : m->k_cache) drop(p);
    for (void *p : m->v_cache) drop(p);
    drop(m->dec_logits); drop(m->dec_h); drop(m->dec_history); drop(m->dec_next); drop(m->dec_attn_ws);
    drop(m->dec_attn_tickets); drop(m->dec_pos); drop(m->dec_stats);
    m->k_cache.clear(); m->v_cache.clear();
    m->dec_logits = m->dec_h = nullptr; m->dec_history = m->dec_next = nullptr; m->dec_attn_ws = nullptr;
    m->dec_attn_tickets = nullptr; m->dec_pos = nullptr; m->dec_stats = nullptr;
    batch = batch > m->cache_batch ? batch : m->cache_batch;
    max_total_len = max_total_len > m->cache_len ? max_total_len : m->cache_len;
    m->cache_batch = m->cache_len = 0;
  }
  const size_t es = dtype_size(m->dt), bytes = batch * max_total_len * m->KV * es;
  m->k_cache.assign(m->L, nullptr); m->v_cache.assign(m->L, nullptr);
  for (size_t l = 0; l < m->L; ++l) {
    TRY(dalloc(m, &m->k_cache[l], bytes)); TRY(dalloc(m, &m->v_cache[l], bytes));
    // positions not yet written are read by whole-tile loads and multiplied by a zero weight: they must be finite
    TRY(b200_fill_zero(ctx, m->k_cache[l], bytes)); TRY(b200_fill_zero(ctx, m->v_cache[l], bytes));
  }
  TRY(dalloc(m, &m->dec_logits, batch * m->V * es));
  TRY(dalloc(m, &m->dec_h, batch * m->H * es));
  TRY(dalloc(m, (void **)&m->dec_history, batch * max_total_len * sizeof(int32_t)));
  TRY(dalloc(m, (void **)&m->dec_next, batch * sizeof(int32_t)));
  TRY(dalloc(m, (void **)&m->dec_attn_ws, attn_decode_workspace_floats(batch, m->nH, m->hd) * sizeof(float)));
  TRY(dalloc(m, (void **)&m->dec_attn_tickets, batch * m->nH * sizeof(int)));
  TRY(b200_fill_zero(ctx, m->dec_attn_tickets, batch * m->nH * sizeof(int)));
  TRY(dalloc(m, (void **)&m->dec_pos, sizeof(int)));
  if (m->dt == B200_BF16) {
    TRY(dalloc(m, (void **)&m->dec_stats, 2 * m->L * batch * 2 * sizeof(unsigned long long)));
  }
  m->cache_batch = batch; m->cache_len = max_total_len;
  return B200_OK;
}

extern "C" int b200_model_prefill(b200_model *m, const int32_t *tok, size_t B, size_t P, void *logits_last) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  TRY(check_shape(m, B, P));
  B200_REQUIRE(ctx, tok && logits_last && B <= m->cache_batch && P <= m->cache_len, "prefill: call decode_begin first");
  TRY(forward_all(m, tok, B, P));
  for (size_t l = 0; l < m->L; ++l)
    TRY(kv_append(ctx, m->acts[l].qkv, m->k_cache[l], m->v_cache[l], B, P, 0, m->cache_len, m->Q, m->KV, m->QKV, m->dt));
  // logits of the last prompt position only
  TRY(gather_rows(ctx, m->fh, m->dec_h, B, P, m->H, P - 1, m->dt));
  return b200_gemm_ld(ctx, m->dec_h, m->P(m->off_out()), logits_last, B, m->V, m->H, 0, 0, 0, m->dt, m->dt, m->H, m->V, m->V);
}

// One decoder layer for one new token per sequence (rows = sequences); h in hs[l], result h_mid/tmpH as in the
// training forward so that the caller fuses the residual add with the next norm.
// pos_dev (optional): device int holding `pos`; the kernels then read the position on the device, which makes the
// enqueued step independent of the position (it can be captured once and replayed).  Needs the few-row GEMM path.
// True when a decode step of B sequences runs every projection on the few-row GEMM kernel with the normalisations and
// residual adds folded into it (bf16; B200_DECODE_FOLD_NORM=0 keeps the separate kernels).
static bool decode_folded(const b200_model *m, size_t B) {
  const char *env = getenv("B200_DECODE_FOLD_NORM");
  if (env && env[0] == '0') return false;
  if (m->dt != B200_BF16 || !m->ctx->gemm_skinny || !gemm_skinny_supported(B, 0, 0, 0) || m->L == 0) return false;
  if (m->H % 8 || m->I % 8 || m->hd % 2 || !m->dec_stats) return false;
  const b200_model::Act &a = m->acts[0];
  const size_t H = m->H, I = m->I;
  return gemm_tc_supported(a.a2, m->P(m->off_qkv(0)), a.qkv, B, m->QKV, H, H, m->QKV, m->QKV, m->dt) &&
         gemm_tc_supported(a.o, m->P(m->off_o(0)), a.h_mid, B, H, m->Q, m->Q, H, H, m->dt) &&
         gemm_tc_supported(a.h_mid, m->P(m->off_gate_up(0)), a.act, B, 2 * I, H, H, 2 * I, I, m->dt) &&
         gemm_tc_supported(a.act, m->P(m->off_down(0)), m->hs[1], B, H, I, I, H, H, m->dt) &&
         gemm_tc_supported(m->fh, m->P(m->off_out()), a.qkv, B, m->V, H, H, m->V, m->V, m->dt);
}

static int layer_decode_core(b200_model *m, size_t l, const void *h_in, size_t B, size_t pos, const int *pos_dev = nullptr,
                             bool fold = false) {
  b200_ctx *ctx = m->ctx;
  const size_t H = m->H, I = m->I;
  const float eps = m->cfg.rms_norm_eps;
  b200_model::Act &a = m->acts[l];
  const b200_dtype dt = m->dt;
  const size_t es = dtype_size(dt), half = m->hd / 2;
  const float *cos_p = m->cos_t + pos * half, *sin_p = m->sin_t + pos * half;    // every row is at position `pos`
  const bool rope_in_gemm = fold || (dt == B200_BF16 && m->hd % 32 == 0 && (pos * half * 4) % 16 == 0 &&
                            gemm_tc_supported(a.a2, m->P(m->off_qkv(l)), a.qkv, B, m->QKV, H, H, m->QKV, m->QKV, dt));
  B200_REQUIRE(ctx, !pos_dev || rope_in_gemm, "decode: device-side positions need the bf16 few-row GEMM path");
  if (rope_in_gemm) {
    GemmEpilogue epi;
    epi.cos_t = cos_p; epi.sin_t = sin_p; epi.S = 1; epi.hd = (int)m->hd; epi.cols = (int)(m->Q + m->KV);
    if (pos_dev) { epi.cos_t = m->cos_t; epi.sin_t = m->sin_t; epi.pos_dev = pos_dev; }
    // folded, layers after the first: a2 holds h * w_attn_norm and slot 2l-1 of dec_stats the row sums, both left by the
    // previous layer's down projection; the scale applies the layer norm and the attention's inner unit norm
    // (cpp/src/Transformer.cpp layer forward: attn_norm, then Attention's own input norm)
    if (fold && l > 0) { epi.row_acc = m->dec_stats + (2 * l - 1) * 2 * m->cache_batch; epi.norm_double = 1; epi.norm_eps = eps; }
    TRY(b200_gemm_ld(ctx, a.a2, m->P(m->off_qkv(l)), a.qkv, B, m->QKV, H, 0, 0, 0, dt, dt, H, m->QKV, m->QKV, &epi));
  } else {
    TRY(b200_gemm_ld(ctx, a.a2, m->P(m->off_qkv(l)), a.qkv, B, m->QKV, H, 0, 0, 0, dt, dt, H, m->QKV, m->QKV));
    TRY(rope_strided(ctx, a.qkv, cos_p, sin_p, B, m->nH + m->nKV, 1, m->hd, (long long)m->QKV, (long long)m->hd, (long long)m->QKV, dt, false));
  }
  // attention over the cache; the new token's K/V rows go from the projection output into the cache in the same kernel
  // when one CTA serves all query heads of a KV head (group sizes 1, 2, 4, 8), else in a copy kernel first
  const size_t Gq = m->nH / m->nKV;
  const bool fused_append = (Gq == 1 || Gq == 2 || Gq == 4 || Gq == 8) && !(m->hd == 256 && Gq > 4);
  B200_REQUIRE(ctx, !pos_dev || fused_append, "decode: device-side positions need the cache append fused into the attention kernel");
  if (!fused_append) TRY(kv_append(ctx, a.qkv, m->k_cache[l], m->v_cache[l], B, 1, pos, m->cache_len, m->Q, m->KV, m->QKV, dt));
  TRY(attn_decode(ctx, a.qkv, fused_append ? (const char *)a.qkv + m->Q * es : nullptr,
                  fused_append ? (const char *)a.qkv + (m->Q + m->KV) * es : nullptr, m->k_cache[l], m->v_cache[l],
                  a.o, B, m->nH, m->nKV, m->hd, m->cache_len, pos + 1, m->QKV, m->Q, m->dec_attn_ws, m->dec_attn_tickets, dt, pos_dev));
  if (fold) {
    const bool last = l + 1 == m->L;
    GemmEpilogue eo;                                // h_mid = h + o Wo;  ffn_in = h_mid * w_ffn_norm, row sums
    eo.residual = h_in; eo.ld_res = H;
    eo.next_norm_w = m->P(m->off_ffn_norm(l)); eo.xw_out = a.ffn_in; eo.ld_xw = H; eo.stat_acc = m->dec_stats + (2 * l) * 2 * m->cache_batch;
    TRY(b200_gemm_ld(ctx, a.o, m->P(m->off_o(l)), a.h_mid, B, H, m->Q, 0, 0, 0, dt, dt, m->Q, H, H, &eo));
    GemmEpilogue eg;                                // act = silu(g) * u of rstd * (ffn_in [Wg | Wu])
    eg.swiglu_I = (int)I; eg.row_acc = eo.stat_acc; eg.norm_eps = eps;
    TRY(b200_gemm_ld(ctx, a.ffn_in, m->P(m->off_gate_up(l)), a.act, B, 2 * I, H, 0, 0, 0, dt, dt, H, 2 * I, I, &eg));
    GemmEpilogue ed;                                // next stream = h_mid + act Wd;  the next norm's input and row sums
    ed.residual = a.h_mid; ed.ld_res = H;
    ed.next_norm_w = m->P(last ? m->off_final_norm() : m->off_attn_norm(l + 1));
    ed.xw_out = last ? m->fh : m->acts[l + 1].a2; ed.ld_xw = H; ed.stat_acc = m->dec_stats + (2 * l + 1) * 2 * m->cache_batch;
    return b200_gemm_ld(ctx, a.act, m->P(m->off_down(l)), m->hs[l + 1], B, H, I, 0, 0, 0, dt, dt, I, H, H, &ed);
  }
  TRY(b200_gemm_ld(ctx, a.o, m->P(m->off_o(l)), m->tmpH, B, H, m->Q, 0, 0, 0, dt, dt, m->Q, H, H));
  TRY(add_norm_oop(ctx, h_in, m->tmpH, a.h_mid, m->P(m->off_ffn_norm(l)), a.ffn_in, B, H, eps, dt));
  if (dt == B200_BF16 && ctx->gemm_skinny && gemm_skinny_supported(B, 0, 0, 0) && I % 8 == 0 &&
      gemm_tc_supported(a.ffn_in, m->P(m->off_gate_up(l)), a.act, B, 2 * I, H, H, 2 * I, I, dt)) {
    GemmEpilogue epi;                               // silu(gate) * up in the GEMM epilogue: no [B, 2I] intermediate
    epi.swiglu_I = (int)I;
    TRY(b200_gemm_ld(ctx, a.ffn_in, m->P(m->off_gate_up(l)), a.act, B, 2 * I, H, 0, 0, 0, dt, dt, H, 2 * I, I, &epi));
  } else {
    TRY(b200_gemm_ld(ctx, a.ffn_in, m->P(m->off_gate_up(l)), a.gate_up, B, 2 * I, H, 0, 0, 0, dt, dt, H, 2 * I, 2 * I));
    TRY(swiglu_fwd_strided(ctx, a.gate_up, (char *)a.gate_up + I * es, a.act, B, I, 2 * I, I, dt));
  }
  TRY(b200_gemm_ld(ctx, a.act, m->P(m->off_down(l)), m->tmpH, B, H, I, 0, 0, 0, dt, dt, I, H, H));
  return B200_OK;
}

static int decode_step_impl(b200_model *m, const int32_t *tok, size_t B, size_t pos, void *logits, const int *pos_dev);
// Every kernel of a decode step supports programmatic dependent launch (it waits before its first dependent access), so
// the step is enqueued with that launch attribute: each kernel's launch and set-up, and the weight prefetch of the
// few-row GEMMs, overlap the tail of the kernel before.  B200_DECODE_PDL=0 turns it off.
static int decode_step_core(b200_model *m, const int32_t *tok, size_t B, size_t pos, void *logits, const int *pos_dev) {
  b200_ctx *ctx = m->ctx;
  const char *env = getenv("B200_DECODE_PDL");
  const bool keep = ctx->pdl;
  ctx->pdl = !(env && env[0] == '0') && m->dt == B200_BF16 && ctx->gemm_skinny && gemm_skinny_supported(B, 0, 0, 0);
  const int rc = decode_step_impl(m, tok, B, pos, logits, pos_dev);
  ctx->pdl = keep;
  return rc;
}
static int decode_step_impl(b200_model *m, const int32_t *tok, size_t B, size_t pos, void *logits, const int *pos_dev) {
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, tok && logits && B > 0 && B <= m->cache_batch && pos < m->cache_len, "decode_step: bad arguments");
  const size_t H = m->H;
  const float eps = m->cfg.rms_norm_eps;
  const b200_dtype dt = m->dt;
  const bool folded = decode_folded(m, B);
  if (folded)      // the row-sum accumulators of the folded normalisations start every step at zero
    B200_CUDA(ctx, cudaMemsetAsync(m->dec_stats, 0, 2 * m->L * m->cache_batch * 2 * sizeof(unsigned long long), ctx->stream));
  {
    // The first kernel of a step is launched WITHOUT programmatic serialization, so it starts only when every kernel of
    // the previous step has completed: programmatic dependent launch orders a kernel against its immediate predecessor
    // only, and the attention kernels load cache tiles (written by the previous step) ahead of their own wait.
    const bool keep = ctx->pdl;
    ctx->pdl = false;
    const int rc = b200_embedding_forward(ctx, (const uint32_t *)tok, m->P(m->off_emb()), m->hs[0], B, H, m->V, dt);
    ctx->pdl = keep;
    TRY(rc);
  }
  if (folded) {
    // five launches per layer: after the first layer's input norm every normalisation and residual add rides in a projection
    TRY(add_norm_norm_oop(ctx, m->hs[0], nullptr, nullptr, m->P(m->off_attn_norm(0)), nullptr, m->ones, m->acts[0].a2, m->acts[0].a1, B, H, eps, dt));
    for (size_t l = 0; l < m->L; ++l) TRY(layer_decode_core(m, l, m->hs[l], B, pos, pos_dev, true));
    GemmEpilogue ev;
    ev.row_acc = m->dec_stats + (2 * m->L - 1) * 2 * m->cache_batch; ev.norm_eps = eps;
    return b200_gemm_ld(ctx, m->fh, m->P(m->off_out()), logits, B, m->V, H, 0, 0, 0, dt, dt, H, m->V, m->V, &ev);
  }
  if (m->L == 0) {
    TRY(b200_rms_norm_forward(ctx, m->hs[0], m->fh, m->P(m->off_final_norm()), nullptr, eps, B, H, dt));
  } else {
    TRY(add_norm_norm_oop(ctx, m->hs[0], nullptr, nullptr, m->P(m->off_attn_norm(0)), nullptr, m->ones, m->acts[0].a2, m->acts[0].a1, B, H, eps, dt));
    for (size_t l = 0; l < m->L; ++l) {
      TRY(layer_decode_core(m, l, m->hs[l], B, pos, pos_dev));
      if (l + 1 < m->L)
        TRY(add_norm_norm_oop(ctx, m->acts[l].h_mid, m->tmpH, m->hs[l + 1], m->P(m->off_attn_norm(l + 1)), nullptr, m->ones,
                              m->acts[l + 1].a2, m->acts[l + 1].a1, B, H, eps, dt));
      else
        TRY(add_norm_oop(ctx, m->acts[l].h_mid, m->tmpH, m->hs[l + 1], m->P(m->off_final_norm()), m->fh, B, H, eps, dt));
    }
  }
  return b200_gemm_ld(ctx, m->fh, m->P(m->off_out()), logits, B, m->V, H, 0, 0, 0, dt, dt, H, m->V, m->V);
}

extern "C" int b200_model_decode_step(b200_model *m, const int32_t *tok, size_t B, size_t pos, void *logits) {
  if (!m) return B200_ERR_INVALID;
  return decode_step_core(m, tok, B, pos, logits, nullptr);
}

extern "C" int b200_model_generate(b200_model *m, const int32_t *host_prompt, size_t B, size_t P, size_t new_tokens,
                                   const b200_sampler_config *cfg, int32_t *host_out, float *prefill_ms, float *decode_ms) {
  if (!m) return B200_ERR_INVALID;
  b200_ctx *ctx = m->ctx;
  B200_REQUIRE(ctx, host_prompt && cfg && host_out && new_tokens > 0, "generate: null pointer");
  TRY(b200_model_decode_begin(m, B, P + new_tokens));
  const size_t ld = m->cache_len;
  // history rows hold prompt then generated ids (the repetition penalty looks at both, sampler.py:130-137)
  B200_CUDA(ctx, cudaMemcpy2DAsync(m->dec_history, ld * 4, host_prompt, P * 4, P * 4, B, cudaMemcpyHostToDevice, ctx->stream));
  int32_t *d_prompt = nullptr;
  TRY(b200_malloc(ctx, B * P * 4, (void **)&d_prompt));
  int rc = b200_memcpy_h2d(ctx, d_prompt, host_prompt, B * P * 4);
  cudaEvent_t e0, e1, e2;
  cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
  cudaEventRecord(e0, ctx->stream);
  if (!rc) rc = b200_model_prefill(m, d_prompt, B, P, m->dec_logits);
  if (!rc) rc = b200_sample(ctx, m->dec_logits, m->dt, B, m->V, m->dec_history, P, ld, 1, cfg, P, m->dec_next, nullptr, nullptr);   // draw counter = history length
  cudaEventRecord(e1, ctx->stream);
  const auto host_t0 = std::chrono::steady_clock::now();
  // The per-token step is a chain of ~230 short kernels: enqueueing it costs more host time than it takes to run.
  // So the position lives in device memory, one step is captured into a CUDA graph and replayed for the rest.
  const char *genv = getenv("B200_DECODE_GRAPH");
  bool use_graph = !(genv && genv[0] == '0') && new_tokens > 3 && m->dt == B200_BF16 && ctx->gemm_skinny &&
                   gemm_skinny_supported(B, 0, 0, 0) && m->hd % 32 == 0 && m->H % 8 == 0 && m->QKV % 8 == 0 && m->L > 0;
  {
    const size_t Gq = m->nH / m->nKV;              // group sizes whose cache append is fused into the attention kernel
    use_graph = use_graph && (Gq == 1 || Gq == 2 || Gq == 4 || Gq == 8) && !(m->hd == 256 && Gq > 4);
  }
  cudaGraphExec_t exec = nullptr;
  bool capture_tried = false;
  if (use_graph && !rc) {
    const int p0 = (int)P;
    cudaError_t ce = cudaMemcpyAsync(m->dec_pos, &p0, sizeof(int), cudaMemcpyHostToDevice, ctx->stream);
    if (ce != cudaSuccess) rc = b200_fail(ctx, B200_ERR_CUDA, "generate: position upload failed: %s", cudaGetErrorString(ce));
  }
  const int *pos_dev = use_graph ? m->dec_pos : nullptr;
  for (size_t t = 1; t < new_tokens && !rc; ++t) {
    if (exec) {
      cudaError_t ce = cudaGraphLaunch(exec, ctx->stream);
      if (ce != cudaSuccess) rc = b200_fail(ctx, B200_ERR_CUDA, "generate: graph launch failed: %s", cudaGetErrorString(ce));
      else ctx->launches += m->dec_graph_nodes;
      continue;
    }
    // t == 1 runs eagerly (one-time attribute calls stay outside the capture); t == 2 is captured
    const bool capturing = use_graph && t == 2 && !capture_tried;
    const uint64_t launches_before = ctx->launches;
    if (capturing) {
      capture_tried = true;
      if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); --t; continue; }
    }
    rc = decode_step_core(m, m->dec_next, B, P + t - 1, m->dec_logits, pos_dev);
    const bool pdl_keep = ctx->pdl;
    ctx->pdl = pos_dev != nullptr && !(getenv("B200_DECODE_PDL") && getenv("B200_DECODE_PDL")[0] == '0');
    if (!rc) rc = sample_launch(ctx, m->dec_logits, m->dt, B, m->V, m->dec_history, P + t, ld, 1, cfg, P + t, m->dec_next, nullptr, nullptr, pos_dev);
    if (!rc && pos_dev) rc = advance_pos(ctx, m->dec_pos);
    ctx->pdl = pdl_keep;
    if (capturing) {
      cudaGraph_t graph = nullptr;
      const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
      if (!rc && ce == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
        m->dec_graph_nodes = ctx->launches - launches_before;
        ctx->launches = launches_before;
      } else {
        exec = nullptr;
        cudaGetLastError();
        ctx->launches = launches_before;
      }
      if (graph) cudaGraphDestroy(graph);
      if (!rc) --t;                                 // nothing ran while capturing: do step t again (replay, or eagerly)
    }
  }
  if (exec) cudaGraphExecDestroy(exec);
  cudaEventRecord(e2, ctx->stream);
  if (getenv("B200_DEBUG_TIMING"))
    fprintf(stderr, "[b200] decode loop enqueued in %.3f ms of host time\n",
            std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - host_t0).count());
  if (!rc) {
    cudaError_t ce = cudaMemcpy2DAsync(host_out, new_tokens * 4, m->dec_history + P, ld * 4, new_tokens * 4, B, cudaMemcpyDeviceToHost, ctx->stream);
    if (ce != cudaSuccess) rc = b200_fail(ctx, B200_ERR_CUDA, "copy of generated ids failed: %s", cudaGetErrorString(ce));
  }
  int rs = b200_sync(ctx);
  float ms = 0.f;
  if (prefill_ms) { cudaEventElapsedTime(&ms, e0, e1); *prefill_ms = ms; }
  if (decode_ms) { cudaEventElapsedTime(&ms, e1, e2); *decode_ms = ms; }
  cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
  b200_free(ctx, d_prompt);
  return rc ? rc : rs;
}
