// Shared declarations of the B200 backend: context, status handling, small
// device helpers.  Internal to csrc/; the public surface is include/b200_bridge.h.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/b200_bridge.h"

typedef __nv_bfloat16 bf16;

struct b200_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  uint64_t launches = 0;
  // device-side status word: kernels with bounded waits record a give-up here
  int *dev_status = nullptr;
  int *host_status = nullptr;  // pinned
  char err[512] = {0};
  // workspace for split reductions etc. (grown on demand, never shrunk)
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  // optional per-launch timing of the tensor-core GEMM (CUDA events on the launching stream)
  // 1: large bf16 GEMMs use the two-CTA (cta_group::2) kernel; 0: always the single-CTA kernel
  int gemm_2cta = 1;
  int gemm_skinny = 1;
  int attn_fwd2 = 1;       // 1: forward attention works on two query tiles per CTA with P and O in tensor memory
  int attn_decode_tc = 1;  // 1: decode attention on the tensor cores when one CTA per (sequence, KV head) fills the GPU
  int attn_bwd2 = 1;       // 1: backward attention (head_dim 128) in its transposed form, P and dS in tensor memory
  // decode step: kernels are launched with programmatic stream serialization, so a kernel's launch and set-up overlap the
  // tail of the one before it; each such kernel waits (griddepcontrol.wait) before it touches anything a predecessor wrote
  bool pdl = false;
  // Bit-reproducible gradients (B200_DETERMINISTIC=1; for chasing a divergence between runs or ranks): no split-K in the
  // GEMMs, attention backward writes dQ per key tile and adds the tiles in order, the embedding gradient is added token
  // by token.  The default paths add fp32 values with device atomics whose order varies from run to run.
  bool deterministic = false;
  bool time_gemm = false;
  struct Timed { cudaEvent_t start, stop; double flops; };
  std::vector<Timed> timed;
  std::vector<cudaEvent_t> event_pool;
  cudaEvent_t batch_t0 = nullptr, batch_t1 = nullptr;   // b200_batch_timer_begin / _end
  bool batch_timing = false;
  // launch trace (b200_internal_trace): one event after every kernel launch, attributed to its source line
  bool trace_on = false;
  struct Mark { cudaEvent_t ev; const char *file; int line; };
  std::vector<Mark> marks;
};

int b200_fail(b200_ctx *ctx, int code, const char *fmt, ...);
// Returns device scratch of at least `bytes` (reallocates if needed; synchronises first when it must grow).
void *b200_scratch(b200_ctx *ctx, size_t bytes);

#define B200_CUDA(ctx, call)                                                        \
  do {                                                                              \
    cudaError_t e_ = (call);                                                        \
    if (e_ != cudaSuccess)                                                          \
      return b200_fail((ctx), B200_ERR_CUDA, "%s failed: %s (%s:%d)", #call,        \
                       cudaGetErrorString(e_), __FILE__, __LINE__);                 \
  } while (0)

void b200_trace_mark(b200_ctx *ctx, const char *file, int line);
#define B200_LAUNCHED(ctx)                                                          \
  do {                                                                              \
    (ctx)->launches++;                                                              \
    if ((ctx)->trace_on) b200_trace_mark((ctx), __FILE__, __LINE__);                \
    cudaError_t e_ = cudaGetLastError();                                            \
    if (e_ != cudaSuccess)                                                          \
      return b200_fail((ctx), B200_ERR_CUDA, "kernel launch failed: %s (%s:%d)",    \
                       cudaGetErrorString(e_), __FILE__, __LINE__);                 \
  } while (0)

#define B200_REQUIRE(ctx, cond, msg)                                                \
  do {                                                                              \
    if (!(cond)) return b200_fail((ctx), B200_ERR_INVALID, "%s (%s)", msg, #cond);  \
  } while (0)

static inline size_t dtype_size(b200_dtype d) { return d == B200_BF16 ? 2 : 4; }

// ---- device helpers ------------------------------------------------------
// Programmatic dependent launch.  Both are no-ops in a kernel launched without the attribute.  pdl_wait() returns once
// every kernel this one depends on has completed and its writes are visible; nothing written by a predecessor may be
// read, and nothing a predecessor reads may be written, before it.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vector of T: 4 floats or 8 bf16.
template <class T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T *p) { raw = *reinterpret_cast<const uint4 *>(p); }
  __device__ __forceinline__ void store(T *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
  __device__ __forceinline__ void unpack(float *f) const {
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f(e[i]);
  }
  __device__ __forceinline__ void pack(const float *f) {
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f<T>(f[i]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is shared float[32]. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float *red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float *red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ---- internal launchers shared between translation units -------------------
int gemm_simt_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta,
                     int tb, int acc, b200_dtype in_dt, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc);
// Optional fused epilogue of the tensor-core GEMM (bf16 output): rotary position embedding applied to the
// fp32 accumulators of columns [0, cols) before rounding -- row r is token position r % S, column c is
// element c % hd of its head; interleaved pairs, tables [S, hd/2] (cpp/src/Positional.cpp:120-147).
struct GemmEpilogue {
  const float *cos_t = nullptr, *sin_t = nullptr;
  int S = 0, hd = 0, cols = 0;
  const int *pos_dev = nullptr;   // few-row kernel only: every row is at token position *pos_dev (decode; read on the device so that a captured step can be replayed)
  // W = [gate | up] (I columns each).  Few-row kernel: C[M, I] = silu(A*gate) * (A*up) and nothing else is written.
  // Two-CTA kernel (act_out set): C[M, 2I] = A*W as usual AND act_out[M, I] = silu(gate) * up computed from the fp32
  // accumulators (slightly more accurate than the separate SwiGLU kernel, which reads the bf16-rounded products back).
  // Few-row kernel only: an RMS normalisation split between the projection that PRODUCES a row h and the one that
  // CONSUMES norm(h), so that a decode step needs no normalisation kernel.
  //   producer: C = h = residual + A*W (residual: type of C, leading dimension ld_res).  With next_norm_w (N elements)
  //     it also writes xw_out = bf16(h * next_norm_w) (leading dimension ld_xw) and adds every row's sums of h^2 and
  //     xw^2 over its columns to stat_acc[row * 2 + {0, 1}] as 2^-32 fixed-point integers (integer atomics: the total
  //     does not depend on the order of the CTAs).  The caller zeroes stat_acc beforehand.
  //   consumer: A = xw.  With row_acc (the producer's stat_acc) the product is scaled by
  //     rstd = rsqrt(sum h^2 / K + norm_eps); norm_double applies the second, unit-weight norm of the normalised row as
  //     well (its statistic is rstd^2 * sum xw^2 / K).
  const void *residual = nullptr;
  size_t ld_res = 0;
  const void *next_norm_w = nullptr;
  void *xw_out = nullptr;
  size_t ld_xw = 0;
  unsigned long long *stat_acc = nullptr;
  const unsigned long long *row_acc = nullptr;
  int norm_double = 0;
  float norm_eps = 0.f;
  int swiglu_I = 0;
  void *act_out = nullptr;
  size_t ld_act = 0;
  // Cross-entropy over the columns of C = A*W (the vocabulary projection), two-CTA kernel only.  Row r has target
  // column ce_targets[r]; a "tile" is one 256-column block of C (gemm_tc2_ce_tiles(N) of them).
  //   ce_mode 1: C is NOT stored.  For every (row, tile) the epilogue writes max_j(x*log2e) to ce_part_max[tile*M + r]
  //              and sum_j exp2(x*log2e - max) to ce_part_sum[tile*M + r]; the tile that holds the target column also
  //              writes that logit to ce_tgt_logit[r].
  //   ce_mode 2: the same statistics, taken from the bf16-rounded values, and C is stored as usual.
  //   ce_mode 3: C = (exp(x - ce_lse[r]) - [column == target]) * ce_scale  (the gradient of the mean loss).
  int ce_mode = 0;
  const uint32_t *ce_targets = nullptr;
  float *ce_part_max = nullptr, *ce_part_sum = nullptr, *ce_tgt_logit = nullptr;
  const float *ce_lse = nullptr;
  float ce_scale = 0.f;
};
size_t gemm_tc2_ce_tiles(size_t N);   // number of column tiles the cross-entropy epilogue reports per row
int gemm_tc_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                   int acc, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi = nullptr);
int gemm_tc2_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                    int acc, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi = nullptr);
// true when b200_gemm_ld would run the two-CTA kernel with the fused SwiGLU output for this [M, 2I] forward GEMM
bool gemm_tc2_swiglu_eligible(const b200_ctx *ctx, size_t M, size_t I);
bool gemm_skinny_supported(size_t M, int ta, int tb, int acc);
int gemm_skinny_launch(b200_ctx *ctx, const void *A, const void *W, void *C, size_t M, size_t N, size_t K, b200_dtype out_dt,
                       size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi = nullptr);
bool gemm_tc_supported(const void *A, const void *B, const void *C, size_t M, size_t N, size_t K, size_t lda,
                       size_t ldb, size_t ldc, b200_dtype out_dt);
// Strided general form used by the engine (leading dimensions in elements).
int b200_gemm_ld(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                 int acc, b200_dtype in_dt, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc,
                 const GemmEpilogue *epi = nullptr);

// Attention on strided head layouts (element strides; head_dim contiguous).
struct AttnStrides {
  long long q_b, q_h, q_s;     // query  (batch, head, seq) strides
  long long k_b, k_h, k_s;     // key
  long long v_b, v_h, v_s;     // value
  long long o_b, o_h, o_s;     // output / dO
};
int attn_fwd_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                    size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt);
int attn_bwd_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                    const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                    size_t hd, const AttnStrides &st, const AttnStrides &gst, b200_dtype dt,
                    const float *rope_cos = nullptr, const float *rope_sin = nullptr);
// true when attn_bwd_launch can apply the inverse rotary embedding to dQ and dK itself (tensor-core path)
bool attn_bwd_fuses_rope(size_t B, size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st,
                         const AttnStrides &gst, b200_dtype dt, const void *Q, const void *K, const void *V,
                         const void *O, const void *dO, const void *dQ, const void *dK, const void *dV);

// Kernel launch on the context's stream; with ctx->pdl the launch carries the programmatic-stream-serialization
// attribute (the kernel must then call pdl_wait() before its first dependent access).  cluster_x > 1 adds a cluster.
template <class... KArgs, class... Args>
inline cudaError_t launch_k(b200_ctx *ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (cluster_x > 0) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = (unsigned)cluster_x; at[n].val.clusterDim.y = 1; at[n].val.clusterDim.z = 1; ++n;
  }
  if (ctx->pdl) { at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[n].val.programmaticStreamSerializationAllowed = 1; ++n; }
  cfg.attrs = at; cfg.numAttrs = (unsigned)n;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}
