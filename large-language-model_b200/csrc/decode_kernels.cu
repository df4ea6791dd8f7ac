// Kernels of the autoregressive decode path: KV-cache append, single-query GQA attention over the
// cache, last-token gather, and the sampler.  The reference C++ engine declares a KVCache
// (cpp/include/TransformerConfig.hpp:121-124) but never reads or writes it and has no generation
// loop; the sampling rules follow the reference's Python sampler
// (python/pipeline/inference/sampler.py:43-108): repetition penalty over the last 128 ids
// (v/p if v>0 else v*p, then -(p-1)*35, whitespace ids exempt), top-k (keep logits >= k-th largest),
// top-p (sorted softmax, keep through the first index whose cumulative probability exceeds p, at
// least two tokens), then a categorical draw from logits/temperature, or argmax at temperature 0.
// All of it is HBM / latency bound small-batch work on CUDA cores.
#include "common.cuh"

namespace {

// ---- cache append: rows of the fused [M, Q+2KV] projection -> K/V caches [B, S_max, KV] ----------
template <class T>
__global__ void kv_append_kernel(const T *__restrict__ qkv, T *__restrict__ kc, T *__restrict__ vc, int B, int T_new,
                                 int pos0, int S_max, int Q, int KV, int ld) {
  constexpr int N = 16 / sizeof(T);
  const int units = KV / N;                                // 16-byte units per K (or V) row
  const size_t n = (size_t)B * T_new * units * 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(i % units); size_t r = i / units;
    const int which = (int)(r & 1); r >>= 1;
    const int t = (int)(r % T_new), b = (int)(r / T_new);
    const T *src = qkv + ((size_t)b * T_new + t) * ld + Q + which * KV + u * N;
    T *dst = (which ? vc : kc) + ((size_t)b * S_max + pos0 + t) * KV + u * N;
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
  }
}

// ---- single-query attention over the cache: one CTA (4 warps) per (batch, head) -----------------
// q [B, Q] (row stride ldq), caches [B, S_max, KV]; keys 0..t_len-1.  Each warp takes keys
// w, w+4, ... in chunks of 32 (lane = key) with an online softmax; the four partial results are merged.
template <class T>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const T *__restrict__ q, const T *__restrict__ kc, const T *__restrict__ vc, T *__restrict__ o,
                   int nH, int nKV, int hd, int S_max, int t_len, int ldq, int ldo, float scale) {
  extern __shared__ float sm[];
  float *qs = sm;                           // hd
  float *part_o = sm + hd;                  // 4 * hd
  float *part_m = part_o + 4 * hd, *part_l = part_m + 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x % nH, b = blockIdx.x / nH, kvh = h / (nH / nKV), KV = nKV * hd;
  const T *qrow = q + (size_t)b * ldq + h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f(qrow[d]);
  __syncthreads();
  const T *kb = kc + (size_t)b * S_max * KV + kvh * hd, *vb = vc + (size_t)b * S_max * KV + kvh * hd;
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int j0 = warp * 32; j0 < t_len; j0 += 128) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < t_len) {
      const T *kr = kb + (size_t)j * KV;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot += qs[d] * to_f(kr[d]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (j < t_len) ? __expf(s - m_new) : 0.f, corr = __expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= corr;
    const int nj = min(32, t_len - j0);
    for (int jj = 0; jj < nj; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T *vr = vb + (size_t)(j0 + jj) * KV;
#pragma unroll
      for (int i = 0; i < 8; ++i) { const int d = lane + 32 * i; if (d < hd) acc[i] += pj * to_f(vr[d]); }
    }
    m = m_new;
  }
  if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < 8; ++i) { const int d = lane + 32 * i; if (d < hd) part_o[warp * hd + d] = acc[i]; }
  __syncthreads();
  const float M = fmaxf(fmaxf(part_m[0], part_m[1]), fmaxf(part_m[2], part_m[3]));
  float L = 0.f;
  for (int w = 0; w < 4; ++w) L += part_l[w] * __expf(part_m[w] - M);
  T *orow = o + (size_t)b * ldo + h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < 4; ++w) v += part_o[w * hd + d] * __expf(part_m[w] - M);
    orow[d] = from_f<T>(v / L);
  }
}

template <class T>
__global__ void gather_rows_kernel(const T *__restrict__ src, T *__restrict__ dst, int B, int S, int H, int pos) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)B * H; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % H), b = (int)(i / H);
    dst[i] = src[((size_t)b * S + pos) * H + c];
  }
}

// ---- sampler: one CTA of 1024 threads per sequence ------------------------------------------------
constexpr int SORT_N = 32768;          // vocabulary padded to a power of two (fp32 keys in 128 KiB of shared memory)

__device__ __forceinline__ float block_reduce_sum(float v, float *red) { return block_sum(v, red); }
__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct SamplerArgs {
  int V, window, hist_len, hist_ld, top_k, n_ws;
  float penalty, top_p, temperature;
  uint64_t seed, step;
  int ws[8];
};

// logits after the repetition penalty (token ids of the last `window` history entries, whitespace exempt)
template <class T>
__device__ __forceinline__ float penalised(const T *row, int v, const int *recent, int n_recent, float penalty) {
  float x = to_f(row[v]);
  if (penalty != 1.0f) {
    bool seen = false;
    for (int i = 0; i < n_recent; ++i) seen |= (recent[i] == v);
    if (seen) x = (x > 0.f ? x / penalty : x * penalty) - (penalty - 1.0f) * 35.0f;
  }
  return x;
}

template <class T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T *__restrict__ logits, int32_t *history, int32_t *__restrict__ out_tokens,
              float *__restrict__ out_threshold, int32_t *__restrict__ out_kept, SamplerArgs a, int append) {
  extern __shared__ float keys[];                  // SORT_N
  __shared__ float red[32];
  __shared__ int recent[128];
  __shared__ int n_recent_s, cutoff_s;
  __shared__ float scan_s[1024];
  const int b = blockIdx.x, tid = threadIdx.x;
  const T *row = logits + (size_t)b * a.V;
  // the distinct non-whitespace ids among the last `window` history entries
  if (tid == 0) {
    int n = 0;
    const int start = a.hist_len > a.window ? a.hist_len - a.window : 0;
    for (int i = start; i < a.hist_len; ++i) {
      const int id = history[(size_t)b * a.hist_ld + i];
      bool skip = false;
      for (int w = 0; w < a.n_ws; ++w) skip |= (a.ws[w] == id);
      for (int j = 0; j < n; ++j) skip |= (recent[j] == id);
      if (!skip && id >= 0 && id < a.V) recent[n++] = id;
    }
    n_recent_s = (a.penalty != 1.0f) ? n : 0;
    cutoff_s = 0x7fffffff;
  }
  __syncthreads();
  const int n_recent = n_recent_s;
  for (int v = tid; v < SORT_N; v += 1024) keys[v] = v < a.V ? penalised(row, v, recent, n_recent, a.penalty) : -INFINITY;
  __syncthreads();
  // bitonic sort, descending
  for (int k = 2; k <= SORT_N; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < SORT_N; i += 1024) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const float x = keys[i], y = keys[ixj];
          const bool desc = (i & k) == 0;
          if (desc ? (x < y) : (x > y)) { keys[i] = y; keys[ixj] = x; }
        }
      }
      __syncthreads();
    }
  }
  const float mx = keys[0];
  float thr = -INFINITY;
  int n_keep = a.V;
  if (a.top_k > 0 && a.top_k < a.V) {
    thr = keys[a.top_k - 1];
    // survivors of top-k: all entries >= thr (ties included)
    int cnt = 0;
    for (int i = tid; i < a.V; i += 1024) cnt += keys[i] >= thr ? 1 : 0;
    n_keep = (int)(block_reduce_sum((float)cnt, red) + 0.5f);
  }
  if (a.top_p < 1.0f) {
    // softmax over the survivors in sorted order; each thread owns a contiguous run of 32 sorted entries
    float local = 0.f;
    const int i0 = tid * 32;
    for (int i = i0; i < i0 + 32; ++i) if (i < n_keep) local += __expf(keys[i] - mx);
    const float Z = block_reduce_sum(local, red);
    scan_s[tid] = local;
    __syncthreads();
    if (tid == 0) {                                  // 1024-entry exclusive scan, then locate the crossing run
      float run = 0.f;
      for (int t = 0; t < 1024; ++t) { const float x = scan_s[t]; scan_s[t] = run; run += x; }
    }
    __syncthreads();
    float cum = scan_s[tid];
    int first = -1;
    for (int i = i0; i < i0 + 32; ++i) {
      if (i < n_keep) { cum += __expf(keys[i] - mx); if (first < 0 && cum / Z > a.top_p) first = i; }
    }
    if (first >= 0) atomicMin(&cutoff_s, first);
    __syncthreads();
    if (cutoff_s != 0x7fffffff) {                    // no crossing (rounding): the reference then filters nothing
      int cutoff = cutoff_s < 1 ? 1 : cutoff_s;
      if (cutoff > a.V - 1) cutoff = a.V - 1;
      thr = fmaxf(thr, keys[cutoff]);
    }
  }
  __syncthreads();
  // kept set and the draw, in token-id order
  int cnt = 0;
  float wsum = 0.f;
  const float invT = a.temperature > 0.f ? 1.0f / a.temperature : 0.f;
  const int per = (a.V + 1023) / 1024, v0 = tid * per;
  for (int v = v0; v < v0 + per && v < a.V; ++v) {
    const float x = penalised(row, v, recent, n_recent, a.penalty);
    if (x >= thr) { ++cnt; wsum += __expf((x - mx) * invT); }
  }
  const int kept = (int)(block_reduce_sum((float)cnt, red) + 0.5f);
  if (tid == 0) { if (out_threshold) out_threshold[b] = thr; if (out_kept) out_kept[b] = kept; }
  __shared__ int pick;
  if (tid == 0) pick = a.V;
  __syncthreads();
  if (a.temperature > 0.f) {
    const float W = block_reduce_sum(wsum, red);
    scan_s[tid] = wsum;
    __syncthreads();
    if (tid == 0) { float run = 0.f; for (int t = 0; t < 1024; ++t) { const float x = scan_s[t]; scan_s[t] = run; run += x; } }
    __syncthreads();
    const uint64_t bits = mix64(a.seed ^ mix64(a.step * 0x10001ull + (uint64_t)b));
    const float u = ((float)(bits >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float target = u * W;
    float cum = scan_s[tid];
    for (int v = v0; v < v0 + per && v < a.V; ++v) {
      const float x = penalised(row, v, recent, n_recent, a.penalty);
      if (x >= thr) { cum += __expf((x - mx) * invT); if (cum >= target) { atomicMin(&pick, v); break; } }
    }
    __syncthreads();
    if (tid == 0 && pick == a.V) {                   // rounding left the target just above the total: take the last kept id
      for (int v = a.V - 1; v >= 0; --v) if (penalised(row, v, recent, n_recent, a.penalty) >= thr) { pick = v; break; }
    }
  } else {
    // greedy: lowest id among the maxima
    for (int v = v0; v < v0 + per && v < a.V; ++v)
      if (penalised(row, v, recent, n_recent, a.penalty) == mx) { atomicMin(&pick, v); break; }
  }
  __syncthreads();
  if (tid == 0) {
    out_tokens[b] = pick;
    if (append) history[(size_t)b * a.hist_ld + a.hist_len] = pick;     // the entry just past the ones read above
  }
}
}  // namespace

int kv_append(b200_ctx *ctx, const void *qkv, void *kc, void *vc, size_t B, size_t T_new, size_t pos0, size_t S_max,
              size_t Q, size_t KV, size_t ld, b200_dtype dt) {
  const size_t N = 16 / dtype_size(dt);
  B200_REQUIRE(ctx, KV % N == 0 && Q % N == 0 && ld % N == 0, "kv_append: widths must be multiples of 16 bytes");
  const size_t n = B * T_new * (KV / N) * 2;
  if (!n) return B200_OK;
  const int grid = (int)((n + 255) / 256 < (size_t)ctx->sm_count * 16 ? (n + 255) / 256 : (size_t)ctx->sm_count * 16);
  if (dt == B200_BF16) kv_append_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)qkv, (bf16 *)kc, (bf16 *)vc, (int)B, (int)T_new, (int)pos0, (int)S_max, (int)Q, (int)KV, (int)ld);
  else kv_append_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)qkv, (float *)kc, (float *)vc, (int)B, (int)T_new, (int)pos0, (int)S_max, (int)Q, (int)KV, (int)ld);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

int attn_decode(b200_ctx *ctx, const void *q, const void *kc, const void *vc, void *o, size_t B, size_t nH, size_t nKV,
                size_t hd, size_t S_max, size_t t_len, size_t ldq, size_t ldo, b200_dtype dt) {
  B200_REQUIRE(ctx, hd <= 256 && t_len >= 1 && t_len <= S_max, "attn_decode: bad shape");
  const size_t smem = (5 * hd + 8) * sizeof(float);
  const float scale = 1.0f / sqrtf((float)hd);
  if (dt == B200_BF16) attn_decode_kernel<bf16><<<(unsigned)(B * nH), 128, smem, ctx->stream>>>((const bf16 *)q, (const bf16 *)kc, (const bf16 *)vc, (bf16 *)o, (int)nH, (int)nKV, (int)hd, (int)S_max, (int)t_len, (int)ldq, (int)ldo, scale);
  else attn_decode_kernel<float><<<(unsigned)(B * nH), 128, smem, ctx->stream>>>((const float *)q, (const float *)kc, (const float *)vc, (float *)o, (int)nH, (int)nKV, (int)hd, (int)S_max, (int)t_len, (int)ldq, (int)ldo, scale);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

int gather_rows(b200_ctx *ctx, const void *src, void *dst, size_t B, size_t S, size_t H, size_t pos, b200_dtype dt) {
  const size_t n = B * H;
  const int grid = (int)((n + 255) / 256);
  if (dt == B200_BF16) gather_rows_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, (int)B, (int)S, (int)H, (int)pos);
  else gather_rows_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, (int)B, (int)S, (int)H, (int)pos);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

extern "C" int b200_sample(b200_ctx *ctx, const void *logits, b200_dtype dt, size_t batch, size_t vocab,
                           int32_t *history, size_t hist_len, size_t hist_ld, int append, const b200_sampler_config *cfg,
                           uint64_t step, int32_t *out_tokens, float *out_threshold, int32_t *out_kept) {
  B200_REQUIRE(ctx, logits && cfg && out_tokens && batch > 0, "sample: null pointer");
  B200_REQUIRE(ctx, vocab >= 2 && vocab <= (size_t)SORT_N, "sample: vocabulary must be in [2, 32768]");
  B200_REQUIRE(ctx, cfg->n_whitespace_ids >= 0 && cfg->n_whitespace_ids <= 8 && (history || (hist_len == 0 && !append)) && (!append || hist_len < hist_ld),
               "sample: bad configuration");
  SamplerArgs a;
  a.V = (int)vocab; a.window = 128; a.hist_len = (int)hist_len; a.hist_ld = (int)hist_ld; a.top_k = cfg->top_k;
  a.n_ws = cfg->n_whitespace_ids; a.penalty = cfg->repetition_penalty; a.top_p = cfg->top_p; a.temperature = cfg->temperature;
  a.seed = cfg->seed; a.step = step;
  for (int i = 0; i < 8; ++i) a.ws[i] = i < a.n_ws ? cfg->whitespace_ids[i] : -1;
  static bool attr[2] = {false, false};
  const size_t smem = SORT_N * sizeof(float);
  if (dt == B200_BF16) {
    if (!attr[1]) { B200_CUDA(ctx, cudaFuncSetAttribute(sample_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[1] = true; }
    sample_kernel<bf16><<<(unsigned)batch, 1024, smem, ctx->stream>>>((const bf16 *)logits, history, out_tokens, out_threshold, out_kept, a, append);
  } else {
    if (!attr[0]) { B200_CUDA(ctx, cudaFuncSetAttribute(sample_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[0] = true; }
    sample_kernel<float><<<(unsigned)batch, 1024, smem, ctx->stream>>>((const float *)logits, history, out_tokens, out_threshold, out_kept, a, append);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}
