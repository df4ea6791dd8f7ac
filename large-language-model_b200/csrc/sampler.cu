// On-device sampler for the decode loop.  Rules follow the reference's Python sampler
// (python/pipeline/inference/sampler.py:43-108): repetition penalty over the last 128 ids
// (v/p if v>0 else v*p, then -(p-1)*35, whitespace ids exempt), top-k (keep logits >= the k-th largest),
// top-p (softmax of the survivors in descending order, keep through the first index whose cumulative
// probability exceeds p, at least two tokens), then a categorical draw from logits/temperature, or the
// lowest-id argmax at temperature 0.
//
// One CTA of 1024 threads per sequence; the penalised logits of the row live in shared memory as fp32 when the
// vocabulary has at most 32768 entries, else in a per-row fp32 work array in global memory (L2-resident: the
// reference's own configurations use vocabularies of 100256 and 100352, cpp/include/TransformerConfig.hpp:92,107).
// Nothing is sorted: the k-th largest value and the top-p crossing value are found by repeated linear
// histograms (2048 bins) over a shrinking value range, walking the bins from the largest values down.
// Probability mass is accumulated as 2^-40 fixed point integers, so the result does not depend on the order
// in which threads add to a bin, and a given (logits, seed, step, row) always yields the same token.  A bin's
// mass is kept as three 14-bit-wide pieces in 32-bit counters (native shared-memory atomics; a piece cannot overflow
// below 2^17 keys) and as one 64-bit counter for larger vocabularies.  Every pass over the keys reads four at a time.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024, BINS = 2048, MAX_V = 32768, WINDOW = 128;
constexpr int PIECE_BITS = 14, PIECE_MAX_V = 1 << 17;   // 2^17 keys * 2^14 < 2^32

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct SamplerArgs {
  int V, hist_len, hist_ld, top_k, n_ws;
  float penalty, top_p, temperature;
  uint64_t seed, step;
  const int *pos_dev;      // when set: hist_len = step = *pos_dev + 1 (read on the device: replayable capture)
  float *gkeys;            // [batch, V] work array for vocabularies that do not fit in shared memory, else null
  int ws[8];
};

struct Scratch {
  uint32_t cnt[BINS];
  union {
    uint32_t piece[3][BINS];          // mass = piece[0] + (piece[1] << 14) + (piece[2] << 28)
    unsigned long long mass[BINS];    // vocabularies of 2^17 entries and more
  };
  unsigned long long total;
  unsigned long long wtot[32], ctot[32];
  float fred[64];
  int ired[32];
  int sel_bin, sel_above_c;
  unsigned long long sel_above_w;
  int pick;
};

__device__ __forceinline__ float block_max(float v, float *red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  return warp_max(r);
}
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long *red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long r = red[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}
// exclusive prefix over the 1024 threads (thread order) of a (64-bit, 32-bit) pair in one round
__device__ __forceinline__ void block_excl_scan2(unsigned long long v, uint32_t c, unsigned long long *red, unsigned long long *red_c,
                                                 unsigned long long &ex_v, uint32_t &ex_c) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v; uint32_t cin = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o); const uint32_t u = __shfl_up_sync(0xffffffffu, cin, o);
    if (lane >= o) { inc += t; cin += u; }
  }
  __syncthreads();
  if (lane == 31) { red[warp] = inc; red_c[warp] = cin; }
  __syncthreads();
  unsigned long long w = red[lane], winc = w; uint32_t wc = (uint32_t)red_c[lane], wcinc = wc;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, winc, o); const uint32_t u = __shfl_up_sync(0xffffffffu, wcinc, o);
    if (lane >= o) { winc += t; wcinc += u; }
  }
  ex_v = __shfl_sync(0xffffffffu, winc - w, warp) + inc - v;
  ex_c = __shfl_sync(0xffffffffu, wcinc - wc, warp) + cin - c;
}
// (max, min) over the block in one round; red holds 64 floats
__device__ __forceinline__ void block_max_min(float &mx, float &mn, float *red) {
  mx = warp_max(mx); mn = -warp_max(-mn);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = mx; red[32 + (threadIdx.x >> 5)] = mn; }
  __syncthreads();
  mx = warp_max(red[threadIdx.x & 31]); mn = -warp_max(-red[32 + (threadIdx.x & 31)]);
}

// Calls f(x, index) for every key, four keys per load when the array allows it.
template <class F>
__device__ __forceinline__ void for_keys(const float *keys, int V, F f) {
  const int tid = threadIdx.x;
  if (((uintptr_t)keys & 15) == 0) {
    const int V4 = V >> 2;
    for (int i = tid; i < V4; i += THREADS) {
      const float4 x = reinterpret_cast<const float4 *>(keys)[i];
      f(x.x, 4 * i); f(x.y, 4 * i + 1); f(x.z, 4 * i + 2); f(x.w, 4 * i + 3);
    }
    for (int i = (V4 << 2) + tid; i < V; i += THREADS) f(keys[i], i);
  } else {
    for (int i = tid; i < V; i += THREADS) f(keys[i], i);
  }
}

__device__ __forceinline__ unsigned long long qmass(float x, float mx) { return (unsigned long long)(__expf(x - mx) * 1099511627776.0f); }

// Walk the finite keys in [lo, mx] from the largest down, adding 1 per key (BY_COUNT) or its fixed-point softmax
// numerator; find the value v* at which the running total first exceeds the target: `target` itself when BY_COUNT,
// else frac * (total mass of the keys in range).  above_c is the count of the keys strictly greater than v*.
// `lo` must be the smallest key of the range.  Returns false when the total never exceeds the target.
// WIDE: 64-bit bin counters (any vocabulary size) instead of three 32-bit pieces.
template <bool BY_COUNT, bool WIDE>
__device__ bool select_desc(const float *keys, int V, float lo, float mx, unsigned long long target, double frac, float &vstar,
                            int &above_c, Scratch *s) {
  const int tid = threadIdx.x;
  float hi = mx;
  above_c = 0;
  unsigned long long above_w = 0;
  if (!(lo <= hi)) return false;                       // no finite key in range
  for (int iter = 0; iter < 8; ++iter) {
    const float scale = hi > lo ? (float)(BINS - 1) / (hi - lo) : 0.f;
    s->cnt[tid] = 0; s->cnt[tid + THREADS] = 0;
    if (!BY_COUNT) {
      if (WIDE) { s->mass[tid] = 0; s->mass[tid + THREADS] = 0; }
      else {
#pragma unroll
        for (int k = 0; k < 3; ++k) { s->piece[k][tid] = 0; s->piece[k][tid + THREADS] = 0; }
      }
    }
    if (tid == 0) s->sel_bin = -1;
    __syncthreads();
    for_keys(keys, V, [&](float x, int) {
      if (x >= lo && x <= hi) {
        const int bin = min(BINS - 1, (int)((hi - x) * scale));
        atomicAdd(&s->cnt[bin], 1u);
        if (!BY_COUNT) {
          const unsigned long long q = qmass(x, mx);
          if (WIDE) atomicAdd(&s->mass[bin], q);
          else {
            const uint32_t q0 = (uint32_t)q & ((1u << PIECE_BITS) - 1), q1 = (uint32_t)(q >> PIECE_BITS) & ((1u << PIECE_BITS) - 1),
                           q2 = (uint32_t)(q >> (2 * PIECE_BITS));
            if (q0) atomicAdd(&s->piece[0][bin], q0);
            if (q1) atomicAdd(&s->piece[1][bin], q1);
            if (q2) atomicAdd(&s->piece[2][bin], q2);
          }
        }
      }
    });
    __syncthreads();
    auto bin_mass = [&](int bin) -> unsigned long long {
      if (BY_COUNT) return s->cnt[bin];
      if (WIDE) return s->mass[bin];
      return (unsigned long long)s->piece[0][bin] + ((unsigned long long)s->piece[1][bin] << PIECE_BITS) +
             ((unsigned long long)s->piece[2][bin] << (2 * PIECE_BITS));
    };
    const uint32_t c0 = s->cnt[2 * tid], c1 = s->cnt[2 * tid + 1];
    const unsigned long long w0 = bin_mass(2 * tid), w1 = bin_mass(2 * tid + 1);
    unsigned long long ex_w; uint32_t ex_c;
    block_excl_scan2(w0 + w1, c0 + c1, s->wtot, s->ctot, ex_w, ex_c);
    if (!BY_COUNT && iter == 0) {
      // the first histogram holds every key of the range: its total is the softmax denominator
      if (tid == THREADS - 1) s->total = ex_w + w0 + w1;
      __syncthreads();
      target = (unsigned long long)(frac * (double)s->total);
    }
    const unsigned long long base = above_w + ex_w;
    if (base <= target && target < base + w0) { s->sel_bin = 2 * tid; s->sel_above_w = base; s->sel_above_c = above_c + (int)ex_c; }
    else if (base + w0 <= target && target < base + w0 + w1) { s->sel_bin = 2 * tid + 1; s->sel_above_w = base + w0; s->sel_above_c = above_c + (int)(ex_c + c0); }
    __syncthreads();
    const int sel = s->sel_bin;
    if (sel < 0) return false;
    above_w = s->sel_above_w; above_c = s->sel_above_c;
    float nlo = INFINITY, nhi = -INFINITY;
    for_keys(keys, V, [&](float x, int) {
      if (x >= lo && x <= hi && min(BINS - 1, (int)((hi - x) * scale)) == sel) { nlo = fminf(nlo, x); nhi = fmaxf(nhi, x); }
    });
    block_max_min(nhi, nlo, s->fred);
    hi = nhi; lo = nlo;
    if (hi == lo) break;
  }
  vstar = hi;
  return true;
}

template <class T>
__global__ void __launch_bounds__(THREADS)
sample_kernel(const T *__restrict__ logits, int32_t *history, int32_t *__restrict__ out_tokens,
              float *__restrict__ out_threshold, int32_t *__restrict__ out_kept, SamplerArgs a, int append) {
  pdl_launch_dependents();
  pdl_wait();
  if (a.pos_dev) { a.hist_len = *a.pos_dev + 1; a.step = (uint64_t)a.hist_len; }
  extern __shared__ __align__(16) float smem_keys[];
  float *keys = a.gkeys ? a.gkeys + (size_t)blockIdx.x * a.V : smem_keys;      // V penalised logits
  __shared__ Scratch sc;
  __shared__ int recent[WINDOW];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T *row = logits + (size_t)b * a.V;
  if (sizeof(T) == 2 && (((uintptr_t)row | (uintptr_t)keys) & 15) == 0) {       // eight bf16 logits per load
    const int V8 = a.V >> 3;
    for (int i = tid; i < V8; i += THREADS) {
      const uint4 x = reinterpret_cast<const uint4 *>(row)[i];
      const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&x.x)), f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&x.y)),
                   f2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&x.z)), f3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&x.w));
      reinterpret_cast<float4 *>(keys)[2 * i] = make_float4(f0.x, f0.y, f1.x, f1.y);
      reinterpret_cast<float4 *>(keys)[2 * i + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
    }
    for (int v = (V8 << 3) + tid; v < a.V; v += THREADS) keys[v] = to_f(row[v]);
  } else {
    for (int v = tid; v < a.V; v += THREADS) keys[v] = to_f(row[v]);
  }
  const int n_hist = a.penalty != 1.0f ? min(a.hist_len, WINDOW) : 0;
  if (tid < n_hist) recent[tid] = history[(size_t)b * a.hist_ld + a.hist_len - n_hist + tid];
  __syncthreads();
  if (tid < n_hist) {                              // each distinct, non-whitespace recent id is penalised once
    const int id = recent[tid];
    bool skip = id < 0 || id >= a.V;
    for (int w = 0; w < a.n_ws; ++w) skip |= (a.ws[w] == id);
    for (int j = 0; j < tid; ++j) skip |= (recent[j] == id);
    if (!skip) { const float x = keys[id]; keys[id] = (x > 0.f ? x / a.penalty : x * a.penalty) - (a.penalty - 1.0f) * 35.0f; }
  }
  __syncthreads();
  float mx = -INFINITY, mn = INFINITY;               // largest key, smallest finite key
  for_keys(keys, a.V, [&](float x, int) { mx = fmaxf(mx, x); if (x > -INFINITY) mn = fminf(mn, x); });
  block_max_min(mx, mn, sc.fred);

  float thr = -INFINITY;
  const bool want_filters = a.temperature > 0.f || out_threshold != nullptr || out_kept != nullptr;
  if (want_filters) {
    int above_c; float vstar;
    if (a.top_k > 0 && a.top_k < a.V) {
      if (select_desc<true, false>(keys, a.V, mn, mx, (unsigned long long)(a.top_k - 1), 0.0, vstar, above_c, &sc)) thr = vstar;
    }
    if (a.top_p < 1.0f) {
      // the range starts at the smallest kept key: the top-k threshold is itself a key
      const float lo = thr > -INFINITY ? thr : mn;
      const bool found = a.V < PIECE_MAX_V ? select_desc<false, false>(keys, a.V, lo, mx, 0ull, (double)a.top_p, vstar, above_c, &sc)
                                           : select_desc<false, true>(keys, a.V, lo, mx, 0ull, (double)a.top_p, vstar, above_c, &sc);
      if (found) {
        float cut = vstar;
        if (above_c == 0 && vstar == mx) {
          // the crossing happens at the largest value.  If one top token alone crosses p, the reference still keeps the
          // second entry of the sorted order; if several share the maximum, the second entry is one of them.
          int n_top = 0; float second_l = -INFINITY;
          for_keys(keys, a.V, [&](float x, int) { if (x == mx) ++n_top; else second_l = fmaxf(second_l, x); });
          const unsigned long long n_max = block_sum_u64((unsigned long long)n_top, sc.ctot);
          const float second = block_max(second_l, sc.fred);
          cut = n_max >= 2 ? mx : second;
        }
        thr = fmaxf(thr, cut);
      }
    }
  }
  // ---- kept set, then the draw in token-id order: warp w owns ids [w*per_w, (w+1)*per_w) ----------------
  const float invT = a.temperature > 0.f ? 1.0f / a.temperature : 0.f;
  const int per_w = ((a.V + 31) / 32 + 31) / 32 * 32, v_lo = warp * per_w, v_hi = min(a.V, v_lo + per_w);
  float wsum = 0.f; int cnt = 0; int last_kept = -1;
  for (int v = v_lo + lane; v < v_hi; v += 32) {
    const float x = keys[v];
    if (x >= thr) { ++cnt; wsum += __expf((x - mx) * invT); last_kept = v; }
  }
  const int kept = (int)block_sum_u64((unsigned long long)cnt, sc.ctot);
  if (tid == 0) { if (out_threshold) out_threshold[b] = thr; if (out_kept) out_kept[b] = kept; sc.pick = a.V; }
  if (a.temperature > 0.f) {
    const float wt = warp_sum(wsum);
    last_kept = __reduce_max_sync(0xffffffffu, last_kept);
    __syncthreads();
    if (lane == 0) { sc.fred[warp] = wt; sc.ired[warp] = last_kept; }
    __syncthreads();
    // every warp scans the 32 warp totals (same arithmetic everywhere)
    const float my = sc.fred[lane];
    float inc = my;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
    const float W = __shfl_sync(0xffffffffu, inc, 31);
    const uint64_t bits = mix64(a.seed ^ mix64(a.step * 0x10001ull + (uint64_t)b));
    const float u = ((float)(bits >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float target = u * W;
    const unsigned hit = __ballot_sync(0xffffffffu, my > 0.f && inc >= target);
    const unsigned any = __ballot_sync(0xffffffffu, my > 0.f);
    const int sel_warp = hit ? __ffs(hit) - 1 : 31 - __clz(any);     // rounding: fall back to the last warp with weight
    if (warp == sel_warp) {
      float run = __shfl_sync(0xffffffffu, inc - my, sel_warp);
      int found = -1;
      for (int v0 = v_lo; v0 < v_hi && found < 0; v0 += 32) {
        const int v = v0 + lane;
        const float x = v < v_hi ? keys[v] : -INFINITY;
        const float w = (v < v_hi && x >= thr) ? __expf((x - mx) * invT) : 0.f;
        float winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, winc, o); if (lane >= o) winc += t; }
        const unsigned h = __ballot_sync(0xffffffffu, w > 0.f && run + winc >= target);
        if (h) found = v0 + __ffs(h) - 1;
        run += __shfl_sync(0xffffffffu, winc, 31);
      }
      if (found < 0) found = sc.ired[sel_warp];
      if (lane == 0) sc.pick = found;
    }
  } else {
    // greedy: lowest id among the maxima
    int best = 0x7fffffff;
    for (int v = v_lo + lane; v < v_hi; v += 32) if (keys[v] == mx) { best = v; break; }
    best = __reduce_min_sync(0xffffffffu, best);
    __syncthreads();
    if (lane == 0 && best != 0x7fffffff) atomicMin(&sc.pick, best);
  }
  __syncthreads();
  if (tid == 0) {
    out_tokens[b] = sc.pick;
    if (append) history[(size_t)b * a.hist_ld + a.hist_len] = sc.pick;     // the entry just past the ones read above
  }
}

__global__ void advance_pos_kernel(int *pos) {
  pdl_launch_dependents();
  pdl_wait();
  *pos += 1;
}
}  // namespace

int advance_pos(b200_ctx *ctx, int *pos) {
  B200_CUDA(ctx, launch_k(ctx, advance_pos_kernel, dim3(1), dim3(1), 0, 0, pos));
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// pos_dev (optional): device int; the kernel then takes hist_len = step = *pos_dev + 1.
int sample_launch(b200_ctx *ctx, const void *logits, b200_dtype dt, size_t batch, size_t vocab, int32_t *history,
                  size_t hist_len, size_t hist_ld, int append, const b200_sampler_config *cfg, uint64_t step,
                  int32_t *out_tokens, float *out_threshold, int32_t *out_kept, const int *pos_dev) {
  B200_REQUIRE(ctx, logits && cfg && out_tokens && batch > 0, "sample: null pointer");
  B200_REQUIRE(ctx, vocab >= 2 && vocab <= (size_t)0x7fffff00, "sample: vocabulary must have at least 2 entries");
  B200_REQUIRE(ctx, cfg->n_whitespace_ids >= 0 && cfg->n_whitespace_ids <= 8 && (history || (hist_len == 0 && !append)) && (!append || hist_len < hist_ld),
               "sample: bad configuration");
  B200_REQUIRE(ctx, cfg->repetition_penalty > 0.f && cfg->temperature >= 0.f, "sample: penalty must be > 0 and temperature >= 0");
  SamplerArgs a;
  a.V = (int)vocab; a.hist_len = (int)hist_len; a.hist_ld = (int)hist_ld; a.top_k = cfg->top_k;
  a.n_ws = cfg->n_whitespace_ids; a.penalty = cfg->repetition_penalty; a.top_p = cfg->top_p; a.temperature = cfg->temperature;
  a.seed = cfg->seed; a.step = step; a.pos_dev = pos_dev; a.gkeys = nullptr;
  for (int i = 0; i < 8; ++i) a.ws[i] = i < a.n_ws ? cfg->whitespace_ids[i] : -1;
  static bool attr[2] = {false, false};
  size_t smem = (size_t)MAX_V * sizeof(float);
  if (vocab > (size_t)MAX_V) {
    // the context workspace only grows; a generation loop makes its first call (which may allocate) before it captures a step
    a.gkeys = (float *)b200_scratch(ctx, batch * vocab * sizeof(float));
    if (!a.gkeys) return B200_ERR_NOMEM;
    smem = 0;
  }
  if (dt == B200_BF16) {
    if (!attr[1]) { B200_CUDA(ctx, cudaFuncSetAttribute(sample_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[1] = true; }
    B200_CUDA(ctx, launch_k(ctx, sample_kernel<bf16>, dim3((unsigned)batch), dim3(THREADS), smem, 0, (const bf16 *)logits, history, out_tokens, out_threshold, out_kept, a, append));
  } else {
    if (!attr[0]) { B200_CUDA(ctx, cudaFuncSetAttribute(sample_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[0] = true; }
    B200_CUDA(ctx, launch_k(ctx, sample_kernel<float>, dim3((unsigned)batch), dim3(THREADS), smem, 0, (const float *)logits, history, out_tokens, out_threshold, out_kept, a, append));
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}

extern "C" int b200_sample(b200_ctx *ctx, const void *logits, b200_dtype dt, size_t batch, size_t vocab,
                           int32_t *history, size_t hist_len, size_t hist_ld, int append, const b200_sampler_config *cfg,
                           uint64_t step, int32_t *out_tokens, float *out_threshold, int32_t *out_kept) {
  return sample_launch(ctx, logits, dt, batch, vocab, history, hist_len, hist_ld, append, cfg, step, out_tokens, out_threshold,
                       out_kept, nullptr);
}
