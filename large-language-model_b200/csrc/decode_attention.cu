// Single-query GQA attention over the KV cache (decode: one new token per sequence).
// The reference engine declares a KVCache (cpp/include/TransformerConfig.hpp:121-124) but never uses it;
// the maths is the causal GQA attention of cpp/src/Attention.cpp:236-280 for the last query position.
//
// HBM/L2-bound: every K and V row of the cache is read once per KV head.  Work split:
//   grid = (key splits, query-head groups, sequences); a CTA of 8 warps takes one contiguous run of
//   keys for GQ query heads that share a KV head (GQ = nH/nKV when that is 1, 2, 4 or 8, so the K/V
//   rows are read once for the whole group); a warp takes one key at a time, the lanes split the head
//   dimension (coalesced row reads), scores are reduced with shuffles and folded into an online softmax.
//   Warps merge through shared memory, splits merge through a small fp32 workspace: the CTA that
//   arrives last at a per-(sequence, group) ticket does the final merge (no waiting anywhere).
// The new token's K/V row is taken from the projection output and appended to the cache here (when the query heads of a
// KV head share a CTA; otherwise the caller appends it first).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

// One lane's EPL consecutive elements of a row: raw load (so that several rows can be in flight before any
// conversion), unpack to fp32, raw store.
template <int BYTES> struct RawVec;
template <> struct RawVec<2> { typedef unsigned short type; };
template <> struct RawVec<4> { typedef uint32_t type; };
template <> struct RawVec<8> { typedef uint2 type; };
template <> struct RawVec<16> { typedef uint4 type; };
template <> struct RawVec<32> { struct type { uint4 a, b; }; };
template <class T, int EPL> struct RowLoad {
  typedef typename RawVec<sizeof(T) * EPL>::type Raw;
  static __device__ __forceinline__ Raw ldg(const T *p) { return *reinterpret_cast<const Raw *>(p); }
  static __device__ __forceinline__ void stg(T *p, const Raw &r) { *reinterpret_cast<Raw *>(p) = r; }
  static __device__ __forceinline__ void unpack(const Raw &r, float *f) {
    const T *e = reinterpret_cast<const T *>(&r);
#pragma unroll
    for (int i = 0; i < EPL; ++i) f[i] = to_f(e[i]);
  }
};

// Sums each of NV per-lane values over the 32 lanes and leaves every total in every lane.  Instead of NV butterflies
// (5 NV shuffles) the values are folded: at each step a lane keeps half of its values and hands the other half to its
// partner, so the totals end up spread over the lanes (NV - 1 + a few shuffles), then each is broadcast (NV shuffles).
template <int NV>
__device__ __forceinline__ void warp_sum_all(float (&v)[NV], int lane) {
  static_assert(NV == 1 || NV == 2 || NV == 4 || NV == 8 || NV == 16 || NV == 32, "value count must be a power of two");
  float w[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) w[i] = v[i];
  int n = NV;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    if (n > 1) {
      const bool up = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) {
        if (i < n / 2) {
          const float a = w[2 * i], b = w[2 * i + 1];
          w[i] = (up ? b : a) + __shfl_xor_sync(0xffffffffu, up ? a : b, off);
        }
      }
      n >>= 1;
    } else {
      w[0] += __shfl_xor_sync(0xffffffffu, w[0], off);
    }
  }
  // the total of value t sits in the lanes whose bits 4,3,2,... spell t's bits 0,1,2,...
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int src = ((t & 1) << 4) | ((t & 2) << 2) | (t & 4) | ((t & 8) >> 2) | ((t & 16) >> 4);
    v[t] = __shfl_sync(0xffffffffu, w[0], src);
  }
}

struct DecodeAttnArgs {
  const void *q, *k_new, *v_new;     // rows of the fused projection output (row stride ldq elements)
  void *kc, *vc, *o;                 // caches [B, S_max, nKV*hd]; output [B, ldo]
  float *ws_o, *ws_ml;               // [B, nH, splits, hd] and [B, nH, splits, 2]
  int *tickets;                      // [B, nH / GQ], zero between launches
  const int *pos_dev;                // when set: length = *pos_dev + 1 (read on the device: replayable capture)
  int nH, nKV, S_max, t_len, ldq, ldo, chunk;
  float scale;
};

// EPL = head_dim / 32 elements per lane; GQ = query heads per CTA (all share one KV head).
template <class T, int EPL, int GQ>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(DecodeAttnArgs a) {
  constexpr int HD = EPL * 32;
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_o[WARPS][GQ][HD];
  __shared__ float s_m[WARPS][GQ], s_l[WARPS][GQ];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, nsplit = gridDim.x, grp = blockIdx.y, b = blockIdx.z;
  const int G = a.nH / a.nKV, h0 = grp * GQ, kvh = h0 / G, KV = a.nKV * HD;
  const int t_len = a.pos_dev ? *a.pos_dev + 1 : a.t_len;      // plain load: written by the previous step's last kernel
  const int k0 = split * a.chunk, k1 = min(t_len, k0 + a.chunk);
  const T *q = (const T *)a.q + (size_t)b * a.ldq + (size_t)h0 * HD + lane * EPL;
  T *kc = (T *)a.kc + (size_t)b * a.S_max * KV + (size_t)kvh * HD + lane * EPL;
  T *vc = (T *)a.vc + (size_t)b * a.S_max * KV + (size_t)kvh * HD + lane * EPL;

  float qf[GQ][EPL], acc[GQ][EPL], m[GQ], l[GQ];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    RowLoad<T, EPL>::unpack(RowLoad<T, EPL>::ldg(q + g * HD), qf[g]);
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { qf[g][e] *= a.scale; acc[g][e] = 0.f; }
  }
  constexpr int KB = 4;                            // keys per warp step
  typedef typename RowLoad<T, EPL>::Raw Raw;
  // The token being decoded: its K/V rows come from the projection output and are appended to the cache by the CTA whose
  // key run holds the last position, before that CTA reads them back (the host passes k_new only when one CTA serves all
  // query heads of the KV head, so nobody else reads that cache row in this launch).
  if (a.k_new != nullptr && k0 <= t_len - 1 && t_len - 1 < k1) {
    if (warp == 0) {
      const size_t src = (size_t)b * a.ldq + (size_t)kvh * HD + lane * EPL, dst = (size_t)(t_len - 1) * KV;
      RowLoad<T, EPL>::stg(kc + dst, RowLoad<T, EPL>::ldg((const T *)a.k_new + src));
      RowLoad<T, EPL>::stg(vc + dst, RowLoad<T, EPL>::ldg((const T *)a.v_new + src));
    }
    __syncthreads();
  }
  // Raw loads of the KB rows of one step, branch-free (rows past the run re-read the step's first row and are masked in
  // the softmax).  The next step's rows are requested before this step's maths, so two steps of rows are in flight.
  auto load_rows = [&](int j, Raw *kr, Raw *vr) {
#pragma unroll
    for (int i = 0; i < KB; ++i) {
      const int ji = j + i * WARPS;
      const size_t off = (size_t)(ji < k1 ? ji : j) * KV;
      kr[i] = RowLoad<T, EPL>::ldg(kc + off);
      vr[i] = RowLoad<T, EPL>::ldg(vc + off);
    }
  };
  Raw kr[KB], vr[KB];
  if (k0 + warp < k1) load_rows(k0 + warp, kr, vr);
  for (int j = k0 + warp; j < k1; j += WARPS * KB) {
    Raw kn[KB], vn[KB];
    const int jn = j + WARPS * KB;
    if (jn < k1) load_rows(jn, kn, vn);
    float sv[KB * GQ];
#pragma unroll
    for (int i = 0; i < KB; ++i) {
      float kf[EPL];
      RowLoad<T, EPL>::unpack(kr[i], kf);
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d += qf[g][e] * kf[e];
        sv[i * GQ + g] = d;
      }
    }
    warp_sum_all<KB * GQ>(sv, lane);
    float s[KB][GQ];
#pragma unroll
    for (int i = 0; i < KB; ++i) {
#pragma unroll
      for (int g = 0; g < GQ; ++g) s[i][g] = sv[i * GQ + g];
    }
    float corr[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      float m_new = m[g];
#pragma unroll
      for (int i = 0; i < KB; ++i) if (j + i * WARPS < k1) m_new = fmaxf(m_new, s[i][g]);
      corr[g] = __expf(m[g] - m_new);
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < KB; ++i) {
        s[i][g] = (j + i * WARPS < k1) ? __expf(s[i][g] - m_new) : 0.f;      // scores become probabilities
        psum += s[i][g];
      }
      l[g] = l[g] * corr[g] + psum;
      m[g] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] *= corr[g];
    }
#pragma unroll
    for (int i = 0; i < KB; ++i) {
      float vf[EPL];
      RowLoad<T, EPL>::unpack(vr[i], vf);
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] += s[i][g] * vf[e];
      }
    }
    if (jn < k1) {
#pragma unroll
      for (int i = 0; i < KB; ++i) { kr[i] = kn[i]; vr[i] = vn[i]; }
    }
  }
  // ---- merge the warps of this CTA ------------------------------------------------------------
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) s_o[warp][g][lane * EPL + e] = acc[g][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < GQ * HD; i += WARPS * 32) {
    const int g = i / HD, d = i % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_m[w][g]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = s_m[w][g] == -INFINITY ? 0.f : __expf(s_m[w][g] - M);
      L += s_l[w][g] * f; O += s_o[w][g][d] * f;
    }
    if (nsplit == 1) {
      ((T *)a.o)[(size_t)b * a.ldo + (size_t)(h0 + g) * HD + d] = from_f<T>(O / L);
    } else {
      const size_t slot = ((size_t)b * a.nH + h0 + g) * nsplit + split;
      a.ws_o[slot * HD + d] = O;
      if (d == 0) { a.ws_ml[slot * 2] = M; a.ws_ml[slot * 2 + 1] = L; }
    }
  }
  if (nsplit == 1) return;
  // ---- the CTA that takes the last ticket merges the splits --------------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int *t = a.tickets + (size_t)b * gridDim.y + grp;
    const int prev = atomicAdd(t, 1);
    s_last = prev == nsplit - 1;
    if (s_last) *t = 0;                            // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < GQ * HD; i += WARPS * 32) {
    const int g = i / HD, d = i % HD;
    const size_t slot0 = ((size_t)b * a.nH + h0 + g) * nsplit;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, __ldcg(a.ws_ml + (slot0 + s) * 2));
    float L = 0.f, O = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = __ldcg(a.ws_ml + (slot0 + s) * 2);
      const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
      L += __ldcg(a.ws_ml + (slot0 + s) * 2 + 1) * f;
      O += __ldcg(a.ws_o + (slot0 + s) * HD + d) * f;
    }
    ((T *)a.o)[(size_t)b * a.ldo + (size_t)(h0 + g) * HD + d] = from_f<T>(O / L);
  }
}

template <class T, int EPL>
int launch_gq(b200_ctx *ctx, const DecodeAttnArgs &a, int gq, dim3 grid) {
  switch (gq) {
    case 8:
      if constexpr (EPL < 8) { B200_CUDA(ctx, launch_k(ctx, attn_decode_kernel<T, EPL, 8>, grid, dim3(WARPS * 32), 0, 0, a)); break; }
      else return b200_fail(ctx, B200_ERR_INVALID, "attn_decode: 8 heads of dimension 256 per CTA exceed shared memory");
    case 4: B200_CUDA(ctx, launch_k(ctx, attn_decode_kernel<T, EPL, 4>, grid, dim3(WARPS * 32), 0, 0, a)); break;
    case 2: B200_CUDA(ctx, launch_k(ctx, attn_decode_kernel<T, EPL, 2>, grid, dim3(WARPS * 32), 0, 0, a)); break;
    default: B200_CUDA(ctx, launch_k(ctx, attn_decode_kernel<T, EPL, 1>, grid, dim3(WARPS * 32), 0, 0, a)); break;
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}
template <class T>
int launch_hd(b200_ctx *ctx, const DecodeAttnArgs &a, int hd, int gq, dim3 grid) {
  switch (hd) {
    case 32: return launch_gq<T, 1>(ctx, a, gq, grid);
    case 64: return launch_gq<T, 2>(ctx, a, gq, grid);
    case 128: return launch_gq<T, 4>(ctx, a, gq, grid);
    default: return launch_gq<T, 8>(ctx, a, gq, grid);   // head_dim 256: the caller keeps gq <= 4 (shared memory)
  }
}

}  // namespace

constexpr int ATTN_DECODE_MAX_SPLITS = 16;

bool attn_decode_tc_supported(const b200_ctx *ctx, const void *q, const void *kc, const void *vc, const void *o, size_t B, size_t nH,
                              size_t nKV, size_t hd, size_t S_max, size_t ldq, size_t ldo, b200_dtype dt);
int attn_decode_tc(b200_ctx *ctx, const void *q, const void *k_new, const void *v_new, void *kc, void *vc, void *o, size_t B,
                   size_t nH, size_t nKV, size_t S_max, size_t t_len, size_t ldq, size_t ldo, const int *pos_dev);

size_t attn_decode_workspace_floats(size_t B, size_t nH, size_t hd) { return B * nH * ATTN_DECODE_MAX_SPLITS * (hd + 2); }

// q/k_new/v_new: rows of the fused projection (stride ldq); k_new/v_new may be null when the cache already
// holds position t_len-1.  pos_dev (optional): device int, length = *pos_dev + 1 instead of t_len.  ws: attn_decode_workspace_floats() floats; tickets: B*nH ints, zero-initialised.
int attn_decode(b200_ctx *ctx, const void *q, const void *k_new, const void *v_new, void *kc, void *vc, void *o, size_t B,
                size_t nH, size_t nKV, size_t hd, size_t S_max, size_t t_len, size_t ldq, size_t ldo, float *ws, int *tickets,
                b200_dtype dt, const int *pos_dev) {
  B200_REQUIRE(ctx, (hd == 32 || hd == 64 || hd == 128 || hd == 256) && t_len >= 1 && t_len <= S_max && nKV > 0 && nH % nKV == 0,
               "attn_decode: head_dim must be 32, 64, 128 or 256 and 1 <= length <= cache length");
  B200_REQUIRE(ctx, ws && tickets && B <= 65535, "attn_decode: workspace missing");
  if (ctx->attn_decode_tc && attn_decode_tc_supported(ctx, q, kc, vc, o, B, nH, nKV, hd, S_max, ldq, ldo, dt))
    return attn_decode_tc(ctx, q, k_new, v_new, kc, vc, o, B, nH, nKV, S_max, t_len, ldq, ldo, pos_dev);
  const size_t G = nH / nKV;
  int gq = (G == 2 || G == 4 || G == 8) ? (int)G : 1;
  if (hd == 256 && gq > 4) gq = 1;
  DecodeAttnArgs a;
  a.q = q; a.k_new = k_new; a.v_new = v_new; a.kc = kc; a.vc = vc; a.o = o;
  B200_REQUIRE(ctx, !k_new || (size_t)gq == G, "attn_decode: the fused cache append needs one CTA per KV-head group");
  a.pos_dev = pos_dev;
  if (pos_dev) t_len = S_max;                      // the grid is sized for the longest length so that it never changes
  a.ws_o = ws; a.ws_ml = ws + B * nH * ATTN_DECODE_MAX_SPLITS * hd; a.tickets = tickets;
  a.nH = (int)nH; a.nKV = (int)nKV; a.S_max = (int)S_max; a.t_len = (int)t_len; a.ldq = (int)ldq; a.ldo = (int)ldo;
  a.scale = 1.0f / sqrtf((float)hd);
  // key runs: one wave of CTAs (two fit per SM), at least 4 keys per warp, at most 16 splits
  const size_t groups = B * (nH / gq);
  size_t want = (2 * (size_t)ctx->sm_count) / groups;        // rounded down: one full wave, never a second, mostly empty one
  if (want < 1) want = 1;
  if (want > (size_t)ATTN_DECODE_MAX_SPLITS) want = ATTN_DECODE_MAX_SPLITS;
  size_t chunk = (t_len + want - 1) / want;
  if (chunk < 32) chunk = 32;
  chunk = (chunk + WARPS - 1) / WARPS * WARPS;
  const size_t nsplit = (t_len + chunk - 1) / chunk;
  a.chunk = (int)chunk;
  dim3 grid((unsigned)nsplit, (unsigned)(nH / gq), (unsigned)B);
  if (dt == B200_BF16) return launch_hd<bf16>(ctx, a, (int)hd, gq, grid);
  return launch_hd<float>(ctx, a, (int)hd, gq, grid);
}
