// Causal grouped-query attention on CUDA cores, fp32 maths, any head_dim <= 256.
// This is the fp32 path of the backend (1e-4 contract against the reference's CPU loops,
// cpp/src/Attention.cpp:236-280 forward, :292-348 backward) and the catch-all for
// shapes the tensor-core kernel does not take.  One warp per query row; keys are
// processed 32 at a time (lane = key) with an online softmax; outputs are owned by
// lanes (lane = head-dim element mod 32).  kv head = h / (nH/nKV).
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_ND = 8;  // head_dim <= 256

template <class T>
__global__ void __launch_bounds__(WARPS * 32)
attn_fwd_simt(const T *__restrict__ Q, const T *__restrict__ K, const T *__restrict__ V, T *__restrict__ O,
              float *__restrict__ lse, int B, int nH, int nKV, int S, int hd, AttnStrides st, float scale) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *qs = sm + warp * hd;
  const int G = nH / nKV;
  const long long rows = (long long)B * nH * S;
  for (long long row = (long long)blockIdx.x * WARPS + warp; row < rows; row += (long long)gridDim.x * WARPS) {
    const int sq = (int)(row % S);
    const int h = (int)((row / S) % nH);
    const int b = (int)(row / ((long long)S * nH));
    const int kvh = h / G;
    const T *q = Q + b * st.q_b + h * st.q_h + (long long)sq * st.q_s;
    const T *kbase = K + b * st.k_b + kvh * st.k_h;
    const T *vbase = V + b * st.v_b + kvh * st.v_h;
    __syncwarp();
    for (int d = lane; d < hd; d += 32) qs[d] = to_f(q[d]);
    __syncwarp();
    float m = -INFINITY, l = 0.f, o[MAX_ND];
#pragma unroll
    for (int i = 0; i < MAX_ND; ++i) o[i] = 0.f;
    for (int j0 = 0; j0 <= sq; j0 += 32) {
      const int j = j0 + lane;
      float s = -INFINITY;
      if (j <= sq) {
        const T *kr = kbase + (long long)j * st.k_s;
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot += qs[d] * to_f(kr[d]);
        s = dot * scale;
      }
      float m_new = fmaxf(m, warp_max(s));
      float p = (j <= sq) ? __expf(s - m_new) : 0.f;
      float corr = __expf(m - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int i = 0; i < MAX_ND; ++i) o[i] *= corr;
      const int nj = min(32, sq - j0 + 1);
      for (int jj = 0; jj < nj; ++jj) {
        float pj = __shfl_sync(0xffffffffu, p, jj);
        const T *vr = vbase + (long long)(j0 + jj) * st.v_s;
#pragma unroll
        for (int i = 0; i < MAX_ND; ++i) {
          int d = lane + 32 * i;
          if (d < hd) o[i] += pj * to_f(vr[d]);
        }
      }
      m = m_new;
    }
    T *orow = O + b * st.o_b + h * st.o_h + (long long)sq * st.o_s;
    float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_ND; ++i) {
      int d = lane + 32 * i;
      if (d < hd) orow[d] = from_f<T>(o[i] * inv);
    }
    if (lse && lane == 0) lse[((long long)b * nH + h) * S + sq] = m + __logf(l);
  }
}

// dQ is owned by the warp; dK/dV are accumulated with fp32 atomics into contiguous
// [B,nKV,S,hd] scratch (several query rows and the G query heads of a kv head all add
// into the same key rows) and converted to the output layout afterwards.
template <class T>
__global__ void __launch_bounds__(WARPS * 32)
attn_bwd_simt(const T *__restrict__ Q, const T *__restrict__ K, const T *__restrict__ V, const T *__restrict__ O,
              const T *__restrict__ dO, const float *__restrict__ lse, T *__restrict__ dQ, float *__restrict__ dKacc,
              float *__restrict__ dVacc, int B, int nH, int nKV, int S, int hd, AttnStrides st, AttnStrides gst,
              float scale) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *qs = sm + warp * 2 * hd, *gs = qs + hd;
  const int G = nH / nKV;
  const long long rows = (long long)B * nH * S;
  for (long long row = (long long)blockIdx.x * WARPS + warp; row < rows; row += (long long)gridDim.x * WARPS) {
    const int sq = (int)(row % S);
    const int h = (int)((row / S) % nH);
    const int b = (int)(row / ((long long)S * nH));
    const int kvh = h / G;
    const T *q = Q + b * st.q_b + h * st.q_h + (long long)sq * st.q_s;
    const T *orow = O + b * st.o_b + h * st.o_h + (long long)sq * st.o_s;
    const T *grow = dO + b * st.o_b + h * st.o_h + (long long)sq * st.o_s;
    const T *kbase = K + b * st.k_b + kvh * st.k_h;
    const T *vbase = V + b * st.v_b + kvh * st.v_h;
    float *dkb = dKacc + ((long long)b * nKV + kvh) * S * hd;
    float *dvb = dVacc + ((long long)b * nKV + kvh) * S * hd;
    __syncwarp();
    float dsum = 0.f;
    for (int d = lane; d < hd; d += 32) {
      float gq = to_f(grow[d]);
      qs[d] = to_f(q[d]); gs[d] = gq;
      dsum += gq * to_f(orow[d]);
    }
    dsum = warp_sum(dsum);           // D = sum_d dO*O = sum_j P_j dP_j
    __syncwarp();
    const float L = lse[((long long)b * nH + h) * S + sq];
    float dq[MAX_ND];
#pragma unroll
    for (int i = 0; i < MAX_ND; ++i) dq[i] = 0.f;
    for (int j0 = 0; j0 <= sq; j0 += 32) {
      const int j = j0 + lane;
      float p = 0.f, ds = 0.f;
      if (j <= sq) {
        const T *kr = kbase + (long long)j * st.k_s;
        const T *vr = vbase + (long long)j * st.v_s;
        float dot = 0.f, dp = 0.f;
        for (int d = 0; d < hd; ++d) { dot += qs[d] * to_f(kr[d]); dp += gs[d] * to_f(vr[d]); }
        p = __expf(dot * scale - L);
        ds = p * (dp - dsum) * scale;
      }
      const int nj = min(32, sq - j0 + 1);
      for (int jj = 0; jj < nj; ++jj) {
        float pj = __shfl_sync(0xffffffffu, p, jj), dsj = __shfl_sync(0xffffffffu, ds, jj);
        const T *kr = kbase + (long long)(j0 + jj) * st.k_s;
#pragma unroll
        for (int i = 0; i < MAX_ND; ++i) {
          int d = lane + 32 * i;
          if (d < hd) {
            dq[i] += dsj * to_f(kr[d]);
            atomicAdd(dkb + (long long)(j0 + jj) * hd + d, dsj * qs[d]);
            atomicAdd(dvb + (long long)(j0 + jj) * hd + d, pj * gs[d]);
          }
        }
      }
    }
    T *dqrow = dQ + b * gst.q_b + h * gst.q_h + (long long)sq * gst.q_s;
#pragma unroll
    for (int i = 0; i < MAX_ND; ++i) {
      int d = lane + 32 * i;
      if (d < hd) dqrow[d] = from_f<T>(dq[i]);
    }
  }
}

template <class T>
__global__ void scatter_kv_grads(const float *__restrict__ acc, T *__restrict__ out, int B, int nKV, int S, int hd,
                                 long long sb, long long sh, long long ss) {
  size_t total = (size_t)B * nKV * S * hd;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    int d = (int)(i % hd); size_t r = i / hd;
    int s = (int)(r % S); r /= S;
    int h = (int)(r % nKV); int b = (int)(r / nKV);
    out[b * sb + h * sh + (long long)s * ss + d] = from_f<T>(acc[i]);
  }
}
}  // namespace

int attn_fwd_simt_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                         size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt) {
  B200_REQUIRE(ctx, hd <= 32 * MAX_ND, "attention: head_dim > 256 unsupported");
  size_t rows = B * nH * S;
  if (!rows) return B200_OK;
  size_t blocks = (rows + WARPS - 1) / WARPS, cap = (size_t)ctx->sm_count * 16;
  int grid = (int)(blocks < cap ? blocks : cap);
  float scale = 1.0f / sqrtf((float)hd);
  size_t smem = WARPS * hd * sizeof(float);
  if (dt == B200_BF16) attn_fwd_simt<bf16><<<grid, WARPS * 32, smem, ctx->stream>>>((const bf16 *)Q, (const bf16 *)K, (const bf16 *)V, (bf16 *)O, lse, (int)B, (int)nH, (int)nKV, (int)S, (int)hd, st, scale);
  else attn_fwd_simt<float><<<grid, WARPS * 32, smem, ctx->stream>>>((const float *)Q, (const float *)K, (const float *)V, (float *)O, lse, (int)B, (int)nH, (int)nKV, (int)S, (int)hd, st, scale);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

// kv_scratch: fp32, 2 * B*nKV*S*hd elements.
int attn_bwd_simt_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                         const float *lse, void *dQ, void *dK, void *dV, float *kv_scratch, size_t B, size_t nH,
                         size_t nKV, size_t S, size_t hd, const AttnStrides &st, const AttnStrides &gst,
                         b200_dtype dt) {
  B200_REQUIRE(ctx, hd <= 32 * MAX_ND, "attention: head_dim > 256 unsupported");
  size_t rows = B * nH * S, kvn = B * nKV * S * hd;
  if (!rows) return B200_OK;
  float *dKacc = kv_scratch, *dVacc = kv_scratch + kvn;
  B200_CUDA(ctx, cudaMemsetAsync(kv_scratch, 0, 2 * kvn * sizeof(float), ctx->stream));
  size_t blocks = (rows + WARPS - 1) / WARPS, cap = (size_t)ctx->sm_count * 16;
  int grid = (int)(blocks < cap ? blocks : cap);
  float scale = 1.0f / sqrtf((float)hd);
  size_t smem = WARPS * 2 * hd * sizeof(float);
  int sgrid = (int)((kvn + 255) / 256 < (size_t)ctx->sm_count * 16 ? (kvn + 255) / 256 : (size_t)ctx->sm_count * 16);
  if (dt == B200_BF16) {
    attn_bwd_simt<bf16><<<grid, WARPS * 32, smem, ctx->stream>>>((const bf16 *)Q, (const bf16 *)K, (const bf16 *)V, (const bf16 *)O, (const bf16 *)dO, lse, (bf16 *)dQ, dKacc, dVacc, (int)B, (int)nH, (int)nKV, (int)S, (int)hd, st, gst, scale);
    B200_LAUNCHED(ctx);
    scatter_kv_grads<bf16><<<sgrid, 256, 0, ctx->stream>>>(dKacc, (bf16 *)dK, (int)B, (int)nKV, (int)S, (int)hd, gst.k_b, gst.k_h, gst.k_s);
    B200_LAUNCHED(ctx);
    scatter_kv_grads<bf16><<<sgrid, 256, 0, ctx->stream>>>(dVacc, (bf16 *)dV, (int)B, (int)nKV, (int)S, (int)hd, gst.v_b, gst.v_h, gst.v_s);
  } else {
    attn_bwd_simt<float><<<grid, WARPS * 32, smem, ctx->stream>>>((const float *)Q, (const float *)K, (const float *)V, (const float *)O, (const float *)dO, lse, (float *)dQ, dKacc, dVacc, (int)B, (int)nH, (int)nKV, (int)S, (int)hd, st, gst, scale);
    B200_LAUNCHED(ctx);
    scatter_kv_grads<float><<<sgrid, 256, 0, ctx->stream>>>(dKacc, (float *)dK, (int)B, (int)nKV, (int)S, (int)hd, gst.k_b, gst.k_h, gst.k_s);
    B200_LAUNCHED(ctx);
    scatter_kv_grads<float><<<sgrid, 256, 0, ctx->stream>>>(dVacc, (float *)dV, (int)B, (int)nKV, (int)S, (int)hd, gst.v_b, gst.v_h, gst.v_s);
  }
  B200_LAUNCHED(ctx);
  return B200_OK;
}
