// Causal grouped-query attention forward on the sm_100a tensor cores (tcgen05 + tensor memory + TMA),
// bf16 operands, fp32 accumulation, head_dim 64 or 128, any head layout whose head_dim is
// contiguous (4-D tensor maps carry the batch / head / sequence strides, so the engine's
// token-major fused QKV rows and the reference's [B,heads,S,hd] tensors are both read in place;
// there are no head split/merge passes).
// Replaces metal_bridge::flash_attn_fwd (cpp/include/gpu_kernel/MetalBridge.hpp:49-51); maths of
// cpp/src/Attention.cpp:236-280.
//
// One CTA per (128-query tile, head, batch); key/value tiles of 128, causal tiles only.
//   warp 9    TMA producer (Q once; K, V double-buffered)
//   warp 8    one lane issues S = Q K^T into one of two tensor-memory score buffers and O_t = P V
//   warps 0-7 online softmax: two threads per query row (64 score columns and half of the
//             head_dim each), scores read from tensor memory once, P written (bf16, 128-byte
//             swizzled) to shared memory, O rescaled and accumulated in registers.
//   The score MMA of tile j+1 is issued before the softmax of tile j finishes, so tensor and
//   CUDA cores overlap.  Saves log-sum-exp per row for the backward.
#include "attention_tc.cuh"

using namespace attn;

namespace {

struct FwdShared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full[2], o_consumed[2], pair[4];
  uint32_t tmem_base;
  int abort_flag;
  float xchg[2][2][128];   // [tile parity][column half][row]: row maxima, then row sums
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, bf16 *__restrict__ O, float *__restrict__ lse,
                   int nH, int nKV, int S, long long o_b, long long o_h, long long o_s, float scale, int *status) {
  constexpr int TILE_BYTES = 128 * HD * 2;
  constexpr int OC = HD / 2;                            // output columns per thread
  // Q | K x2 | V x2 | P x2 fill the 227 KiB of shared memory at head_dim 128, so there is no room for an
  // alignment pad: the dynamic segment is declared 1024-byte aligned and checked below.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  uint8_t *sQ = smem, *sK = sQ + TILE_BYTES, *sV = sK + 2 * TILE_BYTES, *sP = sV + 2 * TILE_BYTES;
  FwdShared *sh = (FwdShared *)(sP + 2 * 32768);
  if (tc::smem_u32(smem) & 1023u) {           // swizzled tiles need 1024-byte alignment: refuse rather than corrupt
    if (threadIdx.x == 0) atomicCAS(status, 0, 299);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (S + TQ - 1) / TQ;
  // grid: x = head (fastest), y = query tile, z = batch... launch order is linear in (x, y, z): all heads and
  // batches of the heaviest (last) query tile are dispatched first, the lightest tiles fill the tail
  const int qi = n_qt - 1 - (int)blockIdx.y;
  const int h = blockIdx.x % nH, b = blockIdx.x / nH, kvh = h / (nH / nKV);
  const int n_kt = qi + 1;                            // causal: key tiles 0..qi
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sh->k_full[i], 1); tc::mbar_init(&sh->k_empty[i], 1);
      tc::mbar_init(&sh->v_full[i], 1); tc::mbar_init(&sh->v_empty[i], 1);
      tc::mbar_init(&sh->s_full[i], 1);
      tc::mbar_init(&sh->p_full[i], COMPUTE_WARPS); tc::mbar_init(&sh->o_full[i], 1); tc::mbar_init(&sh->o_consumed[i], COMPUTE_WARPS);
    }
    for (int i = 0; i < 4; ++i) tc::mbar_init(&sh->pair[i], 64);   // the two warps that share a row quarter
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == MMA_WARP) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      tc::mbar_expect_tx(&sh->q_full, TILE_BYTES);
      load_tile<HD>(sQ, &map_q, qi * TQ, h, b, &sh->q_full);
      for (int j = 0; j < n_kt; ++j) {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->k_empty[s], ph ^ 1, status, abort_flag, 201)) break;
        tc::mbar_expect_tx(&sh->k_full[s], TILE_BYTES);
        load_tile<HD>(sK + s * TILE_BYTES, &map_k, j * TK, kvh, b, &sh->k_full[s]);
        if (!tc::mbar_wait(&sh->v_empty[s], ph ^ 1, status, abort_flag, 202)) break;
        tc::mbar_expect_tx(&sh->v_full[s], TILE_BYTES);
        load_tile<HD>(sV + s * TILE_BYTES, &map_v, j * TK, kvh, b, &sh->v_full[s]);
      }
      if (*abort_flag) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = tc::make_idesc_bf16(128, HD, false, true);
      const uint32_t q_addr = tc::smem_u32(sQ), p_addr = tc::smem_u32(sP);
      bool ok = tc::mbar_wait(&sh->q_full, 0, status, abort_flag, 203);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->k_full[s], ph, status, abort_flag, 204)) return false;
        tc::tc_fence_after();
        const uint32_t k_addr = tc::smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc::umma_ss(tmem_base + s * 128, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->s_full[s]);
        tc::umma_commit(&sh->k_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kt && ok; ++j) {
        // scores of the next tile go into the other buffer (its previous reader finished before p_full(j-1))
        if (j + 1 < n_kt) { if (!issue_s(j + 1)) break; }
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->p_full[s], ph, status, abort_flag, 205)) break;
        if (!tc::mbar_wait(&sh->v_full[s], ph, status, abort_flag, 206)) break;
        // the output buffer of tile j was last used by tile j-2
        if (j > 1 && !tc::mbar_wait(&sh->o_consumed[s], ((j - 2) >> 1) & 1, status, abort_flag, 207)) break;
        tc::tc_fence_after();
        const uint32_t v_addr = tc::smem_u32(sV + s * TILE_BYTES), pj_addr = p_addr + s * 32768;
#pragma unroll
        for (int k = 0; k < TK / 16; ++k)
          tc::umma_ss(tmem_o + s * 128, desc_kmajor(pj_addr, k), desc_mnmajor(v_addr, k), idesc_o, k ? 1u : 0u);
        tc::umma_commit(&sh->o_full[s]);
        tc::umma_commit(&sh->v_empty[s]);
      }
    }
  } else {
    // ---- softmax + output accumulation: two threads per query row ------------------------
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;
    const int q_idx = qi * TQ + r;
    const int q_eff = min(q_idx, S - 1);               // rows past the end behave like the last row (never stored)
    const float sl2 = scale * LOG2E;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    float o[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o[i] = 0.f;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_kt && ok; ++j) {
      const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
      if (!tc::mbar_wait(&sh->s_full[s], ph, status, abort_flag, 208)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t ts = tmem_base + lane_base + s * 128 + half * 64;
      const int kc0 = j * TK + half * 64;              // first key column of this thread
      const bool diag = (j == qi);
      uint32_t v[64];
      tc::tmem_ld_32x32(ts, v);
      tc::tmem_ld_32x32(ts + 32, v + 32);
      tc::tmem_ld_wait();
      float mx8[8];                                   // independent partial maxima: no 64-long dependency chain
#pragma unroll
      for (int a = 0; a < 8; ++a) mx8[a] = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float x = __uint_as_float(v[i]);
        if (diag && (kc0 + i > q_eff)) x = -INFINITY;
        mx8[i & 7] = fmaxf(mx8[i & 7], x);
      }
      float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      // the row's other 64 columns belong to the partner warp: exchange the two partial maxima
      sh->xchg[j & 1][half][r] = mx;
      tc::mbar_arrive(&sh->pair[quarter]);
      if (!tc::mbar_wait(&sh->pair[quarter], j & 1, status, abort_flag, 210)) { ok = false; break; }
      mx = fmaxf(mx, sh->xchg[j & 1][half ^ 1][r]);
      const float m_new = fmaxf(m, mx * sl2);
      const float alpha = fast_exp2(m - m_new);
      float rs8[8];                                   // independent partial sums: no 64-long dependency chain
#pragma unroll
      for (int a = 0; a < 8; ++a) rs8[a] = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float e = fast_exp2(__uint_as_float(v[u * 8 + i]) * sl2 - m_new);
          if (diag && (kc0 + u * 8 + i > q_eff)) e = 0.f;
          p[i] = e; rs8[i] += e;
        }
        uint4 w;
        w.x = pack_bf16(p[0], p[1]); w.y = pack_bf16(p[2], p[3]); w.z = pack_bf16(p[4], p[5]); w.w = pack_bf16(p[6], p[7]);
        *reinterpret_cast<uint4 *>(sP + s * 32768 + swz_unit(r, half * 8 + u)) = w;
      }
      const float rowsum = ((rs8[0] + rs8[1]) + (rs8[2] + rs8[3])) + ((rs8[4] + rs8[5]) + (rs8[6] + rs8[7]));
      l = l * alpha + rowsum;
      m = m_new;
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->p_full[s]);
      // Software pipeline: while the tensor cores compute O_t(j) = P(j) V(j), fold in the PREVIOUS tile's
      // O_t(j-1) (its rescale factor alpha(j-1) was kept), then go straight on to the scores of tile j+1.
      if (j > 0) {
        const int sp = (j - 1) & 1;
        if (!tc::mbar_wait(&sh->o_full[sp], ((j - 1) >> 1) & 1, status, abort_flag, 209)) { ok = false; break; }
        tc::tc_fence_after();
        uint32_t ov[OC];
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) tc::tmem_ld_32x32(tmem_o + sp * 128 + lane_base + half * OC + c * 32, ov + c * 32);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < OC; ++i) o[i] = o[i] * alpha_prev + __uint_as_float(ov[i]);
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&sh->o_consumed[sp]);
      }
      alpha_prev = alpha;
    }
    if (ok) {   // drain: the last tile's product
      const int sp = (n_kt - 1) & 1;
      ok = tc::mbar_wait(&sh->o_full[sp], ((n_kt - 1) >> 1) & 1, status, abort_flag, 212);
      tc::tc_fence_after();
      uint32_t ov[OC];
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) tc::tmem_ld_32x32(tmem_o + sp * 128 + lane_base + half * OC + c * 32, ov + c * 32);
      tc::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < OC; ++i) o[i] = o[i] * alpha_prev + __uint_as_float(ov[i]);
      tc::tc_fence_before();
    }
    if (ok) {
      // combine the two column halves' row sums
      sh->xchg[n_kt & 1][half][r] = l;
      tc::mbar_arrive(&sh->pair[quarter]);
      ok = tc::mbar_wait(&sh->pair[quarter], n_kt & 1, status, abort_flag, 211);
      l += sh->xchg[n_kt & 1][half ^ 1][r];
      if (ok && q_idx < S) {
        const float inv = 1.0f / l;
        bf16 *orow = O + (long long)b * o_b + (long long)h * o_h + (long long)q_idx * o_s + half * OC;
#pragma unroll
        for (int u = 0; u < OC / 8; ++u) {
          uint4 w;
          w.x = pack_bf16(o[u * 8 + 0] * inv, o[u * 8 + 1] * inv); w.y = pack_bf16(o[u * 8 + 2] * inv, o[u * 8 + 3] * inv);
          w.z = pack_bf16(o[u * 8 + 4] * inv, o[u * 8 + 5] * inv); w.w = pack_bf16(o[u * 8 + 6] * inv, o[u * 8 + 7] * inv);
          *reinterpret_cast<uint4 *>(orow + u * 8) = w;
        }
        if (lse && half == 0) lse[((long long)b * nH + h) * S + q_idx] = (m + log2f(l)) * (1.0f / LOG2E);   // natural-log units
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
int fwd_launch_t(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B, size_t nH,
                 size_t nKV, size_t S, const AttnStrides &st) {
  CUtensorMap mq, mk, mv;
  if (make_map_4d(&mq, Q, HD, S, nH, B, st.q_s, st.q_h, st.q_b) || make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) ||
      make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
  constexpr int smem = 5 * 128 * HD * 2 + 2 * 32768 + (int)sizeof(FwdShared);
  static_assert(smem <= 232448, "forward attention tiles exceed the 227 KiB of shared memory per CTA");
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  dim3 grid((unsigned)(nH * B), (unsigned)((S + TQ - 1) / TQ), 1);
  attn_fwd_tc_kernel<HD><<<grid, THREADS, smem, ctx->stream>>>(mq, mk, mv, (bf16 *)O, lse, (int)nH, (int)nKV, (int)S, st.o_b, st.o_h,
                                                              st.o_s, 1.0f / sqrtf((float)HD), ctx->dev_status);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
}  // namespace

bool attn_tc_supported(size_t B, size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt,
                       const void *Q, const void *K, const void *V, const void *O) {
  if (dt != B200_BF16 || (hd != 64 && hd != 128) || B == 0 || S == 0 || nKV == 0 || nH % nKV) return false;
  if (nH * B > 0x7fffffffull || (S + TQ - 1) / TQ > 65535) return false;
  return layout_ok(Q, st.q_b, st.q_h, st.q_s) && layout_ok(K, st.k_b, st.k_h, st.k_s) &&
         layout_ok(V, st.v_b, st.v_h, st.v_s) && layout_ok(O, st.o_b, st.o_h, st.o_s);
}

int attn_fwd_tc_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                       size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st) {
  return hd == 128 ? fwd_launch_t<128>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st) : fwd_launch_t<64>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st);
}
