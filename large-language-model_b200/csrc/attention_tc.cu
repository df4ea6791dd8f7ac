// Causal grouped-query attention on the sm_100a tensor cores (tcgen05 + tensor memory + TMA),
// bf16 operands, fp32 accumulation, head_dim 64 or 128, any head layout whose head_dim is
// contiguous (4-D tensor maps carry the batch / head / sequence strides, so the engine's
// token-major fused QKV rows and the reference's [B,heads,S,hd] tensors are both read in place;
// there are no head split/merge passes).
// Replaces metal_bridge::flash_attn_fwd and fused_attn_bwd
// (cpp/include/gpu_kernel/MetalBridge.hpp:49-57); maths of cpp/src/Attention.cpp:236-280, 292-348.
//
// Forward: one CTA per (128-query tile, head, batch); key/value tiles of 128, causal tiles only.
//   warp 5   TMA producer (Q once; K, V double-buffered)
//   warp 4   one lane issues S = Q K^T into one of two tensor-memory score buffers and O_t = P V
//   warps0-3 online softmax, one query row per thread: read S from tensor memory, write P (bf16,
//            128-byte swizzled) to shared memory, rescale-and-accumulate O in registers.
//   The score MMA of tile j+1 is issued before the softmax of tile j finishes, so tensor and
//   CUDA cores overlap.  Saves log-sum-exp per row for the backward.
// Backward: one CTA per (128-key tile, kv head, batch) owns dK/dV in tensor memory and loops
//   over the G = nH/nKV query heads of its kv head and the query tiles at or below the diagonal:
//   S = Q K^T, dP = dO V^T -> P, dS (registers -> shared) -> dV += P^T dO, dK += dS^T Q,
//   dQ_t = dS K (added to an fp32 dQ accumulator with atomics; K/V-tile owners never race on
//   dK/dV).  P is recomputed from the saved log-sum-exp; D = rowsum(dO * O) is a pre-pass.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int TQ = 128, TK = 128;          // query / key tile
constexpr int FWD_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(tc::smem_u32(dst)), "l"(map), "r"(tc::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Load a [128 rows x HD] tile as HD/64 chunks of [128 rows][128 B] (128-byte swizzle).
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t *dst, const CUtensorMap *map, int row0, int head, int batch,
                                          uint64_t *bar) {
#pragma unroll
  for (int c = 0; c < HD / 64; ++c) tma_load_4d(dst + c * 16384, map, c * 64, row0, head, batch, bar);
}

// Byte offset of the 16-byte unit holding columns [8u, 8u+8) of row r in a [128 x 128] bf16 tile stored
// as 2 chunks of [128 rows][128 B] with the 128-byte swizzle (what TMA would have produced).
__device__ __forceinline__ uint32_t swz_unit(int r, int unit16) {   // unit16 in [0,16)
  int chunk = unit16 >> 3, u = unit16 & 7;
  return (uint32_t)(chunk * 16384 + r * 128 + ((u ^ (r & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// A/B operand descriptors for a tile stored as chunks of [128 rows][128 B]:
//   "row-contraction"  : the contraction index is the column (inside the 128-byte row): K-major.
//       16 columns per MMA: chunk = k/4, 32 bytes per step inside the chunk.
//   "col-contraction"  : the contraction index is the row: MN-major; 16 rows (2 KiB) per MMA,
//       64-column chunks 16 KiB apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int k) {
  return tc::make_smem_desc(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return tc::make_smem_desc(base + k * 2048, 16384, 1024);
}

struct FwdShared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, o_full, o_consumed;
  uint32_t tmem_base;
  int abort_flag;
};

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, bf16 *__restrict__ O, float *__restrict__ lse,
                   int nH, int nKV, int S, long long o_b, long long o_h, long long o_s, float scale, int *status) {
  constexpr int TILE_BYTES = 128 * HD * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sQ = smem, *sK = sQ + TILE_BYTES, *sV = sK + 2 * TILE_BYTES, *sP = sV + 2 * TILE_BYTES;
  FwdShared *sh = (FwdShared *)(sP + 32768);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (S + TQ - 1) / TQ;
  const int qi = n_qt - 1 - (int)blockIdx.x;          // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z, kvh = h / (nH / nKV);
  const int n_kt = qi + 1;                            // causal: key tiles 0..qi
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sh->k_full[i], 1); tc::mbar_init(&sh->k_empty[i], 1);
      tc::mbar_init(&sh->v_full[i], 1); tc::mbar_init(&sh->v_empty[i], 1);
      tc::mbar_init(&sh->s_full[i], 1);
    }
    tc::mbar_init(&sh->p_full, 4); tc::mbar_init(&sh->o_full, 1); tc::mbar_init(&sh->o_consumed, 4);
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == 4) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 5) {
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
  } else if (warp == 4) {
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
        if (!tc::mbar_wait(&sh->p_full, j & 1, status, abort_flag, 205)) break;
        if (!tc::mbar_wait(&sh->v_full[s], ph, status, abort_flag, 206)) break;
        if (j > 0 && !tc::mbar_wait(&sh->o_consumed, (j - 1) & 1, status, abort_flag, 207)) break;
        tc::tc_fence_after();
        const uint32_t v_addr = tc::smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < TK / 16; ++k)
          tc::umma_ss(tmem_o, desc_kmajor(p_addr, k), desc_mnmajor(v_addr, k), idesc_o, k ? 1u : 0u);
        tc::umma_commit(&sh->o_full);
        tc::umma_commit(&sh->v_empty[s]);
      }
    }
  } else {
    // ---- softmax + output accumulation: thread = query row ------------------------------
    const int r = warp * 32 + lane;
    const int q_idx = qi * TQ + r;
    const int q_eff = min(q_idx, S - 1);               // rows past the end behave like the last row (never stored)
    const float sl2 = scale * LOG2E;
    float m = -INFINITY, l = 0.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_kt && ok; ++j) {
      const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
      if (!tc::mbar_wait(&sh->s_full[s], ph, status, abort_flag, 208)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t ts = tmem_base + lane_base + s * 128;
      const int k0 = j * TK;
      const bool diag = (j == qi);
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tc::tmem_ld_32x32(ts + c * 32, v);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(v[i]);
          if (diag && (k0 + c * 32 + i > q_eff)) x = -INFINITY;
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m, mx * sl2);
      const float alpha = exp2f(m - m_new);
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tc::tmem_ld_32x32(ts + c * 32, v);
        tc::tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(v[i]);
          float e = exp2f(x * sl2 - m_new);
          if (diag && (k0 + c * 32 + i > q_eff)) e = 0.f;
          p[i] = e; rowsum += e;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 w;
          w.x = pack_bf16(p[u * 8 + 0], p[u * 8 + 1]); w.y = pack_bf16(p[u * 8 + 2], p[u * 8 + 3]);
          w.z = pack_bf16(p[u * 8 + 4], p[u * 8 + 5]); w.w = pack_bf16(p[u * 8 + 6], p[u * 8 + 7]);
          *reinterpret_cast<uint4 *>(sP + swz_unit(r, c * 4 + u)) = w;
        }
      }
      l = l * alpha + rowsum;
      m = m_new;
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->p_full);
      // O_t = P V of this tile
      if (!tc::mbar_wait(&sh->o_full, j & 1, status, abort_flag, 209)) { ok = false; break; }
      tc::tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tc::tmem_ld_32x32(tmem_o + lane_base + c * 32, v);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->o_consumed);
    }
    if (ok && q_idx < S) {
      const float inv = 1.0f / l;
      bf16 *orow = O + (long long)b * o_b + (long long)h * o_h + (long long)q_idx * o_s;
#pragma unroll
      for (int u = 0; u < HD / 8; ++u) {
        uint4 w;
        w.x = pack_bf16(o[u * 8 + 0] * inv, o[u * 8 + 1] * inv); w.y = pack_bf16(o[u * 8 + 2] * inv, o[u * 8 + 3] * inv);
        w.z = pack_bf16(o[u * 8 + 4] * inv, o[u * 8 + 5] * inv); w.w = pack_bf16(o[u * 8 + 6] * inv, o[u * 8 + 7] * inv);
        *reinterpret_cast<uint4 *>(orow + u * 8) = w;
      }
      if (lse) lse[((long long)b * nH + h) * S + q_idx] = (m + log2f(l)) * (1.0f / LOG2E);   // natural-log units
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ backward --
struct BwdShared {
  uint64_t kv_full, qdo_full, qdo_empty, s_full, dp_full, pds_full, dq_full, dq_consumed, done;
  uint32_t tmem_base;
  int abort_flag;
};

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const float *__restrict__ lse, const float *__restrict__ Dsum, float *__restrict__ dQacc,
                   bf16 *__restrict__ dK, bf16 *__restrict__ dV, int nH, int nKV, int S, long long dk_b,
                   long long dk_h, long long dk_s, long long dv_b, long long dv_h, long long dv_s, float scale,
                   int *status) {
  constexpr int TILE_BYTES = 128 * HD * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sK = smem, *sV = sK + TILE_BYTES, *sQ = sV + TILE_BYTES, *sdO = sQ + TILE_BYTES, *sP = sdO + TILE_BYTES,
          *sdS = sP + 32768;
  BwdShared *sh = (BwdShared *)(sdS + 32768);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (S + TQ - 1) / TQ;
  const int j = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = nH / nKV;
  const int n_steps = G * (n_t - j);                  // (head in group) x (query tiles j..n_t-1)
  volatile int *abort_flag = &sh->abort_flag;
  // tensor memory: [0,128) S then dQ_t | [128,256) dP | [256,256+HD) dV | [384,384+HD) dK
  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->kv_full, 1); tc::mbar_init(&sh->qdo_full, 1); tc::mbar_init(&sh->qdo_empty, 1);
    tc::mbar_init(&sh->s_full, 1); tc::mbar_init(&sh->dp_full, 1); tc::mbar_init(&sh->pds_full, 4);
    tc::mbar_init(&sh->dq_full, 1); tc::mbar_init(&sh->dq_consumed, 4); tc::mbar_init(&sh->done, 1);
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == 4) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 5) {
    if (lane == 0) {
      tc::mbar_expect_tx(&sh->kv_full, 2 * TILE_BYTES);
      load_tile<HD>(sK, &map_k, j * TK, kvh, b, &sh->kv_full);
      load_tile<HD>(sV, &map_v, j * TK, kvh, b, &sh->kv_full);
      for (int st = 0; st < n_steps; ++st) {
        const int h = kvh * G + st / (n_t - j), i = j + st % (n_t - j);
        if (!tc::mbar_wait(&sh->qdo_empty, (st & 1) ^ 1, status, abort_flag, 301)) break;
        tc::mbar_expect_tx(&sh->qdo_full, 2 * TILE_BYTES);
        load_tile<HD>(sQ, &map_q, i * TQ, h, b, &sh->qdo_full);
        load_tile<HD>(sdO, &map_do, i * TQ, h, b, &sh->qdo_full);
      }
      if (*abort_flag) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 128, false, false);   // S, dP
      constexpr uint32_t idesc_kv = tc::make_idesc_bf16(128, HD, true, true);     // dV, dK
      constexpr uint32_t idesc_dq = tc::make_idesc_bf16(128, HD, false, true);    // dQ_t
      const uint32_t k_addr = tc::smem_u32(sK), v_addr = tc::smem_u32(sV), q_addr = tc::smem_u32(sQ),
                     do_addr = tc::smem_u32(sdO), p_addr = tc::smem_u32(sP), ds_addr = tc::smem_u32(sdS);
      bool ok = tc::mbar_wait(&sh->kv_full, 0, status, abort_flag, 302);
      for (int st = 0; st < n_steps && ok; ++st) {
        const uint32_t ph = st & 1;
        if (!tc::mbar_wait(&sh->qdo_full, ph, status, abort_flag, 303)) break;
        if (st > 0 && !tc::mbar_wait(&sh->dq_consumed, (st - 1) & 1, status, abort_flag, 304)) break;
        tc::tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) tc::umma_ss(t_s, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->s_full);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) tc::umma_ss(t_dp, desc_kmajor(do_addr, k), desc_kmajor(v_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->dp_full);
        if (!tc::mbar_wait(&sh->pds_full, ph, status, abort_flag, 305)) break;
        tc::tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 128 query rows)
#pragma unroll
        for (int k = 0; k < TQ / 16; ++k) tc::umma_ss(t_dv, desc_mnmajor(p_addr, k), desc_mnmajor(do_addr, k), idesc_kv, (st | k) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < TQ / 16; ++k) tc::umma_ss(t_dk, desc_mnmajor(ds_addr, k), desc_mnmajor(q_addr, k), idesc_kv, (st | k) ? 1u : 0u);
        tc::umma_commit(&sh->qdo_empty);
        // dQ_t = dS K  (contraction over the 128 keys), into the score columns
#pragma unroll
        for (int k = 0; k < TK / 16; ++k) tc::umma_ss(t_s, desc_kmajor(ds_addr, k), desc_mnmajor(k_addr, k), idesc_dq, k ? 1u : 0u);
        tc::umma_commit(&sh->dq_full);
      }
      if (ok) tc::umma_commit(&sh->done);
    }
  } else {
    const int r = warp * 32 + lane;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float sl2 = scale * LOG2E;
    bool ok = true;
    for (int st = 0; st < n_steps && ok; ++st) {
      const int h = kvh * G + st / (n_t - j), i = j + st % (n_t - j);
      const uint32_t ph = st & 1;
      const int q_idx = i * TQ + r;
      const bool valid = q_idx < S;
      const long long stat_off = ((long long)b * nH + h) * S + q_idx;
      const float L2 = valid ? lse[stat_off] * LOG2E : 0.f;
      const float Dr = valid ? Dsum[stat_off] : 0.f;
      const bool diag = (i == j);
      const int k0 = j * TK;
      if (!tc::mbar_wait(&sh->s_full, ph, status, abort_flag, 306)) { ok = false; break; }
      if (!tc::mbar_wait(&sh->dp_full, ph, status, abort_flag, 307)) { ok = false; break; }
      tc::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tc::tmem_ld_32x32(t_s + lane_base + c * 32, sv);
        tc::tmem_ld_32x32(t_dp + lane_base + c * 32, dv);
        tc::tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          float e = exp2f(__uint_as_float(sv[x]) * sl2 - L2);
          if (!valid || (diag && (k0 + c * 32 + x > q_idx))) e = 0.f;
          p[x] = e;
          ds[x] = e * (__uint_as_float(dv[x]) - Dr) * scale;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 w;
          w.x = pack_bf16(p[u * 8 + 0], p[u * 8 + 1]); w.y = pack_bf16(p[u * 8 + 2], p[u * 8 + 3]);
          w.z = pack_bf16(p[u * 8 + 4], p[u * 8 + 5]); w.w = pack_bf16(p[u * 8 + 6], p[u * 8 + 7]);
          *reinterpret_cast<uint4 *>(sP + swz_unit(r, c * 4 + u)) = w;
          w.x = pack_bf16(ds[u * 8 + 0], ds[u * 8 + 1]); w.y = pack_bf16(ds[u * 8 + 2], ds[u * 8 + 3]);
          w.z = pack_bf16(ds[u * 8 + 4], ds[u * 8 + 5]); w.w = pack_bf16(ds[u * 8 + 6], ds[u * 8 + 7]);
          *reinterpret_cast<uint4 *>(sdS + swz_unit(r, c * 4 + u)) = w;
        }
      }
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->pds_full);
      if (!tc::mbar_wait(&sh->dq_full, ph, status, abort_flag, 308)) { ok = false; break; }
      tc::tc_fence_after();
      float *dqrow = dQacc + (((long long)b * nH + h) * S + q_idx) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tc::tmem_ld_32x32(t_s + lane_base + c * 32, v);
        tc::tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int x = 0; x < 32; ++x) atomicAdd(dqrow + c * 32 + x, __uint_as_float(v[x]));
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->dq_consumed);
    }
    // dK / dV of this key tile: rows = keys
    if (ok && tc::mbar_wait(&sh->done, 0, status, abort_flag, 309)) {
      tc::tc_fence_after();
      const int key = j * TK + r;
      bf16 *dkrow = dK + (long long)b * dk_b + (long long)kvh * dk_h + (long long)key * dk_s;
      bf16 *dvrow = dV + (long long)b * dv_b + (long long)kvh * dv_h + (long long)key * dv_s;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t a[32], g[32];
        tc::tmem_ld_32x32(t_dk + lane_base + c * 32, a);
        tc::tmem_ld_32x32(t_dv + lane_base + c * 32, g);
        tc::tmem_ld_wait();
        if (key < S) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(a[u * 8 + 0]), __uint_as_float(a[u * 8 + 1]));
            w.y = pack_bf16(__uint_as_float(a[u * 8 + 2]), __uint_as_float(a[u * 8 + 3]));
            w.z = pack_bf16(__uint_as_float(a[u * 8 + 4]), __uint_as_float(a[u * 8 + 5]));
            w.w = pack_bf16(__uint_as_float(a[u * 8 + 6]), __uint_as_float(a[u * 8 + 7]));
            *reinterpret_cast<uint4 *>(dkrow + c * 32 + u * 8) = w;
            w.x = pack_bf16(__uint_as_float(g[u * 8 + 0]), __uint_as_float(g[u * 8 + 1]));
            w.y = pack_bf16(__uint_as_float(g[u * 8 + 2]), __uint_as_float(g[u * 8 + 3]));
            w.z = pack_bf16(__uint_as_float(g[u * 8 + 4]), __uint_as_float(g[u * 8 + 5]));
            w.w = pack_bf16(__uint_as_float(g[u * 8 + 6]), __uint_as_float(g[u * 8 + 7]));
            *reinterpret_cast<uint4 *>(dvrow + c * 32 + u * 8) = w;
          }
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

// D[b,h,s] = sum_d dO * O : one warp per (b,h,s) row.
__global__ void attn_dsum_kernel(const bf16 *__restrict__ O, const bf16 *__restrict__ dO, float *__restrict__ D,
                                 int B, int nH, int S, int hd, long long o_b, long long o_h, long long o_s,
                                 long long g_b, long long g_h, long long g_s) {
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)B * nH * S;
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int s = (int)(row % S), h = (int)((row / S) % nH), b = (int)(row / ((long long)S * nH));
    const bf16 *o = O + b * o_b + h * o_h + (long long)s * o_s;
    const bf16 *g = dO + b * g_b + h * g_h + (long long)s * g_s;
    float acc = 0.f;
    for (int d = lane * 2; d < hd; d += 64) {
      __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(o + d), c = *reinterpret_cast<const __nv_bfloat162 *>(g + d);
      acc += __bfloat162float(a.x) * __bfloat162float(c.x) + __bfloat162float(a.y) * __bfloat162float(c.y);
    }
    acc = warp_sum(acc);
    if (lane == 0) D[row] = acc;
  }
}
// fp32 [B,nH,S,hd] accumulator -> strided bf16 dQ
__global__ void attn_dq_store_kernel(const float *__restrict__ acc, bf16 *__restrict__ dQ, int B, int nH, int S,
                                     int hd, long long q_b, long long q_h, long long q_s) {
  const size_t total = (size_t)B * nH * S * (hd / 8);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(idx % (hd / 8)); size_t r = idx / (hd / 8);
    const int s = (int)(r % S); r /= S;
    const int h = (int)(r % nH), b = (int)(r / nH);
    const float4 x = *reinterpret_cast<const float4 *>(acc + idx * 8), y = *reinterpret_cast<const float4 *>(acc + idx * 8 + 4);
    uint4 w;
    w.x = pack_bf16(x.x, x.y); w.y = pack_bf16(x.z, x.w); w.z = pack_bf16(y.x, y.y); w.w = pack_bf16(y.z, y.w);
    *reinterpret_cast<uint4 *>(dQ + b * q_b + h * q_h + (long long)s * q_s + u * 8) = w;
  }
}

int make_map_4d(CUtensorMap *map, const void *base, size_t hd, size_t S, size_t heads, size_t B, long long s_s,
                long long s_h, long long s_b) {
  // dims (d, s, head, batch); strides in bytes for dims 1..3
  return tc_make_map_4d(map, base, hd, S, heads, B, (uint64_t)s_s * 2, (uint64_t)s_h * 2, (uint64_t)s_b * 2, 64, 128);
}

bool layout_ok(const void *p, long long sb, long long sh, long long ss) {
  return p && ((uintptr_t)p % 16 == 0) && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0 && ss > 0 && sh > 0 && sb >= 0;
}
}  // namespace

bool attn_tc_supported(size_t B, size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st, b200_dtype dt,
                       const void *Q, const void *K, const void *V, const void *O) {
  if (dt != B200_BF16 || (hd != 64 && hd != 128) || B == 0 || S == 0 || nKV == 0 || nH % nKV) return false;
  if (B > 65535 || nH > 65535) return false;
  return layout_ok(Q, st.q_b, st.q_h, st.q_s) && layout_ok(K, st.k_b, st.k_h, st.k_s) &&
         layout_ok(V, st.v_b, st.v_h, st.v_s) && layout_ok(O, st.o_b, st.o_h, st.o_s);
}

template <int HD>
static int fwd_launch_t(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                        size_t nH, size_t nKV, size_t S, const AttnStrides &st) {
  CUtensorMap mq, mk, mv;
  if (make_map_4d(&mq, Q, HD, S, nH, B, st.q_s, st.q_h, st.q_b) || make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) ||
      make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
  constexpr int smem = 5 * 128 * HD * 2 + 32768 + 1024 + 256;
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  dim3 grid((unsigned)((S + TQ - 1) / TQ), (unsigned)nH, (unsigned)B);
  attn_fwd_tc_kernel<HD><<<grid, FWD_THREADS, smem, ctx->stream>>>(mq, mk, mv, (bf16 *)O, lse, (int)nH, (int)nKV, (int)S, st.o_b, st.o_h,
                                                                  st.o_s, 1.0f / sqrtf((float)HD), ctx->dev_status);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

int attn_fwd_tc_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                       size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st) {
  return hd == 128 ? fwd_launch_t<128>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st) : fwd_launch_t<64>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st);
}

template <int HD>
static int bwd_launch_t(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                        const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                        const AttnStrides &st, const AttnStrides &gst) {
  const size_t rows = B * nH * S;
  // scratch: D [rows] fp32, dQ accumulator [rows, HD] fp32
  float *scr = (float *)b200_scratch(ctx, (rows + rows * HD) * sizeof(float) + 256);
  if (!scr) return B200_ERR_NOMEM;
  float *Dsum = scr, *dQacc = scr + ((rows + 63) / 64) * 64;
  B200_CUDA(ctx, cudaMemsetAsync(dQacc, 0, rows * HD * sizeof(float), ctx->stream));
  {
    size_t blocks = (rows + 7) / 8, cap = (size_t)ctx->sm_count * 16;
    attn_dsum_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>((const bf16 *)O, (const bf16 *)dO, Dsum, (int)B, (int)nH, (int)S, HD,
                                                                                  st.o_b, st.o_h, st.o_s, st.o_b, st.o_h, st.o_s);
    B200_LAUNCHED(ctx);
  }
  CUtensorMap mq, mk, mv, mdo;
  if (make_map_4d(&mq, Q, HD, S, nH, B, st.q_s, st.q_h, st.q_b) || make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) ||
      make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b) || make_map_4d(&mdo, dO, HD, S, nH, B, st.o_s, st.o_h, st.o_b))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
  constexpr int smem = 4 * 128 * HD * 2 + 2 * 32768 + 1024 + 256;
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  dim3 grid((unsigned)((S + TK - 1) / TK), (unsigned)nKV, (unsigned)B);
  attn_bwd_tc_kernel<HD><<<grid, FWD_THREADS, smem, ctx->stream>>>(mq, mk, mv, mdo, lse, Dsum, dQacc, (bf16 *)dK, (bf16 *)dV, (int)nH, (int)nKV,
                                                                  (int)S, gst.k_b, gst.k_h, gst.k_s, gst.v_b, gst.v_h, gst.v_s,
                                                                  1.0f / sqrtf((float)HD), ctx->dev_status);
  B200_LAUNCHED(ctx);
  {
    size_t items = rows * (HD / 8), blocks = (items + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    attn_dq_store_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(dQacc, (bf16 *)dQ, (int)B, (int)nH, (int)S, HD, gst.q_b, gst.q_h, gst.q_s);
    B200_LAUNCHED(ctx);
  }
  return B200_OK;
}

int attn_bwd_tc_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                       const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                       size_t hd, const AttnStrides &st, const AttnStrides &gst) {
  return hd == 128 ? bwd_launch_t<128>(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, st, gst)
                   : bwd_launch_t<64>(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, st, gst);
}
