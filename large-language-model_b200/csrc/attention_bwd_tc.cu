// Causal grouped-query attention backward on the sm_100a tensor cores, bf16 operands, fp32
// accumulation, head_dim 64 or 128.  Replaces metal_bridge::fused_attn_bwd
// (cpp/include/gpu_kernel/MetalBridge.hpp:54-57); maths of cpp/src/Attention.cpp:292-348.
//
// One CTA per (128-key tile j, kv head, batch) owns dK_j and dV_j in tensor memory and loops
// over the G = nH/nKV query heads of its kv head and the query tiles i >= j:
//     S = Q_i K_j^T,  dP = dO_i V_j^T            (tensor cores -> tensor memory)
//     P = exp(S*scale - lse), dS = P*(dP - D)*scale   (CUDA cores, two threads per query row;
//                                                 P, dS written bf16 / 128-byte swizzled to shared)
//     dV_j += P^T dO_i,  dK_j += dS^T Q_i,  dQ_t = dS K_j     (tensor cores)
//   dQ_t is staged in shared memory (the P/dS buffers, free by then) and added to an fp32 dQ
//   accumulator with TMA reduce-add, so nothing in the kernel issues per-element atomics and the
//   owners of different key tiles never race on dK/dV.  The same shared-memory tiles serve as
//   K-major and MN-major operands (only the descriptors differ), so no transposes are stored.
//   P is recomputed from the forward's log-sum-exp; D = rowsum(dO * O) is a pre-pass.
#include "attention_tc.cuh"

using namespace attn;

namespace {

struct BwdShared {
  uint64_t kv_full, qdo_full, qdo_empty, s_full, dp_full, pds_full, dq_full, dq_consumed, stage_ready, stage_free, done;
  uint32_t tmem_base;
  int abort_flag;
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_dq, const float *__restrict__ lse,
                   const float *__restrict__ Dsum, bf16 *__restrict__ dK, bf16 *__restrict__ dV, int nH, int nKV, int S,
                   long long dk_b, long long dk_h, long long dk_s, long long dv_b, long long dv_h, long long dv_s,
                   float scale, int *status, const float *__restrict__ rope_cos, const float *__restrict__ rope_sin) {
  constexpr int TILE_BYTES = 128 * HD * 2;
  constexpr int CH = HD / 64;                          // 32-column chunks of the head_dim per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sK = smem, *sV = sK + TILE_BYTES, *sQ = sV + TILE_BYTES, *sdO = sQ + TILE_BYTES, *sP = sdO + TILE_BYTES,
          *sdS = sP + 32768;
  BwdShared *sh = (BwdShared *)(sdS + 32768);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (S + TQ - 1) / TQ;
  // x = (batch, kv head) fastest, y = key tile: the heaviest key tiles (small j) are dispatched first
  const int j = blockIdx.y, kvh = blockIdx.x % nKV, b = blockIdx.x / nKV;
  const int G = nH / nKV;
  const int n_steps = G * (n_t - j);                  // (head in group) x (query tiles j..n_t-1)
  volatile int *abort_flag = &sh->abort_flag;
  // tensor memory: [0,128) S then dQ_t | [128,256) dP | [256,256+HD) dV | [384,384+HD) dK
  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->kv_full, 1); tc::mbar_init(&sh->qdo_full, 1); tc::mbar_init(&sh->qdo_empty, 1);
    tc::mbar_init(&sh->s_full, 1); tc::mbar_init(&sh->dp_full, 1); tc::mbar_init(&sh->pds_full, COMPUTE_WARPS);
    tc::mbar_init(&sh->dq_full, 1); tc::mbar_init(&sh->dq_consumed, COMPUTE_WARPS);
    tc::mbar_init(&sh->stage_ready, COMPUTE_WARPS); tc::mbar_init(&sh->stage_free, 1); tc::mbar_init(&sh->done, 1);
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == MMA_WARP) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      tc::mbar_expect_tx(&sh->kv_full, 2 * TILE_BYTES);
      load_tile<HD>(sK, &map_k, j * TK, kvh, b, &sh->kv_full);
      load_tile<HD>(sV, &map_v, j * TK, kvh, b, &sh->kv_full);
      bool ok = true;
      auto load_qdo = [&](int st) {
        const int h = kvh * G + st / (n_t - j), i = j + st % (n_t - j);
        tc::mbar_expect_tx(&sh->qdo_full, 2 * TILE_BYTES);
        load_tile<HD>(sQ, &map_q, i * TQ, h, b, &sh->qdo_full);
        load_tile<HD>(sdO, &map_do, i * TQ, h, b, &sh->qdo_full);
      };
      if (n_steps > 0) load_qdo(0);
      for (int st = 0; st < n_steps && ok; ++st) {
        const int h = kvh * G + st / (n_t - j), i = j + st % (n_t - j);
        // Q/dO of the next step as soon as this step's dV/dK products have read the current ones
        if (st + 1 < n_steps) {
          if (!tc::mbar_wait(&sh->qdo_empty, st & 1, status, abort_flag, 301)) { ok = false; break; }
          load_qdo(st + 1);
        }
        // dQ_t of this step: staged in the P/dS buffers by the compute warps -> reduce-add into global
        if (!tc::mbar_wait(&sh->stage_ready, st & 1, status, abort_flag, 310)) { ok = false; break; }
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) tma_reduce_add_3d(&map_dq, sP + c * 16384, c * 32, i * TQ, b * nH + h);
        bulk_commit();
        bulk_wait_read0();                              // shared memory may be overwritten again
        tc::mbar_arrive(&sh->stage_free);
      }
      bulk_wait0();
      if (*abort_flag) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 128, false, false);   // S, dP
      constexpr uint32_t idesc_kv = tc::make_idesc_bf16(128, HD, true, true);     // dV, dK
      constexpr uint32_t idesc_dq = tc::make_idesc_bf16(128, HD, false, true);    // dQ_t
      const uint32_t k_addr = tc::smem_u32(sK), v_addr = tc::smem_u32(sV), q_addr = tc::smem_u32(sQ),
                     do_addr = tc::smem_u32(sdO), p_addr = tc::smem_u32(sP), ds_addr = tc::smem_u32(sdS);
      bool ok = tc::mbar_wait(&sh->kv_full, 0, status, abort_flag, 302);
      for (int st = 0; st < n_steps && ok; ++st) {
        const uint32_t ph = st & 1;
        if (!tc::mbar_wait(&sh->qdo_full, ph, status, abort_flag, 303)) { ok = false; break; }
        if (st > 0 && !tc::mbar_wait(&sh->dq_consumed, (st - 1) & 1, status, abort_flag, 304)) { ok = false; break; }
        tc::tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) tc::umma_ss(t_s, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->s_full);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) tc::umma_ss(t_dp, desc_kmajor(do_addr, k), desc_kmajor(v_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->dp_full);
        if (!tc::mbar_wait(&sh->pds_full, ph, status, abort_flag, 305)) { ok = false; break; }
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
    // ---- compute warps: two threads per query row, 64 key columns each -----------------------
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
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
      const int kc0 = j * TK + half * 64;
      // the previous step's dQ_t staging (in sP/sdS) must have been read out by the TMA engine
      if (st > 0 && !tc::mbar_wait(&sh->stage_free, (st - 1) & 1, status, abort_flag, 311)) { ok = false; break; }
      if (!tc::mbar_wait(&sh->s_full, ph, status, abort_flag, 306)) { ok = false; break; }
      if (!tc::mbar_wait(&sh->dp_full, ph, status, abort_flag, 307)) { ok = false; break; }
      tc::tc_fence_after();
      // P and dS for this thread's 64 key columns; tiles below the diagonal with all rows valid (almost all of them)
      // take the path without per-element bound checks
      auto p_and_ds = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[32], dv[32];
          tc::tmem_ld_32x32(t_s + lane_base + half * 64 + c * 32, sv);
          tc::tmem_ld_32x32(t_dp + lane_base + half * 64 + c * 32, dv);
          tc::tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float p[8], ds[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              float e = fast_exp2(__uint_as_float(sv[u * 8 + x]) * sl2 - L2);
              if constexpr (MASKED) {
                if (!valid || (diag && (kc0 + c * 32 + u * 8 + x > q_idx))) e = 0.f;
              }
              p[x] = e;
              ds[x] = e * (__uint_as_float(dv[u * 8 + x]) - Dr) * scale;
            }
            uint4 w;
            w.x = pack_bf16(p[0], p[1]); w.y = pack_bf16(p[2], p[3]); w.z = pack_bf16(p[4], p[5]); w.w = pack_bf16(p[6], p[7]);
            *reinterpret_cast<uint4 *>(sP + swz_unit(r, half * 8 + c * 4 + u)) = w;
            w.x = pack_bf16(ds[0], ds[1]); w.y = pack_bf16(ds[2], ds[3]); w.z = pack_bf16(ds[4], ds[5]); w.w = pack_bf16(ds[6], ds[7]);
            *reinterpret_cast<uint4 *>(sdS + swz_unit(r, half * 8 + c * 4 + u)) = w;
          }
        }
      };
      if (diag || (i + 1) * TQ > S) p_and_ds(std::true_type{}); else p_and_ds(std::false_type{});
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->pds_full);
      // dQ_t: this thread's half of the head_dim -> fp32 staging tile [HD/32 chunks][128 rows][32 fp32]
      if (!tc::mbar_wait(&sh->dq_full, ph, status, abort_flag, 308)) { ok = false; break; }
      tc::tc_fence_after();
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int chunk = half * CH + c;
        uint32_t v[32];
        tc::tmem_ld_32x32(t_s + lane_base + chunk * 32, v);
        tc::tmem_ld_wait();
        uint8_t *dst = sP + chunk * 16384 + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4 *>(dst + ((u ^ (r & 7)) << 4)) = make_uint4(v[u * 4], v[u * 4 + 1], v[u * 4 + 2], v[u * 4 + 3]);
      }
      tc::tc_fence_before();
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) { tc::mbar_arrive(&sh->dq_consumed); tc::mbar_arrive(&sh->stage_ready); }
    }
    // dK / dV of this key tile: rows = keys, this thread's half of the head_dim
    if (ok && tc::mbar_wait(&sh->done, 0, status, abort_flag, 309)) {
      tc::tc_fence_after();
      const int key = j * TK + r;
      bf16 *dkrow = dK + (long long)b * dk_b + (long long)kvh * dk_h + (long long)key * dk_s;
      bf16 *dvrow = dV + (long long)b * dv_b + (long long)kvh * dv_h + (long long)key * dv_s;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int col = (half * CH + c) * 32;
        uint32_t a[32], g[32];
        tc::tmem_ld_32x32(t_dk + lane_base + col, a);
        tc::tmem_ld_32x32(t_dv + lane_base + col, g);
        tc::tmem_ld_wait();
        if (key < S) {
          if (rope_cos != nullptr) {
            // gradient of the rotary embedding (inverse rotation, cpp/src/Positional.cpp:207-231) on dK, position = key
            const float *cp = rope_cos + (size_t)key * (HD / 2) + (col >> 1), *sp = rope_sin + (size_t)key * (HD / 2) + (col >> 1);
#pragma unroll
            for (int p2 = 0; p2 < 16; ++p2) {
              const float x0 = __uint_as_float(a[2 * p2]), x1 = __uint_as_float(a[2 * p2 + 1]), cc = __ldg(cp + p2), ss = __ldg(sp + p2);
              a[2 * p2] = __float_as_uint(x0 * cc + x1 * ss);
              a[2 * p2 + 1] = __float_as_uint(-x0 * ss + x1 * cc);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(a[u * 8 + 0]), __uint_as_float(a[u * 8 + 1]));
            w.y = pack_bf16(__uint_as_float(a[u * 8 + 2]), __uint_as_float(a[u * 8 + 3]));
            w.z = pack_bf16(__uint_as_float(a[u * 8 + 4]), __uint_as_float(a[u * 8 + 5]));
            w.w = pack_bf16(__uint_as_float(a[u * 8 + 6]), __uint_as_float(a[u * 8 + 7]));
            *reinterpret_cast<uint4 *>(dkrow + col + u * 8) = w;
            w.x = pack_bf16(__uint_as_float(g[u * 8 + 0]), __uint_as_float(g[u * 8 + 1]));
            w.y = pack_bf16(__uint_as_float(g[u * 8 + 2]), __uint_as_float(g[u * 8 + 3]));
            w.z = pack_bf16(__uint_as_float(g[u * 8 + 4]), __uint_as_float(g[u * 8 + 5]));
            w.w = pack_bf16(__uint_as_float(g[u * 8 + 6]), __uint_as_float(g[u * 8 + 7]));
            *reinterpret_cast<uint4 *>(dvrow + col + u * 8) = w;
          }
        }
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

// D[b,h,s] = sum_d dO * O (and, when asked, lse * log2(e) beside it).  Eight lanes per (b,s,h) row (16-byte loads for head_dim 128), rows visited with the head
// index fastest so that a token-major tensor is read as one contiguous stream; two rows per lane group in flight.
template <int HD>
__global__ void __launch_bounds__(256)
attn_dsum_kernel(const bf16 *__restrict__ O, const bf16 *__restrict__ dO, float *__restrict__ D, int B, int nH, int S,
                 long long o_b, long long o_h, long long o_s, const float *__restrict__ lse, float *__restrict__ lse2,
                 float *__restrict__ zero_acc) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VEC = HD / 8;                       // elements per lane: 16 (32 bytes) or 8 (16 bytes)
  typedef typename std::conditional<VEC == 16, uint4, uint2>::type Raw;   // loaded in 16- or 8-byte pieces
  constexpr int PIECES = VEC * 2 / (int)sizeof(Raw);
  const int sub = threadIdx.x & 7;
  const long long rows = (long long)B * nH * S;
  const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3, n_groups = ((long long)gridDim.x * blockDim.x) >> 3;
  auto dot_row = [&](long long r, Raw (&a)[PIECES], Raw (&c)[PIECES]) {
    const int h = (int)(r % nH), s = (int)((r / nH) % S), b = (int)(r / ((long long)nH * S));
    const long long off = b * o_b + h * o_h + (long long)s * o_s + sub * VEC;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      a[p] = *reinterpret_cast<const Raw *>(O + off + p * (sizeof(Raw) / 2));
      c[p] = *reinterpret_cast<const Raw *>(dO + off + p * (sizeof(Raw) / 2));
    }
  };
  auto reduce_store = [&](long long r, const Raw (&a)[PIECES], const Raw (&c)[PIECES]) {
    float acc = 0.f;
    const __nv_bfloat162 *pa = reinterpret_cast<const __nv_bfloat162 *>(a), *pc = reinterpret_cast<const __nv_bfloat162 *>(c);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pc[i]);
      acc += x.x * y.x + x.y * y.y;
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (r < rows) {
      const int h = (int)(r % nH), s = (int)((r / nH) % S), b = (int)(r / ((long long)nH * S));
      const long long at = ((long long)b * nH + h) * S + s;
      if (sub == 0) {
        D[at] = acc;
        if (lse2) lse2[at] = lse[at] * LOG2E;           // the row's log-sum-exp in base-2 units for the second backward form
      }
      if (zero_acc) {
        // the row of the fp32 dQ accumulator starts at zero: cleared here, 64 bytes per lane, instead of by a memset of
        // its own in front of this kernel
        float4 *z = reinterpret_cast<float4 *>(zero_acc + at * HD + sub * VEC);
#pragma unroll
        for (int p = 0; p < VEC / 4; ++p) z[p] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };
  for (long long r0 = group * 2; r0 < rows; r0 += n_groups * 2) {      // the shuffles need every lane: rows past the end are clamped
    const long long r1 = r0 + 1 < rows ? r0 + 1 : r0;
    Raw a0[PIECES], c0[PIECES], a1[PIECES], c1[PIECES];
    dot_row(r0, a0, c0);
    dot_row(r1, a1, c1);
    reduce_store(r0, a0, c0);
    reduce_store(r0 + 1, a1, c1);
  }
}
// fp32 [B,nH,S,hd] accumulator -> strided bf16 dQ
// tile_stride > 0: acc holds one slice per 128-key tile (slice j covers the queries from 128 j on); they are added in order.
__global__ void attn_dq_store_kernel(const float *__restrict__ acc, bf16 *__restrict__ dQ, int B, int nH, int S,
                                     int hd, long long q_b, long long q_h, long long q_s,
                                     const float *__restrict__ rope_cos, const float *__restrict__ rope_sin, float mul,
                                     long long tile_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)B * nH * S * (hd / 8);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(idx % (hd / 8)); size_t r = idx / (hd / 8);
    const int s = (int)(r % S); r /= S;
    const int h = (int)(r % nH), b = (int)(r / nH);
    float4 x = *reinterpret_cast<const float4 *>(acc + idx * 8), y = *reinterpret_cast<const float4 *>(acc + idx * 8 + 4);
    if (tile_stride) {
      for (int t = 1; t <= s / TK; ++t) {
        const float4 x2 = *reinterpret_cast<const float4 *>(acc + t * tile_stride + idx * 8), y2 = *reinterpret_cast<const float4 *>(acc + t * tile_stride + idx * 8 + 4);
        x.x += x2.x; x.y += x2.y; x.z += x2.z; x.w += x2.w; y.x += y2.x; y.y += y2.y; y.z += y2.z; y.w += y2.w;
      }
    }
    x.x *= mul; x.y *= mul; x.z *= mul; x.w *= mul; y.x *= mul; y.y *= mul; y.z *= mul; y.w *= mul;   // 1, or the softmax scale
    if (rope_cos != nullptr) {   // gradient of the rotary embedding on dQ: inverse rotation at position s
      const float4 c = *reinterpret_cast<const float4 *>(rope_cos + (size_t)s * (hd / 2) + u * 4);
      const float4 n = *reinterpret_cast<const float4 *>(rope_sin + (size_t)s * (hd / 2) + u * 4);
      float4 a = x, d = y;
      x.x = a.x * c.x + a.y * n.x; x.y = -a.x * n.x + a.y * c.x; x.z = a.z * c.y + a.w * n.y; x.w = -a.z * n.y + a.w * c.y;
      y.x = d.x * c.z + d.y * n.z; y.y = -d.x * n.z + d.y * c.z; y.z = d.z * c.w + d.w * n.w; y.w = -d.z * n.w + d.w * c.w;
    }
    uint4 w;
    w.x = pack_bf16(x.x, x.y); w.y = pack_bf16(x.z, x.w); w.z = pack_bf16(y.x, y.y); w.w = pack_bf16(y.z, y.w);
    *reinterpret_cast<uint4 *>(dQ + b * q_b + h * q_h + (long long)s * q_s + u * 8) = w;
  }
}

}  // namespace

bool attn_bwd2_supported(size_t S, size_t hd);
int attn_bwd2_tc_run(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *dO, const float *lse2, const float *Dsum,
                     float *dQacc, long long dq_tile_stride, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S, const AttnStrides &st,
                     const AttnStrides &gst, const float *rope_cos, const float *rope_sin);

namespace {
template <int HD>
int bwd_launch_t(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                 const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                 const AttnStrides &st, const AttnStrides &gst, const float *rope_cos, const float *rope_sin) {
  const size_t rows = B * nH * S;
  // scratch: D [rows] fp32, dQ accumulator [rows, HD] fp32 (zeroed here, added to by TMA reduce)
  const size_t d_elems = ((rows + 63) / 64) * 64;
  const bool second_form = HD == 128 && ctx->attn_bwd2 && attn_bwd2_supported(S, HD);
  // bit-reproducible form (second form only): one dQ slice per key tile instead of one accumulator all tiles add to
  const size_t dq_slices = (ctx->deterministic && second_form) ? (S + TK - 1) / TK : 1;
  const long long dq_tile_stride = dq_slices > 1 ? (long long)(rows * HD) : 0;
  float *scr = (float *)b200_scratch(ctx, (2 * d_elems + dq_slices * rows * HD) * sizeof(float));
  if (!scr) return B200_ERR_NOMEM;
  float *Dsum = scr, *lse2 = scr + d_elems, *dQacc = scr + 2 * d_elems;
  {
    size_t blocks = (rows + 63) / 64, cap = (size_t)ctx->sm_count * 16;      // 32 lane groups x 2 rows per block pass
    B200_CUDA(ctx, launch_k(ctx, attn_dsum_kernel<HD>, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0, 0, (const bf16 *)O, (const bf16 *)dO, Dsum,
                            (int)B, (int)nH, (int)S, st.o_b, st.o_h, st.o_s, lse, second_form ? lse2 : (float *)nullptr, dQacc));
    B200_LAUNCHED(ctx);
  }
  if (second_form) {
    int rc = attn_bwd2_tc_run(ctx, Q, K, V, dO, lse2, Dsum, dQacc, dq_tile_stride, dK, dV, B, nH, nKV, S, st, gst, rope_cos, rope_sin);
    if (rc != B200_OK) return rc;
  } else {
    CUtensorMap mq, mk, mv, mdo, mdq;
    if (make_map_4d(&mq, Q, HD, S, nH, B, st.q_s, st.q_h, st.q_b) || make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) ||
        make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b) || make_map_4d(&mdo, dO, HD, S, nH, B, st.o_s, st.o_h, st.o_b) ||
        tc_make_map_f32_3d(&mdq, dQacc, HD, S, B * nH, (uint64_t)HD * 4, (uint64_t)S * HD * 4, 32, 128))
      return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
    constexpr int smem = 4 * 128 * HD * 2 + 2 * 32768 + 1024 + (int)sizeof(BwdShared);
    static bool attr = false;
    if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
    dim3 grid((unsigned)(nKV * B), (unsigned)((S + TK - 1) / TK), 1);
    attn_bwd_tc_kernel<HD><<<grid, THREADS, smem, ctx->stream>>>(mq, mk, mv, mdo, mdq, lse, Dsum, (bf16 *)dK, (bf16 *)dV, (int)nH, (int)nKV, (int)S,
                                                                gst.k_b, gst.k_h, gst.k_s, gst.v_b, gst.v_h, gst.v_s, 1.0f / sqrtf((float)HD),
                                                                ctx->dev_status, rope_cos, rope_sin);
    B200_LAUNCHED(ctx);
  }
  {
    size_t items = rows * (HD / 8), blocks = (items + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    B200_CUDA(ctx, launch_k(ctx, attn_dq_store_kernel, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0, 0, (const float *)dQacc, (bf16 *)dQ, (int)B, (int)nH,
                            (int)S, (int)HD, gst.q_b, gst.q_h, gst.q_s, rope_cos, rope_sin, second_form ? 1.0f / sqrtf((float)HD) : 1.0f, dq_tile_stride));
    B200_LAUNCHED(ctx);
  }
  return B200_OK;
}
}  // namespace

int attn_bwd_tc_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *O, const void *dO,
                       const float *lse, void *dQ, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S,
                       size_t hd, const AttnStrides &st, const AttnStrides &gst, const float *rope_cos,
                       const float *rope_sin) {
  return hd == 128 ? bwd_launch_t<128>(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, st, gst, rope_cos, rope_sin)
                   : bwd_launch_t<64>(ctx, Q, K, V, O, dO, lse, dQ, dK, dV, B, nH, nKV, S, st, gst, rope_cos, rope_sin);
}
