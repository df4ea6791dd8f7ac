// Causal grouped-query attention forward, second tensor-core form: one CTA works on TWO adjacent 128-query tiles
// of a head at once and keeps both the probabilities and the output accumulators in tensor memory.
// Replaces metal_bridge::flash_attn_fwd (cpp/include/gpu_kernel/MetalBridge.hpp:49-51); maths of
// cpp/src/Attention.cpp:236-280.  Same interface and numerics contract as attention_tc.cu.
//
// Why: with one query tile per CTA the tensor cores wait for the softmax of every key tile and back.  Here
//   * two independent softmax streams (query tiles A and B, one warpgroup each, one thread per query row, so no
//     cross-thread exchange) alternate on the tensor pipe: while A's scores are exponentiated, B's products run;
//   * P is written back over the scores in tensor memory as packed bf16 and is the A operand of the P V product
//     (tcgen05.mma with A from tensor memory): no shared-memory round trip, no proxy fence;
//   * O is accumulated by the MMA itself in tensor memory; it is rescaled only when a row's running maximum grew by
//     more than 2^8 since the value in use (the stale maximum stays exact: numerator and denominator share it);
//   * each K / V tile is loaded once for both query tiles.
// Tensor memory: [S_A 128 | O_A 128 | S_B 128 | O_B 128] columns.  Shared memory: Q_A, Q_B, K x2, V x2.
//   warps 0-3 softmax of tile A, warps 4-7 softmax of tile B, warp 8 MMA issue, warp 9 TMA (warps 10-11 only lend registers).
// tcgen05.mma operations of one thread execute in issue order, which is what lets S(j+1) overwrite the columns that
// P(j) occupied right after the P(j) V(j) product has been issued.
#include "attention_tc.cuh"
#include <type_traits>

using namespace attn;

namespace {

struct Fwd2Shared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr float RESCALE_THRESHOLD = 8.0f;      // log2 units: P stays below 2^8
// Three warpgroups: two of softmax (one thread per query row, the row's 128 scores stay in registers between the
// maximum and the exponentials) and one holding the MMA and TMA warps, which gives most of its registers away.
constexpr int FWD2_THREADS = 384;
constexpr int REGS_SOFTMAX = 232, REGS_SERVICE = 40;
template <int N> __device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int HD>
__global__ void __launch_bounds__(FWD2_THREADS, 1)
attn_fwd2_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, bf16 *__restrict__ O, float *__restrict__ lse,
                    int nH, int nKV, int S, long long o_b, long long o_h, long long o_s, float scale, int *status) {
  pdl_launch_dependents();
  constexpr int TILE_BYTES = 128 * HD * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  uint8_t *sQ = smem, *sK = sQ + 2 * TILE_BYTES, *sV = sK + 2 * TILE_BYTES;
  Fwd2Shared *sh = (Fwd2Shared *)(sV + 2 * TILE_BYTES);
  uint8_t *stage = (uint8_t *)(sh + 1);          // 8 softmax warps x 2 KiB: transposition buffers of the output stores
  if (tc::smem_u32(smem) & 1023u) {           // swizzled tiles need 1024-byte alignment: refuse rather than corrupt
    if (threadIdx.x == 0) atomicCAS(status, 0, 298);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (S + TQ - 1) / TQ, n_pairs = (n_qt + 1) / 2;
  const int pr = n_pairs - 1 - (int)blockIdx.y;          // heaviest pairs are dispatched first
  const int qA = 2 * pr, qB = 2 * pr + 1;
  const bool validB = qB < n_qt;
  const int nA = qA + 1, nB = validB ? qB + 1 : 0, n_kt = validB ? nB : nA;   // causal: key tiles 0..q
  const int h = blockIdx.x % nH, b = blockIdx.x / nH, kvh = h / (nH / nKV);
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sh->k_full[i], 1); tc::mbar_init(&sh->k_empty[i], 1);
      tc::mbar_init(&sh->v_full[i], 1); tc::mbar_init(&sh->v_empty[i], 1);
      tc::mbar_init(&sh->s_full[i], 1); tc::mbar_init(&sh->p_full[i], 4); tc::mbar_init(&sh->o_full[i], 1);
    }
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == MMA_WARP) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  pdl_wait();                          // set-up above may overlap the previous kernel's tail; operands are touched from here on
  const uint32_t tmem_base = sh->tmem_base;

  if (warp >= 8) {
   setmaxnreg_dec<REGS_SERVICE>();
   if (warp == TMA_WARP) {
    if (lane == 0) {
      tc::mbar_expect_tx(&sh->q_full, validB ? 2 * TILE_BYTES : TILE_BYTES);
      load_tile<HD>(sQ, &map_q, qA * TQ, h, b, &sh->q_full);
      if (validB) load_tile<HD>(sQ + TILE_BYTES, &map_q, qB * TQ, h, b, &sh->q_full);
      for (int j = 0; j < n_kt; ++j) {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->k_empty[s], ph ^ 1, status, abort_flag, 221)) break;
        tc::mbar_expect_tx(&sh->k_full[s], TILE_BYTES);
        load_tile<HD>(sK + s * TILE_BYTES, &map_k, j * TK, kvh, b, &sh->k_full[s]);
        if (!tc::mbar_wait(&sh->v_empty[s], ph ^ 1, status, abort_flag, 222)) break;
        tc::mbar_expect_tx(&sh->v_full[s], TILE_BYTES);
        load_tile<HD>(sV + s * TILE_BYTES, &map_v, j * TK, kvh, b, &sh->v_full[s]);
      }
      if (*abort_flag) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = tc::make_idesc_bf16(128, HD, false, true);
      const uint32_t q_addr[2] = {tc::smem_u32(sQ), tc::smem_u32(sQ + TILE_BYTES)};
      bool ok = tc::mbar_wait(&sh->q_full, 0, status, abort_flag, 223);
      // S_X(j) = Q_X K_j^T into tile X's score columns; the K buffer is released after its last reader
      auto issue_s = [&](int X, int j) -> bool {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->k_full[s], ph, status, abort_flag, 224)) return false;
        tc::tc_fence_after();
        const uint32_t k_addr = tc::smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc::umma_ss(tmem_base + X * 256, desc_kmajor(q_addr[X], k), desc_kmajor(k_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->s_full[X]);
        const bool last_reader = X == 1 || j >= nB;      // B reads every key tile A reads, after A
        if (last_reader) tc::umma_commit(&sh->k_empty[s]);
        return true;
      };
      // O_X (+)= P_X(j) V_j with P read from tensor memory (packed bf16 over the first 64 score columns)
      auto issue_pv = [&](int X, int j) -> bool {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tc::mbar_wait(&sh->p_full[X], j & 1, status, abort_flag, 225)) return false;
        if (!tc::mbar_wait(&sh->v_full[s], ph, status, abort_flag, 226)) return false;
        tc::tc_fence_after();
        const uint32_t v_addr = tc::smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < TK / 16; ++k)
          tc::umma_ts(tmem_base + X * 256 + 128, tmem_base + X * 256 + k * 8, desc_mnmajor(v_addr, k), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        tc::umma_commit(&sh->o_full[X]);
        const bool last_reader = X == 1 || j >= nB;
        if (last_reader) tc::umma_commit(&sh->v_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0, 0);
      if (ok && validB) ok = issue_s(1, 0);
      for (int j = 0; j < n_kt && ok; ++j) {
        if (j < nA) { ok = issue_pv(0, j); if (ok && j + 1 < nA) ok = issue_s(0, j + 1); }
        if (ok && j < nB) { ok = issue_pv(1, j); if (ok && j + 1 < nB) ok = issue_s(1, j + 1); }
      }
    }
   }
  } else {
    setmaxnreg_inc<REGS_SOFTMAX>();
    // ---- softmax: warpgroup X owns query tile X, one thread per query row ------------------------------------
    const int X = warp >> 2, quarter = warp & 3;
    const int qt = X ? qB : qA, nX = X ? nB : nA;
    const int r = quarter * 32 + lane;
    const int q_idx = qt * TQ + r;
    const int q_eff = min(q_idx, S - 1);               // rows past the end behave like the last row (never stored)
    const float sl2 = scale * LOG2E;
    const uint32_t tS = tmem_base + ((uint32_t)(quarter * 32) << 16) + X * 256, tO = tS + 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nX && ok; ++j) {
      ok = tc::mbar_wait(&sh->s_full[X], j & 1, status, abort_flag, 228);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }        // the tensor-memory accesses below are warp-collective
      tc::tc_fence_after();
      const bool masked = (j == qt) || ((j + 1) * TK > S);   // diagonal tile, or keys past the end of the sequence
      const int k0 = j * TK;
      // The row's 128 scores are read once and stay in registers.  Tiles below the diagonal (almost all of them)
      // take the path without per-element bound checks.
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc::tmem_ld_32x32(tS + c * 32, v + c * 32);
      tc::tmem_ld_wait();
      if (masked) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > q_eff) v[i] = 0xff800000u;        // -inf: exp2 gives exactly 0 below
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        mx4[0] = max3(mx4[0], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        mx4[1] = max3(mx4[1], __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        mx4[2] = max3(mx4[2], __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
        mx4[3] = max3(mx4[3], __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
      }
      const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2);
      const bool need = (m_new - m_used) > RESCALE_THRESHOLD;
      if (j == 0) {
        m_used = m_new;                                  // nothing accumulated yet
      } else if (__any_sync(0xffffffffu, need)) {
        // a row of this warp outgrew the maximum in use: rescale its output accumulator in tensor memory
        // (the product of tile j-1 must have landed; the product of tile j cannot start before p_full below)
        ok = tc::mbar_wait(&sh->o_full[X], (j - 1) & 1, status, abort_flag, 229);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        tc::tc_fence_after();
        const float f = need ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tc::tmem_ld_32x32(tO + c * 32, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tc::tmem_st_32x32(tO + c * 32, o);
        }
        tc::tmem_st_wait();
        l *= f;
        if (need) m_used = m_new;
      }
      // probabilities, packed bf16 written over the first half of the score columns (all 128 were read above)
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t w[64];
#pragma unroll
      for (int i = 0; i < 128; i += 2) {
        const float e0 = fast_exp2(__uint_as_float(v[i]) * sl2 - m_used), e1 = fast_exp2(__uint_as_float(v[i + 1]) * sl2 - m_used);
        rs4[(i >> 1) & 3] += e0 + e1;
        w[i >> 1] = pack_bf16(e0, e1);
      }
      tc::tmem_st_32x32(tS, w);
      tc::tmem_st_32x32(tS + 32, w + 32);
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tc::tmem_st_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->p_full[X]);
    }
    if (ok && nX > 0) {
      ok = __all_sync(0xffffffffu, tc::mbar_wait(&sh->o_full[X], (nX - 1) & 1, status, abort_flag, 230));
      tc::tc_fence_after();
      if (ok) {
        const float inv = 1.0f / l;
        // rows of the warp: q0w .. q0w+31; whole 64-byte row segments per store instruction (see tc::stage_store_bf16)
        const int q0w = qt * TQ + quarter * 32;
        bf16 *obase = O + (long long)b * o_b + (long long)h * o_h + (long long)q0w * o_s;
        uint8_t *stg = stage + warp * 2048;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tc::tmem_ld_32x32(tO + c * 32, v);
          tc::tmem_ld_wait();
          uint4 w[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            w[u].x = pack_bf16(__uint_as_float(v[u * 8 + 0]) * inv, __uint_as_float(v[u * 8 + 1]) * inv);
            w[u].y = pack_bf16(__uint_as_float(v[u * 8 + 2]) * inv, __uint_as_float(v[u * 8 + 3]) * inv);
            w[u].z = pack_bf16(__uint_as_float(v[u * 8 + 4]) * inv, __uint_as_float(v[u * 8 + 5]) * inv);
            w[u].w = pack_bf16(__uint_as_float(v[u * 8 + 6]) * inv, __uint_as_float(v[u * 8 + 7]) * inv);
          }
          tc::stage_store_bf16(stg, lane, w, obase + c * 32, (size_t)o_s, S - q0w);
        }
        if (lse && q_idx < S) lse[((long long)b * nH + h) * S + q_idx] = (m_used + log2f(l)) * (1.0f / LOG2E);   // natural-log units
      }
      tc::tc_fence_before();
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
int fwd2_launch_t(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B, size_t nH,
                  size_t nKV, size_t S, const AttnStrides &st) {
  CUtensorMap mq, mk, mv;
  if (make_map_4d(&mq, Q, HD, S, nH, B, st.q_s, st.q_h, st.q_b) || make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) ||
      make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
  constexpr int smem = 6 * 128 * HD * 2 + (int)sizeof(Fwd2Shared) + 8 * 2048;
  static_assert(smem <= 232448, "forward attention tiles exceed the 227 KiB of shared memory per CTA");
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd2_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  const size_t n_qt = (S + TQ - 1) / TQ;
  dim3 grid((unsigned)(nH * B), (unsigned)((n_qt + 1) / 2), 1);
  B200_CUDA(ctx, launch_k(ctx, attn_fwd2_tc_kernel<HD>, grid, dim3(FWD2_THREADS), (size_t)smem, 0, mq, mk, mv, (bf16 *)O, lse, (int)nH, (int)nKV, (int)S, st.o_b,
                          st.o_h, st.o_s, 1.0f / sqrtf((float)HD), ctx->dev_status));
  B200_LAUNCHED(ctx);
  return B200_OK;
}
}  // namespace

int attn_fwd2_tc_launch(b200_ctx *ctx, const void *Q, const void *K, const void *V, void *O, float *lse, size_t B,
                        size_t nH, size_t nKV, size_t S, size_t hd, const AttnStrides &st) {
  return hd == 128 ? fwd2_launch_t<128>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st) : fwd2_launch_t<64>(ctx, Q, K, V, O, lse, B, nH, nKV, S, st);
}
