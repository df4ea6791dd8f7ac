// Causal grouped-query attention backward, second tensor-core form (head_dim 128): keys in the tensor-memory lanes,
// 64-query steps handled in pairs.  Replaces metal_bridge::fused_attn_bwd
// (cpp/include/gpu_kernel/MetalBridge.hpp:54-57); maths of cpp/src/Attention.cpp:292-348.  Same contract as
// attention_bwd_tc.cu, which stays for head_dim 64 and for sequence lengths that are not a multiple of 4.
//
// One CTA per (128-key tile j, kv head, batch) owns dK_j and dV_j in tensor memory and walks the query heads of
// its kv head and their 64-query sub-tiles t >= 2j.  Everything is computed TRANSPOSED, keys as rows:
//     S^T  = K_j Q_t^T          dP^T = V_j dO_t^T                    (128 keys x 64 queries each, tensor memory)
//     P^T  = exp(S^T*scale - lse[q]),  dS^T = P^T (dP^T - D[q])         (CUDA cores, two threads per key row; the factor
//                                                                    `scale` of dS is applied to dK at the end and to dQ by
//                                                                    the kernel that stores it; lse comes in base-2 units)
//     dV_j += P^T dO_t          dK_j += dS^T Q_t                     (P^T, dS^T are read FROM tensor memory: they are
//                                                                    written back over S^T / dP^T as packed bf16)
//     dQ_t^T = K_j^T dS^T                                            (dS^T also goes to shared memory, as the B operand)
// The transposition is what lets P and dS feed the two accumulating products without a shared-memory round trip, and
// with 64-query steps the scores of TWO steps fit beside the dK / dV accumulators: while the tensor cores run the
// products of the pair's first step, the CUDA cores turn the second step's scores into P and dS.
//   warps 0-7 compute P^T / dS^T (and the final dK / dV rows), warp 8 issues MMAs, warp 9 loads Q_t / dO_t and the
//   row statistics four steps ahead, warps 10-13 copy each finished dQ_t^T out of tensor memory (so that the slot is
//   free for step s+2 without the compute warps being involved) and add it to the global accumulator straight from
//   registers: a warp's 32 head_dim values of one query are one 128-byte line, so each red instruction is coalesced.
//   (Shared memory bandwidth is what bounds this kernel - MMA operands, TMA writes and ordinary stores share it - so
//   dQ does not take the detour through a staging buffer and a TMA reduce-add.)
//   tensor memory: S^T x 2 steps | dP^T x 2 steps (64 columns each) | dV 128 | dK 128; dQ_t^T lands in the step's dP^T
//   columns.  The scores of a pair of steps are one N = 128 product each (S^T, dP^T); everything else runs per step.
//   shared memory: K, V, (Q, dO, lse and D of the step's queries) x 4, dS^T x 2 = 226 KiB.
// dQ goes into the fp32 accumulator [B*nH*S][head_dim] that the first form fills with TMA reduce-adds.
#include "attention_tc.cuh"

using namespace attn;

namespace {

constexpr int HD = 128;
constexpr int SQ = 64;                                  // queries per step
constexpr int KV_TILE = 128 * HD * 2;                   // 32 KiB
constexpr int Q_TILE = SQ * HD * 2;                     // 16 KiB
constexpr int DS_TILE = 128 * SQ * 2;                   // 16 KiB: [128 keys][64 queries] bf16, one swizzled chunk
constexpr int STAT = 2 * SQ * 4;                        // lse and D of the 64 queries of a step
constexpr int NQ = 4;                                   // Q / dO sub-tiles in flight: two pairs of consecutive steps
constexpr int PAIR_TILE = 2 * Q_TILE;                   // [128 rows: step 2p, step 2p+1][128 columns] as two 64-column chunks
constexpr int DQ_WARPS = 4, BWD2_THREADS = THREADS + 32 * DQ_WARPS;         // warps 10..13 add dQ to global memory

struct Bwd2Shared {
  uint64_t kv_full, qdo_full[NQ], qdo_empty[NQ], s_full[2], sdp_full[2], pds_full[2], dq_full[2], dq_consumed[2], done;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}

// A shared-memory operand descriptor kept as two words: only the low one (the start address field) changes from one MMA
// to the next, so that the issuing thread spends one add per operand and MMA.
struct Desc { uint32_t lo, hi; };
__device__ __forceinline__ Desc desc_of(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  const uint64_t d = tc::make_smem_desc(addr, lbo, sbo);
  return {(uint32_t)d, (uint32_t)(d >> 32)};
}
template <bool ACC>
__device__ __forceinline__ void mma_ss(uint32_t d, Desc a, uint32_t a_off, Desc b, uint32_t b_off, uint32_t idesc) {
  asm volatile("{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
               ::"r"(d), "r"(a.lo + (a_off >> 4)), "r"(a.hi), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, Desc b, uint32_t b_off, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .b64 db;\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
               ::"r"(d), "r"(a_tmem), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "r"(acc) : "memory");
}
// [64 rows x 128 columns] bf16 sub-tile: half of the rows of a pair tile, whose two 64-column chunks are 16 KiB apart
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(tc::smem_u32(dst)), "l"(src), "r"(bytes), "r"(tc::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void load_subtile(uint8_t *dst, const CUtensorMap *map, int row0, int head, int batch, uint64_t *bar) {
  tma_load_4d(dst, map, 0, row0, head, batch, bar);
  tma_load_4d(dst + 16384, map, 64, row0, head, batch, bar);
}

__global__ void __launch_bounds__(BWD2_THREADS, 1)
attn_bwd2_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    float *__restrict__ dQacc, long long dq_tile_stride, const float *__restrict__ lse2,
                    const float *__restrict__ Dsum, bf16 *__restrict__ dK, bf16 *__restrict__ dV, int nH, int nKV, int S,
                    long long dk_b, long long dk_h, long long dk_s, long long dv_b, long long dv_h, long long dv_s,
                    float scale, int *status, const float *__restrict__ rope_cos, const float *__restrict__ rope_sin) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  uint8_t *sK = smem, *sV = sK + KV_TILE, *sQ = sV + KV_TILE, *sdO = sQ + NQ * Q_TILE, *sdS = sdO + NQ * Q_TILE,
          *sStat = sdS + 2 * DS_TILE;
  Bwd2Shared *sh = (Bwd2Shared *)(sStat + NQ * STAT);
  if (tc::smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 297);
    return;
  }
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_sub = (S + SQ - 1) / SQ;
  const int j = blockIdx.y, kvh = blockIdx.x % nKV, b = blockIdx.x / nKV;
  const int G = nH / nKV;
  const int per_head = n_sub - 2 * j;                  // query sub-tiles 2j .. n_sub-1 see this key tile
  const int n_steps = G * per_head;
  volatile int *abort_flag = &sh->abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->kv_full, 1); tc::mbar_init(&sh->done, 1);
    for (int i = 0; i < NQ; ++i) { tc::mbar_init(&sh->qdo_full[i], 1); tc::mbar_init(&sh->qdo_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sh->s_full[i], 1); tc::mbar_init(&sh->sdp_full[i], 1); tc::mbar_init(&sh->pds_full[i], COMPUTE_WARPS);
      tc::mbar_init(&sh->dq_full[i], 1); tc::mbar_init(&sh->dq_consumed[i], DQ_WARPS);
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
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 384;
  auto step_head = [&](int st) { return kvh * G + st / per_head; };
  auto step_q0 = [&](int st) { return (2 * j + st % per_head) * SQ; };

  if (warp == TMA_WARP) {
    if (lane == 0) {
      tc::mbar_expect_tx(&sh->kv_full, 2 * KV_TILE);
      load_tile<HD>(sK, &map_k, j * TK, kvh, b, &sh->kv_full);
      load_tile<HD>(sV, &map_v, j * TK, kvh, b, &sh->kv_full);
      auto load_qdo = [&](int st) {
        const int s = st % NQ, q0 = step_q0(st), h = step_head(st);
        const uint32_t stat_bytes = (uint32_t)min(SQ, S - q0) * 4;      // a multiple of 16: S is a multiple of 4
        const long long stat_off = ((long long)b * nH + h) * S + q0;
        tc::mbar_expect_tx(&sh->qdo_full[s], 2 * Q_TILE + 2 * stat_bytes);
        const int sub_off = ((st >> 1) & 1) * PAIR_TILE + (st & 1) * 8192;
        load_subtile(sQ + sub_off, &map_q, q0, h, b, &sh->qdo_full[s]);
        load_subtile(sdO + sub_off, &map_do, q0, h, b, &sh->qdo_full[s]);
        bulk_load_1d(sStat + s * STAT, lse2 + stat_off, stat_bytes, &sh->qdo_full[s]);
        bulk_load_1d(sStat + s * STAT + SQ * 4, Dsum + stat_off, stat_bytes, &sh->qdo_full[s]);
      };
      for (int st = 0; st < NQ && st < n_steps; ++st) load_qdo(st);
      for (int st = 0; st + NQ < n_steps; ++st) {        // the buffers of step st are free once its dK / dV products have run
        if (!tc::mbar_wait(&sh->qdo_empty[st % NQ], (st / NQ) & 1, status, abort_flag, 332)) break;
        load_qdo(st + NQ);
      }
      if (*abort_flag) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 2 * SQ, false, false);   // S^T, dP^T: keys x queries of a pair
      constexpr uint32_t idesc_kv = tc::make_idesc_bf16(128, HD, false, true);    // dV, dK: A from tensor memory
      constexpr uint32_t idesc_dq = tc::make_idesc_bf16(HD, SQ, true, true);      // dQ_t^T: head_dim x queries
      const Desc dk_k = desc_of(tc::smem_u32(sK), 16, 1024), dv_k = desc_of(tc::smem_u32(sV), 16, 1024), dk_mn = desc_of(tc::smem_u32(sK), 16384, 1024);
      bool ok = tc::mbar_wait(&sh->kv_full, 0, status, abort_flag, 333);
      // scores of the pair of steps (2p, 2p+1): one N = 128 product each for S^T and dP^T (half the operand traffic of
      // two N = 64 products); the second step may not exist, its columns are then never read
      auto issue_scores = [&](int p) -> bool {
        const int a = 2 * p;
        if (!tc::mbar_wait(&sh->qdo_full[a % NQ], (a / NQ) & 1, status, abort_flag, 334)) return false;
        if (a + 1 < n_steps && !tc::mbar_wait(&sh->qdo_full[(a + 1) % NQ], ((a + 1) / NQ) & 1, status, abort_flag, 334)) return false;
        tc::tc_fence_after();
        const Desc dq_k = desc_of(tc::smem_u32(sQ + (p & 1) * PAIR_TILE), 16, 1024), ddo_k = desc_of(tc::smem_u32(sdO + (p & 1) * PAIR_TILE), 16, 1024);
        mma_ss<false>(tmem_base, dk_k, 0, dq_k, 0, idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k) mma_ss<true>(tmem_base, dk_k, (k >> 2) * 16384 + (k & 3) * 32, dq_k, (k >> 2) * 16384 + (k & 3) * 32, idesc_s);
        tc::umma_commit(&sh->s_full[p & 1]);
        // the dP^T columns held dQ^T of steps 2p-2 and 2p-1 until the dQ warps copied them out
        if (p >= 1 && !(tc::mbar_wait(&sh->dq_consumed[0], (p - 1) & 1, status, abort_flag, 335) &&
                        tc::mbar_wait(&sh->dq_consumed[1], (p - 1) & 1, status, abort_flag, 335))) return false;
        tc::tc_fence_after();
        mma_ss<false>(tmem_base + 128, dv_k, 0, ddo_k, 0, idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k) mma_ss<true>(tmem_base + 128, dv_k, (k >> 2) * 16384 + (k & 3) * 32, ddo_k, (k >> 2) * 16384 + (k & 3) * 32, idesc_s);
        tc::umma_commit(&sh->sdp_full[p & 1]);
        return true;
      };
      auto issue_products = [&](int st) -> bool {
        const int s = st & 1; const uint32_t ph = (st >> 1) & 1;
        if (!tc::mbar_wait(&sh->pds_full[s], ph, status, abort_flag, 336)) return false;
        tc::tc_fence_after();
        const int sq = st % NQ;
        const int sub_off = ((st >> 1) & 1) * PAIR_TILE + s * 8192;
        const Desc dq_mn = desc_of(tc::smem_u32(sQ + sub_off), 16384, 1024), ddo_mn = desc_of(tc::smem_u32(sdO + sub_off), 16384, 1024),
                   dds_mn = desc_of(tc::smem_u32(sdS + s * DS_TILE), 16384, 1024);
        const uint32_t t_s = tmem_base + s * 64, t_dp = t_s + 128;
        // dK += dS^T Q_t ; dV += P^T dO_t : A (keys x 64 queries, packed bf16) from tensor memory, 16 queries per MMA;
        // the packed values of queries [0,32) sit in columns [0,16) and those of queries [32,64) in columns [32,48).
        // The tensor pipe runs this thread's MMAs in order, so dQ_t^T may overwrite dS^T right after the dK product; it
        // is issued before the dV product so that the dQ warps get it as early as possible.
#pragma unroll
        for (int k = 0; k < SQ / 16; ++k)
          mma_ts(t_dk, t_dp + (k >> 1) * 32 + (k & 1) * 8, dq_mn, k * 2048, idesc_kv, (st | k) ? 1u : 0u);
        // dQ_t^T = K_j^T dS^T (contraction over the 128 keys, dS^T from shared memory)
        mma_ss<false>(t_dp, dk_mn, 0, dds_mn, 0, idesc_dq);
#pragma unroll
        for (int k = 1; k < TK / 16; ++k) mma_ss<true>(t_dp, dk_mn, k * 2048, dds_mn, k * 2048, idesc_dq);
        tc::umma_commit(&sh->dq_full[s]);
#pragma unroll
        for (int k = 0; k < SQ / 16; ++k)
          mma_ts(t_dv, t_s + (k >> 1) * 32 + (k & 1) * 8, ddo_mn, k * 2048, idesc_kv, (st | k) ? 1u : 0u);
        tc::umma_commit(&sh->qdo_empty[sq]);
        return true;
      };
      // Issue order: scores of pair p+1 follow the products of pair p; the CUDA cores work on step 2p+1 while the tensor
      // pipe runs the products of step 2p.
      if (ok && n_steps > 0) ok = issue_scores(0);
      for (int st = 0; st < n_steps && ok; st += 2) {
        ok = issue_products(st);
        if (ok && st + 1 < n_steps) ok = issue_products(st + 1);
        if (ok && st + 2 < n_steps) ok = issue_scores((st >> 1) + 1);
      }
      if (ok) tc::umma_commit(&sh->done);
    }
  } else if (warp >= 10) {
    // ---- dQ warps: dQ_t^T (rows = head_dim = this thread's lane, 64 queries) -> global fp32 accumulator --------------
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    int sub = 0, head = kvh * G;                                   // step st: query sub-tile 2j + sub of this head
    for (int st = 0; st < n_steps; ++st) {
      const int s = st & 1; const uint32_t ph = (st >> 1) & 1;
      if (!__all_sync(0xffffffffu, tc::mbar_wait(&sh->dq_full[s], ph, status, abort_flag, 342))) break;
      tc::tc_fence_after();
      uint32_t v[64];
      tc::tmem_ld_32x32(tmem_base + lane_base + 128 + s * 64, v);
      tc::tmem_ld_32x32(tmem_base + lane_base + 128 + s * 64 + 32, v + 32);
      tc::tmem_ld_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->dq_consumed[s]);        // the columns may take dP^T of step st+2
      const int q0 = (2 * j + sub) * SQ, nq = min(SQ, S - q0);
      float *dst = dQacc + (long long)j * dq_tile_stride + (((long long)b * nH + head) * S + q0) * HD + quarter * 32 + lane;
      if (++sub == per_head) { sub = 0; ++head; }
      if (dq_tile_stride) {           // bit-reproducible form: this key tile's own slice; the store kernel adds the slices in order
#pragma unroll
        for (int q = 0; q < SQ; ++q)
          if (q < nq) dst[(size_t)q * HD] = __uint_as_float(v[q]);
      } else {
#pragma unroll
        for (int q = 0; q < SQ; ++q)
          if (q < nq) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)q * HD), "f"(__uint_as_float(v[q])) : "memory");
      }
    }
  } else {
    // ---- compute warps: two threads per key row (tensor-memory lane), 32 of the step's 64 queries each ----------
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    const int key = j * TK + r;
    bool ok = true;
    int sub = 0;                                                      // step st: query sub-tile 2j + sub (no division per step)
    for (int st = 0; st < n_steps && ok; ++st) {
      const int s = st & 1;
      const int tile_q0 = (2 * j + sub) * SQ, q0 = tile_q0 + half * 32;     // this thread's first query
      if (++sub == per_head) sub = 0;
      const float *st_l = reinterpret_cast<const float *>(sStat + (st % NQ) * STAT) + half * 32, *st_d = st_l + SQ;
      // bound checks only where the step touches the diagonal or an end of the sequence
      const bool tile_masked = (tile_q0 < (j + 1) * TK) || (tile_q0 + SQ > S) || ((j + 1) * TK > S);
      const uint32_t t_s = tmem_base + lane_base + s * 64, t_dp = t_s + 128;
      const int pr = (st >> 1) & 1; const uint32_t pph = (st >> 2) & 1;      // the pair's score barriers
      uint32_t sv[32], wp[16], wd[16];
      float p[32];
      ok = tc::mbar_wait(&sh->qdo_full[st % NQ], (st / NQ) & 1, status, abort_flag, 346) &&      // lse, D of this step
           tc::mbar_wait(&sh->s_full[pr], pph, status, abort_flag, 343);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc::tc_fence_after();
      tc::tmem_ld_32x32(t_s + half * 32, sv);
      tc::tmem_ld_wait();
      if (!tile_masked) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 L = *reinterpret_cast<const float4 *>(st_l + u * 4);
          p[u * 4 + 0] = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 0]), sl2, -L.x));
          p[u * 4 + 1] = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 1]), sl2, -L.y));
          p[u * 4 + 2] = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 2]), sl2, -L.z));
          p[u * 4 + 3] = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 3]), sl2, -L.w));
        }
      } else {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int q = q0 + x;
          const bool live = q < S && key < S && q >= key;
          p[x] = live ? fast_exp2(fmaf(__uint_as_float(sv[x]), sl2, -st_l[x])) : 0.f;
        }
      }
#pragma unroll
      for (int x = 0; x < 16; ++x) wp[x] = pack_bf16(p[2 * x], p[2 * x + 1]);
      tmem_st_32x16(t_s + half * 32, wp);
      ok = tc::mbar_wait(&sh->sdp_full[pr], pph, status, abort_flag, 345);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc::tc_fence_after();
      tc::tmem_ld_32x32(t_dp + half * 32, sv);
      tc::tmem_ld_wait();
      if (!tile_masked) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 D = *reinterpret_cast<const float4 *>(st_d + u * 4);
          const float d0 = p[u * 4 + 0] * (__uint_as_float(sv[u * 4 + 0]) - D.x), d1 = p[u * 4 + 1] * (__uint_as_float(sv[u * 4 + 1]) - D.y),
                      d2 = p[u * 4 + 2] * (__uint_as_float(sv[u * 4 + 2]) - D.z), d3 = p[u * 4 + 3] * (__uint_as_float(sv[u * 4 + 3]) - D.w);
          wd[u * 2] = pack_bf16(d0, d1); wd[u * 2 + 1] = pack_bf16(d2, d3);
        }
      } else {
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          // p is zero wherever the entry is masked; the statistics of queries past the end are never loaded
          const float d0 = p[x] != 0.f ? p[x] * (__uint_as_float(sv[x]) - st_d[x]) : 0.f;
          const float d1 = p[x + 1] != 0.f ? p[x + 1] * (__uint_as_float(sv[x + 1]) - st_d[x + 1]) : 0.f;
          wd[x >> 1] = pack_bf16(d0, d1);
        }
      }
      // P^T and dS^T back into tensor memory, packed bf16 over the first half of the 32 columns this thread just read
      // (never over columns the other thread of the row still has to read); dS^T also to shared memory
      tmem_st_32x16(t_dp + half * 32, wd);
      {
        uint8_t *row = sdS + s * DS_TILE + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4 *>(row + (((half * 4 + u) ^ (r & 7)) << 4)) = make_uint4(wd[u * 4], wd[u * 4 + 1], wd[u * 4 + 2], wd[u * 4 + 3]);
      }
      tc::tmem_st_wait();
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->pds_full[s]);
    }
    // dK / dV of this key tile: rows = keys, this thread's half of the head_dim
    if (ok && __all_sync(0xffffffffu, tc::mbar_wait(&sh->done, 0, status, abort_flag, 344))) {
      tc::tc_fence_after();
      // every MMA of the CTA has completed: the Q ring is free and serves as the transposition buffers of the stores
      // (whole 64-byte row segments per store instruction, see tc::stage_store_bf16)
      const int key0 = j * TK + quarter * 32;
      bf16 *dkbase = dK + (long long)b * dk_b + (long long)kvh * dk_h + (long long)key0 * dk_s;
      bf16 *dvbase = dV + (long long)b * dv_b + (long long)kvh * dv_h + (long long)key0 * dv_s;
      uint8_t *stg = sQ + warp * 2048;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = (half * 2 + c) * 32;
        uint32_t a[32], g[32];
        tc::tmem_ld_32x32(t_dk + lane_base + col, a);
        tc::tmem_ld_32x32(t_dv + lane_base + col, g);
        tc::tmem_ld_wait();
        {
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] = __float_as_uint(__uint_as_float(a[e]) * scale);       // dS was left unscaled
          if (rope_cos != nullptr && key < S) {
            // gradient of the rotary embedding (inverse rotation, cpp/src/Positional.cpp:207-231) on dK, position = key
            const float *cp = rope_cos + (size_t)key * (HD / 2) + (col >> 1), *sp = rope_sin + (size_t)key * (HD / 2) + (col >> 1);
#pragma unroll
            for (int p2 = 0; p2 < 16; ++p2) {
              const float x0 = __uint_as_float(a[2 * p2]), x1 = __uint_as_float(a[2 * p2 + 1]), cc = __ldg(cp + p2), ss = __ldg(sp + p2);
              a[2 * p2] = __float_as_uint(x0 * cc + x1 * ss);
              a[2 * p2 + 1] = __float_as_uint(-x0 * ss + x1 * cc);
            }
          }
          uint4 wk[4], wv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            wk[u].x = pack_bf16(__uint_as_float(a[u * 8 + 0]), __uint_as_float(a[u * 8 + 1]));
            wk[u].y = pack_bf16(__uint_as_float(a[u * 8 + 2]), __uint_as_float(a[u * 8 + 3]));
            wk[u].z = pack_bf16(__uint_as_float(a[u * 8 + 4]), __uint_as_float(a[u * 8 + 5]));
            wk[u].w = pack_bf16(__uint_as_float(a[u * 8 + 6]), __uint_as_float(a[u * 8 + 7]));
            wv[u].x = pack_bf16(__uint_as_float(g[u * 8 + 0]), __uint_as_float(g[u * 8 + 1]));
            wv[u].y = pack_bf16(__uint_as_float(g[u * 8 + 2]), __uint_as_float(g[u * 8 + 3]));
            wv[u].z = pack_bf16(__uint_as_float(g[u * 8 + 4]), __uint_as_float(g[u * 8 + 5]));
            wv[u].w = pack_bf16(__uint_as_float(g[u * 8 + 6]), __uint_as_float(g[u * 8 + 7]));
          }
          tc::stage_store_bf16(stg, lane, wk, dkbase + col, (size_t)dk_s, S - key0);
          tc::stage_store_bf16(stg, lane, wv, dvbase + col, (size_t)dv_s, S - key0);
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

}  // namespace

bool attn_bwd2_supported(size_t S, size_t hd) { return hd == 128 && S % 4 == 0 && S >= 4; }

// Dsum must hold rowsum(dO * O) and lse2 the log-sum-exp times log2(e) (attn_dsum_kernel of attention_bwd_tc.cu); dQ comes
// out WITHOUT the softmax scale (the caller's store kernel multiplies it in); dQacc: the zeroed fp32 accumulator
// [B*nH*S][128] that the caller afterwards turns into dQ rows.  dq_tile_stride > 0 (elements): key tile j writes its
// contribution to the slice dQacc + j * dq_tile_stride instead of adding to one accumulator (queries from 128 j on).
int attn_bwd2_tc_run(b200_ctx *ctx, const void *Q, const void *K, const void *V, const void *dO, const float *lse2, const float *Dsum,
                     float *dQacc, long long dq_tile_stride, void *dK, void *dV, size_t B, size_t nH, size_t nKV, size_t S, const AttnStrides &st,
                     const AttnStrides &gst, const float *rope_cos, const float *rope_sin) {
  CUtensorMap mq, mk, mv, mdo;
  if (tc_make_map_4d(&mq, Q, HD, S, nH, B, (uint64_t)st.q_s * 2, (uint64_t)st.q_h * 2, (uint64_t)st.q_b * 2, 64, SQ) ||
      make_map_4d(&mk, K, HD, S, nKV, B, st.k_s, st.k_h, st.k_b) || make_map_4d(&mv, V, HD, S, nKV, B, st.v_s, st.v_h, st.v_b) ||
      tc_make_map_4d(&mdo, dO, HD, S, nH, B, (uint64_t)st.o_s * 2, (uint64_t)st.o_h * 2, (uint64_t)st.o_b * 2, 64, SQ))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for attention operands");
  constexpr int smem = 2 * KV_TILE + 2 * NQ * Q_TILE + 2 * DS_TILE + NQ * STAT + (int)sizeof(Bwd2Shared);
  static_assert(smem <= 232448, "backward attention tiles exceed the 227 KiB of shared memory per CTA");
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd2_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  dim3 grid((unsigned)(nKV * B), (unsigned)((S + TK - 1) / TK), 1);
  B200_CUDA(ctx, launch_k(ctx, attn_bwd2_tc_kernel, grid, dim3(BWD2_THREADS), (size_t)smem, 0, mq, mk, mv, mdo, dQacc, dq_tile_stride, lse2, Dsum, (bf16 *)dK, (bf16 *)dV, (int)nH,
                          (int)nKV, (int)S, gst.k_b, gst.k_h, gst.k_s, gst.v_b, gst.v_h, gst.v_s, 1.0f / sqrtf((float)HD), ctx->dev_status, rope_cos, rope_sin));
  B200_LAUNCHED(ctx);
  return B200_OK;
}
