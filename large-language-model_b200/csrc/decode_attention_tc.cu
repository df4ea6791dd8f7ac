// Decode attention on the tensor cores: one new token per sequence against the K/V cache, head_dim 128, bf16.
// Same contract as attn_decode_kernel of decode_attention.cu (single-token attention of
// cpp/src/Attention.cpp:236-280 over the cache of cpp/src/Attention.cpp:121-175); used when one CTA per
// (sequence, KV head) fills the GPU, i.e. when the batch is large enough that key runs need not be split.
//
// The CUDA-core kernel spends its time issuing instructions (a dot product per key and query head); here the cache
// tiles go from HBM to shared memory by TMA and the tensor cores do both products, transposed so that the 128 rows of
// the MMA are 128 keys (scores) or the 128 head dimensions (output) and the MMA's N is the padded group of query heads:
//     S^T_i = K_i Q^T            [128 keys x 16]   for every 128-key tile i of the cache (all tiles stay in tensor memory)
//     one softmax over all tiles (exact maximum first, so the output needs no rescaling)
//     O^T  += V_i^T P_i^T        [128 dims x 16]
// K tiles stream first, then V tiles, through one ring of 32 KiB stages; V tiles are already in flight while the
// softmax runs.  The new token's key and value never pass through the cache read: its score is a CUDA-core dot product
// and its value is added in the epilogue; its rows are appended to the cache for the steps to come.
//   warps 0-3: stage Q, append the new rows, softmax (thread = key), epilogue (thread = head dimension);
//   warp 4: TMA; warp 5: MMA issue.
#include "attention_tc.cuh"

using namespace attn;

namespace {

constexpr int HD = 128, KEYS = 128;
constexpr int TILE = KEYS * HD * 2;                    // 32 KiB: [2 chunks of 64 columns][128 rows][128 B], 128-byte swizzle
constexpr int OPERAND16 = 16 * HD * 2;                 // 4 KiB: a 16-row K-major operand (Q, or P of one tile): 2 chunks of 2 KiB
constexpr int SM_WARPS = 4, TMA_W = 4, MMA_W = 5, DEC_THREADS = 192;
constexpr int MAX_STAGES = 5;

struct DecTcArgs {
  const bf16 *q, *k_new, *v_new;       // rows of the fused projection output (row stride ldq elements); k_new may be null
  bf16 *kc, *vc, *o;                   // caches [B, S_max, nKV*128]; output rows [B, ldo]
  const int *pos_dev;                  // when set: the new token's position is *pos_dev instead of t_len - 1
  int nKV, G, S_max, t_len, ldq, ldo;
  int early_tiles;                     // K tiles that hold only positions written before this step's kernels started
  float scale;
  int *status;
};

struct DecShared {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], q_ready, s_full, p_ready, o_full;
  uint32_t tmem_base;
  int abort_flag;
  float red_max[SM_WARPS][16], red_sum[SM_WARPS][16], s_new[16];
};

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t *r) {
  if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
  } else {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
  }
}
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // warps 0-3
// K-major 16-row operand: 16 columns (32 B) per MMA, 64-column chunks 2 KiB apart
__device__ __forceinline__ uint64_t desc_rows16(uint32_t base, int k) { return tc::make_smem_desc(base + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024); }

// GP: query heads per KV head, padded (columns read per tile); NT: most 128-key tiles a sequence may have.
template <int GP, int NT>
__global__ void __launch_bounds__(DEC_THREADS, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecTcArgs a) {
  constexpr int NS = NT <= 8 ? 5 : 4;                  // ring stages
  constexpr uint32_t TCOLS = NT <= 8 ? 256 : 512;      // 16 columns per score tile + 16 for the output
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *ring = smem_raw, *sQ = ring + NS * TILE, *sP = sQ + OPERAND16;
  DecShared *sh = (DecShared *)(sP + NT * OPERAND16);
  if (tc::smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, 298);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int kvh = blockIdx.x, b = blockIdx.y, G = a.G;
  volatile int *abort_flag = &sh->abort_flag;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) { tc::mbar_init(&sh->full[i], 1); tc::mbar_init(&sh->empty[i], 1); }
    tc::mbar_init(&sh->q_ready, SM_WARPS); tc::mbar_init(&sh->s_full, 1);
    tc::mbar_init(&sh->p_ready, SM_WARPS); tc::mbar_init(&sh->o_full, 1);
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  // tensor memory is taken before the next kernel of the stream may start, so that kernel's CTAs cannot hold the
  // columns this one is still waiting for
  if (warp == MMA_W) tc::tmem_alloc(&sh->tmem_base, TCOLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base, t_o = tmem_base + 16 * NT;
  pdl_launch_dependents();
  // Cache tiles of positions that were complete before this token step began depend on no kernel still running: their
  // loads go out before the wait on the previous kernel (with a captured step the host-side length is a lower bound:
  // replays only move forward).
  const int n_early = min(a.early_tiles, NS);
  if (warp == TMA_W && lane == 0) {
    for (int i = 0; i < n_early; ++i) {
      tc::mbar_expect_tx(&sh->full[i], TILE);
      tma_load_4d(ring + i * TILE, &map_k, 0, i * KEYS, kvh, b, &sh->full[i]);
      tma_load_4d(ring + i * TILE + 16384, &map_k, 64, i * KEYS, kvh, b, &sh->full[i]);
    }
  }
  pdl_wait();

  const int pos = a.pos_dev ? *a.pos_dev : a.t_len - 1;        // position of the new token
  const bool has_new = a.k_new != nullptr;
  const int n_cached = has_new ? pos : pos + 1;                  // keys that come from the cache
  const int nt = min((n_cached + KEYS - 1) / KEYS, NT);

  if (warp == TMA_W) {
    if (lane == 0) {
      for (int i = n_early; i < 2 * nt; ++i) {                    // K tiles, then V tiles
        const int slot = i % NS;
        if (i >= NS && !tc::mbar_wait(&sh->empty[slot], ((i / NS) - 1) & 1, a.status, abort_flag, 351)) break;
        const CUtensorMap *map = i < nt ? &map_k : &map_v;
        const int key0 = (i < nt ? i : i - nt) * KEYS;
        tc::mbar_expect_tx(&sh->full[slot], TILE);
        tma_load_4d(ring + slot * TILE, map, 0, key0, kvh, b, &sh->full[slot]);
        tma_load_4d(ring + slot * TILE + 16384, map, 64, key0, kvh, b, &sh->full[slot]);
      }
      // early loads nobody will consume (only if a captured step were replayed at an earlier position than it was
      // captured at) must still land before the CTA gives its shared memory back
      for (int i = nt; i < n_early; ++i) tc::mbar_wait(&sh->full[i], 0, a.status, abort_flag, 358);
    }
  } else if (warp == MMA_W) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 16, false, false);   // S^T: keys x heads
      constexpr uint32_t idesc_o = tc::make_idesc_bf16(128, 16, true, false);    // O^T: dims x heads, A = V^T (MN-major)
      bool ok = tc::mbar_wait(&sh->q_ready, 0, a.status, abort_flag, 352);
      tc::tc_fence_after();
      const uint32_t q_addr = tc::smem_u32(sQ);
      for (int i = 0; i < nt && ok; ++i) {
        const int slot = i % NS;
        ok = tc::mbar_wait(&sh->full[slot], (i / NS) & 1, a.status, abort_flag, 353);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t k_addr = tc::smem_u32(ring + slot * TILE);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) tc::umma_ss(tmem_base + 16 * i, desc_kmajor(k_addr, k), desc_rows16(q_addr, k), idesc_s, k ? 1u : 0u);
        tc::umma_commit(&sh->empty[slot]);
      }
      if (ok) { if (nt > 0) tc::umma_commit(&sh->s_full); else tc::mbar_arrive(&sh->s_full); }   // no MMA to wait for on an empty cache
      if (ok) ok = tc::mbar_wait(&sh->p_ready, 0, a.status, abort_flag, 354);
      tc::tc_fence_after();
      for (int i = 0; i < nt && ok; ++i) {
        const int j = nt + i, slot = j % NS;
        ok = tc::mbar_wait(&sh->full[slot], (j / NS) & 1, a.status, abort_flag, 355);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t v_addr = tc::smem_u32(ring + slot * TILE), p_addr = tc::smem_u32(sP + i * OPERAND16);
#pragma unroll
        for (int k = 0; k < KEYS / 16; ++k) tc::umma_ss(t_o, desc_mnmajor(v_addr, k), desc_rows16(p_addr, k), idesc_o, (i | k) ? 1u : 0u);
        tc::umma_commit(&sh->empty[slot]);
      }
      if (ok) { if (nt > 0) tc::umma_commit(&sh->o_full); else tc::mbar_arrive(&sh->o_full); }
    }
  } else {
    // ---- warps 0-3 -------------------------------------------------------------------------------------------------
    const float sl2 = a.scale * LOG2E;
    const bf16 *q_row = a.q + (size_t)b * a.ldq + (size_t)kvh * G * HD;
    {   // Q^T operand: 16 rows (heads of the group, zero beyond G) x 128 dims; this thread: row tid/8, 16 dims
      const int q = tid >> 3, seg = tid & 7;
      uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
      if (q < G) {
        const uint4 *src = reinterpret_cast<const uint4 *>(q_row + (size_t)q * HD + seg * 16);
        v0 = src[0]; v1 = src[1];
      }
      uint8_t *dst = sQ + (seg >> 2) * 2048 + q * 128;
      *reinterpret_cast<uint4 *>(dst + ((((seg & 3) * 2) ^ (q & 7)) << 4)) = v0;
      *reinterpret_cast<uint4 *>(dst + ((((seg & 3) * 2 + 1) ^ (q & 7)) << 4)) = v1;
    }
    for (int u = tid; u < nt * (OPERAND16 / 16); u += SM_WARPS * 32) reinterpret_cast<uint4 *>(sP)[u] = make_uint4(0, 0, 0, 0);
    if (has_new) {
      // the new token's rows join the cache for the next steps (this step reads them from the projection output)
      if (tid < 32) {
        const bf16 *src = (tid < 16 ? a.k_new : a.v_new) + (size_t)b * a.ldq + (size_t)kvh * HD;
        bf16 *dst = (tid < 16 ? a.kc : a.vc) + (((size_t)b * a.S_max + pos) * a.nKV + kvh) * HD;
        reinterpret_cast<uint4 *>(dst)[tid & 15] = reinterpret_cast<const uint4 *>(src)[tid & 15];
      }
      // its scores: one head per warp pass, four dims per lane
      const bf16 *kn = a.k_new + (size_t)b * a.ldq + (size_t)kvh * HD + lane * 4;
      const float2 k01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(kn)),
                   k23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(kn + 2));
      for (int q = warp; q < G; q += SM_WARPS) {
        const bf16 *qp = q_row + (size_t)q * HD + lane * 4;
        const float2 q01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(qp)),
                     q23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(qp + 2));
        float s = q01.x * k01.x + q01.y * k01.y + q23.x * k23.x + q23.y * k23.y;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) sh->s_new[q] = s * sl2;
      }
    } else if (tid < 16) {
      sh->s_new[tid] = -INFINITY;
    }
    tc::fence_proxy_async();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sh->q_ready);

    // scores of every tile: this thread is key `tid` of each tile
    bool ok = __all_sync(0xffffffffu, tc::mbar_wait(&sh->s_full, 0, a.status, abort_flag, 356));
    tc::tc_fence_after();
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    uint32_t sv[NT][GP];
#pragma unroll
    for (int i = 0; i < NT; ++i)
      if (i < nt) tmem_ld_cols<GP>(tmem_base + lane_base + 16 * i, sv[i]);
    tc::tmem_ld_wait();
    float m[GP], l[GP];
#pragma unroll
    for (int q = 0; q < GP; ++q) m[q] = -INFINITY;
#pragma unroll
    for (int i = 0; i < NT; ++i)
      if (i < nt && i * KEYS + tid < n_cached) {
#pragma unroll
        for (int q = 0; q < GP; ++q) m[q] = fmaxf(m[q], __uint_as_float(sv[i][q]) * sl2);
      }
#pragma unroll
    for (int q = 0; q < GP; ++q) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) m[q] = fmaxf(m[q], __shfl_xor_sync(0xffffffffu, m[q], off));
      if (lane == 0) sh->red_max[warp][q] = m[q];
    }
    softmax_sync();                                       // also orders the zero fill of sP before the writes below
#pragma unroll
    for (int q = 0; q < GP; ++q) {
      m[q] = fmaxf(fmaxf(sh->red_max[0][q], sh->red_max[1][q]), fmaxf(sh->red_max[2][q], sh->red_max[3][q]));
      if (q < G) m[q] = fmaxf(m[q], sh->s_new[q]);
      l[q] = 0.f;
    }
    // P^T operand of tile i: row = head, this thread's key is one bf16 of the row
#pragma unroll
    for (int i = 0; i < NT; ++i)
      if (i < nt) {
        const bool live = i * KEYS + tid < n_cached;
        uint8_t *col = sP + i * OPERAND16 + (tid >> 6) * 2048 + (tid & 7) * 2;
#pragma unroll
        for (int q = 0; q < GP; ++q) {
          const float p = live ? fast_exp2(__uint_as_float(sv[i][q]) * sl2 - m[q]) : 0.f;
          const bf16 pb = __float2bfloat16_rn(p);
          l[q] += __bfloat162float(pb);                   // the sum of what the tensor cores will multiply
          if (q < G) *reinterpret_cast<bf16 *>(col + q * 128 + (((((tid & 63) >> 3)) ^ (q & 7)) << 4)) = pb;
        }
      }
    tc::fence_proxy_async();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sh->p_ready);
#pragma unroll
    for (int q = 0; q < GP; ++q) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) l[q] += __shfl_xor_sync(0xffffffffu, l[q], off);
      if (lane == 0) sh->red_sum[warp][q] = l[q];
    }
    softmax_sync();
    float p_new[GP];
#pragma unroll
    for (int q = 0; q < GP; ++q) {
      p_new[q] = (has_new && q < G) ? fast_exp2(sh->s_new[q] - m[q]) : 0.f;
      l[q] = sh->red_sum[0][q] + sh->red_sum[1][q] + sh->red_sum[2][q] + sh->red_sum[3][q] + p_new[q];
    }
    // output: this thread is head dimension `tid`
    ok = __all_sync(0xffffffffu, tc::mbar_wait(&sh->o_full, 0, a.status, abort_flag, 357)) && ok;
    tc::tc_fence_after();
    uint32_t ov[GP];
#pragma unroll
    for (int q = 0; q < GP; ++q) ov[q] = 0u;
    if (nt > 0) { tmem_ld_cols<GP>(t_o + lane_base, ov); tc::tmem_ld_wait(); }
    const float vn = has_new ? __bfloat162float(a.v_new[(size_t)b * a.ldq + (size_t)kvh * HD + tid]) : 0.f;
    if (ok) {
#pragma unroll
      for (int q = 0; q < GP; ++q)
        if (q < G) a.o[(size_t)b * a.ldo + ((size_t)kvh * G + q) * HD + tid] = __float2bfloat16_rn((__uint_as_float(ov[q]) + p_new[q] * vn) / l[q]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == MMA_W) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, TCOLS);
  }
}

template <int GP, int NT>
int launch_tc(b200_ctx *ctx, const CUtensorMap &mk, const CUtensorMap &mv, const DecTcArgs &a, dim3 grid) {
  constexpr int NS = NT <= 8 ? 5 : 4;
  constexpr int smem = NS * TILE + OPERAND16 + NT * OPERAND16 + (int)sizeof(DecShared);
  static_assert(smem <= 232448, "decode attention tiles exceed the 227 KiB of shared memory per CTA");
  static bool attr = false;
  if (!attr) { B200_CUDA(ctx, cudaFuncSetAttribute(attn_decode_tc_kernel<GP, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
  B200_CUDA(ctx, launch_k(ctx, attn_decode_tc_kernel<GP, NT>, grid, dim3(DEC_THREADS), (size_t)smem, 0, mk, mv, a));
  B200_LAUNCHED(ctx);
  return B200_OK;
}

}  // namespace

// True when the tensor-core kernel covers the case: bf16, head_dim 128, a group of at most 8 query heads per KV head,
// a cache of at most 2048 positions (1024 for groups above 4), aligned rows, and enough (sequence, KV head) pairs to
// fill the GPU without splitting key runs.
bool attn_decode_tc_supported(const b200_ctx *ctx, const void *q, const void *kc, const void *vc, const void *o, size_t B, size_t nH,
                              size_t nKV, size_t hd, size_t S_max, size_t ldq, size_t ldo, b200_dtype dt) {
  if (dt != B200_BF16 || hd != 128 || nKV == 0 || nH % nKV) return false;
  const size_t G = nH / nKV;
  if (G > 8 || S_max > 2048 || (G > 4 && S_max > 1024)) return false;
  if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)o) % 16 || ldq % 8 || ldo % 8) return false;
  return B * nKV * 2 >= (size_t)ctx->sm_count && B <= 65535;
}

int attn_decode_tc(b200_ctx *ctx, const void *q, const void *k_new, const void *v_new, void *kc, void *vc, void *o, size_t B,
                   size_t nH, size_t nKV, size_t S_max, size_t t_len, size_t ldq, size_t ldo, const int *pos_dev) {
  const size_t G = nH / nKV;
  CUtensorMap mk, mv;
  // cache [B, S_max, nKV, 128]: dims (dim, position, kv head, sequence); box = 64 columns x 128 positions
  if (tc_make_map_4d(&mk, kc, HD, S_max, nKV, B, nKV * HD * 2, HD * 2, S_max * nKV * HD * 2, 64, KEYS) ||
      tc_make_map_4d(&mv, vc, HD, S_max, nKV, B, nKV * HD * 2, HD * 2, S_max * nKV * HD * 2, 64, KEYS))
    return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for the K/V cache");
  DecTcArgs a;
  a.q = (const bf16 *)q; a.k_new = (const bf16 *)k_new; a.v_new = (const bf16 *)v_new;
  a.kc = (bf16 *)kc; a.vc = (bf16 *)vc; a.o = (bf16 *)o; a.pos_dev = pos_dev;
  a.nKV = (int)nKV; a.G = (int)G; a.S_max = (int)S_max; a.t_len = (int)t_len; a.ldq = (int)ldq; a.ldo = (int)ldo;
  a.scale = 1.0f / sqrtf((float)HD);
  a.status = ctx->dev_status;
  {
    const size_t cached_at_least = k_new ? t_len - 1 : t_len;     // positions in the cache (a lower bound when pos_dev is set)
    a.early_tiles = (int)(cached_at_least / KEYS);
  }
  dim3 grid((unsigned)nKV, (unsigned)B, 1);
  if (G > 4) return launch_tc<8, 8>(ctx, mk, mv, a, grid);
  if (S_max <= 1024) return launch_tc<4, 8>(ctx, mk, mv, a, grid);
  return launch_tc<4, 16>(ctx, mk, mv, a, grid);
}
