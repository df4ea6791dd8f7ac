// Weight-streaming bf16 GEMM for a handful of rows (decode: one new token per sequence):
//   C[M,N] = A[M,K] * W[K,N],  M <= 64,  W stored [in,out] as the reference keeps its projections
//   (cpp/src/Tensor.cpp:174-228 via metal_bridge::gemm_bf16, cpp/include/gpu_kernel/MetalBridge.hpp:39-42).
// The work is bound by reading W once from HBM, so the kernel is laid out to keep every SM streaming:
//   * operands are swapped on the tensor core: the 128 rows of the tcgen05.mma tile are 128 OUTPUT FEATURES
//     (W tile, MN-major straight from its [K,N] storage) and the MMA's N is the (padded) row count of A,
//     so no tensor-core work is spent on padding rows;
//   * a thread-block cluster of SPLIT CTAs shares one 128-feature tile and splits K between its CTAs;
//     partial sums meet in distributed shared memory (each CTA owns 128/SPLIT features, receives the other
//     CTAs' partials for them, adds them in a fixed order and writes its slice of C), so the result is
//     deterministic and needs no zero-filled fp32 workspace;
//   * the optional rotary epilogue rotates interleaved feature pairs on the fp32 sums;
//   * the optional SwiGLU epilogue (W = [gate | up], each `swiglu_I` columns wide) puts 64 gate and the matching
//     64 up features in one tile and writes silu(gate) * up, so the [M, 2I] intermediate never exists
//     (metal_bridge::fused_swiglu_gemm, cpp/include/gpu_kernel/MetalBridge.hpp:44-46).
//   * optionally an RMS normalisation (cpp/src/RMSNorm.cpp forward) is split between two projections: the one that
//     produces the residual stream h adds the residual in its epilogue, writes h * w_norm next to h and adds the sums
//     of squares of its columns to per-row accumulators; the one that consumes norm(h) multiplies h * w_norm by W as it
//     is and scales its result by rstd from those sums.  A decoder layer of a decode step then needs no normalisation kernel;
// 128 threads: warp 0 lane 0 issues TMA, warp 1 lane 0 issues the MMAs, all four warps run the epilogue.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int FT = 128;               // output features per cluster tile (rows of the MMA)
constexpr int BK = 64, STAGES = 4;
constexpr int W_STAGE_BYTES = FT * BK * 2;     // 16 KiB: two [64 features x 64 K] swizzled chunks
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int THREADS = 128;

__host__ __device__ constexpr int a_stage_bytes(int nt) { return nt * BK * 2; }
constexpr int STATS_BYTES = 64 * 2 * 4;        // [row][sum h^2, sum (h w)^2] of a normalisation the producing projection started
__host__ __device__ constexpr int smem_bytes(int nt) {
  return STAGES * (W_STAGE_BYTES + a_stage_bytes(nt)) + FT * nt * 4 + STATS_BYTES + 1024 /*align*/ + 128 /*barriers*/;
}

struct Tail {
  uint64_t full[STAGES], empty[STAGES], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_all() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_all() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t cta, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// G consecutive outputs of one row -> C (16 bytes of bf16 or 16/32 bytes of fp32)
template <class TO, int G>
__device__ __forceinline__ void store_group(TO *dst, const float (&v)[G]) {
  if constexpr (sizeof(TO) == 2) {
    uint32_t w[G / 2];
#pragma unroll
    for (int i = 0; i < G / 2; ++i) { __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t *>(&b); }
    if constexpr (G == 8) *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    else *reinterpret_cast<uint2 *>(dst) = make_uint2(w[0], w[1]);
  } else {
#pragma unroll
    for (int i = 0; i < G / 4; ++i) reinterpret_cast<float4 *>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
}
template <class TO, int G>
__device__ __forceinline__ void load_group(const TO *src, float (&v)[G]) {
  if constexpr (sizeof(TO) == 2) {
    uint32_t w[G / 2];
    if constexpr (G == 8) { const uint4 x = *reinterpret_cast<const uint4 *>(src); w[0] = x.x; w[1] = x.y; w[2] = x.z; w[3] = x.w; }
    else { const uint2 x = *reinterpret_cast<const uint2 *>(src); w[0] = x.x; w[1] = x.y; }
#pragma unroll
    for (int i = 0; i < G / 2; ++i) { const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&w[i])); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else {
#pragma unroll
    for (int i = 0; i < G / 4; ++i) { const float4 f = reinterpret_cast<const float4 *>(src)[i]; v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w; }
  }
}

// NT = padded row count of A (32 or 64) = N of the MMA and width of the accumulator in tensor memory.
// `vec`: C (and the residual) allow 16-byte accesses at every group of 4 features.
template <int NT, class TO>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   TO *__restrict__ C, int M, int N, int K, size_t ldc, int split, int *status, GemmEpilogue epi, int vec) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sW = smem, *sA = smem + STAGES * W_STAGE_BYTES;
  float *red = (float *)(sA + STAGES * a_stage_bytes(NT));          // [split][NT][FT/split]
  float *stats = (float *)((uint8_t *)red + FT * NT * 4);           // [NT][2]
  Tail *sh = (Tail *)((uint8_t *)stats + STATS_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = split > 1 ? cluster_rank() : 0;
  const int tile = blockIdx.x / split;
  const bool swiglu = epi.swiglu_I > 0;
  const bool normed = epi.row_acc != nullptr;
  const int n0 = tile * (swiglu ? FT / 2 : FT);   // first output feature of the tile
  const int num_kb = (K + BK - 1) / BK;
  const int kb_lo = (int)((long long)num_kb * rank / split), kb_hi = (int)((long long)num_kb * (rank + 1) / split);
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { tc::mbar_init(&sh->full[i], 1); tc::mbar_init(&sh->empty[i], 1); }
    tc::mbar_init(&sh->acc_full, 1);
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
    tc::tma_prefetch_desc(&map_w);
    tc::tma_prefetch_desc(&map_a);
  }
  if (warp == 0) tc::tmem_alloc(&sh->tmem_base, 64);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  // every CTA of the cluster must be resident before the remote stores of the epilogue: arrive now, wait only there,
  // so the barrier's latency hides behind the main loop
  if (split > 1) cluster_arrive_all();

  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {
    // The weight tiles do not depend on the kernel before this one: the first ring of them is requested before waiting
    // for it (programmatic dependent launch), the activation rows only after.
    const int n_early = min(kb_hi - kb_lo, STAGES);
    auto load_w = [&](int stage, int kb) {
      tc::mbar_expect_tx(&sh->full[stage], W_STAGE_BYTES + a_stage_bytes(NT));
      uint8_t *w = sW + stage * W_STAGE_BYTES;
      tc::tma_load_2d(w, &map_w, n0, kb * BK, &sh->full[stage]);
      tc::tma_load_2d(w + CHUNK_BYTES, &map_w, swiglu ? epi.swiglu_I + n0 : n0 + 64, kb * BK, &sh->full[stage]);
    };
    for (int i = 0; i < n_early; ++i) load_w(i, kb_lo + i);
    pdl_wait();
    for (int i = 0; i < n_early; ++i) tc::tma_load_2d(sA + i * a_stage_bytes(NT), &map_a, (kb_lo + i) * BK, 0, &sh->full[i]);
    int stage = n_early == STAGES ? 0 : n_early; uint32_t phase = n_early == STAGES ? 1 : 0;
    for (int kb = kb_lo + n_early; kb < kb_hi; ++kb) {
      if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1, status, abort_flag, 401)) break;
      load_w(stage, kb);
      tc::tma_load_2d(sA + stage * a_stage_bytes(NT), &map_a, kb * BK, 0, &sh->full[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = tc::make_idesc_bf16(FT, NT, true, false);
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int kb = kb_lo; kb < kb_hi; ++kb) {
      if (!tc::mbar_wait(&sh->full[stage], phase, status, abort_flag, 402)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t w_addr = tc::smem_u32(sW + stage * W_STAGE_BYTES), a_addr = tc::smem_u32(sA + stage * a_stage_bytes(NT));
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        const uint64_t dw = tc::make_smem_desc(w_addr + k * 2048, CHUNK_BYTES, 1024);   // MN-major: 16 K-rows = 2 KiB
        const uint64_t da = tc::make_smem_desc(a_addr + k * 32, 16, 1024);              // K-major: 16 bf16 = 32 B
        tc::umma_ss(tmem_base, dw, da, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
      }
      tc::umma_commit(&sh->empty[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    if (ok) tc::umma_commit(&sh->acc_full);
  }
  __syncwarp();
  pdl_wait();                                   // before any global store (and for the threads that did not load)
  // Values the final loop needs that do not depend on the product: requested now, consumed after the exchange.
  const int pos_row = (epi.cos_t != nullptr && epi.pos_dev) ? *epi.pos_dev : -1;
  if (split > 1) cluster_wait_all();

  // ---- epilogue: tensor memory -> the owning CTA's shared memory ------------------------------
  const int NL = FT / split;                    // features owned per CTA
  if (normed && threadIdx.x >= 64 && threadIdx.x - 64 < NT) {
    // row sums the producing projection accumulated (fixed point, 2^-32); read by the final loop after the barrier below
    const int row = threadIdx.x - 64;
    float a = 0.f, b = 0.f;
    if (row < M) {
      a = (float)((double)__ldg(epi.row_acc + row * 2) * (1.0 / 4294967296.0));
      b = (float)((double)__ldg(epi.row_acc + row * 2 + 1) * (1.0 / 4294967296.0));
    }
    stats[row * 2] = a; stats[row * 2 + 1] = b;
  }
  bool ok = true;
  if (kb_hi > kb_lo) ok = tc::mbar_wait(&sh->acc_full, 0, status, abort_flag, 403);
  ok = __all_sync(0xffffffffu, ok);             // the tensor-memory load below is warp-collective
  tc::tc_fence_after();
  if (ok) {
    const int f = warp * 32 + lane;             // feature of this thread = tensor-memory lane
    // SwiGLU tiles: rows 0..63 are gate features, 64..127 the matching up features; an owner gets both halves
    const int NLh = NL / 2;
    const uint32_t owner = swiglu ? (uint32_t)((f & 63) / NLh) : (uint32_t)(f / NL);
    const int fl = swiglu ? (f >> 6) * NLh + (f & 63) % NLh : f % NL;
    const uint32_t base = tc::smem_u32(red) + (uint32_t)(((int)rank * NT) * NL + fl) * 4u;
#pragma unroll
    for (int c = 0; c < NT / 32; ++c) {
      uint32_t r[32];
      if (kb_hi > kb_lo) {
        tc::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + c * 32, r);
        tc::tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (split > 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) st_cluster_f32(base + (uint32_t)((c * 32 + j) * NL) * 4u, owner, __uint_as_float(r[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) red[(c * 32 + j) * NL + fl] = __uint_as_float(r[j]);
      }
    }
  }
  tc::tc_fence_before();
  if (split > 1) cluster_sync_all(); else __syncthreads();

  // ---- fixed-order sum over the K splits, normalisation scale, rotary embedding, residual, store ------------
  auto row_scale = [&](int m) -> float {
    if (!normed) return 1.f;
    const float a = stats[m * 2], b = stats[m * 2 + 1];
    const float r1 = rsqrtf(a / (float)K + epi.norm_eps);
    return epi.norm_double ? r1 * rsqrtf(r1 * r1 * b / (float)K + epi.norm_eps) : r1;
  };
  if (!*abort_flag && swiglu) {
    const int NLh = NL / 2, nf0 = n0 + (int)rank * NLh;
    if (vec) {                                     // 8 features per item: NLh is 8, 16, 32 or 64; swiglu_I % 8 == 0
      const int gpr = NLh / 8;
      for (int i = threadIdx.x; i < NT * gpr; i += THREADS) {
        const int m = i / gpr, p = (i % gpr) * 8;
        const int n = nf0 + p;
        if (m >= M || n >= epi.swiglu_I) continue;
        float g[8], u[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = u[j] = 0.f;
        for (int s = 0; s < split; ++s) {
          const float4 *r = reinterpret_cast<const float4 *>(red + ((size_t)s * NT + m) * NL + p);
          const float4 *q = reinterpret_cast<const float4 *>(red + ((size_t)s * NT + m) * NL + NLh + p);
          const float4 g0 = r[0], g1 = r[1], u0 = q[0], u1 = q[1];
          g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w; g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
          u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w; u[4] += u1.x; u[5] += u1.y; u[6] += u1.z; u[7] += u1.w;
        }
        const float sc = row_scale(m);
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gv = g[j] * sc;
          y[j] = gv / (1.0f + __expf(-gv)) * (u[j] * sc);
        }
        store_group<TO, 8>(C + (size_t)m * ldc + n, y);
      }
    } else {
      for (int i = threadIdx.x; i < NT * NLh; i += THREADS) {
        const int m = i / NLh, p = i % NLh;
        const int n = nf0 + p;
        if (m >= M || n >= epi.swiglu_I) continue;
        float g = 0.f, u = 0.f;
        for (int s = 0; s < split; ++s) {
          const float *r = red + ((size_t)s * NT + m) * NL;
          g += r[p]; u += r[NLh + p];
        }
        const float sc = row_scale(m);
        g *= sc; u *= sc;
        const float sig = 1.0f / (1.0f + __expf(-g));
        C[(size_t)m * ldc + n] = from_f<TO>(g * sig * u);
      }
    }
  } else if (!*abort_flag) {
    const int gpr = NL / 4, nf0 = n0 + (int)rank * NL;      // 4 features per item (NL is 16 ... 128): gpr lanes per row
    const TO *res = reinterpret_cast<const TO *>(epi.residual);
    const bf16 *nw = reinterpret_cast<const bf16 *>(epi.next_norm_w);
    for (int i0 = 0; i0 < NT * gpr; i0 += THREADS) {         // NT * gpr is a multiple of 128: no thread leaves early
      const int i = i0 + threadIdx.x;
      const int m = i / gpr, p = (i % gpr) * 4;
      const int n = nf0 + p;
      const bool live = m < M && n < N;
      const bool whole = vec && n + 4 <= N;
      // independent of the sums: issue first
      float rv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
      if (live && res) {
        if (whole) load_group<TO, 4>(res + (size_t)m * epi.ld_res + n, rv);
        else for (int j = 0; j < 4 && n + j < N; ++j) rv[j] = to_f(res[(size_t)m * epi.ld_res + n + j]);
      }
      if (live && nw) {
        if (whole) load_group<bf16, 4>(nw + n, wv);
        else for (int j = 0; j < 4 && n + j < N; ++j) wv[j] = to_f(nw[n + j]);
      }
      const bool rot = live && epi.cos_t != nullptr && n < epi.cols;   // cols, hd and n are even
      float2 cv = make_float2(1.f, 1.f), sv = make_float2(0.f, 0.f);
      if (rot) {
        const int prow = epi.pos_dev ? pos_row : m % epi.S;
        const size_t tab = (size_t)prow * (epi.hd >> 1) + ((n % epi.hd) >> 1);
        cv.x = __ldg(epi.cos_t + tab); sv.x = __ldg(epi.sin_t + tab);
        if (n + 2 < epi.cols) {
          const size_t tab1 = (size_t)prow * (epi.hd >> 1) + (((n + 2) % epi.hd) >> 1);
          cv.y = __ldg(epi.cos_t + tab1); sv.y = __ldg(epi.sin_t + tab1);
        }
      }
      float x[4] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        for (int s = 0; s < split; ++s) {
          const float4 v = *reinterpret_cast<const float4 *>(red + ((size_t)s * NT + m) * NL + p);
          x[0] += v.x; x[1] += v.y; x[2] += v.z; x[3] += v.w;
        }
        const float sc = row_scale(m);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] *= sc;
        if (rot) {
          const float y0 = x[0] * cv.x - x[1] * sv.x, y1 = x[0] * sv.x + x[1] * cv.x;
          const float y2 = x[2] * cv.y - x[3] * sv.y, y3 = x[2] * sv.y + x[3] * cv.y;
          x[0] = y0; x[1] = y1; x[2] = y2; x[3] = y3;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] += rv[j];
        TO *dst = C + (size_t)m * ldc + n;
        if (whole) store_group<TO, 4>(dst, x);
        else for (int j = 0; j < 4 && n + j < N; ++j) dst[j] = from_f<TO>(x[j]);
      }
      if (nw) {
        // the next normalisation, as far as this CTA's columns go: h as stored (rounded), h * w rounded, their squares
        float s1 = 0.f, s2 = 0.f, y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float h = (live && n + j < N) ? to_f(from_f<TO>(x[j])) : 0.f;
          y[j] = __bfloat162float(__float2bfloat16_rn(h * wv[j]));
          s1 = fmaf(h, h, s1); s2 = fmaf(y[j], y[j], s2);
        }
        if (live) {
          bf16 *xd = reinterpret_cast<bf16 *>(epi.xw_out) + (size_t)m * epi.ld_xw + n;
          if (whole) store_group<bf16, 4>(xd, y);
          else for (int j = 0; j < 4 && n + j < N; ++j) xd[j] = __float2bfloat16_rn(y[j]);
        }
        for (int o = 1; o < gpr; o <<= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
        if ((threadIdx.x & (gpr - 1)) == 0 && m < M) {
          atomicAdd(epi.stat_acc + m * 2, (unsigned long long)(s1 * 4294967296.0f));
          atomicAdd(epi.stat_acc + m * 2 + 1, (unsigned long long)(s2 * 4294967296.0f));
        }
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 64);
  }
}

template <int NT, class TO>
int launch(b200_ctx *ctx, const CUtensorMap &mw, const CUtensorMap &ma, void *C, int M, int N, int K, size_t ldc, int split,
           const GemmEpilogue &epi) {
  const size_t esz = sizeof(TO);
  const int vec = (uintptr_t)C % 16 == 0 && (ldc * esz) % 16 == 0 &&
                  (!epi.residual || ((uintptr_t)epi.residual % 16 == 0 && (epi.ld_res * esz) % 16 == 0)) &&
                  (!epi.next_norm_w || (((uintptr_t)epi.next_norm_w | (uintptr_t)epi.xw_out) % 16 == 0 && (epi.ld_xw * 2) % 16 == 0));
  auto kern = gemm_skinny_kernel<NT, TO>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(NT)));
    attr_set = true;
  }
  const int ft = epi.swiglu_I > 0 ? FT / 2 : FT;
  B200_CUDA(ctx, launch_k(ctx, kern, dim3(((N + ft - 1) / ft) * split), dim3(THREADS), (size_t)smem_bytes(NT), split, mw, ma, (TO *)C, M, N, K, ldc, split, ctx->dev_status, epi, vec));
  B200_LAUNCHED(ctx);
  return B200_OK;
}

}  // namespace

// K split: as many CTAs per feature tile as keep the grid within two CTAs per SM, each with >= 4 K slices
static int k_split(const b200_ctx *ctx, int tiles, int num_kb) {
  int split = 1;
  while (split < 8 && tiles * split * 2 <= 2 * ctx->sm_count && num_kb >= split * 4) split *= 2;
  return split;
}
bool gemm_skinny_supported(size_t M, int ta, int tb, int acc) { return M > 0 && M <= 64 && !ta && !tb && !acc; }

int gemm_skinny_launch(b200_ctx *ctx, const void *A, const void *W, void *C, size_t M, size_t N, size_t K, b200_dtype out_dt,
                       size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi_in) {
  GemmEpilogue epi;
  if (epi_in) {
    epi = *epi_in;
    B200_REQUIRE(ctx, epi.swiglu_I > 0 || epi.row_acc || epi.residual || epi.next_norm_w || (epi.cos_t && epi.sin_t && epi.S > 0), "gemm: unsupported fused epilogue");
    B200_REQUIRE(ctx, !epi.cos_t || (epi.sin_t && epi.S > 0 && epi.hd % 2 == 0 && epi.cols % 2 == 0), "gemm: unsupported fused rotary epilogue");
    B200_REQUIRE(ctx, !epi.residual || (!epi.swiglu_I && epi.ld_res >= N), "gemm: the residual epilogue needs a plain product");
    B200_REQUIRE(ctx, !epi.next_norm_w || (!epi.swiglu_I && out_dt == B200_BF16 && epi.xw_out && epi.stat_acc && epi.ld_xw >= N),
                 "gemm: the producer half of the folded normalisation needs a plain bf16 product, an output for h*w and one for the row sums");
  }
  const int nt = M <= 32 ? 32 : 64;
  CUtensorMap mw, ma;
  int r = tc_make_map_2d(&mw, W, N, K, ldb * 2, 64, BK);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(W) failed: %d", r);
  r = tc_make_map_2d(&ma, A, K, M, lda * 2, BK, nt);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed: %d", r);
  if (epi.swiglu_I > 0) {
    B200_REQUIRE(ctx, !epi.cos_t && (size_t)epi.swiglu_I * 2 == N && epi.swiglu_I % 8 == 0, "gemm: the SwiGLU epilogue needs W = [gate | up] with N = 2 I");
    N = (size_t)epi.swiglu_I;                      // output width
  }
  const int tiles = (int)((N + (epi.swiglu_I > 0 ? FT / 2 : FT) - 1) / (epi.swiglu_I > 0 ? FT / 2 : FT)), num_kb = (int)((K + BK - 1) / BK);
  const int split = k_split(ctx, tiles, num_kb);
  const int m = (int)M, n = (int)N, k = (int)K;
  if (nt == 32) {
    if (out_dt == B200_BF16) return launch<32, bf16>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
    return launch<32, float>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
  }
  if (out_dt == B200_BF16) return launch<64, bf16>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
  return launch<64, float>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
}
