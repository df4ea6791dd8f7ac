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
__host__ __device__ constexpr int smem_bytes(int nt) {
  return STAGES * (W_STAGE_BYTES + a_stage_bytes(nt)) + FT * nt * 4 + 1024 /*align*/ + 128 /*barriers*/;
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

// NT = padded row count of A (32 or 64) = N of the MMA and width of the accumulator in tensor memory.
template <int NT, class TO>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   TO *__restrict__ C, int M, int N, int K, size_t ldc, int split, int *status, GemmEpilogue epi) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sW = smem, *sA = smem + STAGES * W_STAGE_BYTES;
  float *red = (float *)(sA + STAGES * a_stage_bytes(NT));          // [split][NT][FT/split]
  Tail *sh = (Tail *)((uint8_t *)red + FT * NT * 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = split > 1 ? cluster_rank() : 0;
  const int tile = blockIdx.x / split;
  const bool swiglu = epi.swiglu_I > 0;
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
  if (split > 1) cluster_wait_all();

  // ---- epilogue: tensor memory -> the owning CTA's shared memory ------------------------------
  const int NL = FT / split;                    // features owned per CTA
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

  // ---- fixed-order sum over the K splits, optional rotary embedding, store ---------------------
  if (!*abort_flag && swiglu) {
    const int NLh = NL / 2, nf0 = n0 + (int)rank * NLh;
    for (int i = threadIdx.x; i < NT * NLh; i += THREADS) {
      const int m = i / NLh, p = i % NLh;
      const int n = nf0 + p;
      if (m >= M || n >= epi.swiglu_I) continue;
      float g = 0.f, u = 0.f;
      for (int s = 0; s < split; ++s) {
        const float *r = red + ((size_t)s * NT + m) * NL;
        g += r[p]; u += r[NLh + p];
      }
      const float sig = 1.0f / (1.0f + __expf(-g));
      C[(size_t)m * ldc + n] = from_f<TO>(g * sig * u);
    }
  } else if (!*abort_flag) {
    const int pairs = NL / 2, nf0 = n0 + (int)rank * NL;
    for (int i = threadIdx.x; i < NT * pairs; i += THREADS) {
      const int m = i / pairs, p = i % pairs;
      const int n = nf0 + 2 * p;
      if (m >= M || n >= N) continue;
      float x0 = 0.f, x1 = 0.f;
      for (int s = 0; s < split; ++s) {
        const float2 v = *reinterpret_cast<const float2 *>(red + ((size_t)s * NT + m) * NL + 2 * p);
        x0 += v.x; x1 += v.y;
      }
      if (epi.cos_t != nullptr && n < epi.cols) {
        const int prow = epi.pos_dev ? *epi.pos_dev : m % epi.S;
        const size_t tab = (size_t)prow * (epi.hd >> 1) + ((n % epi.hd) >> 1);
        const float cv = __ldg(epi.cos_t + tab), sv = __ldg(epi.sin_t + tab);
        const float y0 = x0 * cv - x1 * sv, y1 = x0 * sv + x1 * cv;
        x0 = y0; x1 = y1;
      }
      TO *dst = C + (size_t)m * ldc + n;
      if (n + 1 < N) {
        if constexpr (sizeof(TO) == 2) *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(x0, x1);
        else *reinterpret_cast<float2 *>(dst) = make_float2(x0, x1);
      } else {
        dst[0] = from_f<TO>(x0);
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
  auto kern = gemm_skinny_kernel<NT, TO>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(NT)));
    attr_set = true;
  }
  const int ft = epi.swiglu_I > 0 ? FT / 2 : FT;
  B200_CUDA(ctx, launch_k(ctx, kern, dim3(((N + ft - 1) / ft) * split), dim3(THREADS), (size_t)smem_bytes(NT), split, mw, ma, (TO *)C, M, N, K, ldc, split, ctx->dev_status, epi));
  B200_LAUNCHED(ctx);
  return B200_OK;
}

}  // namespace

bool gemm_skinny_supported(size_t M, int ta, int tb, int acc) { return M > 0 && M <= 64 && !ta && !tb && !acc; }

int gemm_skinny_launch(b200_ctx *ctx, const void *A, const void *W, void *C, size_t M, size_t N, size_t K, b200_dtype out_dt,
                       size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi_in) {
  GemmEpilogue epi;
  if (epi_in) {
    epi = *epi_in;
    B200_REQUIRE(ctx, epi.swiglu_I > 0 || (epi.cos_t && epi.sin_t && epi.S > 0 && epi.hd % 2 == 0 && epi.cols % 2 == 0), "gemm: unsupported fused epilogue");
  }
  const int nt = M <= 32 ? 32 : 64;
  CUtensorMap mw, ma;
  int r = tc_make_map_2d(&mw, W, N, K, ldb * 2, 64, BK);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(W) failed: %d", r);
  r = tc_make_map_2d(&ma, A, K, M, lda * 2, BK, nt);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed: %d", r);
  // K split: as many CTAs per feature tile as keep the grid within two CTAs per SM, each with >= 2 K slices
  if (epi.swiglu_I > 0) {
    B200_REQUIRE(ctx, !epi.cos_t && (size_t)epi.swiglu_I * 2 == N && epi.swiglu_I % 8 == 0, "gemm: the SwiGLU epilogue needs W = [gate | up] with N = 2 I");
    N = (size_t)epi.swiglu_I;                      // output width
  }
  const int tiles = (int)((N + (epi.swiglu_I > 0 ? FT / 2 : FT) - 1) / (epi.swiglu_I > 0 ? FT / 2 : FT)), num_kb = (int)((K + BK - 1) / BK);
  int split = 1;
  while (split < 8 && tiles * split * 2 <= 2 * ctx->sm_count && num_kb >= split * 4) split *= 2;
  const int m = (int)M, n = (int)N, k = (int)K;
  if (nt == 32) {
    if (out_dt == B200_BF16) return launch<32, bf16>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
    return launch<32, float>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
  }
  if (out_dt == B200_BF16) return launch<64, bf16>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
  return launch<64, float>(ctx, mw, ma, C, m, n, k, ldc, split, epi);
}
