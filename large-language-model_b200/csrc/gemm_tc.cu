// bf16 tensor-core GEMM for sm_100a: C[M,N] (+)= op(A)[M,K] * op(B)[K,N],
// fp32 accumulation in tensor memory, bf16 or fp32 output.
// Replaces metal_bridge::gemm_bf16 and its NT / TN aliases
// (cpp/include/gpu_kernel/MetalBridge.hpp:39-42, 119-122).
//
// Design (one persistent CTA per SM, 192 threads):
//   warp 0        TMA producer: 128-byte-swizzled A/B tiles, 64-deep K slices, STAGES-deep ring
//   warp 1        allocates tensor memory; one lane issues tcgen05.mma 128x256x16
//   warps 2..5    epilogue: tcgen05.ld 32 columns at a time -> convert -> 16-byte global stores
//   tensor memory holds two 128x256 fp32 accumulators, so the epilogue of tile i overlaps
//   the main loop of tile i+1.
// Operand majorness is handled in the descriptors, not by copying:
//   A stored [M,K] -> K-major; stored [K,M] (trans_a, weight-gradient GEMMs) -> MN-major
//   B stored [N,K] (trans_b, data-gradient GEMMs) -> K-major; stored [K,N] (forward) -> MN-major
// Ragged M/N/K edges are zero-filled by TMA and masked in the epilogue.
#include "common.cuh"
#include "tc_common.cuh"
#include <cudaTypedefs.h>
#include <mutex>

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int CHUNK_BYTES = 64 * BK * 2;     // one [64 MN x 64 K] MN-major chunk = 8 KiB
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
constexpr int THREADS = 192;
constexpr int GROUP_M = 16;                  // m-tiles per rasterisation group

struct SharedTail {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <bool A_MN, bool B_MN, class TO, bool ACC>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               TO *__restrict__ C, int M, int N, int K, size_t ldc, int *status, GemmEpilogue epi) {
  // MN-major descriptor fields (bytes): stride between 64-wide chunks, 8-row group stride, advance per 16-deep MMA
  constexpr uint32_t mn_lbo = CHUNK_BYTES, mn_sbo = 1024, mn_kadv = 2048;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sA = smem, *sB = smem + STAGES * A_STAGE_BYTES;
  SharedTail *sh = (SharedTail *)(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, total = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { tc::mbar_init(&sh->full[i], 1); tc::mbar_init(&sh->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&sh->acc_full[i], 1); tc::mbar_init(&sh->acc_empty[i], 4); }
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
    tc::tma_prefetch_desc(&map_a);
    tc::tma_prefetch_desc(&map_b);
  }
  if (warp == 1) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  auto tile_coords = [&](int t, int &tm, int &tn) {
    int per_group = GROUP_M * tiles_n;
    int g = t / per_group, r = t % per_group;
    int gm = min(GROUP_M, tiles_m - g * GROUP_M);
    tm = g * GROUP_M + r % gm;
    tn = r / gm;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int tm, tn; tile_coords(t, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1, status, abort_flag, 101)) { ok = false; break; }
          tc::mbar_expect_tx(&sh->full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t *a = sA + stage * A_STAGE_BYTES, *b = sB + stage * B_STAGE_BYTES;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tc::tma_load_2d(a + c * CHUNK_BYTES, &map_a, tm * BM + c * 64, kb * BK, &sh->full[stage]);
          } else {
            tc::tma_load_2d(a, &map_a, kb * BK, tm * BM, &sh->full[stage]);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tc::tma_load_2d(b + c * CHUNK_BYTES, &map_b, tn * BN + c * 64, kb * BK, &sh->full[stage]);
          } else {
            tc::tma_load_2d(b, &map_b, kb * BK, tn * BN, &sh->full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {   // let copies already in flight land before the CTA's shared memory is released
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        if (!tc::mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, status, abort_flag, 102)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&sh->full[stage], phase, status, abort_flag, 103)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t a_addr = tc::smem_u32(sA + stage * A_STAGE_BYTES), b_addr = tc::smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 bf16 = 32 B further along the swizzled row; MN-major: 16 K-rows = 2 KiB further
            uint64_t da = A_MN ? tc::make_smem_desc(a_addr + k * mn_kadv, mn_lbo, mn_sbo) : tc::make_smem_desc(a_addr + k * 32, 16, 1024);
            uint64_t db = B_MN ? tc::make_smem_desc(b_addr + k * mn_kadv, mn_lbo, mn_sbo) : tc::make_smem_desc(b_addr + k * 32, 16, 1024);
            tc::umma_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc::umma_commit(&sh->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&sh->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int tm, tn; tile_coords(t, tm, tn);
      if (!tc::mbar_wait(&sh->acc_full[acc], acc_phase, status, abort_flag, 104)) { ok = false; break; }
      tc::tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      TO *crow = C + (size_t)row * ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + c * 32, r);
        tc::tmem_ld_wait();
        const int col = tn * BN + c * 32;
        if (row < M && col < N) {
          if (col + 32 <= N) {
            if constexpr (sizeof(TO) == 2) {
              if (epi.cos_t != nullptr && col < epi.cols) {
                // fused rotary embedding on the fp32 accumulators: 16 interleaved pairs of this 32-column chunk
                const int half = epi.hd >> 1;
                const size_t tab = (size_t)(row % epi.S) * half + ((col % epi.hd) >> 1);
                const float4 *c4 = reinterpret_cast<const float4 *>(epi.cos_t + tab), *s4 = reinterpret_cast<const float4 *>(epi.sin_t + tab);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const float4 cc = __ldg(c4 + g), ss = __ldg(s4 + g);
                  const float cv[4] = {cc.x, cc.y, cc.z, cc.w}, sv[4] = {ss.x, ss.y, ss.z, ss.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float x0 = __uint_as_float(r[g * 8 + 2 * j]), x1 = __uint_as_float(r[g * 8 + 2 * j + 1]);
                    r[g * 8 + 2 * j] = __float_as_uint(x0 * cv[j] - x1 * sv[j]);
                    r[g * 8 + 2 * j + 1] = __float_as_uint(x0 * sv[j] + x1 * cv[j]);
                  }
                }
              }
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                uint32_t *po = &o.x;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                  po[j] = *reinterpret_cast<uint32_t *>(&h);
                }
                *reinterpret_cast<uint4 *>(crow + col + v * 8) = o;
              }
            } else {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
                if (ACC) {
                  float4 p = *reinterpret_cast<const float4 *>(crow + col + v * 4);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4 *>(crow + col + v * 4) = o;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < N) {
                float v = __uint_as_float(r[j]);
                if (ACC) v += to_f(crow[col + j]);
                crow[col + j] = from_f<TO>(v);
              }
            }
          }
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_encode_once;

void load_encode() {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
}

template <bool A_MN, bool B_MN, class TO, bool ACC>
int launch_variant(b200_ctx *ctx, const CUtensorMap &ma, const CUtensorMap &mb, void *C, int M, int N, int K,
                   size_t ldc, const GemmEpilogue &epi) {
  auto kern = gemm_tc_kernel<A_MN, B_MN, TO, ACC>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set = true;
  }
  int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  b200_ctx::Timed tm{};
  if (ctx->time_gemm) {
    auto ev = [&]() { cudaEvent_t e; if (ctx->event_pool.empty()) cudaEventCreate(&e); else { e = ctx->event_pool.back(); ctx->event_pool.pop_back(); } return e; };
    tm.start = ev(); tm.stop = ev(); tm.flops = 2.0 * M * N * K;
    cudaEventRecord(tm.start, ctx->stream);
  }
  kern<<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(ma, mb, (TO *)C, M, N, K, ldc, ctx->dev_status, epi);
  B200_LAUNCHED(ctx);
  if (ctx->time_gemm) { cudaEventRecord(tm.stop, ctx->stream); ctx->timed.push_back(tm); }
  return B200_OK;
}

template <bool A_MN, bool B_MN>
int launch_out(b200_ctx *ctx, const CUtensorMap &ma, const CUtensorMap &mb, void *C, int M, int N, int K, size_t ldc,
               b200_dtype out_dt, int acc, const GemmEpilogue &epi) {
  if (out_dt == B200_BF16) return launch_variant<A_MN, B_MN, bf16, false>(ctx, ma, mb, C, M, N, K, ldc, epi);
  if (acc) return launch_variant<A_MN, B_MN, float, true>(ctx, ma, mb, C, M, N, K, ldc, epi);
  return launch_variant<A_MN, B_MN, float, false>(ctx, ma, mb, C, M, N, K, ldc, epi);
}

}  // namespace

int tc_make_map_2d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
int tc_make_map_store_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base),
                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        elem_bytes == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
int tc_make_map_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                   uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int tc_make_map_4d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes, uint32_t box0, uint32_t box1) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
  cuuint32_t box[4] = {box0, box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int tc_make_map_f32_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                       uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

bool gemm_tc_supported(const void *A, const void *B, const void *C, size_t M, size_t N, size_t K, size_t lda,
                       size_t ldb, size_t ldc, b200_dtype out_dt) {
  if (M == 0 || N == 0 || K == 0) return false;
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return false;
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) % 16) return false;
  if ((lda * 2) % 16 || (ldb * 2) % 16) return false;             // TMA global strides
  if ((ldc * dtype_size(out_dt)) % 16) return false;              // vector epilogue stores
  return true;
}

int gemm_tc_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                   int acc, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi_in) {
  B200_REQUIRE(ctx, !(acc && out_dt == B200_BF16), "gemm: accumulate needs an fp32 C on the tensor-core path");
  GemmEpilogue epi;
  if (epi_in) {
    epi = *epi_in;
    B200_REQUIRE(ctx, out_dt == B200_BF16 && epi.cos_t && epi.sin_t && epi.S > 0 && epi.hd % 32 == 0 && epi.cols % 32 == 0 &&
                 ((uintptr_t)epi.cos_t | (uintptr_t)epi.sin_t) % 16 == 0, "gemm: unsupported fused rotary epilogue");
  }
  CUtensorMap ma, mb;
  int r;
  // A: stored [M,K] (K inner) or, transposed, [K,M] (M inner)
  if (!ta) r = tc_make_map_2d(&ma, A, K, M, lda * 2, BK, BM);
  else r = tc_make_map_2d(&ma, A, M, K, lda * 2, 64, BK);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed: %d", r);
  // B: stored [K,N] (N inner) or, transposed, [N,K] (K inner)
  if (!tb) r = tc_make_map_2d(&mb, B, N, K, ldb * 2, 64, BK);
  else r = tc_make_map_2d(&mb, B, K, N, ldb * 2, BK, BN);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed: %d", r);
  const bool a_mn = ta != 0, b_mn = tb == 0;
  int m = (int)M, n = (int)N, k = (int)K;
  if (a_mn && b_mn) return launch_out<true, true>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  if (a_mn && !b_mn) return launch_out<true, false>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  if (!a_mn && b_mn) return launch_out<false, true>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  return launch_out<false, false>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
}

// ---- test hook for the bounded-wait error path (not part of the public header) -----------------------------------
// One thread waits on an mbarrier that nothing ever arrives on, with a limit of `limit_cycles` SM clocks (about a
// millisecond in the test).  The wait gives up, records code 199 in the context's device status word and the kernel
// returns normally: the next b200_sync reports B200_ERR_DEVICE_WAIT and the context stays usable.  This is the same
// mbar_wait every tensor-core kernel uses, so the test covers the give-up path without faulting or hanging anything.
namespace {
__global__ void wait_probe_kernel(int *status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
    tc::mbar_wait(&bar, 0, status, &abort_flag, 199, limit_cycles);
  }
}
}  // namespace
extern "C" int b200_internal_wait_probe(b200_ctx *ctx, long long limit_cycles) {
  if (!ctx) return B200_ERR_INVALID;
  B200_REQUIRE(ctx, limit_cycles > 0 && limit_cycles <= 200000000ll, "wait_probe: limit must be at most 2e8 cycles");
  wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, limit_cycles);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
