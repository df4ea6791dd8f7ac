// Two-CTA form of the bf16 tensor-core GEMM (tcgen05 cta_group::2): a cluster of two CTAs on one
// SM pair computes a 256x256 output tile.  Each CTA stages its own 128 rows of A and only HALF of the
// B tile (128 of the 256 columns); the pair's tensor cores read both halves, so the shared-memory
// fill per SM drops from 48 KiB to 32 KiB per 64-deep K slice (the single-CTA kernel is bound by that
// fill bandwidth) and the ring deepens from 4 to 6 stages.
//   both CTAs:  warp 0 = TMA producer (loads signal the LEADER's "full" barrier),
//               warps 2..5 = epilogue of the CTA's own 128 accumulator rows
//   leader CTA: warp 1 lane 0 issues tcgen05.mma.cta_group::2 (M = 256) and commits completion to the
//               "empty" / "accumulator full" barriers of both CTAs
// Same operand handling as gemm_tc.cu (K-major / MN-major through descriptors, ragged edges by TMA
// zero fill), same optional rotary epilogue.  No load uses multicast; the only cross-CTA traffic is
// mbarrier arrivals and the tensor cores reading the peer's B half.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KiB: this CTA's 128 rows
constexpr int B_STAGE_BYTES = (BN / 2) * BK * 2;  // 16 KiB: this CTA's half of the 256 columns
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int STORE_STAGE_BYTES = 2 * 32 * 128;   // per epilogue warp: two boxes of 32 rows x 128 B for the result stores
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 + 1024 + 4 * STORE_STAGE_BYTES;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;                        // 256-row tile pairs per rasterisation group
constexpr uint32_t LEADER_MASK = 0xFEFFFFFFu;     // clears the CTA-rank bit of a shared::cluster address (rank 0)
constexpr uint32_t PEER_BIT = 0x01000000u;        // rank 1 of the pair

struct SharedTail {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_2sm(void *dst, const CUtensorMap *map, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(tc::smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_ss_2sm(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// completion of everything issued so far -> the same barrier in both CTAs of the pair
__device__ __forceinline__ void umma_commit_both(uint64_t *bar) {
  const uint32_t a = tc::smem_u32(bar) & LEADER_MASK;
  umma_commit_2sm(a);
  umma_commit_2sm(a | PEER_BIT);
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t *dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void red_add_v4(float *p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// Rotary embedding of one 32-column chunk of an accumulator row (cpp/src/Positional.cpp:120-147): the 16 (cos, sin)
// pairs of the chunk are fetched by rope_fetch -- early, so that their latency hides behind the wait for the accumulator
// or the previous chunk's arithmetic -- and applied by rope_apply to the fp32 values before they are rounded.
struct RopeVals { float4 c[4], s[4]; };
__device__ __forceinline__ bool rope_wanted(const GemmEpilogue &epi, int row, int col, int M, int N) {
  return epi.cos_t != nullptr && col < epi.cols && col + 32 <= N && row < M;
}
__device__ __forceinline__ void rope_fetch(RopeVals &v, const GemmEpilogue &epi, int row, int col) {
  const int half = epi.hd >> 1;
  const size_t tab = (size_t)(row % epi.S) * half + ((col % epi.hd) >> 1);
  const float4 *c4 = reinterpret_cast<const float4 *>(epi.cos_t + tab), *s4 = reinterpret_cast<const float4 *>(epi.sin_t + tab);
#pragma unroll
  for (int g = 0; g < 4; ++g) { v.c[g] = __ldg(c4 + g); v.s[g] = __ldg(s4 + g); }
}
__device__ __forceinline__ void rope_apply(uint32_t (&r)[32], const RopeVals &v) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const float cv[4] = {v.c[g].x, v.c[g].y, v.c[g].z, v.c[g].w}, sv[4] = {v.s[g].x, v.s[g].y, v.s[g].z, v.s[g].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x0 = __uint_as_float(r[g * 8 + 2 * j]), x1 = __uint_as_float(r[g * 8 + 2 * j + 1]);
      r[g * 8 + 2 * j] = __float_as_uint(x0 * cv[j] - x1 * sv[j]);
      r[g * 8 + 2 * j + 1] = __float_as_uint(x0 * sv[j] + x1 * cv[j]);
    }
  }
}
// Result stores.  An epilogue thread owns one accumulator ROW; written directly, one warp store instruction would touch
// 32 rows with 16 bytes each (32 half-used sectors) -- measured, those stores, not the MMAs, bounded the kernel (a 756 GFLOP
// GEMM took 0.49 ms without them, 0.55 ms with its bf16 result, 0.64 ms with a third output).  So each warp transposes
// its 32-row chunk through a private, swizzled shared-memory buffer and writes whole row segments: one instruction covers
// 8 rows x 64 B (bf16) or 4 rows x 128 B (fp32).  All 32 lanes must call; rows at or beyond rows_valid are not written.
// base points at (first row of the warp, first column of the chunk).
using tc::stage_store_bf16;
__device__ __forceinline__ void pack_chunk_bf16(const uint32_t (&r)[32], uint4 (&v)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t *po = &v[k].x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[k * 8 + 2 * j]), __uint_as_float(r[k * 8 + 2 * j + 1]));
      po[j] = *reinterpret_cast<uint32_t *>(&h);
    }
  }
}
// Bulk-store route of a warp: its boxes alternate between two 4 KiB buffers; a buffer is rewritten only after the bulk
// store issued from it two boxes ago has finished reading it.  Box layout = the tensor map's swizzle (64-byte for bf16
// rows of 64 B, 128-byte for fp32 rows of 128 B), which is also what makes the st.shared of 32 rows conflict-free.
struct BulkOut {
  uint8_t *buf;      // 1024-byte aligned, 2 x 4096 bytes; null: the route is off
  int n;             // boxes issued so far
};
__device__ __forceinline__ uint8_t *bulk_box_begin(BulkOut &o, int lane) {
  if (lane == 0) tc::bulk_wait_read<1>();
  __syncwarp();
  return o.buf + (o.n & 1) * 4096;
}
__device__ __forceinline__ void bulk_box_issue(BulkOut &o, int lane, const uint8_t *box, const CUtensorMap *map, int col, int row, bool add) {
  tc::fence_proxy_async();           // this thread's st.shared become visible to the bulk-copy engine
  __syncwarp();
  if (lane == 0) {
    if (add) tc::tma_reduce_add_2d(map, box, col, row); else tc::tma_store_2d(map, box, col, row);
    tc::bulk_commit();
  }
  ++o.n;
}
__device__ __forceinline__ void bulk_store_bf16(BulkOut &o, int lane, const uint4 (&v)[4], const CUtensorMap *map, int col, int row) {
  uint8_t *box = bulk_box_begin(o, lane);
#pragma unroll
  for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4 *>(box + lane * 64 + ((k ^ ((lane >> 1) & 3)) << 4)) = v[k];
  bulk_box_issue(o, lane, box, map, col, row, false);
}
// One 32-column chunk of the warp's 32 accumulator rows -> global memory.  Warp-collective: every lane calls it with its
// own row's values (lane = row - row0); `red`: this tile is one K-split of several -> add into C with vector reductions.
template <class TO, bool ACC>
__device__ __forceinline__ void store_chunk(uint32_t (&r)[32], TO *C, size_t ldc, int row0, int lane, int col, int M, int N,
                                            uint8_t *stg, bool red, BulkOut &bo, const CUtensorMap *map_c) {
  if (bo.buf) {                     // bulk tensor store: clipped at the edges of C by the copy engine
    if (row0 >= M) return;
    if constexpr (sizeof(TO) == 2) {
      uint4 v[4];
      pack_chunk_bf16(r, v);
      bulk_store_bf16(bo, lane, v, map_c, col, row0);
    } else {
      uint8_t *box = bulk_box_begin(bo, lane);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        *reinterpret_cast<uint4 *>(box + lane * 128 + ((k ^ (lane & 7)) << 4)) = make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
      bulk_box_issue(bo, lane, box, map_c, col, row0, red || ACC);
    }
    return;
  }
  const int rows_valid = M - row0;
  if (col + 32 <= N) {
    if constexpr (sizeof(TO) == 2) {
      uint4 v[4];
      pack_chunk_bf16(r, v);
      stage_store_bf16(stg, lane, v, reinterpret_cast<bf16 *>(C) + (size_t)row0 * ldc + col, ldc, rows_valid);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        *reinterpret_cast<uint4 *>(stg + lane * 128 + ((k ^ (lane & 7)) << 4)) = make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
      __syncwarp();
      float *base = reinterpret_cast<float *>(C) + (size_t)row0 * ldc + col;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), w = lane & 7;
        const uint4 x = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((w ^ (rr & 7)) << 4));
        if (rr < rows_valid) {
          float *p = base + (size_t)rr * ldc + w * 4;
          float4 o = make_float4(__uint_as_float(x.x), __uint_as_float(x.y), __uint_as_float(x.z), __uint_as_float(x.w));
          if (red) { red_add_v4(p, o.x, o.y, o.z, o.w); continue; }
          if (ACC) { const float4 q = *reinterpret_cast<const float4 *>(p); o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w; }
          *reinterpret_cast<float4 *>(p) = o;
        }
      }
      __syncwarp();
    }
  } else if (lane < rows_valid) {
    // ragged last columns: each thread writes its own row element by element
    TO *crow = C + (size_t)(row0 + lane) * ldc;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col + j < N) {
        float v = __uint_as_float(r[j]);
        if constexpr (sizeof(TO) == 4) {
          if (red) { atomicAdd(reinterpret_cast<float *>(crow + col + j), v); continue; }
        }
        if (ACC) v += to_f(crow[col + j]);
        crow[col + j] = from_f<TO>(v);
      }
    }
  }
}

__device__ __forceinline__ float tanh_approx(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
constexpr float LOG2E = 1.4426950408889634f;

// Cross-entropy epilogue of one accumulator row (one thread) over the 256 columns of a tile; see GemmEpilogue::ce_mode.
// Softmax statistics are kept in base-2 units (x * log2e): one FMA and one ex2 per element.
__device__ __forceinline__ void ce_row_epilogue(uint32_t taddr, bf16 *C, size_t ldc, int row0, int lane, int tn, int M, int N,
                                                const GemmEpilogue &epi, uint8_t *stg, BulkOut &bo, const CUtensorMap *map_c) {
  const int row = row0 + lane;
  const bool row_ok = row < M;
  const uint32_t tgt = row_ok ? __ldg(epi.ce_targets + row) : 0xffffffffu;
  const int col0 = tn * BN;
  if (epi.ce_mode == 3) {
    const float lse2 = row_ok ? __ldg(epi.ce_lse + row) * LOG2E : 0.f;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      __syncwarp();                 // rows past M skip the arithmetic below; the tensor-memory load wants the whole warp
      tc::tmem_ld_32x32(taddr + c * 32, r);
      tc::tmem_ld_wait();
      const int col = col0 + c * 32;
      if (col < N) {
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float p = ex2(fmaf(__uint_as_float(r[j]), LOG2E, -lse2));
            if ((uint32_t)(col + j) == tgt) p -= 1.0f;
            r[j] = __float_as_uint(p * epi.ce_scale);
          }
        }
        store_chunk<bf16, false>(r, C, ldc, row0, lane, col, M, N, stg, false, bo, map_c);
      }
    }
    return;
  }
  float m2 = -1e30f, s = 0.f, tl = 0.f;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    __syncwarp();
    tc::tmem_ld_32x32(taddr + c * 32, r);
    tc::tmem_ld_wait();
    const int col = col0 + c * 32;
    if (col >= N) continue;                                   // warp-uniform
    if (epi.ce_mode == 2) {
      // the stored logits are bf16: take the statistics from the rounded values, which is what a later pass reads back
      store_chunk<bf16, false>(r, C, ldc, row0, lane, col, M, N, stg, false, bo, map_c);
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j]))));
    }
    if (!row_ok) continue;
    if (tgt - (uint32_t)col < 32u) {
#pragma unroll
      for (int j = 0; j < 32; ++j) if ((uint32_t)(col + j) == tgt) tl = __uint_as_float(r[j]);
    }
    if (col + 32 > N) {             // ragged last chunk: columns past N hold the zero fill of the weight tile
#pragma unroll
      for (int j = 0; j < 32; ++j) if (col + j >= N) r[j] = __float_as_uint(-1e30f);
    }
    float t[32], cm = -1e30f;
#pragma unroll
    for (int j = 0; j < 32; ++j) { t[j] = __uint_as_float(r[j]) * LOG2E; cm = fmaxf(cm, t[j]); }
    const float mn = fmaxf(m2, cm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) acc += ex2(t[j] - mn);
    s = s * ex2(m2 - mn) + acc;
    m2 = mn;
  }
  if (row_ok) {
    epi.ce_part_max[(size_t)tn * M + row] = m2;
    epi.ce_part_sum[(size_t)tn * M + row] = s;
    if (tgt - (uint32_t)col0 < (uint32_t)BN && tgt < (uint32_t)N) epi.ce_tgt_logit[row] = tl;
  }
}

template <bool A_MN, bool B_MN, class TO, bool ACC>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_act,
                TO *__restrict__ C, int M, int N, int K, size_t ldc, int *status, GemmEpilogue epi, int splits, int bulk_store) {
  pdl_launch_dependents();             // the next kernel of the stream may be scheduled onto SMs as this grid leaves them
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sA = smem, *sB = smem + STAGES * A_STAGE_BYTES;
  SharedTail *sh = (SharedTail *)(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  // fused SwiGLU output: a tile is 128 gate columns (staged by the leader CTA) next to the matching 128 up columns
  // (staged by its peer), so one accumulator row holds both values of 128 activation features
  const bool swiglu = epi.swiglu_I > 0;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = swiglu ? (epi.swiglu_I + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN,
            total = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int items = total * splits;                 // work item = (tile pair, K split); all tiles of split 0 first
  volatile int *abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { tc::mbar_init(&sh->full[i], 1); tc::mbar_init(&sh->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&sh->acc_full[i], 1); tc::mbar_init(&sh->acc_empty[i], 8); }
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::fence_proxy_async();
    tc::tma_prefetch_desc(&map_a);
    tc::tma_prefetch_desc(&map_b);
  }
  if (warp == 1) tmem_alloc_2sm(&sh->tmem_base, 512);
  tc::tc_fence_before();
  __syncthreads();
  cluster_sync();                      // the peer's barriers are initialised before anything arrives on them
  tc::tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  // Everything above (barriers, tensor-memory allocation, descriptor prefetch) touched nothing another kernel owns and may
  // have overlapped the tail of the kernel before; from here on operands are read and results written.
  pdl_wait();

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
      for (int it = cluster_id; it < items && ok; it += n_clusters) {
        int tm, tn; tile_coords(it % total, tm, tn);
        const int sp = it / total, kb0 = sp * num_kb / splits, kb1 = (sp + 1) * num_kb / splits;
        const int m0 = tm * 2 * BM + (int)rank * BM;            // this CTA's rows
        const int n0 = swiglu ? tn * (BN / 2) + (int)rank * epi.swiglu_I       // gate columns | matching up columns
                              : tn * BN + (int)rank * (BN / 2);              // this CTA's half of the B columns
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1, status, abort_flag, 111)) { ok = false; break; }
          const uint32_t full_leader = tc::smem_u32(&sh->full[stage]) & LEADER_MASK;
          if (leader) tc::mbar_expect_tx(&sh->full[stage], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          uint8_t *a = sA + stage * A_STAGE_BYTES, *b = sB + stage * B_STAGE_BYTES;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_2sm(a + c * CHUNK_BYTES, &map_a, m0 + c * 64, kb * BK, full_leader);
          } else {
            tma_load_2d_2sm(a, &map_a, kb * BK, m0, full_leader);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c) tma_load_2d_2sm(b + c * CHUNK_BYTES, &map_b, n0 + c * 64, kb * BK, full_leader);
          } else {
            tma_load_2d_2sm(b, &map_b, kb * BK, n0, full_leader);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { long long t0 = clock64(); while (clock64() - t0 < 2000000ll) {} }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = tc::make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int it = cluster_id; it < items && ok; it += n_clusters) {
        const int sp = it / total, kb0 = sp * num_kb / splits, kb1 = (sp + 1) * num_kb / splits;
        if (!tc::mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, status, abort_flag, 112)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc::mbar_wait(&sh->full[stage], phase, status, abort_flag, 113)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t a_addr = tc::smem_u32(sA + stage * A_STAGE_BYTES), b_addr = tc::smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t da = A_MN ? tc::make_smem_desc(a_addr + k * 2048, CHUNK_BYTES, 1024) : tc::make_smem_desc(a_addr + k * 32, 16, 1024);
            uint64_t db = B_MN ? tc::make_smem_desc(b_addr + k * 2048, CHUNK_BYTES, 1024) : tc::make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_ss_2sm(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_both(&sh->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_both(&sh->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;                        // tensor-memory lane quarter this warp may read
    uint8_t *stg = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 + (warp - 2) * STORE_STAGE_BYTES;
    BulkOut bo{bulk_store ? stg : nullptr, 0};
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int it = cluster_id; it < items && ok; it += n_clusters) {
      int tm, tn; tile_coords(it % total, tm, tn);
      const int row0 = tm * 2 * BM + (int)rank * BM + q * 32, row = row0 + lane;
      RopeVals rope_now, rope_next;
      bool rope0 = false;
      if constexpr (sizeof(TO) == 2 && !ACC) {
        rope0 = !swiglu && !epi.ce_mode && rope_wanted(epi, row, tn * BN, M, N);
        if (rope0) rope_fetch(rope_now, epi, row, tn * BN);        // in flight while this warp waits for the MMAs
      }
      if (!tc::mbar_wait(&sh->acc_full[acc], acc_phase, status, abort_flag, 114)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if constexpr (sizeof(TO) == 2 && !ACC) {
        if (epi.ce_mode) {
          ce_row_epilogue(taddr, (bf16 *)C, ldc, row0, lane, tn, M, N, epi, stg, bo, &map_c);
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tc::smem_u32(&sh->acc_empty[acc]) & LEADER_MASK);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
        if (swiglu) {
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t g[32], u[32];
            tc::tmem_ld_32x32(taddr + c * 32, g);
            tc::tmem_ld_32x32(taddr + BN / 2 + c * 32, u);
            tc::tmem_ld_wait();
            const int col = tn * (BN / 2) + c * 32;
            if (col < epi.swiglu_I) {               // warp-uniform; swiglu_I is a multiple of 32
              uint4 vg[4], vu[4], va[4];
              pack_chunk_bf16(g, vg);
              pack_chunk_bf16(u, vu);
              // silu(x) = x * sigmoid(x) = h + h * tanh(h) with h = x / 2: one special-function op and two FMA-pipe ops
              // per element, taken from the fp32 accumulators
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float h = 0.5f * __uint_as_float(g[j]);
                g[j] = __float_as_uint(fmaf(h, tanh_approx(h), h) * __uint_as_float(u[j]));
              }
              pack_chunk_bf16(g, va);
              if (bo.buf) {
                if (row0 < M) {
                bulk_store_bf16(bo, lane, vg, &map_c, col, row0);
                bulk_store_bf16(bo, lane, vu, &map_c, col + epi.swiglu_I, row0);
                bulk_store_bf16(bo, lane, va, &map_act, col, row0);
                }
              } else {
                bf16 *cbase = (bf16 *)C + (size_t)row0 * ldc + col;
                stage_store_bf16(stg, lane, vg, cbase, ldc, M - row0);
                stage_store_bf16(stg, lane, vu, cbase + epi.swiglu_I, ldc, M - row0);
                stage_store_bf16(stg, lane, va, (bf16 *)epi.act_out + (size_t)row0 * epi.ld_act + col, epi.ld_act, M - row0);
              }
            }
          }
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tc::smem_u32(&sh->acc_empty[acc]) & LEADER_MASK);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + c * 32, r);
        const int col = tn * BN + c * 32;
        bool rope_ahead = false;
        if constexpr (sizeof(TO) == 2 && !ACC) {
          rope_ahead = c + 1 < BN / 32 && rope_wanted(epi, row, col + 32, M, N);
          if (rope_ahead) rope_fetch(rope_next, epi, row, col + 32);
        }
        tc::tmem_ld_wait();
        if constexpr (sizeof(TO) == 2 && !ACC) {
          if (rope0) rope_apply(r, rope_now);
          rope0 = rope_ahead;
          if (rope_ahead) rope_now = rope_next;
        }
        if (col < N) store_chunk<TO, ACC>(r, C, ldc, row0, lane, col, M, N, stg, splits > 1, bo, &map_c);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tc::smem_u32(&sh->acc_empty[acc]) & LEADER_MASK);   // the leader issues the MMAs
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (bo.buf && lane == 0) tc::bulk_wait_all();      // the bulk stores have landed before the CTA exits
  }
  tc::tc_fence_before();
  __syncthreads();
  cluster_sync();                      // neither CTA leaves while the pair may still touch its shared / tensor memory
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, class TO, bool ACC>
int launch_variant(b200_ctx *ctx, const CUtensorMap &ma, const CUtensorMap &mb, void *C, int M, int N, int K,
                   size_t ldc, const GemmEpilogue &epi) {
  auto kern = gemm_tc2_kernel<A_MN, B_MN, TO, ACC>;
  // Results leave through bulk tensor stores when C (and the activation output) can carry a tensor map.
  static const bool bulk_wanted = [] { const char *e = getenv("B200_GEMM_BULK_STORE"); return !(e && e[0] == '0'); }();
  CUtensorMap mc = ma, mact = ma;    // placeholders when the route is off (never dereferenced)
  int bulk = 0;
  // (not for the vocabulary-sized products: with bulk stores the three vocabulary GEMMs of a step read 1.70 / 2.94 / 4.03 GB
  // from DRAM, with vector stores 1.17-1.36 / 2.13-2.41 / 2.80-3.45 GB over two captures, at the same speed)
  if (bulk_wanted && C && (uintptr_t)C % 16 == 0 && (ldc * sizeof(TO)) % 16 == 0 && N <= 16384 && K <= 16384) {
    bulk = tc_make_map_store_2d(&mc, C, (int)sizeof(TO), (uint64_t)N, (uint64_t)M, ldc * sizeof(TO)) == 0;
    if (bulk && epi.swiglu_I > 0)
      bulk = tc_make_map_store_2d(&mact, epi.act_out, 2, (uint64_t)epi.swiglu_I, (uint64_t)M, (uint64_t)epi.ld_act * 2) == 0;
  }
  static bool attr_set = false;
  static int max_clusters = 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = ctx->stream; cfg.attrs = attr; cfg.numAttrs = ctx->pdl ? 2 : 1;
  if (!attr_set) {
    B200_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    cfg.gridDim = dim3(ctx->sm_count & ~1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = ctx->sm_count / 2; }
    max_clusters = n;
    attr_set = true;
  }
  const int pairs = ((M + 2 * BM - 1) / (2 * BM)) * (epi.swiglu_I > 0 ? (epi.swiglu_I + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN);
  // Split K (fp32 output only: partial tiles are added with vector reductions) when whole tile pairs fill the
  // SM pairs badly -- the weight-gradient GEMMs have few tiles and a 16384-deep K.
  int splits = 1;
  if (sizeof(TO) == 4 && ldc == (size_t)N) {
    const int num_kb = (K + BK - 1) / BK;
    auto eff = [&](int s) { int items = pairs * s; int waves = (items + max_clusters - 1) / max_clusters; return (double)items / ((double)waves * max_clusters); };
    double best = eff(1);
    for (int s = 2; s <= 4; ++s)
      if (num_kb / s >= 16 && eff(s) > best + 0.08) { best = eff(s); splits = s; }
  }
  if (ctx->deterministic) splits = 1;          // partial tiles would be added in an order that varies
  const int items = pairs * splits;
  const int clusters = items < max_clusters ? items : max_clusters;
  cfg.gridDim = dim3(2 * clusters);
  b200_ctx::Timed tm{};
  if (ctx->time_gemm) {
    auto ev = [&]() { cudaEvent_t e; if (ctx->event_pool.empty()) cudaEventCreate(&e); else { e = ctx->event_pool.back(); ctx->event_pool.pop_back(); } return e; };
    tm.start = ev(); tm.stop = ev(); tm.flops = 2.0 * M * N * K;
    cudaEventRecord(tm.start, ctx->stream);
  }
  // the clear that split-K needs is part of the GEMM's cost: it sits inside the timed interval
  if (splits > 1 && !ACC) B200_CUDA(ctx, cudaMemsetAsync(C, 0, (size_t)M * N * sizeof(float), ctx->stream));
  B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, mact, (TO *)C, M, N, K, ldc, ctx->dev_status, epi, splits, bulk));
  ctx->launches++;
  if (ctx->trace_on) {      // one trace site per GEMM shape and form
    static std::vector<std::string *> keys;
    char buf[96];
    snprintf(buf, sizeof(buf), "gemm2 %dx%dx%d %s%s%s ce%d sk%d", M, N, K, A_MN ? "T" : "N", B_MN ? "N" : "T", sizeof(TO) == 4 ? " f32" : "", epi.ce_mode, splits);
    std::string *k = nullptr;
    for (auto *p : keys) if (*p == buf) k = p;
    if (!k) { k = new std::string(buf); keys.push_back(k); }
    b200_trace_mark(ctx, k->c_str(), 0);
  }
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

// Same contract as gemm_tc_launch (gemm_tc.cu); worthwhile when there are enough 256x256 tile pairs.
int gemm_tc2_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta, int tb,
                    int acc, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc, const GemmEpilogue *epi_in) {
  B200_REQUIRE(ctx, !(acc && out_dt == B200_BF16), "gemm: accumulate needs an fp32 C on the tensor-core path");
  GemmEpilogue epi;
  if (epi_in && epi_in->swiglu_I > 0) {
    epi = *epi_in;
    B200_REQUIRE(ctx, out_dt == B200_BF16 && !acc && !ta && !tb && !epi.cos_t && epi.act_out && (size_t)epi.swiglu_I * 2 == N &&
                 epi.swiglu_I % 32 == 0 && (epi.ld_act * 2) % 16 == 0 && (uintptr_t)epi.act_out % 16 == 0,
                 "gemm: the fused SwiGLU output needs a bf16 forward GEMM on W = [gate | up] with I a multiple of 32");
  } else if (epi_in && epi_in->ce_mode) {
    epi = *epi_in;
    B200_REQUIRE(ctx, out_dt == B200_BF16 && !acc && !epi.cos_t && epi.ce_mode >= 1 && epi.ce_mode <= 3 && epi.ce_targets &&
                 (epi.ce_mode == 3 ? epi.ce_lse != nullptr : (epi.ce_part_max && epi.ce_part_sum && epi.ce_tgt_logit)),
                 "gemm: the cross-entropy epilogue needs a bf16 product, the target ids and its statistics arrays");
  } else if (epi_in) {
    epi = *epi_in;
    B200_REQUIRE(ctx, out_dt == B200_BF16 && epi.cos_t && epi.sin_t && epi.S > 0 && epi.hd % 32 == 0 && epi.cols % 32 == 0 &&
                 ((uintptr_t)epi.cos_t | (uintptr_t)epi.sin_t) % 16 == 0, "gemm: unsupported fused rotary epilogue");
  }
  CUtensorMap ma, mb;
  int r;
  if (!ta) r = tc_make_map_2d(&ma, A, K, M, lda * 2, BK, BM);
  else r = tc_make_map_2d(&ma, A, M, K, lda * 2, 64, BK);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed: %d", r);
  if (!tb) r = tc_make_map_2d(&mb, B, N, K, ldb * 2, 64, BK);
  else r = tc_make_map_2d(&mb, B, K, N, ldb * 2, BK, BN / 2);
  if (r) return b200_fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed: %d", r);
  const bool a_mn = ta != 0, b_mn = tb == 0;
  int m = (int)M, n = (int)N, k = (int)K;
  if (a_mn && b_mn) return launch_out<true, true>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  if (a_mn && !b_mn) return launch_out<true, false>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  if (!a_mn && b_mn) return launch_out<false, true>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
  return launch_out<false, false>(ctx, ma, mb, C, m, n, k, ldc, out_dt, acc, epi);
}

size_t gemm_tc2_ce_tiles(size_t N) { return (N + BN - 1) / BN; }

bool gemm_tc2_swiglu_eligible(const b200_ctx *ctx, size_t M, size_t I) {
  const size_t pairs = ((M + 2 * BM - 1) / (2 * BM)) * ((I + BN / 2 - 1) / (BN / 2));
  return ctx->gemm_2cta && I % 32 == 0 && pairs >= (size_t)ctx->sm_count / 4;
}
