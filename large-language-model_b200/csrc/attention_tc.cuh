// Helpers shared by the tensor-core attention forward and backward kernels.
#pragma once
#include "common.cuh"
#include "tc_common.cuh"

namespace attn {

constexpr int TQ = 128, TK = 128;                 // query / key tile
constexpr int COMPUTE_WARPS = 8;                  // softmax / gradient warps (2 per scheduler)
constexpr int MMA_WARP = 8, TMA_WARP = 9;
constexpr int THREADS = 320;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(tc::smem_u32(dst)), "l"(map), "r"(tc::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// shared -> global element-wise add of a [rows x 32 fp32] box (3-D map: column, row, batch*head)
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap *map, const void *src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(tc::smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Load a [128 rows x HD] bf16 tile as HD/64 chunks of [128 rows][128 B] (128-byte swizzle).
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t *dst, const CUtensorMap *map, int row0, int head, int batch,
                                          uint64_t *bar) {
#pragma unroll
  for (int c = 0; c < HD / 64; ++c) tma_load_4d(dst + c * 16384, map, c * 64, row0, head, batch, bar);
}

// Byte offset of 16-byte unit `unit16` (0..15 = columns [8u, 8u+8)) of row r in a [128 x 128] bf16 tile
// stored as 2 chunks of [128 rows][128 B] with the 128-byte swizzle (what TMA would have produced).
__device__ __forceinline__ uint32_t swz_unit(int r, int unit16) {
  int chunk = unit16 >> 3, u = unit16 & 7;
  return (uint32_t)(chunk * 16384 + r * 128 + ((u ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
// Operand descriptors for a tile stored as chunks of [128 rows][128 B]:
//   contraction along the columns (inside the 128-byte row): K-major, 16 columns = 32 B per MMA,
//     64-column chunks 16 KiB apart;
//   contraction along the rows: MN-major, 16 rows = 2 KiB per MMA, 64-column chunks 16 KiB apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int k) {
  return tc::make_smem_desc(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return tc::make_smem_desc(base + k * 2048, 16384, 1024);
}

inline int make_map_4d(CUtensorMap *map, const void *base, size_t hd, size_t S, size_t heads, size_t B, long long s_s,
                       long long s_h, long long s_b) {
  // dims (d, s, head, batch); strides in bytes for dims 1..3; box = 64 columns x 128 rows
  return tc_make_map_4d(map, base, hd, S, heads, B, (uint64_t)s_s * 2, (uint64_t)s_h * 2, (uint64_t)s_b * 2, 64, 128);
}
inline bool layout_ok(const void *p, long long sb, long long sh, long long ss) {
  return p && ((uintptr_t)p % 16 == 0) && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0 && ss > 0 && sh > 0 && sb >= 0;
}

}  // namespace attn
