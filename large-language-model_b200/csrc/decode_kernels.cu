// Small data-movement kernels of the autoregressive decode path: KV-cache append after the prefill
// (rows of the fused [M, Q+2KV] projection -> caches [B, S_max, KV]) and the last-token gather.
// The reference C++ engine declares a KVCache (cpp/include/TransformerConfig.hpp:121-124) but never fills it.
#include "common.cuh"

namespace {

// ---- cache append: rows of the fused [M, Q+2KV] projection -> K/V caches [B, S_max, KV] ----------
template <class T>
__global__ void kv_append_kernel(const T *__restrict__ qkv, T *__restrict__ kc, T *__restrict__ vc, int B, int T_new,
                                 int pos0, int S_max, int Q, int KV, int ld) {
  constexpr int N = 16 / sizeof(T);
  const int units = KV / N;                                // 16-byte units per K (or V) row
  const size_t n = (size_t)B * T_new * units * 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(i % units); size_t r = i / units;
    const int which = (int)(r & 1); r >>= 1;
    const int t = (int)(r % T_new), b = (int)(r / T_new);
    const T *src = qkv + ((size_t)b * T_new + t) * ld + Q + which * KV + u * N;
    T *dst = (which ? vc : kc) + ((size_t)b * S_max + pos0 + t) * KV + u * N;
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
  }
}

template <class T>
__global__ void gather_rows_kernel(const T *__restrict__ src, T *__restrict__ dst, int B, int S, int H, int pos) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)B * H; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % H), b = (int)(i / H);
    dst[i] = src[((size_t)b * S + pos) * H + c];
  }
}

}  // namespace

int kv_append(b200_ctx *ctx, const void *qkv, void *kc, void *vc, size_t B, size_t T_new, size_t pos0, size_t S_max,
              size_t Q, size_t KV, size_t ld, b200_dtype dt) {
  const size_t N = 16 / dtype_size(dt);
  B200_REQUIRE(ctx, KV % N == 0 && Q % N == 0 && ld % N == 0, "kv_append: widths must be multiples of 16 bytes");
  const size_t n = B * T_new * (KV / N) * 2;
  if (!n) return B200_OK;
  const int grid = (int)((n + 255) / 256 < (size_t)ctx->sm_count * 16 ? (n + 255) / 256 : (size_t)ctx->sm_count * 16);
  if (dt == B200_BF16) kv_append_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)qkv, (bf16 *)kc, (bf16 *)vc, (int)B, (int)T_new, (int)pos0, (int)S_max, (int)Q, (int)KV, (int)ld);
  else kv_append_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)qkv, (float *)kc, (float *)vc, (int)B, (int)T_new, (int)pos0, (int)S_max, (int)Q, (int)KV, (int)ld);
  B200_LAUNCHED(ctx);
  return B200_OK;
}

int gather_rows(b200_ctx *ctx, const void *src, void *dst, size_t B, size_t S, size_t H, size_t pos, b200_dtype dt) {
  const size_t n = B * H;
  const int grid = (int)((n + 255) / 256);
  if (dt == B200_BF16) gather_rows_kernel<bf16><<<grid, 256, 0, ctx->stream>>>((const bf16 *)src, (bf16 *)dst, (int)B, (int)S, (int)H, (int)pos);
  else gather_rows_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)src, (float *)dst, (int)B, (int)S, (int)H, (int)pos);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
