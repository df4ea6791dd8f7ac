// CUDA-core GEMM with fp32 accumulation: C[M,N] (+)= op(A)[M,K] * op(B)[K,N].
// This is the fp32 path of the backend (the reference's 1e-4 fp32 contract
// cannot be met on bf16 tensor cores) and the catch-all for bf16 operands
// whose strides TMA cannot address.  64x64 tile, 16-deep K slices, 256
// threads, 4x4 outputs per thread, all four transpose combinations by index
// arithmetic (cf. cpp/src/gpu_kernel/gemm_bf16.metal:45,63).
#include "common.cuh"

namespace {
constexpr int TM = 64, TN = 64, TK = 16;

template <class TI, class TO, bool TA, bool TB, bool ACC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI *__restrict__ A, const TI *__restrict__ B, TO *__restrict__ C, int M, int N, int K,
                 size_t lda, size_t ldb, size_t ldc) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;       // 16x16 threads, each 4x4 outputs
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    // A tile: TM x TK
    for (int i = tid; i < TM * TK; i += 256) {
      int m, k;
      if (TA) { m = i % TM; k = i / TM; } else { k = i % TK; m = i / TK; }
      int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < K) v = to_f(TA ? A[(size_t)gk * lda + gm] : A[(size_t)gm * lda + gk]);
      As[k][m] = v;
    }
    for (int i = tid; i < TN * TK; i += 256) {
      int n, k;
      if (TB) { k = i % TK; n = i / TK; } else { n = i % TN; k = i / TN; }
      int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < N && gk < K) v = to_f(TB ? B[(size_t)gn * ldb + gk] : B[(size_t)gk * ldb + gn]);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      size_t o = (size_t)gm * ldc + gn;
      float v = acc[i][j];
      if (ACC) v += to_f(C[o]);
      C[o] = from_f<TO>(v);
    }
  }
}

template <class TI, class TO>
void dispatch(cudaStream_t s, dim3 grid, const void *A, const void *B, void *C, int M, int N, int K, int ta, int tb,
              int acc, size_t lda, size_t ldb, size_t ldc) {
#define L(TA_, TB_, AC_) gemm_simt_kernel<TI, TO, TA_, TB_, AC_><<<grid, 256, 0, s>>>((const TI *)A, (const TI *)B, (TO *)C, M, N, K, lda, ldb, ldc)
  int code = (ta ? 4 : 0) | (tb ? 2 : 0) | (acc ? 1 : 0);
  switch (code) {
    case 0: L(false, false, false); break;
    case 1: L(false, false, true); break;
    case 2: L(false, true, false); break;
    case 3: L(false, true, true); break;
    case 4: L(true, false, false); break;
    case 5: L(true, false, true); break;
    case 6: L(true, true, false); break;
    default: L(true, true, true); break;
  }
#undef L
}
}  // namespace

int gemm_simt_launch(b200_ctx *ctx, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, int ta,
                     int tb, int acc, b200_dtype in_dt, b200_dtype out_dt, size_t lda, size_t ldb, size_t ldc) {
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  B200_REQUIRE(ctx, grid.y <= 65535, "gemm: M too large for the CUDA-core kernel");
  if (in_dt == B200_F32 && out_dt == B200_F32) dispatch<float, float>(ctx->stream, grid, A, B, C, (int)M, (int)N, (int)K, ta, tb, acc, lda, ldb, ldc);
  else if (in_dt == B200_F32) dispatch<float, bf16>(ctx->stream, grid, A, B, C, (int)M, (int)N, (int)K, ta, tb, acc, lda, ldb, ldc);
  else if (out_dt == B200_F32) dispatch<bf16, float>(ctx->stream, grid, A, B, C, (int)M, (int)N, (int)K, ta, tb, acc, lda, ldb, ldc);
  else dispatch<bf16, bf16>(ctx->stream, grid, A, B, C, (int)M, (int)N, (int)K, ta, tb, acc, lda, ldb, ldc);
  B200_LAUNCHED(ctx);
  return B200_OK;
}
