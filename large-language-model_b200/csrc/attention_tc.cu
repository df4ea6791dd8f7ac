// Tensor-core (tcgen05) causal GQA attention -- placeholder until the kernels land:
// reports "unsupported" so that the dispatcher uses the CUDA-core kernels.
#include "common.cuh"
bool attn_tc_supported(size_t, size_t, size_t, size_t, size_t, const AttnStrides &, b200_dtype, const void *,
                       const void *, const void *, const void *) { return false; }
int attn_fwd_tc_launch(b200_ctx *ctx, const void *, const void *, const void *, void *, float *, size_t, size_t, size_t,
                       size_t, size_t, const AttnStrides &) { return b200_fail(ctx, B200_ERR_UNSUPPORTED, "no tensor-core attention"); }
int attn_bwd_tc_launch(b200_ctx *ctx, const void *, const void *, const void *, const void *, const void *,
                       const float *, void *, void *, void *, size_t, size_t, size_t, size_t, size_t,
                       const AttnStrides &, const AttnStrides &) { return b200_fail(ctx, B200_ERR_UNSUPPORTED, "no tensor-core attention"); }
