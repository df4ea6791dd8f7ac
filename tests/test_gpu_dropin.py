"""Drop-in check of the boundary: the REFERENCE's own C++ engine sources (Tensor, Attention,
Transformer, Loss ...), compiled by oracle/build_ref.sh and linked against this backend's
`namespace metal_bridge` adaptor instead of the CPU stub, run with GPU_ENABLED=1 so that every op goes
through host pointers into the CUDA kernels -- and must reproduce the CPU checker within 1e-4.
The library is built where the reference checkout is available and travels as a built artefact."""
import os

import numpy as np
import pytest

from gpu_util import FP32_TOL, rel, synth  # noqa: F401
from oracle import oracle

pytestmark = pytest.mark.gpu
LIB = os.path.join(os.path.dirname(oracle.ref_path()), "libref_on_b200.so")
SEED = 20240


@pytest.fixture(scope="module")
def ref_on_gpu():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libref_on_b200.so has not been built (needs the reference checkout)")
    os.environ["GPU_ENABLED"] = "1"          # the reference re-reads this in every op (cpp/src/Attention.cpp:183-190)
    yield oracle.Oracle(LIB, prefix="ref_")
    os.environ["GPU_ENABLED"] = "0"


def test_reference_ops_run_on_the_cuda_backend(ref_on_gpu, orc):
    A, B = synth.normal(SEED, "dA", (37, 19)), synth.normal(SEED, "dB", (19, 23))
    assert rel(ref_on_gpu.gemm(A, B, 37, 23, 19), orc.gemm(A, B, 37, 23, 19)) < 1e-5
    x, w = synth.normal(SEED, "dx", (11, 64)), 1 + 0.1 * synth.normal(SEED, "dw", (64,))
    assert rel(ref_on_gpu.rms_norm_forward(x, w), orc.rms_norm_forward(x, w)) < 1e-5
    lg, tg = synth.normal(SEED, "dl", (9, 70), 2.0), synth.token_ids(SEED, "dt", (9,), 70)
    l1, g1 = ref_on_gpu.cross_entropy(lg, tg)
    l2, g2 = orc.cross_entropy(lg, tg)
    assert abs(l1 - l2) < 1e-5 and rel(g1, g2) < 1e-5


@pytest.mark.parametrize("cfgd", [dict(B=2, S=8, H=32, I=48, nH=4, nKV=2, hd=8, V=64, L=2),
                                  dict(B=2, S=128, H=256, I=688, nH=8, nKV=2, hd=32, V=4096, L=1)],
                         ids=["toy", "single_layer_benchmark_config"])
def test_reference_engine_forward_backward_on_the_cuda_backend(ref_on_gpu, orc, cfgd):
    cfg = oracle.Config(**cfgd)
    params = synth.model_params(SEED, cfg)
    tok = synth.token_ids(SEED, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    t, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    loss, grads, logits = ref_on_gpu.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    eloss, egrads, elogits = orc.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    assert rel(logits, elogits) < FP32_TOL
    assert abs(loss - eloss) < 1e-4 * max(1.0, abs(eloss))
    nz = grads != 0                      # the reference discards norm-weight gradients
    assert nz.sum() > grads.size // 4
    assert rel(grads[nz], egrads[nz]) < FP32_TOL
