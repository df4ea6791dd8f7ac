"""Drop-in check of the boundary: the REFERENCE's own C++ engine sources (Tensor, Attention,
Transformer, Loss ...), compiled by oracle/build_ref.sh and linked against this backend's
`namespace metal_bridge` adaptor instead of the CPU stub, run with GPU_ENABLED=1 so that every op goes
through host pointers into the CUDA kernels -- and must reproduce the CPU checker within 1e-4.
A second build of the same sources keeps bf16 device mirrors (what the reference's Metal shaders read): the
reference engine then runs on the tcgen05 kernels and must stay within 2e-2.  The backend's profiling externs
(device time, GPU calls) and the loss read-back after end_scope are checked through the same libraries.
The libraries are built where the reference checkout is available and travel as built artefacts."""
import ctypes
import os

import numpy as np
import pytest

from gpu_util import FP32_TOL, rel, synth  # noqa: F401
from oracle import oracle

pytestmark = pytest.mark.gpu
LIB = os.path.join(os.path.dirname(oracle.ref_path()), "libref_on_b200.so")
LIB_BF16 = os.path.join(os.path.dirname(oracle.ref_path()), "libref_on_b200_bf16.so")
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


@pytest.fixture(scope="module")
def ref_on_gpu_bf16():
    if not os.path.exists(LIB_BF16):
        pytest.skip("oracle/_ref/libref_on_b200_bf16.so has not been built (needs the reference checkout)")
    os.environ["GPU_ENABLED"] = "1"
    yield oracle.Oracle(LIB_BF16, prefix="ref_")
    os.environ["GPU_ENABLED"] = "0"


def test_reference_engine_on_the_tensor_core_kernels(ref_on_gpu_bf16, orc):
    """head_dim 128, 512 tokens: the reference's Transformer::forward / ::backward through bf16 mirrors reach the
    tcgen05 GEMM and attention kernels; every stored tensor is rounded to bf16 between ops, as on the Metal backend."""
    cfg = oracle.Config(B=2, S=256, H=512, I=1024, nH=4, nKV=2, hd=128, V=2048, L=1)
    params = synth.bf16_round(synth.model_params(SEED, cfg))
    tok = synth.token_ids(SEED, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    t, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    loss, grads, logits = ref_on_gpu_bf16.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    eloss, egrads, elogits = orc.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    assert rel(logits, elogits) < 2e-2
    assert abs(loss - eloss) < 5e-3 * abs(eloss)
    nz = grads != 0
    assert nz.sum() > grads.size // 4
    assert rel(grads[nz], egrads[nz]) < 3e-2      # bf16 between every op of the reference's unfused backward


@pytest.mark.parametrize("which", ["fp32", "bf16"])
def test_profiling_counters_and_loss_read_back(which, request):
    lib_path = LIB if which == "fp32" else LIB_BF16
    if not os.path.exists(lib_path):
        pytest.skip("drop-in library has not been built (needs the reference checkout)")
    os.environ["GPU_ENABLED"] = "1"
    try:
        orc_gpu = oracle.Oracle(lib_path, prefix="ref_")
        L = orc_gpu.lib
        L.ref_backend_stats.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_float)]
        L.ref_scoped_cross_entropy.restype = ctypes.c_float
        L.ref_scoped_cross_entropy.argtypes = [np.ctypeslib.ndpointer(np.float32, flags="C"), np.ctypeslib.ndpointer(np.int32, flags="C"),
                                               ctypes.c_size_t, ctypes.c_size_t]

        def stats():
            ms, calls, loss = ctypes.c_double(), ctypes.c_uint64(), ctypes.c_float()
            L.ref_backend_stats(ctypes.byref(ms), ctypes.byref(calls), ctypes.byref(loss))
            return ms.value, calls.value, loss.value

        L.ref_backend_reset_stats()
        assert stats()[:2] == (0.0, 0)
        A, B = synth.normal(SEED, "cA", (256, 128)), synth.normal(SEED, "cB", (128, 64))
        orc_gpu.gemm(A, B, 256, 64, 128)          # outside a scope: one commit-and-wait per op (cpp/src/gpu_kernel/MetalBridge.mm:1384-1406)
        ms1, calls1, _ = stats()
        assert calls1 >= 1 and ms1 > 0.0
        lg = synth.normal(SEED, "cl", (32, 128), 2.0)
        tg = synth.token_ids(SEED, "ct", (32,), 128)
        scoped = float(L.ref_scoped_cross_entropy(np.ascontiguousarray(lg, np.float32), np.ascontiguousarray(tg, np.int32), 32, 128))
        from oracle import oracle as omod
        expected, _ = omod.Oracle().cross_entropy(lg, tg)
        assert abs(scoped - expected) < (1e-5 if which == "fp32" else 2e-2) * max(1.0, abs(expected))    # get_last_loss() after end_scope
        ms2, calls2, last = stats()
        assert calls2 == calls1 + 1 and ms2 > ms1 and last == scoped     # the whole scope is ONE GPU call (MetalBridge.mm:2195-2207)
    finally:
        os.environ["GPU_ENABLED"] = "0"
