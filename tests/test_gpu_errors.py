"""Error paths of the backend, exercised without faulting or hanging the GPU.
* A bounded device-side wait that runs out: a probe kernel waits (about a millisecond) on an mbarrier nothing arrives on,
  through the same mbar_wait every tensor-core kernel uses; the kernel returns, b200_sync reports B200_ERR_DEVICE_WAIT,
  and the context keeps working.
* A failing gradient exchange, injected on the host (the NCCL call is replaced by an error code, nothing is launched):
  the step reports B200_ERR_COMM, the communicator is torn down with ncclCommAbort, and the model trains on."""
import numpy as np
import pytest

from gpu_util import bridge, ctx, rel, synth  # noqa: F401

pytestmark = pytest.mark.gpu


def test_a_device_wait_that_runs_out_is_reported_and_the_context_survives(ctx):
    lib = ctx.lib
    lib.b200_internal_wait_probe.argtypes = [bridge._vp, bridge.C.c_longlong]
    lib.b200_internal_wait_probe.restype = bridge._i
    ctx.sync()
    assert lib.b200_internal_wait_probe(ctx.h, 2_000_000) == 0          # ~1 ms at 2 GHz
    rc = lib.b200_sync(ctx.h)
    assert rc == -5, rc                                                  # B200_ERR_DEVICE_WAIT
    assert b"wait gave up (code 199)" in lib.b200_last_error(ctx.h)
    # the status word is cleared and the next call works
    A = synth.normal(1, "ea", (64, 32))
    B = synth.normal(1, "eb", (32, 48))
    out = ctx.gemm(ctx.array(A), ctx.array(B), 64, 48, 32).download()
    assert rel(out, A.astype(np.float64) @ B.astype(np.float64)) < 1e-5
    ctx.sync()
    with pytest.raises(bridge.B200Error):                                # limits beyond 2e8 cycles are refused, nothing is launched
        ctx._check(lib.b200_internal_wait_probe(ctx.h, 10_000_000_000))


def test_an_injected_collective_failure_is_reported_and_the_communicator_is_aborted(ctx):
    import torch  # noqa: F401  (brings libnccl.so.2 into the process, as the benchmark does)
    from oracle import oracle
    lib = ctx.lib
    lib.b200_internal_dp_inject_failure.argtypes = [bridge._vp, bridge._i]
    lib.b200_internal_dp_comm_failed.argtypes = [bridge._vp]
    cfg = oracle.Config(B=2, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=128, L=2)
    model = bridge.Model(ctx, cfg, "f32")
    model.init_synthetic(3, 0.05)
    tok = synth.token_ids(6, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    t, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    ok_loss = model.loss_and_grads_host(t, y)
    model.dp_init(bridge.dp_unique_id(), 0, 1)                           # a one-rank communicator on this GPU
    assert abs(model.loss_and_grads_host(t, y) - ok_loss) < 1e-6
    lib.b200_internal_dp_inject_failure(model.h, 1)                      # ncclUnhandledCudaError, host side only
    with pytest.raises(bridge.B200Error, match="ncclAllReduce failed"):
        model.loss_and_grads_host(t, y)
    assert lib.b200_internal_dp_comm_failed(model.h) == 1
    ctx._check(lib.b200_dp_shutdown(model.h))                            # ncclCommAbort path; must return
    assert lib.b200_internal_dp_comm_failed(model.h) == 0
    ctx.sync()
    assert abs(model.loss_and_grads_host(t, y) - ok_loss) < 1e-6         # single-device steps go on
    model.close()
