"""The cross-entropy entry point for hosts that cannot allocate device memory at call time
(b200_cross_entropy_noalloc: per-token losses in a fixed array inside the library, no cudaMalloc).

Some embedders hand this library a fixed memory budget at start-up, forbid allocation afterwards, or
sit on a path where an allocation's implicit synchronisation is unacceptable; they pass every buffer
themselves.  The test calls the entry point through the C ABI twice in a row -- with different
inputs, so stale contents of the shared array would show -- and checks loss and gradient against the
regular entry point; it also checks that an input beyond the fixed capacity is refused.
Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

from gpu_util import bridge, ctx, synth  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-6), ("bf16", 1e-6)])
def test_matches_the_regular_entry_point_on_two_calls_in_a_row(ctx, dtype, tol):
    # every buffer is created up front; the calls under test allocate nothing
    shapes = [(300, 1000), (41, 4096)]          # second call: fewer tokens than the first
    loss_na = ctx.empty((1,), "f32")
    for call, (T, V) in enumerate(shapes):
        lg = synth.normal(50 + call, "logits", (T, V), 3.0)
        if dtype == "bf16":
            lg = synth.bf16_round(lg)
        tg = synth.token_ids(50 + call, "targets", (T,), V).astype(np.uint32)
        d_lg, d_tg = ctx.array(lg, dtype), ctx.array(tg, "u32")
        grad_na = ctx.empty((T, V), dtype)
        ctx.cross_entropy_noalloc(d_lg, d_tg, loss_na, grad_na)
        got_loss, got_grad = float(loss_na.download()[0]), grad_na.download()
        ref_loss, ref_grad = ctx.cross_entropy(d_lg, d_tg)
        ref_loss, ref_grad = float(ref_loss.download()[0]), ref_grad.download()
        assert abs(got_loss - ref_loss) <= tol * max(1.0, abs(ref_loss)), (call, got_loss, ref_loss)
        np.testing.assert_allclose(got_grad, ref_grad, rtol=tol, atol=1e-9)
        ctx.cross_entropy_noalloc(d_lg, d_tg, loss_na, None)          # loss only
        assert abs(float(loss_na.download()[0]) - ref_loss) <= tol * max(1.0, abs(ref_loss))


def test_more_tokens_than_the_fixed_capacity_are_refused(ctx):
    T, V = 65537, 8
    d_lg = ctx.empty((T, V), "f32").zero()
    d_tg = ctx.empty((T,), "u32").zero()
    loss = ctx.empty((1,), "f32")
    with pytest.raises(bridge.B200Error, match="exceed the fixed scratch"):
        ctx.cross_entropy_noalloc(d_lg, d_tg, loss)
    ok_lg, ok_tg = ctx.empty((65536, V), "f32").zero(), ctx.empty((65536,), "u32").zero()
    ctx.cross_entropy_noalloc(ok_lg, ok_tg, loss)                      # exactly at the limit is accepted
    assert abs(float(loss.download()[0]) - np.log(V)) < 1e-5
