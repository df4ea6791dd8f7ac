"""ctypes binding of ``libb200bridge.so`` (the C ABI in ``include/b200_bridge.h``).

Host-side mirror of the reference's backend interface for tests, the smoke check
and the benchmark: numpy arrays in, numpy arrays out, every compute call goes
through the C ABI into the CUDA kernels.  There is no CPU fallback: loading
fails loudly when the library is missing, and ``Context`` fails when no
sm_100 device is present.
"""
from __future__ import annotations

import ctypes as C
import importlib
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200_BRIDGE_LIB names another build of the same library (A/B measurements of two kernel versions in one run)
LIB_PATH = os.environ.get("B200_BRIDGE_LIB") or os.path.join(_HERE, "libb200bridge.so")
F32, BF16 = 0, 1
_synth = importlib.import_module(__package__ + ".synth") if __package__ else None

_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float


class B200Error(RuntimeError):
    pass


class ModelConfig(C.Structure):
    """Mirrors the reference's ModelConfig (cpp/include/TransformerConfig.hpp:16-98)."""
    _fields_ = [(n, _sz) for n in ("vocab_size", "hidden_dim", "intermediate_dim", "n_layers", "n_heads",
                                   "n_kv_heads", "head_dim", "max_seq_len")] + [("rope_base", _f), ("rms_norm_eps", _f)]


class Shape:
    """Problem shape for Model (names follow the reference's ModelConfig plus batch/sequence)."""

    def __init__(self, B, S, H, I, nH, nKV, hd, V, L=1, eps=1e-5, rope_base=10000.0):
        self.B, self.S, self.H, self.I, self.nH, self.nKV, self.hd, self.V, self.L = B, S, H, I, nH, nKV, hd, V, L
        self.eps, self.rope_base = eps, rope_base


class SamplerConfig(C.Structure):
    """Decode hyper-parameters (python/pipeline/inference/sampler.py:18-28 of the reference)."""
    _fields_ = [("temperature", _f), ("top_p", _f), ("repetition_penalty", _f), ("top_k", _i), ("seed", C.c_uint64),
                ("n_whitespace_ids", _i), ("whitespace_ids", _i * 8)]

    @classmethod
    def make(cls, temperature=0.0, top_p=1.0, repetition_penalty=1.0, top_k=0, seed=0, whitespace_ids=()):
        ws = (list(whitespace_ids) + [-1] * 8)[:8]
        return cls(temperature, top_p, repetition_penalty, top_k, seed, min(len(whitespace_ids), 8), (_i * 8)(*ws))


class AdamWParams(C.Structure):
    _fields_ = [(n, _f) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "bias_correction1",
                                  "bias_correction2")]


_SIGS = {
    "b200_init": (_i, [_i, C.POINTER(_vp)]),
    "b200_destroy": (_i, [_vp]),
    "b200_is_available": (_i, []),
    "b200_last_error": (C.c_char_p, [_vp]),
    "b200_stream": (_vp, [_vp]),
    "b200_set_stream": (_i, [_vp, _vp]),
    "b200_sync": (_i, [_vp]),
    "b200_launch_count": (C.c_uint64, [_vp]),
    "b200_profile_gemm": (_i, [_vp, _i]),
    "b200_profile_gemm_read": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "b200_batch_timer_begin": (_i, [_vp]),
    "b200_batch_timer_end": (_i, [_vp, C.POINTER(_f)]),
    "b200_malloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "b200_free": (_i, [_vp, _vp]),
    "b200_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "b200_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "b200_fill_zero": (_i, [_vp, _vp, _sz]),
    "b200_copy": (_i, [_vp, _vp, _vp, _sz]),
    "b200_convert": (_i, [_vp, _vp, _i, _vp, _i, _sz]),
    "b200_fill_normal": (_i, [_vp, _vp, _i, _sz, C.c_uint64, _f]),
    "b200_gemm": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _i]),
    "b200_rms_norm_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _i]),
    "b200_rms_norm_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _i]),
    "b200_fused_add_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i]),
    "b200_fused_backward_add_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i]),
    "b200_rope_tables": (_i, [_vp, _vp, _vp, _sz, _sz, _f]),
    "b200_rope_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "b200_rope_backward": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _i]),
    "b200_swiglu_forward": (_i, [_vp, _vp, _vp, _vp, _sz, _i]),
    "b200_swiglu_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i]),
    "b200_fused_swiglu_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_gemm_ffn": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_residual_add": (_i, [_vp, _vp, _vp, _sz, _i]),
    "b200_reshape_to_4d": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _i]),
    "b200_reshape_to_3d": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _i]),
    "b200_flash_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "b200_fused_attn_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "b200_flash_attn_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "b200_embedding_forward": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_embedding_backward": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_cross_entropy": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _i]),
    "b200_cross_entropy_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _i]),
    "b200_vocab_ce_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_vocab_ce_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _sz, _sz, _sz, _i]),
    "b200_adamw_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, C.POINTER(AdamWParams)]),
    "b200_model_create": (_i, [_vp, C.POINTER(ModelConfig), _i, _sz, _i, C.POINTER(_vp)]),
    "b200_model_destroy": (_i, [_vp]),
    "b200_model_param_count": (_sz, [_vp]),
    "b200_model_load_params": (_i, [_vp, _vp]),
    "b200_model_read_params": (_i, [_vp, _vp]),
    "b200_model_read_grads": (_i, [_vp, _vp]),
    "b200_model_get_config": (_i, [_vp, _vp]),
    "b200_checkpoint_param_count": (_sz, [_vp]),
    "b200_checkpoint_write_flat": (_i, [_vp, _vp, _vp, _vp, C.c_uint64, C.c_char_p]),
    "b200_checkpoint_read_flat": (_i, [_vp, C.c_char_p, _vp, _vp, _vp, _vp, _vp]),
    "b200_checkpoint_save": (_i, [_vp, C.c_char_p, C.c_uint64, _i]),
    "b200_checkpoint_load": (_i, [_vp, C.c_char_p, _i, _vp]),
    "b200_checkpoint_last_error": (C.c_char_p, []),
    "b200_scheduled_lr": (_f, [_sz, _sz, _sz, _f, _f]),
    "b200_metrics_begin": (_i, [C.c_char_p, _sz]),
    "b200_metrics_append": (_i, [C.c_char_p, _sz, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double,
                                C.c_uint64, C.c_double, C.c_uint64, C.c_double, C.c_double]),
    "b200_model_read_opt_state": (_i, [_vp, _vp, _vp, _vp]),
    "b200_model_load_opt_state": (_i, [_vp, _vp, _vp, C.c_uint64]),
    "b200_model_init_synthetic": (_i, [_vp, C.c_uint64, _f]),
    "b200_model_forward": (_i, [_vp, _vp, _sz, _sz, _vp]),
    "b200_model_loss_and_grads": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "b200_model_adamw_step": (_i, [_vp, _f, _f, _f, _f, _f]),
    "b200_model_set_grad_clip": (_i, [_vp, _f]),
    "b200_model_last_grad_norm": (_i, [_vp, C.POINTER(_f), C.POINTER(_f)]),
    "b200_model_train_step_host": (_i, [_vp, _vp, _vp, _sz, _sz, _f, _f, _f, _f, _f, C.POINTER(_f)]),
    "b200_model_train_step": (_i, [_vp, _vp, _vp, _sz, _sz, _f, _f, _f, _f, _f, _vp]),
    "b200_model_layer_forward": (_i, [_vp, _sz, _vp, _vp, _sz, _sz]),
    "b200_model_layer_backward": (_i, [_vp, _sz, _vp, _vp, _sz, _sz]),
    "b200_sample": (_i, [_vp, _vp, _i, _sz, _sz, _vp, _sz, _sz, _i, C.POINTER(SamplerConfig), C.c_uint64, _vp, _vp, _vp]),
    "b200_model_decode_begin": (_i, [_vp, _sz, _sz]),
    "b200_model_prefill": (_i, [_vp, _vp, _sz, _sz, _vp]),
    "b200_model_decode_step": (_i, [_vp, _vp, _sz, _sz, _vp]),
    "b200_model_generate": (_i, [_vp, _vp, _sz, _sz, _sz, C.POINTER(SamplerConfig), _vp, C.POINTER(_f), C.POINTER(_f)]),
    "b200_dp_unique_id": (_i, [_vp]),
    "b200_dp_init": (_i, [_vp, _vp, _i, _i]),
    "b200_dp_shutdown": (_i, [_vp]),
    "b200_model_param_checksum": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "b200_host_gemm": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _i, _i, _i]),
    "b200_host_rms_norm_forward": (_i, [_vp, _vp, _vp, _vp, _f, _sz, _sz]),
    "b200_host_flash_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz]),
    "b200_host_fused_attn_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz]),
    "b200_host_cross_entropy": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz]),
}

EXPORTED_SYMBOLS = tuple(_SIGS)
_lib = None


def load_library() -> C.CDLL:
    """Loads the CUDA extension; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` (nvcc, sm_100a)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(_vp)


class DeviceArray:
    """A device allocation with shape and element type ("f32", "bf16", "i32", "u32")."""

    def __init__(self, ctx: "Context", shape, dtype: str):
        self.ctx, self.shape, self.dtype = ctx, tuple(int(s) for s in np.atleast_1d(shape)), dtype
        self.itemsize = 2 if dtype == "bf16" else 4
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1
        self.nbytes = self.size * self.itemsize
        p = _vp()
        ctx._check(ctx.lib.b200_malloc(ctx.h, self.nbytes, C.byref(p)))
        self.ptr = p.value
        ctx._live.append(self)

    @property
    def code(self):
        return BF16 if self.dtype == "bf16" else F32

    def at(self, elem_offset: int) -> int:
        return self.ptr + elem_offset * self.itemsize

    def upload(self, a: np.ndarray):
        if self.dtype == "bf16":
            host = _synth.to_bf16_bits(np.ascontiguousarray(a, np.float32))
        elif self.dtype == "f32":
            host = np.ascontiguousarray(a, np.float32)
        elif self.dtype == "i32":
            host = np.ascontiguousarray(a, np.int32)
        else:
            host = np.ascontiguousarray(a, np.uint32)
        assert host.size == self.size, (host.size, self.size)
        self.ctx._check(self.ctx.lib.b200_memcpy_h2d(self.ctx.h, self.ptr, _np_ptr(host), self.nbytes))
        self.ctx.sync()          # host staging array may be freed after return
        return self

    def download(self) -> np.ndarray:
        npdt = {"bf16": np.uint16, "f32": np.float32, "i32": np.int32, "u32": np.uint32}[self.dtype]
        host = np.empty(self.shape, npdt)
        self.ctx._check(self.ctx.lib.b200_memcpy_d2h(self.ctx.h, _np_ptr(host), self.ptr, self.nbytes))
        self.ctx.sync()
        return _synth.from_bf16_bits(host).reshape(self.shape) if self.dtype == "bf16" else host

    def zero(self):
        self.ctx._check(self.ctx.lib.b200_fill_zero(self.ctx.h, self.ptr, self.nbytes))
        return self

    def free(self):
        if self.ptr:
            self.ctx.lib.b200_free(self.ctx.h, self.ptr)
            self.ptr = None


class Context:
    """One CUDA device + stream (metal_bridge::initialize / begin_scope / end_scope)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = _vp()
        rc = self.lib.b200_init(device, C.byref(h))
        if rc != 0:
            raise B200Error(f"b200_init(device={device}) failed with {rc}: no sm_100 GPU visible?")
        self.h = h
        self._live: list[DeviceArray] = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def close(self):
        if self.h:
            for a in self._live:
                a.free()
            self._live.clear()
            self.lib.b200_destroy(self.h)
            self.h = None

    def _check(self, rc: int):
        if rc != 0:
            raise B200Error(f"b200 call failed ({rc}): {self.lib.b200_last_error(self.h).decode()}")

    def sync(self):
        self._check(self.lib.b200_sync(self.h))

    def stream_ptr(self) -> int:
        return self.lib.b200_stream(self.h) or 0

    def launch_count(self) -> int:
        return int(self.lib.b200_launch_count(self.h))

    def profile_gemm(self, enable: bool):
        self._check(self.lib.b200_profile_gemm(self.h, int(enable)))

    def profile_gemm_read(self):
        """(total ms, total flops, launches) of the tensor-core GEMM since the last read."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_uint64()
        self._check(self.lib.b200_profile_gemm_read(self.h, C.byref(ms), C.byref(fl), C.byref(n)))
        return ms.value, fl.value, int(n.value)

    def empty(self, shape, dtype="f32") -> DeviceArray:
        return DeviceArray(self, shape, dtype)

    def array(self, a: np.ndarray, dtype="f32") -> DeviceArray:
        return DeviceArray(self, a.shape, dtype).upload(a)

    # ---- ops (device arrays) ------------------------------------------------
    def gemm(self, A, B, M, N, K, trans_a=False, trans_b=False, out_dtype=None, C_acc=None):
        out_dtype = out_dtype or A.dtype
        out = C_acc if C_acc is not None else self.empty((M, N), out_dtype)
        self._check(self.lib.b200_gemm(self.h, A.ptr, B.ptr, out.ptr, M, N, K, int(trans_a), int(trans_b),
                                       int(C_acc is not None), A.code, out.code))
        return out

    def rms_norm_forward(self, x, w, eps=1e-5, want_rstd=False):
        D = x.shape[-1]
        y = self.empty(x.shape, x.dtype)
        rstd = self.empty((x.size // D,), "f32") if want_rstd else None
        self._check(self.lib.b200_rms_norm_forward(self.h, x.ptr, y.ptr, w.ptr, rstd.ptr if rstd else None, eps,
                                                   x.size // D, D, x.code))
        return (y, rstd) if want_rstd else y

    def rms_norm_backward(self, g, x, w, eps=1e-5, want_dw=True):
        D = x.shape[-1]
        dx = self.empty(x.shape, x.dtype)
        dw = self.empty((D,), "f32").zero() if want_dw else None
        self._check(self.lib.b200_rms_norm_backward(self.h, g.ptr, x.ptr, w.ptr, dx.ptr, dw.ptr if dw else None, eps,
                                                    x.size // D, D, x.code))
        return dx, dw

    def fused_add_norm(self, h, r, w, eps=1e-5):
        D = h.shape[-1]
        out = self.empty(h.shape, h.dtype)
        self._check(self.lib.b200_fused_add_norm(self.h, h.ptr, r.ptr, w.ptr, out.ptr, h.size // D, D, eps, h.code))
        return out

    def fused_backward_add_norm(self, g, x, w, res_grad, eps=1e-5):
        D = x.shape[-1]
        dx = self.empty(x.shape, x.dtype)
        self._check(self.lib.b200_fused_backward_add_norm(self.h, g.ptr, x.ptr, w.ptr, res_grad.ptr, dx.ptr,
                                                          x.size // D, D, eps, x.code))
        return dx

    def rope_tables(self, max_seq, hd, base=10000.0):
        c, s = self.empty((max_seq, hd // 2)), self.empty((max_seq, hd // 2))
        self._check(self.lib.b200_rope_tables(self.h, c.ptr, s.ptr, max_seq, hd, base))
        return c, s

    def rope_forward(self, q, k, cos, sin):
        B, qh, S, hd = q.shape
        self._check(self.lib.b200_rope_forward(self.h, q.ptr, k.ptr, cos.ptr, sin.ptr, B, qh, k.shape[1], S, hd, q.code))

    def rope_backward(self, g, cos, sin):
        B, h, S, hd = g.shape
        self._check(self.lib.b200_rope_backward(self.h, g.ptr, cos.ptr, sin.ptr, B, h, S, hd, g.code))

    def swiglu_forward(self, gate, up):
        out = self.empty(gate.shape, gate.dtype)
        self._check(self.lib.b200_swiglu_forward(self.h, gate.ptr, up.ptr, out.ptr, gate.size, gate.code))
        return out

    def swiglu_backward(self, dy, gate, up):
        dg, du = self.empty(gate.shape, gate.dtype), self.empty(gate.shape, gate.dtype)
        self._check(self.lib.b200_swiglu_backward(self.h, dy.ptr, gate.ptr, up.ptr, dg.ptr, du.ptr, gate.size, gate.code))
        return dg, du

    def gemm_ffn(self, a, w_gate_up, M, N, K, want_gate_up=False):
        """silu(a @ W_gate) * (a @ W_up) for w_gate_up = [gate | up] ([K, 2N]); optionally also the two products."""
        out = self.empty((M, N), a.dtype)
        gu = self.empty((M, 2 * N), a.dtype) if want_gate_up else None
        self._check(self.lib.b200_gemm_ffn(self.h, a.ptr, w_gate_up.ptr, gu.ptr if gu is not None else None, out.ptr, M, N, K, a.code))
        return (out, gu) if want_gate_up else out

    def residual_add(self, a, b):
        self._check(self.lib.b200_residual_add(self.h, a.ptr, b.ptr, a.size, a.code))

    def reshape_to_4d(self, src, B, n, S, hd):
        dst = self.empty((B, n, S, hd), src.dtype)
        self._check(self.lib.b200_reshape_to_4d(self.h, src.ptr, dst.ptr, B, n, S, hd, src.code))
        return dst

    def reshape_to_3d(self, src, B, n, S, hd):
        dst = self.empty((B, S, n * hd), src.dtype)
        self._check(self.lib.b200_reshape_to_3d(self.h, src.ptr, dst.ptr, B, n, S, hd, src.code))
        return dst

    def flash_attn_fwd(self, q, k, v, want_lse=False):
        B, nH, S, hd = q.shape
        o = self.empty((B, S, nH * hd), q.dtype)
        lse = self.empty((B, nH, S), "f32") if want_lse else None
        self._check(self.lib.b200_flash_attn_fwd(self.h, q.ptr, k.ptr, v.ptr, o.ptr, lse.ptr if lse else None, B, nH,
                                                 k.shape[1], S, hd, q.code))
        return (o, lse) if want_lse else o

    def fused_attn_bwd(self, q, k, v, dO):
        B, nH, S, hd = q.shape
        dq, dk, dv = self.empty(q.shape, q.dtype), self.empty(k.shape, q.dtype), self.empty(v.shape, q.dtype)
        self._check(self.lib.b200_fused_attn_bwd(self.h, q.ptr, k.ptr, v.ptr, dO.ptr, dq.ptr, dk.ptr, dv.ptr, B, nH,
                                                 k.shape[1], S, hd, q.code))
        return dq, dk, dv

    def flash_attn_bwd(self, q, k, v, o, dO, lse, out=None):
        """Backward from the forward call's saved output and log-sum-exp; returns (dq, dk, dv)."""
        B, nH, S, hd = q.shape
        dq, dk, dv = out if out is not None else (self.empty(q.shape, q.dtype), self.empty(k.shape, q.dtype), self.empty(v.shape, q.dtype))
        self._check(self.lib.b200_flash_attn_bwd(self.h, q.ptr, k.ptr, v.ptr, o.ptr, dO.ptr, lse.ptr, dq.ptr, dk.ptr, dv.ptr,
                                                 B, nH, k.shape[1], S, hd, q.code))
        return dq, dk, dv

    def embedding_forward(self, ids, table):
        V, H = table.shape
        out = self.empty((ids.size, H), table.dtype)
        self._check(self.lib.b200_embedding_forward(self.h, ids.ptr, table.ptr, out.ptr, ids.size, H, V, table.code))
        return out

    def embedding_backward(self, ids, gh, V):
        H = gh.shape[-1]
        gt = self.empty((V, H), "f32")
        self._check(self.lib.b200_embedding_backward(self.h, ids.ptr, gh.ptr, gt.ptr, ids.size, H, V, gh.code))
        return gt

    def cross_entropy(self, logits, targets, want_grad=True, in_place=False):
        """Mean loss and (softmax - onehot)/tokens; in_place writes the gradient over the logits."""
        T, V = logits.size // logits.shape[-1], logits.shape[-1]
        loss = self.empty((1,), "f32")
        grad = (logits if in_place else self.empty(logits.shape, logits.dtype)) if want_grad else None
        self._check(self.lib.b200_cross_entropy(self.h, logits.ptr, targets.ptr, loss.ptr, grad.ptr if grad else None,
                                                T, V, logits.code))
        return loss, grad

    def vocab_ce_forward(self, x, w, targets, want_logits=False):
        """Vocabulary projection + mean cross-entropy in one call: (loss, lse[, logits]) device arrays."""
        (T, H), V = x.shape, w.shape[1]
        loss, lse = self.empty((1,), "f32"), self.empty((T,), "f32")
        logits = self.empty((T, V), x.dtype) if want_logits else None
        self._check(self.lib.b200_vocab_ce_forward(self.h, x.ptr, w.ptr, targets.ptr, loss.ptr, lse.ptr,
                                                   logits.ptr if want_logits else None, T, V, H, x.code))
        return (loss, lse, logits) if want_logits else (loss, lse)

    def vocab_ce_backward(self, x, w, targets, lse, logits=None):
        """Gradients of the mean loss: (dlogits, grad_w fp32 [H,V], grad_x [T,H]).  `logits` (from the forward call) is
        converted in place; without it the projection is run again with the gradient as its epilogue."""
        (T, H), V = x.shape, w.shape[1]
        dl = logits if logits is not None else self.empty((T, V), x.dtype)
        gw, gx = self.empty((H, V), "f32"), self.empty((T, H), x.dtype)
        self._check(self.lib.b200_vocab_ce_backward(self.h, x.ptr, w.ptr, targets.ptr, lse.ptr, dl.ptr, int(logits is not None),
                                                    gw.ptr, gx.ptr, T, V, H, x.code))
        return dl, gw, gx

    def cross_entropy_noalloc(self, logits, targets, loss, grad=None):
        """Cross-entropy through the entry point that allocates nothing: the caller supplies every
        buffer (``loss`` is a 1-element f32 device array, ``grad`` optional, like ``logits``); at most
        65536 tokens.  For hosts that cannot allocate device memory at call time."""
        T, V = logits.size // logits.shape[-1], logits.shape[-1]
        self._check(self.lib.b200_cross_entropy_noalloc(self.h, logits.ptr, targets.ptr, loss.ptr,
                                                        grad.ptr if grad is not None else None, T, V, logits.code))

    def sample(self, logits, history, hist_len, sampler: "SamplerConfig", step=0, append=False):
        """One sampling step; returns (tokens, threshold, kept) device arrays."""
        B, V = logits.shape
        tok, thr, kept = self.empty((B,), "i32"), self.empty((B,), "f32"), self.empty((B,), "i32")
        self._check(self.lib.b200_sample(self.h, logits.ptr, logits.code, B, V, history.ptr if history is not None else None,
                                         hist_len, history.shape[1] if history is not None else 0, int(append),
                                         C.byref(sampler), step, tok.ptr, thr.ptr, kept.ptr))
        return tok, thr, kept

    def adamw_step(self, p, g, m, v, lr, beta1, beta2, eps, wd, step, shadow=None):
        bc1 = float(np.float32(1.0) - np.float32(beta1) ** np.float32(step))
        bc2 = float(np.float32(1.0) - np.float32(beta2) ** np.float32(step))
        prm = AdamWParams(lr, beta1, beta2, eps, wd, bc1, bc2)
        self._check(self.lib.b200_adamw_step(self.h, p.ptr, g.ptr, m.ptr, v.ptr, shadow.ptr if shadow else None, p.size,
                                             C.byref(prm)))

    # ---- host-pointer calls (reference calling convention) --------------------
    def host_gemm(self, A, B, M, N, K, trans_a=False, trans_b=False):
        A, B = np.ascontiguousarray(A, np.float32), np.ascontiguousarray(B, np.float32)
        out = np.empty((M, N), np.float32)
        self._check(self.lib.b200_host_gemm(self.h, _np_ptr(A), _np_ptr(B), _np_ptr(out), M, N, K, int(trans_a),
                                            int(trans_b), F32))
        return out

    def host_rms_norm_forward(self, x, w, eps=1e-5):
        x, w = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w, np.float32)
        y = np.empty_like(x)
        self._check(self.lib.b200_host_rms_norm_forward(self.h, _np_ptr(x), _np_ptr(y), _np_ptr(w), eps,
                                                        x.size // x.shape[-1], x.shape[-1]))
        return y

    def host_flash_attn_fwd(self, q, k, v):
        q, k, v = (np.ascontiguousarray(a, np.float32) for a in (q, k, v))
        B, nH, S, hd = q.shape
        o = np.empty((B, S, nH * hd), np.float32)
        self._check(self.lib.b200_host_flash_attn_fwd(self.h, _np_ptr(q), _np_ptr(k), _np_ptr(v), _np_ptr(o), B, nH,
                                                      k.shape[1], S, hd))
        return o

    def host_fused_attn_bwd(self, q, k, v, dO):
        q, k, v, dO = (np.ascontiguousarray(a, np.float32) for a in (q, k, v, dO))
        B, nH, S, hd = q.shape
        dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
        self._check(self.lib.b200_host_fused_attn_bwd(self.h, _np_ptr(q), _np_ptr(k), _np_ptr(v), _np_ptr(dO),
                                                      _np_ptr(dq), _np_ptr(dk), _np_ptr(dv), B, nH, k.shape[1], S, hd))
        return dq, dk, dv

    def host_cross_entropy(self, logits, targets, want_grad=True):
        logits = np.ascontiguousarray(logits, np.float32)
        targets = np.ascontiguousarray(targets, np.uint32).reshape(-1)
        V = logits.shape[-1]
        loss = np.zeros(1, np.float32)
        grad = np.empty_like(logits) if want_grad else None
        self._check(self.lib.b200_host_cross_entropy(self.h, _np_ptr(logits), _np_ptr(targets), _np_ptr(loss),
                                                     _np_ptr(grad) if want_grad else None, logits.size // V, V))
        return float(loss[0]), grad


class Model:
    """Device-resident decoder-only GQA transformer (Transformer + CrossEntropyLoss + AdamW of the reference)."""

    def __init__(self, ctx: Context, cfg, dtype: str = "bf16", max_batch: int | None = None, with_optimizer=True):
        self.ctx, self.cfg, self.dtype = ctx, cfg, dtype
        mc = ModelConfig(cfg.V, cfg.H, cfg.I, cfg.L, cfg.nH, cfg.nKV, cfg.hd, cfg.S, cfg.rope_base, cfg.eps)
        h = _vp()
        ctx._check(ctx.lib.b200_model_create(ctx.h, C.byref(mc), BF16 if dtype == "bf16" else F32,
                                             max_batch or cfg.B, int(with_optimizer), C.byref(h)))
        self.h = h
        self.n_params = int(ctx.lib.b200_model_param_count(h))
        self._loss = ctx.empty((1,), "f32")

    def close(self):
        if self.h:
            self.ctx.lib.b200_model_destroy(self.h)
            self.h = None

    def load_params(self, flat: np.ndarray):
        flat = np.ascontiguousarray(flat, np.float32)
        assert flat.size == self.n_params, (flat.size, self.n_params)
        self.ctx._check(self.ctx.lib.b200_model_load_params(self.h, _np_ptr(flat)))

    def init_synthetic(self, seed: int, std: float = 0.02):
        self.ctx._check(self.ctx.lib.b200_model_init_synthetic(self.h, seed, std))

    def read_params(self) -> np.ndarray:
        out = np.empty(self.n_params, np.float32)
        self.ctx._check(self.ctx.lib.b200_model_read_params(self.h, _np_ptr(out)))
        return out

    def read_grads(self) -> np.ndarray:
        out = np.empty(self.n_params, np.float32)
        self.ctx._check(self.ctx.lib.b200_model_read_grads(self.h, _np_ptr(out)))
        return out

    def read_opt_state(self):
        """(m, v, step): AdamW moments in the parameter order, and the optimizer step counter."""
        mm, vv = np.empty(self.n_params, np.float32), np.empty(self.n_params, np.float32)
        step = C.c_uint64(0)
        self.ctx._check(self.ctx.lib.b200_model_read_opt_state(self.h, _np_ptr(mm), _np_ptr(vv), C.byref(step)))
        return mm, vv, int(step.value)

    def load_opt_state(self, m: np.ndarray, v: np.ndarray, step: int):
        m, v = np.ascontiguousarray(m, np.float32), np.ascontiguousarray(v, np.float32)
        assert m.size == self.n_params and v.size == self.n_params
        self.ctx._check(self.ctx.lib.b200_model_load_opt_state(self.h, _np_ptr(m), _np_ptr(v), int(step)))

    def forward(self, tokens_dev: DeviceArray, B: int, S: int) -> DeviceArray:
        logits = self.ctx.empty((B * S, self.cfg.V), self.dtype)
        self.ctx._check(self.ctx.lib.b200_model_forward(self.h, tokens_dev.ptr, B, S, logits.ptr))
        return logits

    def loss_and_grads(self, tokens_dev, targets_dev, B, S) -> DeviceArray:
        self.ctx._check(self.ctx.lib.b200_model_loss_and_grads(self.h, tokens_dev.ptr, targets_dev.ptr, B, S,
                                                               self._loss.ptr))
        return self._loss

    def loss_and_grads_host(self, tokens: np.ndarray, targets: np.ndarray) -> float:
        B, S = tokens.shape
        t, y = self.ctx.array(tokens, "i32"), self.ctx.array(targets, "i32")
        loss = self.loss_and_grads(t, y, B, S).download()
        return float(loss[0])

    def adamw_step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1):
        self.ctx._check(self.ctx.lib.b200_model_adamw_step(self.h, lr, beta1, beta2, eps, wd))

    def set_grad_clip(self, max_norm: float):
        """Global-norm gradient clipping of the optimizer step (0 turns it off)."""
        self.ctx._check(self.ctx.lib.b200_model_set_grad_clip(self.h, max_norm))

    def last_grad_norm(self):
        """(gradient norm, factor applied) of the last clipped optimizer step."""
        n, f = _f(0.0), _f(1.0)
        self.ctx._check(self.ctx.lib.b200_model_last_grad_norm(self.h, C.byref(n), C.byref(f)))
        return float(n.value), float(f.value)

    def train_step(self, tokens_dev, targets_dev, B, S, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1):
        self.ctx._check(self.ctx.lib.b200_model_train_step(self.h, tokens_dev.ptr, targets_dev.ptr, B, S, lr, beta1,
                                                           beta2, eps, wd, self._loss.ptr))
        return self._loss

    def train_step_host(self, tokens: np.ndarray, targets: np.ndarray, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                        wd=0.1) -> float:
        B, S = tokens.shape
        tokens, targets = np.ascontiguousarray(tokens, np.int32), np.ascontiguousarray(targets, np.int32)
        loss = _f(0.0)
        self.ctx._check(self.ctx.lib.b200_model_train_step_host(self.h, _np_ptr(tokens), _np_ptr(targets), B, S, lr,
                                                                beta1, beta2, eps, wd, C.byref(loss)))
        return float(loss.value)

    def layer_forward(self, layer: int, h_in: DeviceArray, B: int, S: int) -> DeviceArray:
        out = self.ctx.empty(h_in.shape, h_in.dtype)
        self.ctx._check(self.ctx.lib.b200_model_layer_forward(self.h, layer, h_in.ptr, out.ptr, B, S))
        return out

    def layer_backward(self, layer: int, grad_out: DeviceArray, B: int, S: int) -> DeviceArray:
        out = self.ctx.empty(grad_out.shape, grad_out.dtype)
        self.ctx._check(self.ctx.lib.b200_model_layer_backward(self.h, layer, grad_out.ptr, out.ptr, B, S))
        return out

    # ---- decode -------------------------------------------------------------
    def decode_begin(self, batch: int, max_total_len: int):
        self.ctx._check(self.ctx.lib.b200_model_decode_begin(self.h, batch, max_total_len))

    def prefill(self, tokens_dev: DeviceArray, B: int, P: int) -> DeviceArray:
        logits = self.ctx.empty((B, self.cfg.V), self.dtype)
        self.ctx._check(self.ctx.lib.b200_model_prefill(self.h, tokens_dev.ptr, B, P, logits.ptr))
        return logits

    def decode_step(self, tokens_dev: DeviceArray, B: int, pos: int) -> DeviceArray:
        logits = self.ctx.empty((B, self.cfg.V), self.dtype)
        self.ctx._check(self.ctx.lib.b200_model_decode_step(self.h, tokens_dev.ptr, B, pos, logits.ptr))
        return logits

    def generate(self, prompt: np.ndarray, new_tokens: int, sampler: "SamplerConfig"):
        """prompt [B, P] host ids -> ([B, new_tokens] ids, prefill ms, decode ms)."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        B, P = prompt.shape
        out = np.empty((B, new_tokens), np.int32)
        pm, dm = _f(0.0), _f(0.0)
        self.ctx._check(self.ctx.lib.b200_model_generate(self.h, _np_ptr(prompt), B, P, new_tokens, C.byref(sampler),
                                                         _np_ptr(out), C.byref(pm), C.byref(dm)))
        return out, float(pm.value), float(dm.value)

    def param_checksum(self):
        """(sum, sum of squares) of the fp32 master weights, fixed summation order (replica-drift check)."""
        a, b = C.c_double(), C.c_double()
        self.ctx._check(self.ctx.lib.b200_model_param_checksum(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def dp_init(self, unique_id: bytes, rank: int, world: int):
        buf = C.create_string_buffer(unique_id, 128)
        self.ctx._check(self.ctx.lib.b200_dp_init(self.h, buf, rank, world))


def dp_unique_id() -> bytes:
    lib = load_library()
    buf = C.create_string_buffer(128)
    if lib.b200_dp_unique_id(buf) != 0:
        raise B200Error("ncclGetUniqueId failed (NCCL not found?)")
    return buf.raw
