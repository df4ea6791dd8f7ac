"""ctypes front end of the CPU checker (``liboracle.so`` built from
``block_oracle.c``) and, when it has been built, of ``_ref/libref_oracle.so``
(the reference's own C++ CPU ops compiled by ``build_ref.sh``).

TEST INFRASTRUCTURE ONLY.  Tests, the smoke check and the benchmark's CPU
baseline leg may import this module; the product package must not.
All arrays are C-contiguous float32 / int32 numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_I = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_sz = C.c_size_t


class _Cfg(C.Structure):
    _fields_ = [(n, _sz) for n in ("B", "S", "H", "I", "nH", "nKV", "hd", "V", "L")] + [
        ("eps", C.c_float), ("rope_base", C.c_float)]


@dataclass
class Config:
    """Shape of one problem instance (names follow the reference's ModelConfig,
    cpp/include/TransformerConfig.hpp:16-98)."""
    B: int
    S: int
    H: int
    I: int
    nH: int
    nKV: int
    hd: int
    V: int = 1
    L: int = 1
    eps: float = 1e-5
    rope_base: float = 10000.0

    def c(self) -> _Cfg:
        return _Cfg(self.B, self.S, self.H, self.I, self.nH, self.nKV, self.hd, self.V, self.L,
                    self.eps, self.rope_base)

    @property
    def layer_params(self) -> int:
        q, kv = self.nH * self.hd, self.nKV * self.hd
        return self.H + self.H * q + 2 * self.H * kv + q * self.H + self.H + 3 * self.H * self.I

    @property
    def model_params(self) -> int:
        return self.V * self.H + self.L * self.layer_params + self.H + self.H * self.V

    def layer_slices(self):
        """name -> (offset, shape) inside one layer's flat parameter block."""
        q, kv, H, I = self.nH * self.hd, self.nKV * self.hd, self.H, self.I
        out, off = {}, 0
        for name, shape in (("attn_norm_w", (H,)), ("Wq", (H, q)), ("Wk", (H, kv)), ("Wv", (H, kv)),
                            ("Wo", (q, H)), ("ffn_norm_w", (H,)), ("w_gate", (H, I)), ("w_up", (H, I)),
                            ("w_down", (I, H))):
            n = int(np.prod(shape))
            out[name] = (off, shape)
            off += n
        return out


def _build_if_needed() -> str:
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "block_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


class Oracle:
    """Thin numpy wrapper over the exported ``orc_*`` (or ``ref_*``) symbols."""

    def __init__(self, path: str | None = None, prefix: str = "orc_"):
        self.path = path or _build_if_needed()
        self.lib = C.CDLL(self.path)
        self.p = prefix
        L = self.lib

        def sig(name, res, *args):
            fn = getattr(L, prefix + name)
            fn.restype = res
            fn.argtypes = list(args)
            return fn

        self._gemm = sig("gemm", None, _F, _F, _F, _sz, _sz, _sz, C.c_int, C.c_int, C.c_int)
        self._rmsf = sig("rms_norm_forward", None, _F, _F, _F, C.c_float, _sz, _sz)
        self._rmsb = sig("rms_norm_backward", None, _F, _F, _F, _F, C.c_void_p, C.c_float, _sz, _sz)
        self._ropet = sig("rope_tables", None, _F, _F, _sz, _sz, C.c_float)
        self._rope = sig("rope_apply", None, _F, _F, _F, _sz, _sz, _sz, _sz, C.c_int)
        self._swf = sig("swiglu_forward", None, _F, _F, _F, _sz)
        self._swb = sig("swiglu_backward", None, _F, _F, _F, _F, _F, _sz)
        self._attf = sig("attention_forward", None, _F, _F, _F, _F, _sz, _sz, _sz, _sz, _sz)
        self._attb = sig("attention_backward", None, _F, _F, _F, _F, _F, _F, _F, _sz, _sz, _sz, _sz, _sz)
        self._ce = sig("cross_entropy", C.c_float, _F, _I, C.c_void_p, _sz, _sz)
        self._adamw = sig("adamw_step", None, _F, _F, _F, _F, _sz, *([C.c_float] * 7))
        self._attn_layer = sig("attention_layer", None, C.POINTER(_Cfg), _F, _F, _F, _F, _F, _F,
                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p)
        self._layer_f = sig("layer_forward", None, C.POINTER(_Cfg), _F, _F, _F)
        self._layer_b = sig("layer_backward", None, C.POINTER(_Cfg), _F, _F, _F, _F, _F)
        self._model = sig("model_loss_and_grads", C.c_float, C.POINTER(_Cfg), _I, _I, _F, C.c_void_p,
                          C.c_void_p)
        # training-driver files: only the reference build has them (its own Checkpoint / Trainer classes)
        if hasattr(L, prefix + "checkpoint_save"):
            self._ck_save = sig("checkpoint_save", C.c_int, C.POINTER(_Cfg), _F, _F, _F, C.c_uint64, C.c_char_p)
            self._ck_load = sig("checkpoint_load", C.c_int, C.POINTER(_Cfg), C.c_char_p, _F, _F, _F, C.POINTER(C.c_uint64))
            self._lr = sig("scheduled_lr", C.c_float, _sz, _sz, _sz, C.c_float, C.c_float)

    # ---- primitive ops -------------------------------------------------
    def gemm(self, A, B, M, N, K, transA=False, transB=False, C_in=None):
        out = np.zeros((M, N), np.float32) if C_in is None else np.ascontiguousarray(C_in, np.float32).copy()
        self._gemm(_f(A), _f(B), out, M, N, K, int(transA), int(transB), int(C_in is not None))
        return out

    def rms_norm_forward(self, x, w, eps=1e-5):
        x = _f(x)
        y = np.empty_like(x)
        D = x.shape[-1]
        self._rmsf(x, y, _f(w), eps, x.size // D, D)
        return y

    def rms_norm_backward(self, g, x, w, eps=1e-5, want_dw=True):
        x = _f(x)
        dx = np.empty_like(x)
        D = x.shape[-1]
        dw = np.zeros(D, np.float32) if want_dw else None
        self._rmsb(_f(g), x, _f(w), dx, dw.ctypes.data if want_dw else None, eps, x.size // D, D)
        return dx, dw

    def rope_tables(self, max_seq, hd, base=10000.0):
        c = np.empty((max_seq, hd // 2), np.float32)
        s = np.empty_like(c)
        self._ropet(c, s, max_seq, hd, base)
        return c, s

    def rope(self, t4, cos, sin, backward=False):
        """t4 is [B, heads, S, hd]; returns a rotated copy."""
        t = _f(t4).copy()
        B, h, S, hd = t.shape
        self._rope(t, _f(cos), _f(sin), B, h, S, hd, int(backward))
        return t

    def swiglu_forward(self, gate, up):
        gate = _f(gate)
        out = np.empty_like(gate)
        self._swf(gate, _f(up), out, gate.size)
        return out

    def swiglu_backward(self, dy, gate, up):
        gate = _f(gate)
        dg, du = np.empty_like(gate), np.empty_like(gate)
        self._swb(_f(dy), gate, _f(up), dg, du, gate.size)
        return dg, du

    def attention_forward(self, q4, k4, v4):
        q4, k4, v4 = _f(q4), _f(k4), _f(v4)
        B, nH, S, hd = q4.shape
        nKV = k4.shape[1]
        out = np.empty((B, S, nH * hd), np.float32)
        self._attf(q4, k4, v4, out, B, nH, nKV, S, hd)
        return out

    def attention_backward(self, q4, k4, v4, dO):
        q4, k4, v4 = _f(q4), _f(k4), _f(v4)
        B, nH, S, hd = q4.shape
        nKV = k4.shape[1]
        dq, dk, dv = np.empty_like(q4), np.empty_like(k4), np.empty_like(v4)
        self._attb(q4, k4, v4, _f(dO), dq, dk, dv, B, nH, nKV, S, hd)
        return dq, dk, dv

    def cross_entropy(self, logits, targets, want_grad=True):
        logits = _f(logits)
        V = logits.shape[-1]
        T = logits.size // V
        d = np.empty_like(logits) if want_grad else None
        loss = self._ce(logits, np.ascontiguousarray(targets, np.int32).reshape(-1),
                        d.ctypes.data if want_grad else None, T, V)
        return float(loss), d

    def adamw_step(self, p, g, m, v, lr, beta1, beta2, eps, wd, step):
        p, m, v = _f(p).copy(), _f(m).copy(), _f(v).copy()
        bc1 = np.float32(1.0) - np.float32(beta1) ** np.float32(step)
        bc2 = np.float32(1.0) - np.float32(beta2) ** np.float32(step)
        self._adamw(p, _f(g), m, v, p.size, lr, beta1, beta2, eps, wd, float(bc1), float(bc2))
        return p, m, v

    # ---- compositions ----------------------------------------------------
    def attention_layer(self, cfg: Config, x, Wq, Wk, Wv, Wo, gout=None):
        x = _f(x)
        out = np.empty_like(x)
        if gout is None:
            self._attn_layer(C.byref(cfg.c()), x, _f(Wq), _f(Wk), _f(Wv), _f(Wo), out, *([None] * 6))
            return out
        gx = np.empty_like(x)
        g = [np.zeros_like(_f(w)) for w in (Wq, Wk, Wv, Wo)]
        gout = _f(gout)
        self._attn_layer(C.byref(cfg.c()), x, _f(Wq), _f(Wk), _f(Wv), _f(Wo), out, gout.ctypes.data,
                         gx.ctypes.data, *[a.ctypes.data for a in g])
        return out, gx, g

    def layer_forward(self, cfg: Config, h_in, params):
        h_in = _f(h_in)
        out = np.empty_like(h_in)
        self._layer_f(C.byref(cfg.c()), h_in, _f(params), out)
        return out

    def layer_backward(self, cfg: Config, grad_out, h_in, params, grads_in=None):
        h_in = _f(h_in)
        grads = np.zeros(cfg.layer_params, np.float32) if grads_in is None else _f(grads_in).copy()
        gh = np.empty_like(h_in)
        self._layer_b(C.byref(cfg.c()), _f(grad_out), h_in, _f(params), grads, gh)
        return gh, grads

    def model_loss_and_grads(self, cfg: Config, tokens, targets, params, want_grads=True, want_logits=False):
        tokens = np.ascontiguousarray(tokens, np.int32).reshape(-1)
        targets = np.ascontiguousarray(targets, np.int32).reshape(-1)
        grads = np.zeros(cfg.model_params, np.float32) if want_grads else None
        logits = np.empty((cfg.B * cfg.S, cfg.V), np.float32) if want_logits else None
        loss = self._model(C.byref(cfg.c()), tokens, targets, _f(params),
                           grads.ctypes.data if want_grads else None,
                           logits.ctypes.data if want_logits else None)
        return float(loss), grads, logits


    # ---- the reference's Checkpoint::save / ::load and Trainer::get_scheduled_lr (reference build only) ----
    def checkpoint_save(self, cfg: Config, path: str, params, m, v, step: int):
        rc = self._ck_save(C.byref(cfg.c()), _f(params), _f(m), _f(v), int(step), path.encode())
        if rc:
            raise RuntimeError(f"reference Checkpoint::save failed for {path}")

    def checkpoint_load(self, cfg: Config, path: str):
        n = cfg.model_params
        p, m, v = np.empty(n, np.float32), np.empty(n, np.float32), np.empty(n, np.float32)
        step = C.c_uint64(0)
        rc = self._ck_load(C.byref(cfg.c()), path.encode(), p, m, v, C.byref(step))
        if rc:
            raise RuntimeError(f"reference Checkpoint::load failed for {path}")
        return p, m, v, int(step.value)

    def scheduled_lr(self, step, warmup, max_steps, lr_max, lr_min) -> float:
        return float(self._lr(step, warmup, max_steps, lr_max, lr_min))


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def ref_path() -> str:
    return os.path.join(_HERE, "_ref", "libref_oracle.so")


def have_ref() -> bool:
    return os.path.exists(ref_path())


def load_ref() -> Oracle:
    """The reference's own C++ CPU ops behind the same call surface."""
    return Oracle(ref_path(), prefix="ref_")
