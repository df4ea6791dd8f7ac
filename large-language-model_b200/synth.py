"""Seeded synthetic inputs shared by the parity tests, the fixture generator
and the benchmark.

Counter-based (SplitMix64 of ``stream_key + index``), so a value depends only
on (seed, tensor name, element index) -- never on thread count or call order.
Distributions follow the benchmark configurations: weights and embedding
tables N(0, 0.02), activations / Q / K / V / upstream gradients N(0, 1), token
ids uniform in [0, vocab).  (The reference trainer's own initialiser is
N(0, 1/sqrt(H)) from mt19937(42), cpp/src/RunTrainer.cpp:68-105; shapes are
the same.)
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def stream_key(seed: int, name: str) -> np.uint64:
    """64-bit FNV-1a of the tensor name, mixed with the run seed."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return _splitmix64(np.array([h ^ (seed * 0x9E3779B97F4A7C15 & 0xFFFFFFFFFFFFFFFF)], np.uint64))[0]


def uniform01(seed: int, name: str, n: int, lane: int = 0) -> np.ndarray:
    """n doubles in (0, 1)."""
    key = stream_key(seed, name)
    with np.errstate(over="ignore"):
        ctr = (np.arange(n, dtype=np.uint64) * np.uint64(2) + np.uint64(lane) + key) & _M64
    bits = _splitmix64(ctr) >> np.uint64(11)
    return (bits.astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed: int, name: str, shape, std: float = 1.0) -> np.ndarray:
    """float32 N(0, std) of the given shape (Box-Muller on two uniform lanes)."""
    n = int(np.prod(shape))
    u1, u2 = uniform01(seed, name, n, 0), uniform01(seed, name, n, 1)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32).reshape(shape)


def token_ids(seed: int, name: str, shape, vocab: int) -> np.ndarray:
    n = int(np.prod(shape))
    return np.minimum((uniform01(seed, name, n) * vocab).astype(np.int64), vocab - 1).astype(np.int32).reshape(shape)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) << np.uint64(16)
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> uint16 bfloat16 bit patterns (round to nearest even)."""
    return (bf16_round(a).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def layer_params(seed: int, cfg, layer: int = 0, std: float = 0.02) -> np.ndarray:
    """One decoder layer's flat parameter block (norm weights 1, projections
    N(0, std)), in the order attn_norm_w, Wq, Wk, Wv, Wo, ffn_norm_w, w_gate,
    w_up, w_down; every matrix row-major [in, out]."""
    q, kv, H, I = cfg.nH * cfg.hd, cfg.nKV * cfg.hd, cfg.H, cfg.I
    parts = [np.ones(H, np.float32)]
    for nm, shp in (("Wq", (H, q)), ("Wk", (H, kv)), ("Wv", (H, kv)), ("Wo", (q, H))):
        parts.append(normal(seed, f"layer{layer}.{nm}", shp, std).ravel())
    parts.append(np.ones(H, np.float32))
    for nm, shp in (("w_gate", (H, I)), ("w_up", (H, I)), ("w_down", (I, H))):
        parts.append(normal(seed, f"layer{layer}.{nm}", shp, std).ravel())
    return np.concatenate(parts)


def model_params(seed: int, cfg, std: float = 0.02) -> np.ndarray:
    """Whole-model flat parameters: embedding [V,H], L layer blocks,
    final_norm_w [H], output projection [H,V]."""
    parts = [normal(seed, "tok_embeddings", (cfg.V, cfg.H), std).ravel()]
    parts += [layer_params(seed, cfg, l, std) for l in range(cfg.L)]
    parts += [np.ones(cfg.H, np.float32), normal(seed, "output_projection", (cfg.H, cfg.V), std).ravel()]
    return np.concatenate(parts)
