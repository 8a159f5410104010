"""Seeded synthetic operands in the reference's block formats (numpy only).

The reference's benchmarks and tests use random weight bytes and normal
activations (benchmarks/vecq_bench.cc:119-121, tests/unit/dsv4_fast_test.cc:73-95);
these generators pack such values DIRECTLY into the block layouts, since no
Q4_K quantizer is part of the path.
"""
from __future__ import annotations

import numpy as np


def q8_0_weights(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """uint8 [n, k/32*34]: per block FP16 d = |N(0,0.02)|/127, 32 int8 in [-127,127]."""
    nb = k // 32
    d = (np.abs(rng.normal(0.0, 0.02, size=(n, nb))) / 127.0).astype(np.float16)
    q = rng.integers(-127, 128, size=(n, nb, 32), dtype=np.int16).astype(np.int8)
    out = np.empty((n, nb, 34), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(n, nb * 34)


def pack_q4_k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """sc, mn uint8 [..., 8] in 0..63 -> the 12 packed bytes [..., 12]."""
    s = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    for g in range(4):
        s[..., g] = sc[..., g] | ((sc[..., g + 4] >> 4) << 6)
        s[..., g + 4] = mn[..., g] | ((mn[..., g + 4] >> 4) << 6)
        s[..., g + 8] = (sc[..., g + 4] & 15) | ((mn[..., g + 4] & 15) << 4)
    return s


def q4_k_weights(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """uint8 [n, k/256*144]: codes U{0..15}; 6-bit scales/minima U{0..63};
    d = FP16(|N(0,0.02)|/(15*32)), dmin = FP16(|N(0,0.02)|/32)."""
    nb = k // 256
    out = np.empty((n, nb, 144), np.uint8)
    d = (np.abs(rng.normal(0.0, 0.02, size=(n, nb))) / (15.0 * 32.0)).astype(np.float16)
    dmin = (np.abs(rng.normal(0.0, 0.02, size=(n, nb))) / 32.0).astype(np.float16)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    out[:, :, 2:4] = dmin.view(np.uint8).reshape(n, nb, 2)
    sc = rng.integers(0, 64, size=(n, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(n, nb, 8), dtype=np.uint8)
    out[:, :, 4:16] = pack_q4_k_scales(sc, mn)
    out[:, :, 16:] = rng.integers(0, 256, size=(n, nb, 128), dtype=np.uint8)
    return out.reshape(n, nb * 144)


def more_weights(rng: np.random.Generator, wtype: int, n: int, k: int) -> np.ndarray:
    """uint8 [n, row bytes] of random blocks of GGML type `wtype` (2 Q4_0, 6 Q5_0, 20 IQ4_NL,
    13 Q5_K, 14 Q6_K): every code and scale field uniform over its range, FP16 scales
    |N(0, 0.02)| over the codes' span."""
    def halves(scale, shape):
        return (np.abs(rng.normal(0.0, 0.02, size=shape)) / scale).astype(np.float16).view(np.uint8)
    if wtype in (2, 20, 6):
        size = 22 if wtype == 6 else 18
        nb = k // 32
        out = rng.integers(0, 256, size=(n, nb, size), dtype=np.uint8)
        out[:, :, 0:2] = halves(127.0 if wtype == 20 else 16.0, (n, nb)).reshape(n, nb, 2)
        return out.reshape(n, nb * size)
    nb = k // 256
    if wtype == 13:
        out = rng.integers(0, 256, size=(n, nb, 176), dtype=np.uint8)
        out[:, :, 0:2] = halves(31.0 * 32.0, (n, nb)).reshape(n, nb, 2)
        out[:, :, 2:4] = halves(32.0, (n, nb)).reshape(n, nb, 2)
        return out.reshape(n, nb * 176)
    if wtype == 14:
        out = rng.integers(0, 256, size=(n, nb, 210), dtype=np.uint8)
        out[:, :, 208:210] = halves(32.0 * 64.0, (n, nb)).reshape(n, nb, 2)
        return out.reshape(n, nb * 210)
    raise ValueError(wtype)


def topk_route(rng: np.random.Generator, tokens: int, experts: int, used: int):
    """Router of the MoE config: logits N(0,1) -> softmax -> top-`used` (ties to the
    lower index), weights renormalised.  Returns (ids I32 [tokens, used], w F32)."""
    logits = rng.normal(0.0, 1.0, size=(tokens, experts)).astype(np.float32)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p = p / p.sum(axis=1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :used]
    w = np.take_along_axis(p, order, axis=1)
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return order.astype(np.int32), w
