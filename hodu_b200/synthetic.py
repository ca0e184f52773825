"""Seeded synthetic operands for the five benchmark configurations.

`Tensor::randn` in the reference draws from an unseeded generator
(crates/hodu_core/src/be_cpu/device.rs:163-166), so "seed s" can only mean a generator
owned by the harness.  This one is numpy's counter-based Philox keyed by the seed;
values are produced in f32 on the host (integers for the i8 case) and narrowed by
the caller -- on the device with this library's cast kernels, or on the host with
the oracle's codecs -- so both sides start from the same f32 numbers.

`scale` divides every extent (rounded up to a multiple of `multiple`) to get
small cases with the same value distributions for tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=seed))


def _dim(n: int, scale: int, multiple: int = 8) -> int:
    if scale <= 1:
        return n
    return max(multiple, int(math.ceil(n / scale / multiple)) * multiple)


def config1(scale: int = 1) -> Dict[str, np.ndarray]:
    """f32 A[512,1024] @ B[1024,768], N(0,1), seed 0."""
    m, k, n = _dim(512, scale), _dim(1024, scale), _dim(768, scale)
    g = _rng(0)
    return {"a": g.standard_normal((m, k), dtype=np.float32), "b": g.standard_normal((k, n), dtype=np.float32)}


def config2(scale: int = 1, batches: int = 16) -> Dict[str, np.ndarray]:
    """bf16 A[16,2048,2048] @ B[16,2048,2048]; N(0,1)/sqrt(2048) in f32, seed 1, A then B."""
    d = _dim(2048, scale)
    g = _rng(1)
    s = np.float32(1.0 / math.sqrt(2048.0))
    a = g.standard_normal((batches, d, d), dtype=np.float32) * s
    b = g.standard_normal((batches, d, d), dtype=np.float32) * s
    return {"a": a, "b": b}


def config3(scale: int = 1) -> Dict[str, np.ndarray]:
    """f8e4m3 A[8192,8192] @ B[8192,8192]; N(0,1)*64 clamped to +-448, seed 2; scales 1/64."""
    d = _dim(8192, scale, 16)
    g = _rng(2)
    a = np.clip(g.standard_normal((d, d), dtype=np.float32) * np.float32(64), -448, 448)
    b = np.clip(g.standard_normal((d, d), dtype=np.float32) * np.float32(64), -448, 448)
    return {"a": a, "b": b, "scale_a": 1.0 / 64.0, "scale_b": 1.0 / 64.0}


def config4(scale: int = 1) -> Dict[str, np.ndarray]:
    """i8 A[8192,8192] @ B[8192,8192]; uniform integers in [-127,127], seed 3."""
    d = _dim(8192, scale, 16)
    g = _rng(3)
    a = g.integers(-127, 128, size=(d, d), dtype=np.int8)
    b = g.integers(-127, 128, size=(d, d), dtype=np.int8)
    return {"a": a, "b": b}


def config5(scale: int = 1, tokens: int = 16384) -> Dict[str, np.ndarray]:
    """SwiGLU MLP: X[16384,4096] N(0,1) seed 4; W_gate, W_up [4096,14336], W_down [14336,4096]
    N(0,0.02) seed 5 (gate, up, down in that order).  Weights are given as [K,N] matrices."""
    t, d, h = _dim(tokens, scale), _dim(4096, scale), _dim(14336, scale)
    x = _rng(4).standard_normal((t, d), dtype=np.float32)
    g = _rng(5)
    std = np.float32(0.02)
    wg = g.standard_normal((d, h), dtype=np.float32) * std
    wu = g.standard_normal((d, h), dtype=np.float32) * std
    wd = g.standard_normal((h, d), dtype=np.float32) * std
    return {"x": x, "w_gate": wg, "w_up": wu, "w_down": wd}


FLOPS = {  # 2*M*N*K*batch at full size
    1: 2 * 512 * 1024 * 768,
    2: 2 * 16 * 2048 ** 3,
    3: 2 * 8192 ** 3,
    4: 2 * 8192 ** 3,
    5: 3 * 2 * 16384 * 4096 * 14336,
}
