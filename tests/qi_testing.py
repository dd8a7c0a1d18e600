"""Seeded inputs with the benchmark's distributions, and small helpers shared by the tests,
the smoke check and the bench: W ~ N(0, 0.02) rounded to fp16 and packed by the oracle packer;
X fp16 ~ N(0, 1) with a seeded 1 % of the input channels scaled by 20."""
from __future__ import annotations

import numpy as np

from oracle import qipack_oracle as qo


def make_weights(rng, n: int, k: int) -> np.ndarray:
    return rng.standard_normal((n, k), dtype=np.float32).__mul__(np.float32(0.02)).astype(np.float16)


def make_activations(rng, m: int, k: int, kind: str = "outliers") -> np.ndarray:
    """fp16 activations: 'outliers' (N(0,1), 1 % of channels x20), 'gelu' (GELU-tanh of N(0,1),
    the fc2 input), 'silu' (SiLU of N(0,1), the modulation input)."""
    x = rng.standard_normal((m, k), dtype=np.float32)
    if kind == "outliers":
        channels = rng.choice(k, size=max(1, k // 100), replace=False)
        x[:, channels] *= np.float32(20.0)
    elif kind == "gelu":
        x = (0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))).astype(np.float32)
    elif kind == "silu":
        x = (x / (1.0 + np.exp(-x))).astype(np.float32)
    else:
        raise ValueError(kind)
    return x.astype(np.float16)


def make_bias(rng, n: int) -> np.ndarray:
    return (rng.standard_normal(n, dtype=np.float32) * np.float32(0.01)).astype(np.float32)


def pack_w4a16(w16: np.ndarray, clip: bool = False):
    return qo.pack_matrix(w16, qo.SCHEME_W4A16, clip)


def pack_w4a4(w16: np.ndarray, clip: bool = True):
    codes, scales, _ = qo.pack_matrix(w16, qo.SCHEME_W4A4_H256, clip)
    return codes, scales


def random_w4a16_pack(rng, n: int, k: int):
    """Arbitrary (not packer-made) but valid W4A16 records: cheap for large shapes."""
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.uniform(2e-3, 8e-3, size=(n, k // 64)).astype(np.float16)
    minimums = (-8.0 * scales.astype(np.float32) * rng.uniform(0.8, 1.2, size=scales.shape)).astype(np.float16)
    return codes, scales.view(np.uint16), minimums.view(np.uint16)


def random_w4a4_pack(rng, rows: int, k: int, scale_low: float, scale_high: float):
    """Arbitrary signed codes in -7..7 (never -8, as the format promises) and fp16 scales."""
    values = rng.integers(-7, 8, size=(rows, k), dtype=np.int8).astype(np.int16) & 0xF
    codes = (values[:, 0::2] | (values[:, 1::2] << 4)).astype(np.uint8)
    scales = rng.uniform(scale_low, scale_high, size=(rows, k // 64)).astype(np.float16)
    return codes, scales.view(np.uint16)


def max_relative_error(actual: np.ndarray, expected: np.ndarray) -> float:
    """max |actual - expected| / max |expected|: the bench programs' scale-free error
    (bench_w4a4.cu:445-456 prints the RMS form of the same ratio)."""
    return float(np.max(np.abs(actual.astype(np.float64) - expected.astype(np.float64))) /
                 max(float(np.max(np.abs(expected))), 1e-30))


def fp16_store_error(actual_f16: np.ndarray, expected_f32: np.ndarray):
    """How far stored fp16 outputs are from the fp32 oracle rounded to fp16, in fp16 units in the
    last place. Returns (largest distance over elements that are not tiny, fraction of elements
    checked that way). An element counts as tiny when |expected| < 2^-6 * max|expected|: there a
    distance in its own ulps says nothing (the fp32 sums already differ by more than that through
    summation order), and it is covered by the absolute check of max_relative_error instead."""
    expected = expected_f32.astype(np.float32)
    a = actual_f16.astype(np.float16).view(np.int16).astype(np.int32)
    e = expected.astype(np.float16).view(np.int16).astype(np.int32)
    a = np.where(a < 0, -32768 - a, a)  # order-preserving map of sign-magnitude to two's complement
    e = np.where(e < 0, -32768 - e, e)
    large = np.abs(expected) >= np.max(np.abs(expected)) * np.float32(2.0 ** -6)
    return int(np.max(np.abs(a - e)[large])), float(large.mean())
