"""Seeded synthetic layers for the parity tests, built with the numpy oracle only."""

import functools

import numpy as np

from oracle import bitstream, codec

CODEBOOK3 = np.array([-1, -0.5, -0.25, 0, 0.25, 0.5, 1.0], dtype=np.float32)


def grid_values(kind: str, bits: int) -> tuple[np.ndarray, bool]:
    if kind == "int":
        return codec.int_values(bits), True
    if kind == "nf4":
        return codec.NF4_VALUES, False
    if kind == "codebook3":
        return CODEBOOK3, False
    raise ValueError(kind)


@functools.lru_cache(maxsize=8)
def make_layer(rows: int, width: int, bits: int, group: int, kind: str = "int", seed: int = 0,
               scale: str = "absmax", asym: bool = False):
    """RTN-quantise a seeded N(0, 0.02) fp16 weight; returns a dict of numpy arrays."""
    rng = np.random.default_rng(seed)
    weight = (rng.standard_normal((rows, width), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    values, integer = grid_values(kind, bits)
    codes, scales, zero = codec.rtn_encode(weight.astype(np.float32), values, group, integer=integer,
                                           scale=scale, asym=asym)
    return {
        "rows": rows, "width": width, "bits": bits, "group": min(group, width), "values": values,
        "codes": codes, "packed": bitstream.pack(codes, bits), "scales16": scales.astype(np.float16),
        "zero16": None if zero is None else zero.astype(np.float16), "integer": integer,
    }


def random_layer(rows: int, width: int, bits: int, group: int, seed: int = 0, *, lut_len=None,
                 zeros: bool = False):
    """Uniform random codes with random positive fp16 scales: any shape, no encode cost."""
    rng = np.random.default_rng(seed)
    lut_len = lut_len or 2**bits
    codes = rng.integers(0, lut_len, size=(rows, width), dtype=np.uint8)
    groups = -(-width // group)
    scales = (rng.random((rows, groups), dtype=np.float32) * 0.01 + 0.001).astype(np.float16)
    zero = (rng.standard_normal((rows, groups), dtype=np.float32) * 0.01).astype(np.float16) if zeros else None
    values = np.sort(rng.standard_normal(lut_len).astype(np.float32))
    return {
        "rows": rows, "width": width, "bits": bits, "group": group, "values": values, "codes": codes,
        "packed": bitstream.pack(codes, bits), "scales16": scales, "zero16": zero, "integer": False,
    }


def activations(rows: int, width: int, seed: int = 1, outliers: bool = False) -> np.ndarray:
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, width), dtype=np.float32)
    if outliers:
        picks = rng.permutation(width)[: max(1, width // 100)]
        x[:, picks] *= 50
    return x.astype(np.float16)
