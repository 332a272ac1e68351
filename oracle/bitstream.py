"""Oracle (test infrastructure): unsigned little-endian bit streams.

Stream rule of the reference (``quantization/operations/bit_packing.py:13-29``
for ``pack`` and ``:80-99`` for ``unpack``): codes are flattened in row-major
order; bit ``j`` of code ``i`` is stream bit ``i*bits + j``; stream bit ``t`` is
bit ``t % 8`` (least significant first) of byte ``t // 8``; the final byte is
zero padded.  The reference reaches that layout through three code paths
(within-byte ``:32-43``, across-byte ``:46-77`` and sixteen-bit ``:22-24``);
here one bit-matrix formulation covers every width from 1 to 16.
"""

import math

import numpy as np


def pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """Bytes of the stream that holds ``codes`` at ``bits`` bits each.

    Validation mirrors ``bit_packing.py:15-21``: widths outside 1..16, floating
    codes and codes outside ``[0, 2**bits)`` are rejected.
    """
    if not 1 <= bits <= 16:
        raise ValueError("packing supports one through sixteen bits")
    flat = np.asarray(codes).reshape(-1)
    if flat.dtype.kind == "f":
        raise TypeError("codes must have an integer dtype")
    if flat.size and (int(flat.min()) < 0 or int(flat.max()) >= 2**bits):
        raise ValueError("codes exceed the declared unsigned bit capacity")
    wide = flat.astype(np.uint32)
    planes = ((wide[:, None] >> np.arange(bits, dtype=np.uint32)) & 1).astype(np.uint8)
    return np.packbits(planes.reshape(-1), bitorder="little")


def unpack(packed: np.ndarray, bits: int, shape: tuple) -> np.ndarray:
    """Codes of a stream; uint8 up to eight bits, int32 above (``bit_packing.py:92-99,116-135``)."""
    packed = np.asarray(packed)
    if not 1 <= bits <= 16 or packed.dtype != np.uint8:
        raise ValueError("unpack requires uint8 storage and one through sixteen bits")
    if any(d < 0 for d in shape):
        raise ValueError("shape dimensions must be nonnegative")
    count = math.prod(shape)
    if packed.size != math.ceil(count * bits / 8):
        raise ValueError("packed byte count does not match the declared shape and precision")
    planes = np.unpackbits(packed.reshape(-1), bitorder="little")[: count * bits]
    planes = planes.reshape(count, bits).astype(np.uint32)
    codes = (planes << np.arange(bits, dtype=np.uint32)).sum(axis=1, dtype=np.uint32)
    return codes.astype(np.uint8 if bits <= 8 else np.int32).reshape(shape)


def word_geometry(bits: int) -> tuple[int, int]:
    """(bytes per word, codes per word): the period of the stream (``kernels/packed_linear.py:66-69``)."""
    divisor = math.gcd(bits, 8)
    return bits // divisor, 8 // divisor


def fused_layout(bits: int, width: int, group: int):
    """Eligibility of a layer for the fused matvec, as ``layout_for`` decides it.

    Follows ``kernels/packed_linear.py:63-79``: rows and scale groups must hold
    whole words; the tile is the largest power-of-two word count dividing a
    group, capped at 128 codes; tiles under 16 codes are refused.  Returns
    ``(bits, bytes_per_word, codes_per_word, tile_words)`` or ``None``.
    """
    if not 1 <= bits <= 8:
        return None
    bytes_per_word, codes_per_word = word_geometry(bits)
    if width % codes_per_word or group % codes_per_word:
        return None
    group_words = group // codes_per_word
    tile_words = min(128 // codes_per_word, group_words & -group_words)
    if tile_words * codes_per_word < 16:
        return None
    return bits, bytes_per_word, codes_per_word, tile_words
