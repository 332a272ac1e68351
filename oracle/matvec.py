"""Oracle (test infrastructure): reconstruct-then-matmul, the matvec reference result.

The fused kernel of the reference (``kernels/packed_linear.py:107-173``) and the
kernels of this repository are both compared with the dense route that
``PackedLinear.forward`` itself takes for more than eight rows
(``inference/packed_linear.py:152-154``): unpack the stream, reconstruct the
weight in the storage dtype, multiply.  The product is formed in fp32 (fp64
accumulate is offered for a tighter yardstick).
"""

import numpy as np

from oracle import bitstream, codec

F32 = np.float32


def reconstruct_then_matmul(x, packed, scales16, values, group, bits, shape, *, zero16=None,
                            bias=None, storage=np.float16, accumulate=np.float32):
    """``y = x @ W_ref.T (+ bias)`` with ``W_ref`` the storage-dtype reconstruction."""
    codes = bitstream.unpack(np.asarray(packed), bits, shape)
    dense = codec.reconstruct_weight(codes, scales16, values, group, zero16, storage)
    y = np.asarray(x).astype(accumulate) @ dense.astype(accumulate).T
    if bias is not None:
        y = y + np.asarray(bias).astype(accumulate)
    return y


def relative_l2(actual, expected) -> float:
    """``||actual - expected|| / ||expected||`` in float64."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    denominator = np.linalg.norm(e)
    return float(np.linalg.norm(a - e) / denominator) if denominator else float(np.linalg.norm(a))


def gemv_bytes(rows_out: int, width: int, bits: int, group: int, rows_in: int, *,
               lut_len: int = 0, scale_bytes: int = 2, act_bytes: int = 2, bias: bool = False,
               zeros: bool = False) -> int:
    """Algorithmic bytes of one packed matvec: codes + scales (+offsets) + x + y (+ LUT, bias)."""
    groups = -(-width // group)
    total = rows_out * width * bits // 8 + rows_out * groups * scale_bytes * (2 if zeros else 1)
    total += rows_in * width * act_bytes + rows_in * rows_out * act_bytes + 4 * lut_len
    return total + (rows_out * act_bytes if bias else 0)
