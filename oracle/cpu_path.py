"""Oracle (test infrastructure): the reference's CPU route, written with torch CPU ops.

mlkit has no CPU inference module, but its reconstruct-plus-matmul arithmetic is
ordinary tensor code that runs on host cores: ``unpack``
(``quantization/operations/bit_packing.py:80-99``), ``decode_scaled``
(``quantization/codecs/scaled.py:53-61``), a cast to the storage dtype
(``inference/packed_linear.py:122``) and ``torch.nn.functional.linear``
(``:154``).  This module restates those steps with the same torch operators so
that timing it on the host measures what the reference would do there, with all
the intra-op threads torch uses.  It is the timed CPU baseline and the
benchmark's reference arm; nothing in the product calls it.
"""

import math
import time

import torch


def unpack_torch(packed: torch.Tensor, bits: int, shape: tuple) -> torch.Tensor:
    """Stream to uint8 codes for widths up to eight bits, with byte arithmetic like the reference."""
    count = math.prod(shape)
    stream = packed.reshape(-1)
    if bits == 8:
        return stream.reshape(shape).clone()
    if 8 % bits == 0:
        mask = (1 << bits) - 1
        lanes = [(stream >> s) & mask for s in range(0, 8, bits)]
        return torch.stack(lanes, 1).reshape(-1)[:count].reshape(shape)
    divisor = math.gcd(bits, 8)
    word_bytes, word_codes = bits // divisor, 8 // divisor
    pad = (-stream.numel()) % word_bytes
    if pad:
        stream = torch.cat((stream, stream.new_zeros(pad)))
    words = stream.reshape(-1, word_bytes)
    out = torch.empty((len(words), word_codes), dtype=torch.uint8)
    mask = (1 << bits) - 1
    for column in range(word_codes):
        byte, shift = divmod(column * bits, 8)
        code = words[:, byte] >> shift
        if shift + bits > 8:
            code = code | (words[:, byte + 1] << (8 - shift))
        out[:, column] = code & mask
    return out.reshape(-1)[:count].reshape(shape)


def reconstruct_torch(packed, scales16, values, group, bits, shape, zero16=None,
                      storage=torch.float16) -> torch.Tensor:
    codes = unpack_torch(packed, bits, shape)
    rows, width = shape
    dense = values[codes.int()]
    scales = scales16.float()
    if width % group == 0:
        dense = dense.reshape(rows, -1, group) * scales[:, :, None]
        if zero16 is not None:
            dense = dense + zero16.float()[:, :, None]
        dense = dense.reshape(rows, width)
    else:
        columns = torch.arange(width) // group
        dense = dense * scales[:, columns]
        if zero16 is not None:
            dense = dense + zero16.float()[:, columns]
    return dense.to(storage)


def reconstruct_plus_matmul(x, packed, scales16, values, group, bits, shape, zero16=None, bias=None):
    """One CPU "step": reconstruct the storage-dtype weight, then ``F.linear`` in the input dtype."""
    dense = reconstruct_torch(packed, scales16, values, group, bits, shape, zero16, storage=x.dtype)
    return torch.nn.functional.linear(x, dense, bias)


def time_reconstruct_plus_matmul(layers, rows_in: int, repetitions: int, warmup: int = 1):
    """Median seconds for one pass over ``layers`` (dicts with packed/scales/values/group/bits/shape).

    Returns ``(median_seconds, threads)``.
    """
    inputs = [torch.randn(rows_in, layer["shape"][1]).half() for layer in layers]
    samples = []
    with torch.inference_mode():
        for iteration in range(warmup + repetitions):
            start = time.perf_counter()
            for layer, x in zip(layers, inputs):
                reconstruct_plus_matmul(x, layer["packed"], layer["scales"], layer["values"],
                                        layer["group"], layer["bits"], layer["shape"])
            if iteration >= warmup:
                samples.append(time.perf_counter() - start)
    samples.sort()
    return samples[len(samples) // 2], torch.get_num_threads()
