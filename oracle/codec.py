"""Oracle (test infrastructure): grouped scalar codec, decode and round-to-nearest encode.

Decode restates ``quantization/codecs/scaled.py:19-78`` (tensor path ``:53-61``):
``values[codes] * scales[:, col // group] (+ zero[:, col // group])`` as one
binary32 multiply followed, when offsets exist, by one separate binary32 add.

Encode restates ``quantization/formats/grouped_scaling.py``:
``_initial_scales`` (``:274-289``), ``store_scale`` for fp16
(``formats/scale_storage.py:18-19``), ``_search_scales`` (``:291-351``) and
``_scalar_codes`` (``:353-392``) with ``nearest_codes`` (``:46-51``).
"""

import numpy as np

F32 = np.float32


def group_columns(width: int, group: int) -> np.ndarray:
    return np.arange(width) // group


def decode_scaled(codes, scales, values, group, zero=None) -> np.ndarray:
    """fp32 reconstruction of grouped scalar codes (``codecs/scaled.py:53-61``)."""
    codes = np.asarray(codes)
    scales = np.asarray(scales, dtype=F32)
    values = np.asarray(values, dtype=F32)
    columns = group_columns(codes.shape[1], group)
    weights = values[codes.astype(np.int64)] * scales[:, columns]
    if zero is not None:
        weights = weights + np.asarray(zero, dtype=F32)[:, columns]
    return weights.astype(F32, copy=False)


def reconstruct_weight(codes, scales16, values, group, zero16=None, storage=np.float16):
    """Dense weight in the storage dtype, the way ``PackedLinear.weight`` forms it.

    ``inference/packed_linear.py:115-122``: scales (and offsets) are held in half
    precision, widened to fp32, the fp32 reconstruction is rounded once.
    """
    zero = None if zero16 is None else np.asarray(zero16).astype(F32)
    dense = decode_scaled(codes, np.asarray(scales16).astype(F32), values, group, zero)
    return dense.astype(storage)


def fp32_reciprocal(value: float) -> np.float32:
    """``single_precision_reciprocal`` (``grouped_scaling.py:25-28``)."""
    return F32(1.0) / F32(value)


def group_extrema(weight: np.ndarray, group: int):
    """Per-group minimum and maximum; a short last group keeps only its columns (``:30-43``)."""
    rows, width = weight.shape
    whole = width - width % group
    lows, highs = [], []
    if whole:
        blocks = weight[:, :whole].reshape(rows, -1, group)
        lows.append(blocks.min(-1))
        highs.append(blocks.max(-1))
    if whole < width:
        rest = weight[:, whole:]
        lows.append(rest.min(-1, keepdims=True))
        highs.append(rest.max(-1, keepdims=True))
    return np.concatenate(lows, 1), np.concatenate(highs, 1)


def store_fp16(value: np.ndarray) -> np.ndarray:
    """fp16 round trip with the clamp of ``scale_storage.py:18-19``."""
    return np.clip(value, F32(2.0**-24), F32(65504.0)).astype(np.float16).astype(F32)


def nearest_codes(normalized: np.ndarray, values: np.ndarray) -> np.ndarray:
    """Index of the nearest ascending codebook entry, ties to the lower (``:46-51``)."""
    upper = np.minimum(np.searchsorted(values, normalized, side="left"), values.size - 1)
    lower = np.maximum(upper - 1, 0)
    pick_lower = np.abs(normalized - values[lower]) <= np.abs(normalized - values[upper])
    return np.where(pick_lower, lower, upper)


def torch_like_linspace(start: float, end: float, steps: int) -> np.ndarray:
    """fp32 ``torch.linspace``: forward from ``start`` in the first half, backward from ``end`` after."""
    step = (F32(end) - F32(start)) / F32(steps - 1)
    out = np.empty(steps, dtype=F32)
    half = steps // 2
    for i in range(steps):
        out[i] = F32(start) + step * F32(i) if i < half else F32(end) - step * F32(steps - i - 1)
    return out


def rtn_encode(weight, values, group, *, integer, scale="absmax", asym=False, search_steps=20):
    """Round-to-nearest encode of a weight matrix onto a scaled scalar grid.

    Returns ``(codes uint8, scales fp32 holding fp16 values, zero or None)``.
    """
    weight = np.asarray(weight, dtype=F32)
    values = np.asarray(values, dtype=F32)
    rows, width = weight.shape
    group = min(group or width, width)
    low_value, high_value = F32(values.min()), F32(values.max())
    low, high = group_extrema(weight, group)
    if asym:
        reciprocal = fp32_reciprocal(float(high_value - low_value))
        scales = np.maximum(high - low, F32(1e-12)) * reciprocal
        zero = low - low_value * scales
    else:
        reciprocal = fp32_reciprocal(float(np.abs(values).max()))
        scales = np.maximum(np.maximum(high, -low), F32(1e-12)) * reciprocal
        zero = None
    scales = store_fp16(scales.astype(F32))
    columns = group_columns(width, group)

    def snap(normalized):
        if integer:
            return np.clip(np.round(normalized), low_value, high_value)
        return values[nearest_codes(normalized, values)]

    if scale == "mse":
        pad = (-width) % group
        blocks = np.pad(weight, ((0, 0), (0, pad))).reshape(rows, -1, group)
        occupied = None
        if pad:
            occupied = (np.arange(blocks.shape[1] * group) < width).reshape(1, -1, group)
        centered = blocks if zero is None else blocks - zero[..., None]

        def group_error(candidate):
            normalized = centered / candidate[..., None]
            error = np.square(snap(normalized) * candidate[..., None] - centered)
            if occupied is not None:
                error = error * occupied
            return error.sum(-1, dtype=F32)

        selected = scales.copy()
        best = group_error(scales)
        for fraction in torch_like_linspace(0.5, 1.0, search_steps):
            candidate = store_fp16(scales * fraction)
            error = group_error(candidate)
            improved = error < best
            selected = np.where(improved, candidate, selected)
            best = np.minimum(best, error)
        scales = selected
    if zero is not None:
        magnitude = store_fp16(np.maximum(np.abs(zero), F32(1e-12)))
        zero = (magnitude * np.sign(zero)).astype(F32)
    centered = weight if zero is None else weight - zero[:, columns]
    normalized = centered / scales[:, columns]
    if integer:
        codes = np.clip(np.round(normalized), low_value, high_value) - low_value
    else:
        codes = nearest_codes(normalized, values)
    return codes.astype(np.uint8), scales.astype(F32), zero


NF4_VALUES = np.array(
    [-1.0, -0.6961928, -0.52507305, -0.39491749, -0.28444138, -0.18477343, -0.09105004, 0.0,
     0.07958030, 0.16093020, 0.24611230, 0.33791524, 0.44070983, 0.56261700, 0.72295684, 1.0],
    dtype=F32,
)
"""The sixteen normal-float levels; data of the format (``grids/factory.py:148-152``)."""


def int_values(bits: int) -> np.ndarray:
    """Signed integer grid levels ``-2**(b-1) .. 2**(b-1)-1`` (``grids/factory.py:58-62``)."""
    return np.arange(-(2 ** (bits - 1)), 2 ** (bits - 1), dtype=F32)
