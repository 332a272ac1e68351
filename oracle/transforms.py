"""Oracle (test infrastructure): Walsh-Hadamard and structured orthogonal transforms.

Restates ``quantization/operations/orthogonal_transforms.py``:
``hadamard`` stage-by-stage path (``:23-31``), ``paley_matrix`` (``:38-68``),
``transform_factor`` (``:71-98``), ``structured_transform`` (``:101-109``) and
``randomized_transform`` (``:112-118``).  The sign vector of the randomized
transform is an explicit argument here: the reference draws it from a torch
generator on the tensor's device, and CPU and CUDA generators yield different
vectors for one seed, so parity is only meaningful with the signs given.
"""

import math

import numpy as np

F32 = np.float32


def fwht_stagewise(value: np.ndarray) -> np.ndarray:
    """Unnormalised FWHT over the last axis, butterflies in ascending stride (``:25-30``)."""
    value = np.asarray(value)
    width = value.shape[-1]
    if width <= 0 or width & (width - 1):
        raise ValueError("hadamard currently requires a power-of-two final dimension")
    out = value.copy()
    stride = 1
    while stride < width:
        pairs = out.reshape(*value.shape[:-1], -1, 2, stride)
        first, second = pairs[..., 0, :], pairs[..., 1, :]
        out = np.stack((first + second, first - second), axis=-2).reshape(value.shape)
        stride *= 2
    return out


def hadamard(value: np.ndarray, normalize: bool = True, *, by_multiply: bool = False) -> np.ndarray:
    """Normalised FWHT.

    The tensor path divides by ``sqrt(width)`` (``:31``).  The reference's fused
    CUDA kernel instead multiplies by the fp32 reciprocal
    (``kernels/hadamard.py:115``); ``by_multiply`` selects that rounding.
    """
    out = fwht_stagewise(value)
    if not normalize:
        return out
    width = value.shape[-1]
    dtype = out.dtype.type
    if by_multiply:
        return out * (dtype(1.0) / dtype(math.sqrt(width)))
    return out / dtype(math.sqrt(width))


def is_prime(value: int) -> bool:
    return value >= 2 and all(value % d for d in range(2, math.isqrt(value) + 1))


def _quadratic_characters(field: int) -> np.ndarray:
    """Jacobsthal matrix chi(i - j) over GF(field): 0 on the diagonal, +-1 elsewhere."""
    index = np.arange(field)
    difference = (index[:, None] - index[None, :]) % field
    residue = np.zeros(field, dtype=F32)
    residue[(index[1:] ** 2) % field] = 1
    return np.where(difference == 0, F32(0), 2 * residue[difference] - 1).astype(F32)


def paley_matrix(order: int) -> np.ndarray:
    """Orthonormal Hadamard matrix of a prime-field Paley design (``:38-68``).

    Construction I when ``order - 1`` is a prime congruent to 3 mod 4, else
    construction II when ``order / 2 - 1`` is a prime congruent to 1 mod 4.
    """
    if is_prime(order - 1) and (order - 1) % 4 == 3:
        field = order - 1
        matrix = np.ones((order, order), dtype=F32)
        matrix[1:, 0] = -1
        matrix[1:, 1:] = _quadratic_characters(field) + np.eye(field, dtype=F32)
        return (matrix / F32(math.sqrt(order))).astype(F32)
    field = order // 2 - 1
    if order % 2 == 0 and is_prime(field) and field % 4 == 1:
        conference = np.ones((field + 1, field + 1), dtype=F32)
        conference[0, 0] = 0
        conference[1:, 1:] = _quadratic_characters(field)
        eye = np.eye(field + 1, dtype=F32)
        matrix = np.block([[conference + eye, conference - eye],
                           [conference - eye, -conference - eye]])
        return (matrix / F32(math.sqrt(order))).astype(F32)
    raise ValueError(f"no prime-field Paley construction for order {order}")


def transform_factor(width: int):
    """``(factor, power, basis or None)`` with ``width == factor * power`` (``:71-98``)."""
    if width < 1:
        raise ValueError("transform width must be positive")
    if width & (width - 1) == 0:
        return 1, width, None
    odd = width
    while odd % 2 == 0:
        odd //= 2
    power = width // odd
    for multiplier in (1, 2, 4, 8, 16):
        if power % multiplier:
            continue
        try:
            return odd * multiplier, power // multiplier, paley_matrix(odd * multiplier)
        except ValueError:
            continue
    index = np.arange(odd, dtype=np.float64)
    matrix = np.cos(math.pi / odd * (index[None, :] + 0.5) * index[:, None])
    matrix[0] *= 1 / math.sqrt(odd)
    matrix[1:] *= math.sqrt(2 / odd)
    return odd, power, matrix.astype(F32)


def structured_transform(value: np.ndarray, inverse: bool = False, *, by_multiply: bool = False):
    """``(B_factor kron H_power)`` applied over the last axis (``:101-109``)."""
    value = np.asarray(value)
    factor, power, basis = transform_factor(value.shape[-1])
    if basis is None:
        return hadamard(value, by_multiply=by_multiply)
    blocks = value.reshape(*value.shape[:-1], factor, power)
    basis = basis.astype(value.dtype)
    mixed = np.swapaxes(hadamard(blocks, by_multiply=by_multiply), -1, -2)
    mixed = mixed @ (basis if inverse else basis.T)
    return np.swapaxes(mixed, -1, -2).reshape(value.shape)


def randomized_transform(value, signs, inverse: bool = False, *, by_multiply: bool = False):
    """``S(value * signs)``, or its inverse ``S^-1(value) * signs`` (``:112-118``)."""
    signs = np.asarray(signs).astype(np.asarray(value).dtype)
    if inverse:
        return structured_transform(value, inverse=True, by_multiply=by_multiply) * signs
    return structured_transform(value * signs, by_multiply=by_multiply)
