"""Structured orthogonal transforms: Walsh-Hadamard times a small dense factor, optionally randomised.

API of ``src/mlkit/quantization/operations/orthogonal_transforms.py`` (``hadamard`` ``:12-31``,
``paley_matrix`` ``:38-68``, ``transform_factor`` ``:71-98``, ``structured_transform`` ``:101-109``,
``randomized_transform`` / ``rht`` ``:112-122``).  The factorisation and the factor bases are built on
the host exactly as the reference builds them; the transform itself is one fused CUDA launch
(``csrc/hadamard.cu``) in the dtype of the input, where the reference chains casts, a sign multiply,
several butterfly launches, two transposes and a library matmul.

Inputs must be CUDA tensors: this package has no CPU arithmetic path.
"""

import functools
import math

import torch
from torch import Tensor

from mlkit_b200 import kernels


def _is_prime(value: int) -> bool:
    return value >= 2 and all(value % divisor for divisor in range(2, math.isqrt(value) + 1))


def _jacobsthal(field: int) -> Tensor:
    """chi(i - j) over GF(field): 0 on the diagonal, +1 for squares, -1 otherwise."""
    index = torch.arange(field, device="cpu")
    difference = (index[:, None] - index[None, :]) % field
    square = torch.zeros(field, device="cpu")
    square[(index[1:] ** 2) % field] = 1
    return torch.where(difference == 0, 0.0, 2 * square[difference] - 1)


@functools.lru_cache(maxsize=32)
def paley_matrix(order: int) -> Tensor:
    """Orthonormal Hadamard matrix from a prime-field Paley design (construction I or II)."""
    if _is_prime(order - 1) and (order - 1) % 4 == 3:
        matrix = torch.ones(order, order, device="cpu")
        matrix[1:, 0] = -1
        matrix[1:, 1:] = _jacobsthal(order - 1) + torch.eye(order - 1, device="cpu")
        return matrix / math.sqrt(order)
    field = order // 2 - 1
    if order % 2 == 0 and _is_prime(field) and field % 4 == 1:
        conference = torch.ones(field + 1, field + 1, device="cpu")
        conference[0, 0] = 0
        conference[1:, 1:] = _jacobsthal(field)
        eye = torch.eye(field + 1, device="cpu")
        top = torch.cat((conference + eye, conference - eye), dim=1)
        bottom = torch.cat((conference - eye, -conference - eye), dim=1)
        return torch.cat((top, bottom), dim=0) / math.sqrt(order)
    raise ValueError(f"no prime-field Paley construction for order {order}")


@functools.lru_cache(maxsize=128)
def transform_factor(width: int) -> tuple[int, int, Tensor | None]:
    """``(factor, power, basis)`` with ``width == factor * power`` and ``power`` a power of two.

    A power-of-two width needs no basis.  Otherwise the odd part, times 1, 2, 4, 8 or 16, is tried as
    a Paley order; failing all, the odd part keeps an orthonormal DCT-II basis.
    """
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
    index = torch.arange(odd, dtype=torch.float64, device="cpu")
    matrix = torch.cos(math.pi / odd * (index[None, :] + 0.5) * index[:, None])
    matrix[0] *= 1 / math.sqrt(odd)
    matrix[1:] *= math.sqrt(2 / odd)
    return odd, power, matrix.float()


@functools.lru_cache(maxsize=64)
def _device_basis(width: int, device: torch.device) -> Tensor | None:
    basis = transform_factor(width)[2]
    return None if basis is None else basis.to(device).contiguous()


def sign_vector(width: int, seed: int, device: torch.device | str) -> Tensor:
    """The +-1 vector of the randomised transform for ``seed``, drawn as the reference draws it:
    ``randint(2, (width,))`` from a generator of the tensor's own device, so a checkpoint rotated on
    CUDA by the reference is un-rotated by the same signs here.  Returned as int8."""
    device = torch.device(device)
    generator = torch.Generator(device=device).manual_seed(seed)
    bits = torch.randint(2, (width,), generator=generator, device=device)
    return (bits * 2 - 1).to(torch.int8)


def _require_cuda(value: Tensor) -> None:
    if not value.is_cuda:
        raise ValueError("mlkit_b200 transforms run on CUDA tensors only")
    if value.requires_grad and torch.is_grad_enabled():
        raise RuntimeError("the fused transform does not support autograd")


def hadamard(value: Tensor, *, normalize: bool = True) -> Tensor:
    """Fast Walsh-Hadamard transform along the last axis (a power of two)."""
    width = value.shape[-1]
    if width <= 0 or width & (width - 1):
        raise ValueError("hadamard currently requires a power-of-two final dimension")
    _require_cuda(value)
    return kernels.structured_transform(value, factor=1, power=width, normalize=normalize)


def structured_transform(value: Tensor, *, inverse: bool = False, signs: Tensor | None = None) -> Tensor:
    """``(B kron H)`` over the last axis; with ``signs`` the randomised form ``S(x * signs)``."""
    _require_cuda(value)
    width = value.shape[-1]
    factor, power, _ = transform_factor(width)
    return kernels.structured_transform(value, factor=factor, power=power, basis=_device_basis(width, value.device),
                                        signs=signs, inverse=inverse)


def randomized_transform(value: Tensor, *, seed: int = 0, inverse: bool = False,
                         signs: Tensor | None = None) -> Tensor:
    """``S(value * signs)`` (or ``S^-1(value) * signs``); ``signs`` defaults to ``sign_vector(seed)``."""
    if signs is None:
        signs = sign_vector(value.shape[-1], seed, value.device)
    return structured_transform(value, inverse=inverse, signs=signs)


rht = randomized_transform
