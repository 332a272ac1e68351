"""Quantised-weight carrier, codec registry, bit streams, grids and round-to-nearest formats.

These are the host-side pieces of mlkit's API that the packed-inference path touches.  They keep the
reference's names, argument meaning and error behaviour so that code written against ``mlkit``
(``mk.Q``, ``mk.codec``, ``mk.pack``, ``mk.int`` ...) runs unchanged:

* ``Q``, ``as_q``                       ``src/mlkit/quantization/representation.py:9-75``
* ``codec``, ``decoder``, ``registered``  ``src/mlkit/quantization/codecs/registry.py:11-46``
* ``decode_scaled``, ``decode_feedback``  ``src/mlkit/quantization/codecs/scaled.py:19-101``
* ``pack``, ``unpack``                    ``src/mlkit/quantization/operations/bit_packing.py:13-135``
* ``grid``                                ``src/mlkit/quantization/grids/factory.py:17-152``
* ``scaled``, ``int``, ``nf4``            ``src/mlkit/quantization/formats/grouped_scaling.py:54-414``,
                                          ``formats/standard.py:10-19``, ``formats/scale_storage.py:11-26``
* ``Ctx``, ``layer_seed``                 ``src/mlkit/quantization/context.py:11-13,34-73``

Encoding is conversion-time work and runs as ordinary tensor operations on whatever device the
weight lives on.  Decoding on CUDA goes through the bit-exact dequantisation kernel.
"""

import builtins
import hashlib
import math
from collections.abc import Callable, Mapping
from typing import Any

import torch
from torch import Tensor

# ------------------------------------------------------------------------------------------- Q


class Q:
    """A quantised weight: either a dense reconstruction, or codes with the decoder that expands them.

    ``bits`` counts every stored bit including side information (``None``: unknown).
    """

    def __init__(self, w: Tensor | None = None, *, bits: float | None = None, codes: Tensor | None = None,
                 params: Mapping[str, Any] | None = None, decode: Callable[..., Tensor] | None = None,
                 codec: str | None = None, metadata: Mapping[str, Any] | None = None) -> None:
        if w is None and (codes is None or decode is None):
            raise ValueError("Q requires a reconstruction or codes and a decoder")
        if bits is not None and bits < 0:
            raise ValueError("bits must be nonnegative")
        self._weight = w
        self.bits = bits
        self.codes = codes
        self.params = dict(params or {})
        self.decode = decode
        self.codec = codec
        self.metadata = dict(metadata or {})
        self._stream: tuple[Tensor, Tensor, int, int] | None = None   # (packed, codes it came from, their version, bits)

    def packed_stream(self, bits: int) -> Tensor:
        """``pack(self.codes, bits)``; the stream the device encoder wrote beside the codes is returned
        as it is while the codes are the same tensor, unmodified."""
        held = self._stream
        if (held is not None and held[1] is self.codes and held[2] == _version_of(self.codes) and held[3] == bits):
            return held[0]
        return pack(self.codes, bits)

    @property
    def w(self) -> Tensor:
        """The reconstruction; decoded on every access when codes and a decoder are present."""
        if self.codes is not None and self.decode is not None:
            return self.decode(self.codes, **self.params)
        assert self._weight is not None
        return self._weight

    @property
    def bpw(self) -> float | None:
        return None if self.bits is None else float(self.bits) / self.w.numel()

    def to(self, device: str | torch.device, *, detach: bool = False) -> "Q":
        def move(value: Any) -> Any:
            if isinstance(value, Tensor):
                return (value.detach() if detach else value).to(device)
            if isinstance(value, dict):
                return {key: move(item) for key, item in value.items()}
            return value

        return Q(move(self._weight), bits=self.bits, codes=move(self.codes), params=move(self.params),
                 decode=self.decode, codec=self.codec, metadata=self.metadata)

    def __repr__(self) -> str:
        return f"Q(shape={tuple(self.w.shape)}, bits={self.bits}, codec={self.codec!r})"


def as_q(value: "Q | Tensor") -> Q:
    if isinstance(value, Q):
        return value
    if isinstance(value, Tensor):
        return Q(value)
    raise TypeError(f"quantizers must return a Tensor or Q, received {type(value).__name__}")


# ---------------------------------------------------------------------------- codec registry

_decoders: dict[str, Callable[..., Tensor]] = {}
_row_parameters: dict[str, tuple[str, ...]] = {}


def codec(name: str, *, row_parameters: tuple[str, ...] | None = None) -> Callable[[Callable], Callable]:
    """Decorator that registers a decoder under ``name``; checkpoints store the name."""

    def register(function: Callable[..., Tensor]) -> Callable[..., Tensor]:
        if not name or name in _decoders:
            raise ValueError(f"codec name {name!r} is empty or already registered")
        _decoders[name] = function
        if row_parameters is not None:
            _row_parameters[name] = tuple(row_parameters)
        return function

    return register


def decoder(name: str) -> Callable[..., Tensor]:
    try:
        return _decoders[name]
    except KeyError:
        raise ValueError(f"checkpoint requires registered codec {name!r}") from None


def registered(name: str | None) -> bool:
    return name in _decoders


def row_parameters(name: str | None) -> tuple[str, ...] | None:
    return None if name is None else _row_parameters.get(name)


def _decode_columns(codes: Tensor, scales: Tensor, values: Tensor, columns: Tensor, zero: Tensor | None) -> Tensor:
    dense = values[codes.long()] * scales[:, columns]
    return dense if zero is None else dense + zero[:, columns]


@codec("scaled", row_parameters=("scales", "zero"))
def decode_scaled(codes: Tensor, *, scales: Tensor, values: Tensor, group: int, offset: int = 0,
                  zero: Tensor | None = None) -> Tensor:
    """``values[codes] * scales[:, (offset + col) // group] (+ zero)`` as separate fp32 operations.

    fp32 parameters with uint8 codes on CUDA take the dequantisation kernel (identical bits).
    """
    width = codes.shape[1]
    if (offset == 0 and codes.is_cuda and codes.dtype == torch.uint8 and scales.dtype == torch.float32
            and values.dtype == torch.float32 and values.numel() <= 256
            and not (torch.is_grad_enabled() and (scales.requires_grad or values.requires_grad
                                                  or (zero is not None and zero.requires_grad)))):
        from mlkit_b200 import kernels

        weight, _ = kernels.dequantize(codes.contiguous().reshape(-1), scales.contiguous(), values.contiguous(),
                                       None if zero is None else zero.contiguous(), shape=tuple(codes.shape),
                                       group=group, bits=8, dtype=torch.float32)
        return weight
    columns = torch.arange(offset, offset + width, device=codes.device) // group
    return _decode_columns(codes, scales, values, columns, zero)


@codec("feedback", row_parameters=("scales", "zero"))
def decode_feedback(codes: Tensor, *, scales: Tensor, values: Tensor, group: int, refit: int,
                    zero: Tensor | None = None, permutation: Tensor | None = None) -> Tensor:
    """Error-feedback codes: scale groups restart at every ``refit`` boundary."""
    if refit % group == 0:
        dense = decode_scaled(codes, scales=scales, values=values, group=group, zero=zero)
    else:
        position = torch.arange(codes.shape[1], device=codes.device)
        per_region = -(-refit // group)
        dense = _decode_columns(codes, scales, values,
                                (position // refit) * per_region + (position % refit) // group, zero)
    return dense if permutation is None else dense[:, permutation.argsort()]


# --------------------------------------------------------------------------------- bit streams

_CHUNK_CODES = 1 << 22  # a multiple of eight codes, so every chunk ends on a byte


def _version_of(tensor: Tensor) -> int:
    return 0 if tensor.is_inference() else tensor._version


def pack(codes: Tensor, bits: int) -> Tensor:
    """Little-endian unsigned bit stream: bit ``j`` of code ``i`` is stream bit ``i * bits + j``."""
    if not 1 <= bits <= 16:
        raise ValueError("packing supports one through sixteen bits")
    flat = codes.detach().reshape(-1)
    if flat.is_floating_point():
        raise TypeError("codes must have an integer dtype")
    if flat.numel() and (builtins.int(flat.min()) < 0 or builtins.int(flat.max()) >= 2**bits):
        raise ValueError("codes exceed the declared unsigned bit capacity")
    if bits == 8:
        return flat.to(torch.uint8)
    device = flat.device
    lane = torch.arange(bits, device=device, dtype=torch.int32)
    byte_weights = (1 << torch.arange(8, device=device, dtype=torch.int32))
    pieces = []
    for start in range(0, flat.numel(), _CHUNK_CODES):
        part = flat[start:start + _CHUNK_CODES].to(torch.int32)
        planes = ((part[:, None] >> lane) & 1).reshape(-1)
        tail = (-planes.numel()) % 8
        if tail:
            planes = torch.cat((planes, planes.new_zeros(tail)))
        pieces.append((planes.reshape(-1, 8) * byte_weights).sum(1).to(torch.uint8))
    return torch.cat(pieces) if pieces else torch.empty(0, dtype=torch.uint8, device=device)


def unpack(packed: Tensor, bits: int, shape: tuple[int, ...]) -> Tensor:
    """Inverse of ``pack``: uint8 codes up to eight bits, int32 above."""
    if not 1 <= bits <= 16 or packed.dtype != torch.uint8:
        raise ValueError("unpack requires uint8 storage and one through sixteen bits")
    shape = tuple(shape)
    if any(dimension < 0 for dimension in shape):
        raise ValueError("shape dimensions must be nonnegative")
    count = math.prod(shape)
    if packed.numel() != math.ceil(count * bits / 8):
        raise ValueError("packed byte count does not match the declared shape and precision")
    stream = packed.reshape(-1)
    result_dtype = torch.uint8 if bits <= 8 else torch.int32
    if bits <= 8 and stream.is_cuda and count:
        from mlkit_b200 import kernels

        _, codes = kernels.dequantize(stream.contiguous(), None, None, None, shape=(1, count), group=1,
                                      bits=bits, dtype=None, codes=True)
        return codes.reshape(shape)
    if bits == 8:
        return stream.reshape(shape).clone()
    device = stream.device
    bit = torch.arange(8, device=device, dtype=torch.int32)
    lane_weights = (1 << torch.arange(bits, device=device, dtype=torch.int32))
    pieces = []
    chunk_bytes = _CHUNK_CODES // 8 * bits
    for start in range(0, stream.numel(), chunk_bytes):
        part = stream[start:start + chunk_bytes].to(torch.int32)
        planes = ((part[:, None] >> bit) & 1).reshape(-1)
        whole = planes.numel() // bits
        pieces.append((planes[: whole * bits].reshape(-1, bits) * lane_weights).sum(1))
    codes = torch.cat(pieces)[:count] if pieces else torch.empty(0, dtype=torch.int32, device=device)
    return codes.to(result_dtype).reshape(shape)


# --------------------------------------------------------------------------------------- grids


class Grid:
    """A rounding function with its bit cost; ``values`` lists the levels of a scalar grid."""

    def __init__(self, function: Callable[[Tensor], Tensor], bits: int, dim: int = 1, *,
                 values: Tensor | None = None, name: str = "custom", integer: bool = False) -> None:
        if bits < 1 or dim < 1:
            raise ValueError("grid bits and dimension must be positive")
        self.function, self.bits, self.dim = function, bits, dim
        self.values, self.name, self.integer = values, name, integer

    def __call__(self, value: Tensor) -> Tensor:
        return self.function(value)

    def __repr__(self) -> str:
        return f"Grid({self.name}, bits={self.bits}, dim={self.dim})"


def nearest_level(normalized: Tensor, levels: Tensor) -> Tensor:
    """Index of the nearest ascending level; a tie goes to the lower level."""
    above = torch.searchsorted(levels, normalized.contiguous()).clamp_max(levels.numel() - 1)
    below = (above - 1).clamp_min(0)
    take_below = (normalized - levels[below]).abs() <= (normalized - levels[above]).abs()
    return torch.where(take_below, below, above)


class _GridFactory:
    def int(self, bits: builtins.int) -> Grid:
        if not 2 <= bits <= 16:
            raise ValueError("signed integer grids support 2 through 16 bits")
        low, high = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
        levels = torch.arange(low, high + 1, dtype=torch.float32, device="cpu")
        return Grid(lambda x: x.round().clamp(low, high), bits, values=levels, name=f"int{bits}", integer=True)

    def values(self, values: Any, *, bits: builtins.int | None = None, name: str = "values") -> Grid:
        levels = torch.as_tensor(values, dtype=torch.float32).detach().cpu().flatten().sort().values
        if not levels.numel() or not torch.isfinite(levels).all():
            raise ValueError("a scalar codebook must contain finite values")
        width = max(1, math.ceil(math.log2(levels.numel()))) if bits is None else bits
        if levels.numel() > 2**width:
            raise ValueError("codebook size exceeds the declared bit capacity")

        def snap(x: Tensor) -> Tensor:
            table = levels.to(device=x.device, dtype=x.dtype)
            return table[nearest_level(x, table)]

        return Grid(snap, width, values=levels, name=name)

    def fp(self, format: str) -> Grid:
        """Miniature floating-point grids (e2m1, e3m2, e2m3, e4m3, e5m2) as explicit level tables."""
        if format == "e2m1":
            half = [0.5, 1, 1.5, 2, 3, 4, 6]
            return self.values(torch.tensor([-v for v in reversed(half)] + [0, *half]), bits=4, name=format)
        if format not in {"e3m2", "e2m3", "e4m3", "e5m2"}:
            raise ValueError(f"unsupported floating-point grid {format!r}")
        exponent_bits, mantissa_bits = builtins.int(format[1]), builtins.int(format[3])
        bias = 2 ** (exponent_bits - 1) - 1
        levels = {0.0}
        for exponent in range(2**exponent_bits - 1):
            for mantissa in range(2**mantissa_bits):
                fraction = mantissa / 2**mantissa_bits
                magnitude = fraction * 2 ** (1 - bias) if exponent == 0 else (1 + fraction) * 2 ** (exponent - bias)
                levels.update((magnitude, -magnitude))
        return self.values(torch.tensor(sorted(levels)), bits=1 + exponent_bits + mantissa_bits, name=format)


grid = _GridFactory()

NF4_VALUES = torch.tensor([
    -1.0, -0.6961928, -0.52507305, -0.39491749, -0.28444138, -0.18477343, -0.09105004, 0.0,
    0.07958030, 0.16093020, 0.24611230, 0.33791524, 0.44070983, 0.56261700, 0.72295684, 1.0,
])
"""Normal-float levels: data of the NF4 format."""

SCALE_FORMAT_BITS = {"fp32": 32, "fp16": 16, "bf16": 16}


def store_scale(value: Tensor, format: str) -> tuple[Tensor, int]:
    """Round scales to their storage format and widen back to fp32."""
    if format == "fp32":
        return value.float(), 32
    if format == "fp16":
        return value.clamp(2**-24, 65504).half().float(), 16
    if format == "bf16":
        return value.bfloat16().float(), 16
    raise ValueError(f"unsupported scale storage format {format!r}")


# ------------------------------------------------------------------------------------- context


def layer_seed(name: str, seed: int = 0) -> int:
    """Per-layer seed: first eight bytes of sha256("seed:name"), little endian, mod 2**63 - 1."""
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return builtins.int.from_bytes(digest[:8], "little") % (2**63 - 1)


class Ctx:
    """Layer context handed to a format.  Round-to-nearest needs no statistics, so this carries
    only the identity of the layer and a seeded generator."""

    def __init__(self, name: str = "", module: Any = None, *, seed: int = 0,
                 device: str | torch.device | None = None) -> None:
        self.name, self.module = name, module
        self.cache: dict[str, Any] = {}
        self._device = torch.device("cpu" if device is None else device)
        self.rng = torch.Generator(device=self._device).manual_seed(layer_seed(name, seed))
        self._additional_bits = 0.0

    def add_bits(self, bits: float) -> None:
        if bits < 0:
            raise ValueError("additional bits must be nonnegative")
        self._additional_bits += bits

    @property
    def additional_bits(self) -> float:
        return self._additional_bits


# ------------------------------------------------------------------------------------- formats


def _fp32_reciprocal(value: float) -> float:
    one = torch.tensor(1.0, dtype=torch.float32, device="cpu")
    return float(one / torch.tensor(value, dtype=torch.float32, device="cpu"))


def _group_range(weight: Tensor, group: int) -> tuple[Tensor, Tensor]:
    rows, width = weight.shape
    full = width - width % group
    low, high = [], []
    if full:
        blocks = weight[:, :full].reshape(rows, -1, group)
        low.append(blocks.amin(-1))
        high.append(blocks.amax(-1))
    if full < width:
        low.append(weight[:, full:].amin(-1, keepdim=True))
        high.append(weight[:, full:].amax(-1, keepdim=True))
    return torch.cat(low, 1), torch.cat(high, 1)


class Scaled:
    """Round-to-nearest onto a scalar grid with one stored scale (and optional offset) per row group."""

    row_separable = True

    def __init__(self, grid: Grid, group: builtins.int | None = 128, scale: str = "absmax",
                 scale_fmt: str = "fp16", asym: bool = False, *, search_steps: builtins.int = 20) -> None:
        if group is not None and group <= 0:
            raise ValueError("group must be positive or None")
        if scale not in {"absmax", "mse"}:
            raise ValueError("scale must be absmax, mse, or callable")
        if search_steps < 1:
            raise ValueError("search_steps must be positive")
        if grid.dim != 1 or grid.values is None:
            raise NotImplementedError("mlkit_b200 encodes scalar grids with explicit values only")
        if scale_fmt not in SCALE_FORMAT_BITS:
            raise ValueError(f"unsupported scale storage format {scale_fmt!r}")
        self.grid, self.group, self.scale, self.scale_fmt = grid, group, scale, scale_fmt
        self.asym, self.search_steps = asym, search_steps
        levels = grid.values.detach().cpu()
        self._low, self._high = float(levels.min()), float(levels.max())
        if asym and self._high - self._low <= 0:
            raise ValueError("asymmetric quantization requires at least two distinct grid values")
        self._reciprocal = _fp32_reciprocal(self._high - self._low if asym else float(levels.abs().max()))

    def _snap_codes(self, normalized: Tensor, levels: Tensor) -> Tensor:
        if self.grid.integer:
            return normalized.round().clamp(self._low, self._high) - self._low
        return nearest_level(normalized, levels)

    def _snap_values(self, normalized: Tensor, levels: Tensor) -> Tensor:
        if self.grid.integer:
            return normalized.round().clamp(self._low, self._high)
        return levels[nearest_level(normalized, levels)]

    def __call__(self, w: Tensor, ctx: Ctx | None = None) -> Q:
        if w.ndim != 2 or not w.is_floating_point():
            raise ValueError("scaled requires a finite floating-point weight matrix")
        weight = w.float()
        rows, width = weight.shape
        group = width if self.group is None else min(self.group, width)
        levels = self.grid.values.to(weight.device).contiguous()
        bits = self.grid.bits
        if (weight.is_cuda and self.scale == "absmax" and not self.asym and self.scale_fmt == "fp16" and bits <= 8
                and group <= 1024 and (group * bits) % 8 == 0 and (width * bits) % 8 == 0 and rows > 0):
            # one launch on the device: the same arithmetic, operation for operation (mkb_rtn_encode)
            from mlkit_b200 import kernels

            if not torch.isfinite(weight).all():
                raise ValueError("scaled requires a finite floating-point weight matrix")
            stream, scales16, codes = kernels.rtn_encode(weight, levels, group=group, bits=bits, integer_grid=self.grid.integer,
                                                    low=self._low, high=self._high, reciprocal=self._reciprocal, codes=True)
            scales = scales16.float()
            encoded = Q(
                bits=bits * weight.numel() + scales.numel() * 16, codes=codes,
                params={"scales": scales, "values": levels, "group": group, "offset": 0, "zero": None},
                decode=decode_scaled, codec="scaled",
                metadata={"code_bits": bits, "scale_fmt": self.scale_fmt, "trainable": ["scales"]},
            )
            encoded._stream = (stream, codes, _version_of(codes), bits)
            return encoded
        low, high = _group_range(weight, group)
        if not (torch.isfinite(low).all() and torch.isfinite(high).all()):
            raise ValueError("scaled requires a finite floating-point weight matrix")
        if self.asym:
            scales = (high - low).clamp_min(1e-12) * self._reciprocal
            zero = low - self._low * scales
        else:
            scales, zero = torch.maximum(high, -low).clamp_min(1e-12) * self._reciprocal, None
        scales, scale_bits = store_scale(scales, self.scale_fmt)
        if self.scale == "mse":
            scales = self._search(weight, scales, zero, group, levels)
        if zero is not None:
            zero = store_scale(zero.abs().clamp_min(1e-12), self.scale_fmt)[0] * zero.sign()
        columns = torch.arange(width, device=weight.device) // group
        centered = weight if zero is None else weight - zero[:, columns]
        codes = self._snap_codes(centered / scales[:, columns], levels)
        side_bits = scales.numel() * scale_bits * (2 if zero is not None else 1)
        return Q(
            bits=self.grid.bits * weight.numel() + side_bits,
            codes=codes.to(torch.uint8 if self.grid.bits <= 8 else torch.int32),
            params={"scales": scales, "values": levels, "group": group, "offset": 0, "zero": zero},
            decode=decode_scaled, codec="scaled",
            metadata={"code_bits": self.grid.bits, "scale_fmt": self.scale_fmt,
                      "trainable": ["scales"] + (["zero"] if zero is not None else [])},
        )

    def _search(self, weight: Tensor, scales: Tensor, zero: Tensor | None, group: int, levels: Tensor) -> Tensor:
        """Per group, the stored scale among ``search_steps`` shrunken candidates with least squared error."""
        rows, width = weight.shape
        pad = (-width) % group
        blocks = torch.nn.functional.pad(weight, (0, pad)).reshape(rows, -1, group)
        occupied = None
        if pad:
            occupied = (torch.arange(blocks.shape[1] * group, device=weight.device) < width).reshape(1, -1, group)
        centered = blocks if zero is None else blocks - zero[..., None]

        def error_of(candidate: Tensor) -> Tensor:
            snapped = self._snap_values(centered / candidate[..., None], levels)
            error = (snapped * candidate[..., None] - centered).square()
            return (error if occupied is None else error * occupied).sum(-1)

        best_scale, best_error = scales.clone(), error_of(scales)
        for fraction in torch.linspace(0.5, 1.0, self.search_steps, device=weight.device).tolist():
            candidate, _ = store_scale(scales * fraction, self.scale_fmt)
            error = error_of(candidate)
            better = error < best_error
            best_scale = torch.where(better, candidate, best_scale)
            best_error = torch.minimum(best_error, error)
        return best_scale

    def __repr__(self) -> str:
        text = f"scaled({self.grid!r}, group={self.group}, scale={self.scale!r}"
        if self.scale_fmt != "fp16":
            text += f", scale_fmt={self.scale_fmt!r}"
        return text + (", asym=True)" if self.asym else ")")


def scaled(grid: Grid, group: builtins.int | None = 128, scale: str = "absmax", scale_fmt: str = "fp16",
           asym: bool = False, **options: Any) -> Scaled:
    return Scaled(grid, group, scale, scale_fmt, asym, **options)


def int(bits: builtins.int = 4, group: builtins.int | None = 128, **options: Any) -> Scaled:  # noqa: A001
    return scaled(grid.int(bits), group=group, **options)


def nf4(group: builtins.int | None = 64, **options: Any) -> Scaled:
    return scaled(grid.values(NF4_VALUES, bits=4, name="nf4"), group=group, **options)
