"""Tensor-level wrappers of the C ABI: they take CUDA tensors, pass raw pointers and the current stream.

Counterpart of the reference's launch wrappers in ``src/mlkit/kernels/packed_linear.py:181-313``,
``src/mlkit/kernels/hadamard.py:108-136`` and ``src/mlkit/kernels/launching.py:33-52``: work is queued
on the current CUDA stream of the tensor's device, nothing is synchronised and, apart from the
output tensor the caller passes in, nothing is allocated.
"""

import torch
from torch import Tensor

from mlkit_b200 import _native

DTYPE_TAGS = {torch.float16: _native.F16, torch.bfloat16: _native.BF16, torch.float32: _native.F32}
KERNEL_CHOICES = {"auto": _native.GEMV_AUTO, "scalar": _native.GEMV_SCALAR, "tiled": _native.GEMV_TILED,
                  "tmem": _native.GEMV_TMEM, "bulk": _native.GEMV_BULK, "stream": _native.GEMV_STREAM}

_workspaces: dict[tuple[int, int], Tensor] = {}


def matvec_workspace(device: torch.device, rows: int, outputs: int, width: int, bits: int) -> Tensor | None:
    """Zero-initialised scratch the tensor-memory matvec meets through (it splits K over CTAs), or
    ``None`` when the shape cannot use it.  One buffer per (device, stream) grows to the largest request;
    the kernel leaves it zeroed where it must be, so it is cleared only when (re)allocated.  Launches on
    one stream run in order and may share it."""
    need = _native.library().mkb_gemv_workspace_bytes(rows, outputs, width, bits)
    if need <= 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    held = _workspaces.get(key)
    if held is None or held.numel() < need:
        held = _workspaces[key] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
    return held


def workspace_status() -> int:
    """Non-zero when a bounded wait expired inside any matvec that used one of the pooled workspaces
    (its results are not valid); synchronises with the devices."""
    import ctypes

    worst = 0
    for held in _workspaces.values():
        value = ctypes.c_int(0)
        with torch.cuda.device(held.device):
            check = _native.library().mkb_gemv_workspace_status(held.data_ptr(), held.numel(), ctypes.byref(value))
        _native.check(check, "workspace_status")
        worst = max(worst, value.value)
    return worst


def _tag(dtype: torch.dtype, what: str) -> int:
    try:
        return DTYPE_TAGS[dtype]
    except KeyError:
        raise ValueError(f"{what} dtype {dtype} is not supported (fp16, bf16, fp32)") from None


def _pointer(tensor: Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(*tensors: Tensor | None) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise ValueError("mlkit_b200 kernels require CUDA tensors")
        if device is not None and tensor.device != device:
            raise ValueError("all tensors of one call must live on one device")
        device = tensor.device
    assert device is not None
    return device


def integer_grid_of(values: Tensor) -> tuple[bool, float]:
    """Whether ``values[c] == values[0] + c`` exactly with an integer ``values[0]``; and ``values[0]``."""
    table = values.detach().float().cpu()
    if table.numel() == 0:
        return False, 0.0
    low = float(table[0])
    exact = low == int(low) and abs(low) <= 512 and bool(
        torch.equal(table, low + torch.arange(table.numel(), dtype=torch.float32, device="cpu")))
    return exact, low


ROTATED_MAXIMUM_BYTES = 65536     # of fp32 activations the fused rotation holds in shared memory
ROTATED_PROFITABLE_BYTES = 16384  # up to here the fused launch measured faster than transform + matvec


def rotated_matvec_supported(rows: int, width: int, dtype: torch.dtype, *, profitable: bool = False) -> bool:
    """Whether ``packed_matvec_rotated`` may cover the input (the C entry point checks the layer as well).
    Every CTA of the matvec redoes the rotation, so its cost grows with the rows: measured on B200 at
    K = 4096 the fused launch wins at one row (6.4 against 7.0 us), ties at two and loses at four;
    ``profitable`` asks for the range where it wins."""
    limit = ROTATED_PROFITABLE_BYTES if profitable else ROTATED_MAXIMUM_BYTES
    return (dtype == torch.float16 and 1 <= rows <= 8 and width >= 512 and width & (width - 1) == 0
            and rows * width * 4 <= limit)


def packed_matvec_rotated(x: Tensor, signs: Tensor | None, packed: Tensor, scales: Tensor, values: Tensor,
                          bias: Tensor | None, out: Tensor, *, group: int, bits: int, integer_grid: bool,
                          grid_minimum: float, normalize: bool = True) -> Tensor:
    """``out = matvec(S(x * signs))`` in one launch (``mkb_gemv_hadamard``): equal to ``structured_transform``
    followed by ``packed_matvec`` bit for bit.  Raises ``ValueError`` where the fused launch does not apply."""
    device = _require_cuda(x, signs, packed, scales, values, bias, out)
    rows, width = x.shape
    if signs is not None and signs.dtype != torch.int8:
        raise ValueError("signs must be int8")
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    with torch.cuda.device(device):
        status = _native.library().mkb_gemv_hadamard(
            x.data_ptr(), _pointer(signs), packed.data_ptr(), scales.data_ptr(), values.data_ptr(), _pointer(bias),
            out.data_ptr(), rows, out.shape[1], width, group, bits, values.numel(), _tag(x.dtype, "activation"),
            _tag(scales.dtype, "scale"), width * bits // 8, scales.stride(0) if scales.dim() == 2 else -(-width // group),
            int(integer_grid), float(grid_minimum), int(normalize), torch.cuda.current_stream().cuda_stream)
    _native.check(status, "packed_matvec_rotated")
    return out


_gemm_workspaces: dict[tuple[int, int], Tensor] = {}
GEMM_MAXIMUM_ROWS = 128


def gemm_workspace(device: torch.device, rows: int, outputs: int, width: int) -> Tensor:
    """Zero-initialised scratch of the fused dequantise + GEMM kernel, one per (device, stream), grown to
    the largest request; the kernel leaves it zeroed where it must be."""
    need = _native.library().mkb_gemm_workspace_bytes(rows, outputs, width)
    if need <= 0:
        raise ValueError(f"no fused GEMM for {rows} rows, {outputs} outputs, width {width}")
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    held = _gemm_workspaces.get(key)
    if held is None or held.numel() < need:
        held = _gemm_workspaces[key] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
    return held


def gemm_status() -> int:
    """Non-zero when a bounded wait expired inside a fused GEMM that used a pooled workspace."""
    import ctypes

    worst = 0
    for held in _gemm_workspaces.values():
        value = ctypes.c_int(0)
        with torch.cuda.device(held.device):
            _native.check(_native.library().mkb_gemm_status(held.data_ptr(), ctypes.byref(value)), "gemm_status")
        worst = max(worst, value.value)
    return worst


def gemm_supported(rows: int, *, width: int, group: int, bits: int, dtype: torch.dtype, scales: Tensor,
                   zeros: Tensor | None, integer_grid: bool, grid_minimum: float, levels: int,
                   outputs: int | None = None) -> bool:
    """Whether ``packed_gemm`` covers the layer (the C entry point checks the same and more).  With
    ``outputs`` given, also whether it is the faster route: measured on B200 against reconstruct +
    library GEMM it wins at every shape up to 32 rows, and up to 128 rows once the weight has 2^25
    codes (4096 x 8192) or more; small weights with many rows are quicker through the dense route."""
    if not (1 <= rows <= GEMM_MAXIMUM_ROWS and bits == 4 and group == 128 and width % 128 == 0 and zeros is None
            and dtype == torch.float16 and scales.dtype == torch.float16 and bool(integer_grid)
            and float(grid_minimum) == -8.0 and levels == 16):
        return False
    return outputs is None or rows <= 32 or outputs * width >= 1 << 25


def packed_gemm(x: Tensor, packed: Tensor, scales: Tensor, values: Tensor, bias: Tensor | None, out: Tensor, *,
                group: int, bits: int, integer_grid: bool, grid_minimum: float) -> Tensor:
    """``out[M, N] = x[M, K] @ dequant(packed)^T (+ bias)`` for up to 128 rows in one launch (``mkb_gemm``)."""
    device = _require_cuda(x, packed, scales, values, bias, out)
    rows, width = x.shape
    outputs = out.shape[1]
    if not x.is_contiguous() or not out.is_contiguous():
        raise ValueError("packed_gemm needs contiguous activations and outputs")
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    with torch.cuda.device(device):
        workspace = gemm_workspace(device, rows, outputs, width)
        status = _native.library().mkb_gemm(
            x.data_ptr(), packed.data_ptr(), scales.data_ptr(), values.data_ptr(), None, _pointer(bias), out.data_ptr(),
            rows, outputs, width, group, bits, values.numel(), _tag(x.dtype, "activation"), _tag(scales.dtype, "scale"),
            width * bits // 8, scales.stride(0) if scales.dim() == 2 else -(-width // group), int(integer_grid),
            float(grid_minimum), workspace.data_ptr(), workspace.numel(), torch.cuda.current_stream().cuda_stream)
    _native.check(status, "packed_gemm")
    return out


def packed_matvec(x: Tensor, packed: Tensor, scales: Tensor, values: Tensor, zeros: Tensor | None,
                  bias: Tensor | None, out: Tensor, *, group: int, bits: int, integer_grid: bool = False,
                  grid_minimum: float = 0.0, kernel: str = "auto", packed_row_stride: int | None = None,
                  scale_row_stride: int | None = None, workspace: Tensor | None = None,
                  gated: bool = False) -> Tensor:
    """``out[m, n] = sum_k x[m, k] * (values[code[n, k]] * scales[n, k // group] (+ zeros)) (+ bias[n])``.

    ``x`` is ``[M, K]`` contiguous with ``M <= 8``; ``out`` is ``[M, N]`` in the dtype of ``x``.
    """
    device = _require_cuda(x, packed, scales, values, zeros, bias, out)
    rows, width = x.shape
    if gated:   # x is [rows, 2 * width] = gate | up; the kernel forms silu(gate) * up on load
        if width % 2:
            raise ValueError("a gated input has an even number of columns")
        width //= 2
    outputs = out.shape[-1]
    if not (x.is_contiguous() and out.is_contiguous()):
        raise ValueError("packed_matvec needs contiguous activations and output")
    if out.dtype != x.dtype or out.shape[0] != rows:
        raise ValueError("output must match the activations in dtype and rows")
    if zeros is not None and zeros.dtype != scales.dtype:
        raise ValueError("offsets must share the dtype of the scales")
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    if packed_row_stride is None:
        packed_row_stride = width * bits // 8
    if scale_row_stride is None:
        scale_row_stride = scales.stride(0) if scales.dim() == 2 else -(-width // group)
    with torch.cuda.device(device):
        if workspace is None and kernel in ("auto", "tmem", "bulk") and x.dtype == torch.float16 and integer_grid:
            workspace = matvec_workspace(device, rows, outputs, width, bits)
        status = _native.library().mkb_gemv_ws(
            x.data_ptr(), packed.data_ptr(), scales.data_ptr(), values.data_ptr(), _pointer(zeros),
            _pointer(bias), out.data_ptr(), rows, outputs, width, group, bits, values.numel(),
            _tag(x.dtype, "activation"), _tag(scales.dtype, "scale"), packed_row_stride,
            scale_row_stride, int(integer_grid), float(grid_minimum),
            KERNEL_CHOICES[kernel] | (_native.GEMV_GATED if gated else 0), _pointer(workspace), 0 if workspace is None else workspace.numel(), _stream(device))
    _native.check(status, "packed_matvec")
    return out


class MatvecPlan:
    """The constant arguments of one layer's matvec, bound once.

    The per-call work is what the reference's direct launcher leaves
    (``src/mlkit/inference/packed_linear.py:181-245``): pass the activation and output pointers,
    the row count and the current stream.  The plan holds raw device pointers, so it must be rebuilt
    whenever the layer's buffers move (``PackedLinear._apply`` drops it).
    """

    __slots__ = ("function", "head", "tail", "outputs", "width", "bits", "dtype", "device", "device_index", "keep",
                 "integer_grid", "workspaces")

    def __init__(self, packed: Tensor, scales: Tensor, values: Tensor, zeros: Tensor | None, bias: Tensor | None,
                 *, outputs: int, width: int, group: int, bits: int, dtype: torch.dtype, integer_grid: bool,
                 grid_minimum: float, gated: bool = False) -> None:
        device = _require_cuda(packed, scales, values, zeros, bias)
        if zeros is not None and zeros.dtype != scales.dtype:
            raise ValueError("offsets must share the dtype of the scales")
        if bias is not None and bias.dtype != dtype:
            bias = bias.to(dtype)
        self.function = _native.library().mkb_gemv_ws
        self.head = (packed.data_ptr(), scales.data_ptr(), values.data_ptr(), _pointer(zeros), _pointer(bias))
        self.tail = (outputs, width, group, bits, values.numel(), _tag(dtype, "activation"),
                     _tag(scales.dtype, "scale"), width * bits // 8,
                     scales.stride(0) if scales.dim() == 2 else -(-width // group), int(integer_grid),
                     float(grid_minimum), _native.GEMV_AUTO | (_native.GEMV_GATED if gated else 0))
        self.outputs, self.width, self.bits, self.dtype, self.device = outputs, width, bits, dtype, device
        self.integer_grid = bool(integer_grid) and dtype == torch.float16 and zeros is None
        self.workspaces: dict[tuple[int, int], tuple[int | None, int, Tensor | None]] = {}
        self.device_index = device.index
        self.keep = (packed, scales, values, zeros, bias)  # the pointers above stay valid while these live

    def __call__(self, x: Tensor, out: Tensor) -> Tensor:
        """``x`` [M, width] and ``out`` [M, outputs]: contiguous, on the plan's device, dtype of the plan."""
        if torch.cuda.current_device() != self.device_index:
            with torch.cuda.device(self.device):
                return self(x, out)
        stream = torch.cuda.current_stream().cuda_stream
        rows = x.shape[0]
        held = self.workspaces.get((rows, stream))
        if held is None:  # (pointer, bytes, tensor kept alive) of the scratch for this row count and stream
            tensor = matvec_workspace(self.device, rows, self.outputs, self.width, self.bits) if self.integer_grid else None
            held = self.workspaces[(rows, stream)] = (_pointer(tensor), 0 if tensor is None else tensor.numel(), tensor)
        status = self.function(x.data_ptr(), *self.head, out.data_ptr(), rows, *self.tail, held[0], held[1], stream)
        if status:
            _native.check(status, "packed_matvec")
        return out


def dequantize(packed: Tensor, scales: Tensor | None, values: Tensor | None, zeros: Tensor | None, *,
               shape: tuple[int, int], group: int, bits: int, dtype: torch.dtype | None = torch.float16,
               codes: bool = False) -> tuple[Tensor | None, Tensor | None]:
    """Bit-exact reconstruction of a packed weight; returns ``(weight or None, codes or None)``."""
    device = _require_cuda(packed, scales, values, zeros)
    rows, width = shape
    weight = None if dtype is None else torch.empty(shape, device=device, dtype=dtype)
    unpacked = torch.empty(shape, device=device, dtype=torch.uint8) if codes else None
    if weight is None and unpacked is None:
        raise ValueError("dequantize needs at least one output")
    if weight is not None and (scales is None or values is None):
        raise ValueError("a dense weight needs scales and values")
    if rows * width == 0:
        return weight, unpacked
    if scales is not None and not scales.is_contiguous():
        raise ValueError("scales must be contiguous")
    stride = 0 if scales is None else (scales.stride(0) if scales.dim() == 2 else -(-width // group))
    with torch.cuda.device(device):
        status = _native.library().mkb_dequant(
            packed.data_ptr(), _pointer(scales), _pointer(values), _pointer(zeros), _pointer(weight),
            _pointer(unpacked), rows, width, group, bits, 0 if values is None else values.numel(),
            _native.F32 if scales is None else _tag(scales.dtype, "scale"),
            _native.F16 if dtype is None else _tag(dtype, "output"), stride, _stream(device))
    _native.check(status, "dequantize")
    return weight, unpacked


def rtn_encode(weight: Tensor, levels: Tensor, *, group: int, bits: int, integer_grid: bool, low: float, high: float,
               reciprocal: float, codes: bool = False) -> tuple[Tensor, Tensor, Tensor | None]:
    """Round-to-nearest encode and pack on the device: returns ``(packed uint8, scales fp16 [N, groups],
    codes uint8 [N, K] or None)``.  Raises ``ValueError`` for layouts whose groups or rows do not end
    on a byte (the caller then takes the tensor route)."""
    device = _require_cuda(weight, levels)
    rows, width = weight.shape
    source = weight if weight.is_contiguous() else weight.contiguous()
    group = min(group, width)
    packed = torch.empty(rows * width * bits // 8, dtype=torch.uint8, device=device)
    scales = torch.empty((rows, -(-width // group)), dtype=torch.float16, device=device)
    unpacked = torch.empty((rows, width), dtype=torch.uint8, device=device) if codes else None
    with torch.cuda.device(device):
        status = _native.library().mkb_rtn_encode(
            source.data_ptr(), levels.data_ptr(), packed.data_ptr(), scales.data_ptr(), _pointer(unpacked), rows, width,
            group, bits, levels.numel(), int(integer_grid), float(low), float(high), float(reciprocal),
            _tag(source.dtype, "weight"), _stream(device))
    _native.check(status, "rtn_encode")
    return packed, scales, unpacked


def dequantize_rows(packed: Tensor, scales: Tensor, values: Tensor, zeros: Tensor | None, rows: Tensor, *,
                    shape: tuple[int, int], group: int, bits: int, dtype: torch.dtype) -> Tensor:
    """Reconstruct the listed rows only: ``out[i] = weight[rows[i]]``."""
    device = _require_cuda(packed, scales, values, zeros, rows)
    total, width = shape
    rows = rows.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((rows.numel(), width), device=device, dtype=dtype)
    if rows.numel() == 0:
        return out
    with torch.cuda.device(device):
        status = _native.library().mkb_dequant_rows(
            packed.data_ptr(), scales.data_ptr(), values.data_ptr(), _pointer(zeros), rows.data_ptr(),
            out.data_ptr(), rows.numel(), total, width, group, bits, values.numel(),
            _tag(scales.dtype, "scale"), _tag(dtype, "output"), scales.stride(0), _stream(device))
    _native.check(status, "dequantize_rows")
    return out


def structured_transform(x: Tensor, *, factor: int, power: int, basis: Tensor | None = None,
                         signs: Tensor | None = None, inverse: bool = False, normalize: bool = True,
                         out: Tensor | None = None) -> Tensor:
    """``(basis kron H_power)(x * signs)`` over the last axis, one fused launch; dtype preserved."""
    device = _require_cuda(x, basis, signs, out)
    width = x.shape[-1]
    if factor * power != width:
        raise ValueError("factor * power must equal the transform width")
    source = x if x.is_contiguous() else x.contiguous()
    if out is None:
        out = torch.empty_like(source)
    if signs is not None and (signs.dtype != torch.int8 or signs.numel() != width):
        raise ValueError("signs must be an int8 vector of the transform width")
    if basis is not None and (basis.dtype != torch.float32 or not basis.is_contiguous()):
        raise ValueError("basis must be a contiguous fp32 matrix")
    rows = source.numel() // width if width else 0
    with torch.cuda.device(device):
        status = _native.library().mkb_hadamard(
            source.data_ptr(), _pointer(signs), _pointer(basis), out.data_ptr(), rows, width, factor,
            power, _tag(x.dtype, "activation"), int(inverse), int(normalize), _stream(device))
    _native.check(status, "structured_transform")
    return out


# ---- operators between the matvecs of a decode step (fp16, contiguous, caller-provided outputs) ----

def add_rmsnorm(residual: Tensor, delta: Tensor | None, weight: Tensor, normed: Tensor, eps: float) -> None:
    """``residual += delta`` (in place, when given) and ``normed = rms_norm(residual) * weight``."""
    rows, hidden = residual.shape
    status = _native.library().mkb_add_rmsnorm(residual.data_ptr(), _pointer(delta), weight.data_ptr(),
                                               normed.data_ptr(), rows, hidden, eps, _stream(residual.device))
    _native.check(status, "add_rmsnorm")


def rope_append(qkv: Tensor, positions: Tensor, k_cache: Tensor, v_cache: Tensor, *, q_heads: int, kv_heads: int,
                head_dim: int, theta: float) -> None:
    """Rotary embedding of the q and k heads of ``qkv`` in place, then k and v into the caches."""
    status = _native.library().mkb_rope_append(qkv.data_ptr(), positions.data_ptr(), k_cache.data_ptr(),
                                               v_cache.data_ptr(), qkv.shape[0], q_heads, kv_heads, head_dim,
                                               k_cache.shape[2], theta, _stream(qkv.device))
    _native.check(status, "rope_append")


def attention_decode(qkv: Tensor, positions: Tensor, k_cache: Tensor, v_cache: Tensor, out: Tensor, *,
                     q_heads: int, kv_heads: int, head_dim: int) -> None:
    """Single-token grouped-query attention over the cached positions ``0..positions[m]``."""
    status = _native.library().mkb_attention_decode(qkv.data_ptr(), positions.data_ptr(), k_cache.data_ptr(),
                                                    v_cache.data_ptr(), out.data_ptr(), qkv.shape[0], q_heads,
                                                    kv_heads, head_dim, k_cache.shape[2], head_dim ** -0.5,
                                                    _stream(qkv.device))
    _native.check(status, "attention_decode")


def rope_attention_decode(qkv: Tensor, positions: Tensor, k_cache: Tensor, v_cache: Tensor, out: Tensor, *,
                          q_heads: int, kv_heads: int, head_dim: int, theta: float, scale: float | None = None) -> None:
    """``rope_append`` and ``attention_decode`` in one launch (at most 8 query heads per key-value head);
    ``qkv`` is left unrotated."""
    if scale is None:
        scale = head_dim ** -0.5
    status = _native.library().mkb_rope_attention_decode(
        qkv.data_ptr(), positions.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), qkv.shape[0],
        q_heads, kv_heads, head_dim, k_cache.shape[2], theta, scale, _stream(qkv.device))
    _native.check(status, "rope_attention_decode")


def silu_mul(gate_up: Tensor, out: Tensor) -> None:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    status = _native.library().mkb_silu_mul(gate_up.data_ptr(), out.data_ptr(), gate_up.shape[0], out.shape[1],
                                            _stream(gate_up.device))
    _native.check(status, "silu_mul")


def argmax_keys(logits: Tensor, best: Tensor, offset: int = 0) -> Tensor:
    """``best[m]`` (int64 storage of an unsigned word) = sortable key of the row maximum of ``logits``
    ([M, width] fp16) in the high half, ``0xffffffff - (argmax + offset)`` in the low half."""
    status = _native.library().mkb_argmax(logits.data_ptr(), best.data_ptr(), logits.shape[0], logits.shape[1],
                                          logits.stride(0), offset, _stream(logits.device))
    _native.check(status, "argmax")
    return best


def tokens_of_keys(keys: Tensor) -> Tensor:
    """The token ids inside ``argmax_keys`` words."""
    return 0xFFFFFFFF - (keys & 0xFFFFFFFF)


def decode_status() -> int:
    """Non-zero when a decode operator since the last call saw a cache position outside ``[0, capacity)``
    (it clamped the position and skipped the append; that step's results are not valid).  Synchronises."""
    import ctypes

    value = ctypes.c_int(0)
    _native.check(_native.library().mkb_decode_status(ctypes.byref(value)), "decode_status")
    return value.value
