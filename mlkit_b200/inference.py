"""Packed execution of quantised linear layers: ``PackedLinear``, ``PackedEmbedding``, ``optimize``.

Drop-in counterparts of ``src/mlkit/inference/packed_linear.py`` (``PackedLinear`` ``:41-245``,
``PackedEmbedding`` ``:248-287``, ``packed_compatible`` ``:290-304``), ``layout_for`` /
``PackedLayout`` (``src/mlkit/kernels/packed_linear.py:43-79``), ``optimize``
(``src/mlkit/inference/optimization.py:11-100``) and ``benchmark``
(``src/mlkit/inference/benchmarking.py:17-71``).  Buffer names, attributes, dispatch rule (at most
eight input rows take the fused matvec, more rows reconstruct the dense weight and use a matrix
product) and error behaviour follow the reference; every device computation goes through
``libmlkit_b200`` and there is no Triton and no CPU path.
"""

import copy
import math
import statistics
import time
from collections.abc import Callable
from dataclasses import asdict, dataclass
from typing import Any

import torch
import torch.nn.functional as functional
from torch import Tensor, nn

from mlkit_b200 import kernels
from mlkit_b200.models import Model, QModel
from mlkit_b200.quantization import Q, pack

SCALE_STORAGE_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
MAXIMUM_FUSED_ROWS = 8
MAXIMUM_CODE_BITS = 8
MAXIMUM_TILE_CODES = 128
MINIMUM_TILE_CODES = 16


@dataclass(frozen=True)
class PackedLayout:
    """Word structure of a packed stream: the fewest whole bytes that hold whole codes."""

    bits: int
    bytes_per_word: int
    codes_per_word: int
    tile_words: int

    @property
    def tile_codes(self) -> int:
        return self.tile_words * self.codes_per_word

    def row_bytes(self, input_width: int) -> int:
        return input_width // self.codes_per_word * self.bytes_per_word

    def tiles_per_row(self, input_width: int) -> int:
        return -(-input_width // self.tile_codes)


def layout_for(bits: int, input_width: int, group: int) -> PackedLayout | None:
    """The layout a layer can run the fused matvec with, or ``None`` when a row or a scale group
    would split a packing word (such layers keep packed storage but always reconstruct)."""
    if not 1 <= bits <= MAXIMUM_CODE_BITS:
        return None
    shared = math.gcd(bits, 8)
    bytes_per_word, codes_per_word = bits // shared, 8 // shared
    if input_width % codes_per_word or group % codes_per_word:
        return None
    words = group // codes_per_word
    tile_words = min(MAXIMUM_TILE_CODES // codes_per_word, words & -words)
    if tile_words * codes_per_word < MINIMUM_TILE_CODES:
        return None
    return PackedLayout(bits, bytes_per_word, codes_per_word, tile_words)


def packed_compatible(quantized: Q) -> bool:
    """A complete scalar codec of at most eight bits, original column order, group-aligned refits."""
    if quantized.codec not in {"scaled", "feedback"}:
        return False
    group = quantized.params["group"]
    bits = quantized.metadata.get("code_bits")
    return (isinstance(bits, int) and 1 <= bits <= MAXIMUM_CODE_BITS and quantized.codes is not None
            and quantized.params["values"].numel() <= 2**bits and quantized.params.get("offset", 0) == 0
            and quantized.params.get("permutation") is None and quantized.params.get("refit", group) % group == 0)


def preserve_input_processing(original: nn.Module, replacement: nn.Module) -> None:
    """Carry online input transforms (pre-hooks and their ``_mlkit_*`` buffers) to the substitute."""
    replacement._forward_pre_hooks = original._forward_pre_hooks.copy()
    replacement._forward_pre_hooks_with_kwargs = original._forward_pre_hooks_with_kwargs.copy()
    for name, value in original.named_buffers(recurse=False):
        if name.startswith("_mlkit_"):
            replacement.register_buffer(name, value.detach().clone())


@torch.library.custom_op("mlkit_b200::packed_matvec", mutates_args=())
def _packed_matvec_op(x: Tensor, packed: Tensor, scales: Tensor, values: Tensor, zeros: Tensor | None,
                      bias: Tensor | None, outputs: int, group: int, bits: int, integer_grid: bool,
                      grid_minimum: float) -> Tensor:
    out = x.new_empty((x.shape[0], outputs))
    kernels.packed_matvec(x, packed, scales, values, zeros, bias, out, group=group, bits=bits,
                          integer_grid=integer_grid, grid_minimum=grid_minimum)
    return out


@_packed_matvec_op.register_fake
def _(x, packed, scales, values, zeros, bias, outputs, group, bits, integer_grid, grid_minimum):
    return x.new_empty((x.shape[0], outputs))


class PackedLinear(nn.Module):
    """Scalar-grid codes of one to eight bits executed from their packed stream.

    Up to ``maximum_fused_rows`` input rows go through the packed matvec kernel.  More rows
    reconstruct the dense weight (bit-exact dequantisation kernel) and use a matrix product.
    """

    packed: Tensor
    scales: Tensor
    values: Tensor
    zeros: Tensor | None
    bias: Tensor | None
    _dense_weight: Tensor | None

    def __init__(self, original: nn.Linear, quantized: Q, *, cache_dense: bool = False) -> None:
        super().__init__()
        if not packed_compatible(quantized):
            raise ValueError(
                "PackedLinear requires a complete scalar-grid codec of at most eight bits in "
                "its original column order with refit boundaries aligned to scale groups")
        device = original.weight.device
        if device.type != "cuda":
            raise ValueError("PackedLinear requires CUDA weights")
        self.in_features, self.out_features = original.in_features, original.out_features
        self.group = int(quantized.params["group"])
        self.code_bits = int(quantized.metadata["code_bits"])
        self.storage_dtype = original.weight.dtype
        self.cache_dense = cache_dense
        scales = quantized.params["scales"]
        scale_dtype = SCALE_STORAGE_DTYPES.get(str(quantized.metadata.get("scale_fmt")), scales.dtype)
        zero = quantized.params.get("zero")
        self.register_buffer("packed", quantized.packed_stream(self.code_bits).to(device))
        self.register_buffer("scales", scales.to(device=device, dtype=scale_dtype).contiguous())
        self.register_buffer("values", quantized.params["values"].to(device=device, dtype=torch.float32).contiguous())
        self.register_buffer("zeros", None if zero is None else zero.to(device=device, dtype=scale_dtype).contiguous())
        self.register_buffer("bias", None if original.bias is None else original.bias.detach().clone())
        self.register_buffer("_dense_weight", None, persistent=False)
        levels = quantized.params["values"].detach().cpu().float()
        steps = levels.diff()
        self.uniform_grid = bool(len(steps) and torch.allclose(steps, steps[0].expand_as(steps)))
        self.grid_minimum = float(levels[0])
        self.grid_step = float(steps[0]) if len(steps) else 1.0
        # the arithmetic decode is only taken when the table is an integer ramp, bit for bit
        self.integer_grid, _ = kernels.integer_grid_of(levels)
        self.layout = layout_for(self.code_bits, self.in_features, self.group)
        self.maximum_fused_rows = 0 if self.layout is None else MAXIMUM_FUSED_ROWS
        self._rotation_refused = False
        self._plans: dict[torch.dtype, kernels.MatvecPlan] = {}
        self._siblings: SiblingLaunch | None = None
        preserve_input_processing(original, self)

    def _apply(self, fn: Callable[[Tensor], Tensor], recurse: bool = True) -> "PackedLinear":
        self._dense_weight = None
        self._plans = {}  # bound device pointers are stale once buffers move or change dtype
        if self._siblings is not None:
            self._siblings.dissolve()  # the members' buffers stop being views of one allocation
        return super()._apply(fn, recurse)

    def __deepcopy__(self, memo: dict) -> "PackedLinear":
        """Copy everything but the bound launch plans, which point into this instance's buffers."""
        duplicate = self.__class__.__new__(self.__class__)
        memo[id(self)] = duplicate
        for key, value in self.__dict__.items():
            if key == "_plans":
                duplicate.__dict__[key] = {}
            elif key == "_siblings":
                duplicate.__dict__[key] = None  # a copy launches on its own until it is grouped again
            else:
                duplicate.__dict__[key] = copy.deepcopy(value, memo)
        return duplicate

    def _plan(self, dtype: torch.dtype) -> "kernels.MatvecPlan":
        plan = self._plans.get(dtype)
        if plan is None:
            plan = self._plans[dtype] = kernels.MatvecPlan(
                self.packed, self.scales, self.values, self.zeros, self.bias, outputs=self.out_features,
                width=self.in_features, group=self.group, bits=self.code_bits, dtype=dtype,
                integer_grid=self.integer_grid, grid_minimum=self.grid_minimum)
        return plan

    @property
    def weight(self) -> Tensor:
        """The dense reconstruction in the storage dtype: fp32 multiply (and add), one rounding."""
        if self._dense_weight is not None:
            return self._dense_weight
        dense, _ = kernels.dequantize(self.packed, self.scales, self.values, self.zeros,
                                      shape=(self.out_features, self.in_features), group=self.group,
                                      bits=self.code_bits, dtype=self.storage_dtype)
        if self.cache_dense:
            self._dense_weight = dense
        return dense

    def take_rotation(self, inputs: Tensor, signs: Tensor) -> bool:
        """Called by the rotation pre-hook: ``True`` when the coming ``forward`` will rotate ``inputs`` itself,
        inside the matvec launch (``mkb_gemv_hadamard``); the hook then leaves the input as it is."""
        rows = inputs.numel() // max(self.in_features, 1)
        if (self.layout is None or self._siblings is not None or self.zeros is not None or torch.compiler.is_compiling()
                or inputs.shape[-1] != self.in_features or not inputs.is_cuda or rows > self.maximum_fused_rows
                or not kernels.rotated_matvec_supported(rows, self.in_features, inputs.dtype, profitable=True)
                or self.scales.dtype != torch.float16
                or self._rotation_refused):
            return False
        self._pending_rotation = signs
        return True

    def forward(self, inputs: Tensor) -> Tensor:
        # (under torch.compile nothing is ever pending: take_rotation refuses while a graph is being traced)
        signs = None if torch.compiler.is_compiling() else self.__dict__.pop("_pending_rotation", None)
        if signs is not None:
            rows = inputs.numel() // self.in_features
            flat = inputs.reshape(rows, self.in_features).contiguous()
            out = inputs.new_empty((rows, self.out_features))
            try:
                kernels.packed_matvec_rotated(flat, signs, self.packed, self.scales, self.values, self.bias, out,
                                              group=self.group, bits=self.code_bits, integer_grid=self.integer_grid,
                                              grid_minimum=self.grid_minimum)
                return out.view(inputs.shape[:-1] + (self.out_features,))
            except ValueError:
                # the layer's codec is outside the fused launch: rotate with the transform's own launch from now on
                self._rotation_refused = True
                from mlkit_b200 import transforms

                inputs = transforms.structured_transform(inputs, signs=signs)
        width = self.in_features
        if inputs.shape[-1] != width:
            raise ValueError("input width does not match the packed linear")
        if not inputs.is_cuda:
            raise ValueError("packed inference requires CUDA inputs")
        rows = inputs.numel() // width
        if rows > self.maximum_fused_rows or rows == 0:
            fused_gemm = (rows > 0 and self.layout is not None and inputs.is_cuda
                          and kernels.gemm_supported(rows, width=width, group=self.group, bits=self.code_bits,
                                                     dtype=inputs.dtype, scales=self.scales, zeros=self.zeros,
                                                     integer_grid=self.integer_grid, grid_minimum=self.grid_minimum,
                                                     levels=self.values.numel(), outputs=self.out_features))
            chunked_rows = 2 * self.maximum_fused_rows if fused_gemm else 4 * self.maximum_fused_rows
            if (0 < rows <= chunked_rows and self.layout is not None and not torch.compiler.is_compiling()
                    and self._dense_weight is None and not (inputs.requires_grad and torch.is_grad_enabled())
                    and inputs.dtype == torch.float16 and inputs.is_cuda):
                # a few rows more than one matvec takes: the matvec on chunks of eight rows streams the packed
                # weight once per chunk, which measured faster than the fused GEMM up to 16 rows (16.9 against
                # 19.4 us on 4096 -> 14336) and than reconstruct + library GEMM up to 32 rows for every codec
                flat = inputs.reshape(rows, width).contiguous()
                out = inputs.new_empty((rows, self.out_features))
                plan = self._plan(inputs.dtype)
                for start in range(0, rows, self.maximum_fused_rows):
                    plan(flat[start:start + self.maximum_fused_rows], out[start:start + self.maximum_fused_rows])
                return out.view(inputs.shape[:-1] + (self.out_features,))
            if (fused_gemm and not torch.compiler.is_compiling() and self._dense_weight is None
                    and not (inputs.requires_grad and torch.is_grad_enabled())):
                # up to 128 rows: the weight is reconstructed inside the GEMM kernel, tile by tile
                flat = inputs.reshape(rows, width).contiguous()
                out = kernels.packed_gemm(flat, self.packed, self.scales, self.values, self.bias,
                                          inputs.new_empty((rows, self.out_features)), group=self.group,
                                          bits=self.code_bits, integer_grid=True, grid_minimum=self.grid_minimum)
                return out.view(inputs.shape[:-1] + (self.out_features,))
            return functional.linear(inputs, self.weight.to(inputs.dtype), self.bias)
        if inputs.requires_grad and torch.is_grad_enabled():
            raise RuntimeError("packed CUDA inference does not support autograd")
        flat = inputs.reshape(rows, width)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        if torch.compiler.is_compiling():
            bias = self.bias
            if bias is not None and bias.dtype != inputs.dtype:
                bias = bias.to(inputs.dtype)
            out = _packed_matvec_op(flat, self.packed, self.scales, self.values, self.zeros, bias,
                                    self.out_features, self.group, self.code_bits, self.integer_grid,
                                    self.grid_minimum)
        else:
            if inputs.dtype not in kernels.DTYPE_TAGS:
                raise ValueError(f"activation dtype {inputs.dtype} is not supported (fp16, bf16, fp32)")
            siblings = self._siblings
            if siblings is not None and flat.data_ptr() == inputs.data_ptr():
                out = siblings.output_of(self, flat)
            else:
                out = self._plan(inputs.dtype)(flat, inputs.new_empty((rows, self.out_features)))
        return out.view(inputs.shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.code_bits}, "
                f"group={self.group}, fused={'yes' if self.layout is not None else 'no'}")


class SiblingLaunch:
    """One packed matvec for linears that read the same input (q | k | v, gate | up).

    The reference launches one kernel per ``PackedLinear``
    (``src/mlkit/inference/packed_linear.py:145-179``); a decode step of a Llama block is then seven
    launches of which four stream less than a launch costs.  Here the members' ``packed``, ``scales``
    (and ``zeros``, ``bias``) buffers become views of one allocation each, concatenated along the
    output rows, so checkpoints and state dicts are unchanged while one launch computes every member.
    The first member that is called with an input runs the launch; the others return their columns of
    that result when they are called with the same tensor (same storage, same version) and have not
    taken it yet.  The launch keeps a reference to its input, so a new tensor cannot reuse the address.
    Rows of the weight are independent, so every output equals the member's own launch bit for bit.
    """

    def __init__(self, members: list["PackedLinear"]) -> None:
        first = members[0]
        self.members = list(members)
        self.offsets = [0]
        for member in members:
            self.offsets.append(self.offsets[-1] + member.out_features)
        self.total = self.offsets[-1]
        self.packed = torch.cat([member.packed for member in members])
        self.scales = torch.cat([member.scales for member in members])
        self.zeros = None if first.zeros is None else torch.cat([member.zeros for member in members])
        self.bias = None if first.bias is None else torch.cat([member.bias for member in members])
        row_bytes = first.in_features * first.code_bits // 8
        for index, member in enumerate(members):
            low, high = self.offsets[index], self.offsets[index + 1]
            member.packed = self.packed[low * row_bytes:high * row_bytes]
            member.scales = self.scales[low:high]
            if self.zeros is not None:
                member.zeros = self.zeros[low:high]
            if self.bias is not None:
                member.bias = self.bias[low:high]
            member._plans = {}
            member._siblings = self
        self._plans: dict[torch.dtype, kernels.MatvecPlan] = {}
        self._input: Tensor | None = None
        self._version = -1
        self._output: Tensor | None = None
        self._taken: set[int] = set()

    @staticmethod
    def compatible(members: list["PackedLinear"]) -> bool:
        first = members[0]
        if len(members) < 2 or any(member._siblings is not None for member in members):
            return False
        for member in members:
            if (member.layout is None or member.in_features != first.in_features or member.group != first.group
                    or member.code_bits != first.code_bits or member.scales.dtype != first.scales.dtype
                    or member.packed.device != first.packed.device or (member.zeros is None) != (first.zeros is None)
                    or (member.bias is None) != (first.bias is None) or member.scales.dim() != 2
                    or member.scales.shape[1] != first.scales.shape[1] or member._forward_pre_hooks
                    or (member.bias is not None and member.bias.dtype != first.bias.dtype)
                    or not torch.equal(member.values, first.values)):
                return False
        return True

    def dissolve(self) -> None:
        for member in self.members:
            member._siblings = None
        self._input = self._output = None

    def plan(self, dtype: torch.dtype) -> "kernels.MatvecPlan":
        """The bound launch of the whole group: ``plan(x, out)`` with ``out`` of ``[rows, total]``."""
        plan = self._plans.get(dtype)
        if plan is None:
            first = self.members[0]
            plan = self._plans[dtype] = kernels.MatvecPlan(
                self.packed, self.scales, first.values, self.zeros, self.bias, outputs=self.total,
                width=first.in_features, group=first.group, bits=first.code_bits, dtype=dtype,
                integer_grid=first.integer_grid, grid_minimum=first.grid_minimum)
        return plan

    def output_of(self, member: "PackedLinear", flat: Tensor) -> Tensor:
        index = self.members.index(member)
        current = self._input
        version = 0 if flat.is_inference() else flat._version  # inference tensors carry no version counter
        if (current is None or index in self._taken or current.data_ptr() != flat.data_ptr()
                or current.shape != flat.shape or current.dtype != flat.dtype or self._version != version):
            self._output = self.plan(flat.dtype)(flat, flat.new_empty((flat.shape[0], self.total)))
            self._input, self._version = flat, version
            self._taken = set()
        self._taken.add(index)
        if len(self._taken) == len(self.members):
            self._input = None  # everybody has its columns: let the activation go
        return self._output[:, self.offsets[index]:self.offsets[index + 1]]


SIBLING_NAMES = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def fuse_siblings(module: nn.Module, names: tuple[tuple[str, ...], ...] = SIBLING_NAMES) -> int:
    """Group ``PackedLinear`` children that read the same input into one launch each.  ``names`` lists
    the attribute names of such siblings under a common parent (the Llama naming by default); groups
    whose members differ in codec, width or input hooks are left alone.  Returns the number of groups."""
    groups = 0
    for parent in module.modules():
        for group in names:
            members = [getattr(parent, name, None) for name in group]
            if all(isinstance(member, PackedLinear) for member in members) and SiblingLaunch.compatible(members):
                SiblingLaunch(members)
                groups += 1
    return groups


class PackedEmbedding(nn.Module):
    """Token embedding read from the packed codes of a tied output projection; only the requested
    rows are decoded.  The projection is referenced, not registered: the model owns it as its head."""

    def __init__(self, projection: PackedLinear, original: nn.Embedding) -> None:
        super().__init__()
        if projection.layout is None:
            raise ValueError("a packed embedding requires rows that hold whole packing words")
        self._projection = (projection,)
        self.num_embeddings, self.embedding_dim = projection.out_features, projection.in_features
        self.padding_idx = original.padding_idx

    @property
    def projection(self) -> PackedLinear:
        return self._projection[0]

    @property
    def weight(self) -> Tensor:
        return self.projection.weight

    def forward(self, indices: Tensor) -> Tensor:
        head = self.projection
        rows = kernels.dequantize_rows(head.packed, head.scales, head.values, head.zeros, indices.reshape(-1),
                                       shape=(self.num_embeddings, self.embedding_dim), group=head.group,
                                       bits=head.code_bits, dtype=head.storage_dtype)
        return rows.view(*indices.shape, self.embedding_dim)


def optimize(model: Model | nn.Module, backend: str = "auto", *, compile: bool = False,
             mode: str = "reduce-overhead", cache_dense: bool = False, inplace: bool = False,
             siblings: tuple[tuple[str, ...], ...] | None = SIBLING_NAMES) -> Model:
    """Choose dense or packed execution; packed swaps every compatible ``nn.Linear`` of a ``QModel``
    for a ``PackedLinear`` and a tied embedding for a ``PackedEmbedding``.  ``siblings`` names linears
    under one parent that read the same input; each such group runs as one launch (``None``: never)."""
    if backend not in {"auto", "dense", "packed"}:
        raise ValueError("backend must be auto, dense, or packed")
    wrapped = model if isinstance(model, Model) else Model(model)
    if isinstance(wrapped, QModel):
        _ = wrapped.model_bpw
    if backend == "auto":
        backend = "packed" if isinstance(wrapped, QModel) else "dense"
    if backend == "packed":
        if not isinstance(wrapped, QModel):
            raise ValueError("packed inference requires a QModel with codec state")
        substitutes: dict[str, nn.Module] = {}
        for name, quantized in wrapped.quantized.items():
            target = wrapped.module.get_submodule(name)
            if isinstance(target, nn.Linear) and packed_compatible(quantized):
                substitutes[name] = PackedLinear(target, quantized, cache_dense=cache_dense)
        count = len(substitutes)
        for parameter_name, layer_name in wrapped.tied_weights.items():
            owner_name = parameter_name.rpartition(".")[0]
            owner = wrapped.module.get_submodule(owner_name)
            head = substitutes.get(layer_name)
            if isinstance(owner, nn.Embedding) and isinstance(head, PackedLinear) and head.layout is not None:
                substitutes[owner_name] = PackedEmbedding(head, owner)
        if inplace:
            for name, substitute in substitutes.items():
                if name:
                    wrapped.module.set_submodule(name, substitute)
                else:
                    wrapped.module = substitute
                    wrapped.architecture.model = substitute
            converted = wrapped
        else:
            memo = {id(wrapped.module.get_submodule(name)): substitute for name, substitute in substitutes.items()}
            converted = copy.deepcopy(wrapped, memo)
            for module in converted.module.modules():
                if isinstance(module, PackedLinear):
                    module._forward_pre_hooks = copy.deepcopy(module._forward_pre_hooks, memo)
        converted.execution_backend = f"packed:{count}"
        if siblings and not compile:
            fuse_siblings(converted.module, siblings)
    else:
        converted = wrapped if inplace else copy.deepcopy(wrapped)
        converted.execution_backend = "dense"
    if not inplace or backend == "packed":
        for attribute in ("_compiled_call", "_compiled_call_impl", "_last_compile_config", "_cache"):
            if attribute in converted.module.__dict__:
                delattr(converted.module, attribute)
    if compile:
        configuration = getattr(converted.module, "generation_config", None)
        if configuration is not None and hasattr(converted.module, "get_compiled_call"):
            from transformers import CompileConfig

            configuration = copy.deepcopy(configuration)
            configuration.cache_implementation = "static"
            configuration.compile_config = CompileConfig(mode=mode)
            converted.module.generation_config = configuration
        else:
            converted.module.compile(mode=mode)
        converted.execution_backend += "+compiled"
    return converted


class CapturedCall:
    """A module call replayed as one CUDA graph, host copies included.

    The reference removes the per-launch host cost of a decode step with ``optimize(compile=True)``
    (``torch.compile`` in ``reduce-overhead`` mode, ``src/mlkit/inference/optimization.py:86-99``); here
    the call is captured directly with stream capture, once per input signature (shapes, dtypes,
    devices).  A host input becomes a host-to-device copy node of the graph: from the caller's own
    tensor when it is pinned (its address is part of the signature), from a pinned staging buffer
    otherwise.  With host inputs the results are device-to-host copy nodes into pinned tensors.

    The tensors a call returns are owned by the capture and are overwritten by the next call with the
    same signature.  ``synchronize=False`` returns host results without waiting for them: the caller
    synchronises the stream (or calls ``wait``) before reading.
    """

    def __init__(self, function: Callable[..., Any], *, host_outputs: bool | None = None,
                 synchronize: bool = True) -> None:
        self.function = function
        self.host_outputs = host_outputs
        self.synchronize = synchronize
        self.entries: dict[tuple, dict[str, Any]] = {}
        self.device = next((t.device for t in _module_tensors(function) if t.is_cuda), None)
        self._last: torch.cuda.Event | None = None
        self._by_identity: dict[tuple[int, ...], dict[str, Any]] = {}

    MAXIMUM_PINNED_CAPTURES = 32   # distinct pinned input tensors that get a graph of their own

    def _signature(self, inputs: tuple[Tensor, ...]) -> tuple:
        # a pinned host input is read in place, so its address is part of the signature; a caller that passes
        # a new pinned tensor every time would grow a graph per call, so beyond a bound pinned inputs are
        # staged like pageable ones (one graph per shape)
        in_place = len(self.entries) < self.MAXIMUM_PINNED_CAPTURES
        return tuple((tuple(t.shape), t.dtype, t.device,
                      t.data_ptr() if in_place and not t.is_cuda and t.is_pinned() else 0) for t in inputs)

    def _capture(self, inputs: tuple[Tensor, ...], signature: tuple) -> dict[str, Any]:
        device = self.device or next((t.device for t in inputs if t.is_cuda), None)
        if device is None:
            raise ValueError("capture needs a CUDA module or a CUDA input")
        to_host = self.host_outputs if self.host_outputs is not None else all(not t.is_cuda for t in inputs)
        statics, sources = [], []
        for given, (_, _, _, address) in zip(inputs, signature):
            statics.append(torch.empty(given.shape, dtype=given.dtype, device=device))
            if given.is_cuda:
                sources.append(None)
            else:
                in_place = given.is_pinned() and address != 0
                sources.append(given if in_place else torch.empty(given.shape, dtype=given.dtype, device="cpu").pin_memory())
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        results: list[Tensor] = []
        with torch.cuda.stream(side), torch.inference_mode():
            for static, source, given in zip(statics, sources, inputs):
                if source is not None and source is not given:
                    source.copy_(given)
                static.copy_(given if source is None else source, non_blocking=True)
            self.function(*statics)   # first run outside capture: plans, workspaces, lazy state
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for static, source in zip(statics, sources):
                    if source is not None:
                        static.copy_(source, non_blocking=True)
                produced = self.function(*statics)
                single = isinstance(produced, Tensor)
                tensors = (produced,) if single else tuple(produced)
                first = tensors[0]
                if not to_host:
                    results.extend(tensors)
                elif len(tensors) > 1 and all(t.dtype == first.dtype and t.shape[:-1] == first.shape[:-1] for t in tensors):
                    # results that differ in their last dimension only travel as one copy: a copy node
                    # costs several microseconds whatever its size
                    joined = torch.cat(tensors, dim=-1)
                    host = torch.empty(joined.shape, dtype=joined.dtype, device="cpu").pin_memory()
                    host.copy_(joined, non_blocking=True)
                    start = 0
                    for tensor in tensors:
                        results.append(host[..., start:start + tensor.shape[-1]])
                        start += tensor.shape[-1]
                else:
                    for tensor in tensors:
                        host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu").pin_memory()
                        host.copy_(tensor, non_blocking=True)
                        results.append(host)
        torch.cuda.current_stream(device).wait_stream(side)
        return {"graph": graph, "statics": statics, "sources": sources, "results": results, "single": single,
                "to_host": to_host}

    def wait(self) -> None:
        """Block until the results of the last call are complete."""
        if self._last is not None:
            self._last.synchronize()

    def __call__(self, *inputs: Tensor) -> Any:
        # the same pinned tensors again (the steady state of a serving loop): no signature to compute, nothing to
        # copy on the host; the entry keeps those tensors alive, so the identities cannot be reused
        identity = tuple(map(id, inputs))
        entry = self._by_identity.get(identity)
        if entry is not None and all(given is source and given.shape == static.shape
                                     for given, source, static in zip(inputs, entry["sources"], entry["statics"])):
            entry["graph"].replay()
            if entry["to_host"]:
                self._last.record()
                if self.synchronize:
                    self._last.synchronize()
            return entry["results"][0] if entry["single"] else entry["tuple"]
        signature = self._signature(inputs)
        entry = self.entries.get(signature)
        if entry is None:
            entry = self.entries[signature] = self._capture(inputs, signature)
            entry["tuple"] = tuple(entry["results"])
            if self._last is None:
                self._last = torch.cuda.Event()
            if inputs and all(source is given for source, given in zip(entry["sources"], inputs)):
                self._by_identity[identity] = entry      # every input is a pinned tensor read in place
        for static, source, given in zip(entry["statics"], entry["sources"], inputs):
            if source is None:
                static.copy_(given, non_blocking=True)
            elif source is not given:
                self.wait()            # the staging buffer may still feed the previous replay
                source.copy_(given)
        entry["graph"].replay()
        if entry["to_host"]:
            if self._last is None:
                self._last = torch.cuda.Event()
            self._last.record()
            if self.synchronize:
                self._last.synchronize()
        return entry["results"][0] if entry["single"] else entry["tuple"]


def _module_tensors(function: Any):
    if isinstance(function, Model):
        function = function.module
    if isinstance(function, nn.Module):
        yield from function.parameters()
        yield from function.buffers()


def capture(function: Callable[..., Any], *, host_outputs: bool | None = None, synchronize: bool = True) -> CapturedCall:
    """``function`` (a module or any callable of tensors) as a ``CapturedCall``."""
    return CapturedCall(function, host_outputs=host_outputs, synchronize=synchronize)


@dataclass
class BenchmarkResult:
    median_ms: float
    minimum_ms: float
    percentile_95_ms: float
    repetitions: int
    device: str
    peak_memory_bytes: int | None

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def benchmark(operation: Callable[[], Any], *, warmup: int = 10, repetitions: int = 50,
              inference_mode: bool = True) -> BenchmarkResult:
    """Wall-clock samples with a device synchronisation on both sides of every call."""
    if warmup < 0 or repetitions < 1:
        raise ValueError("warmup must be nonnegative and repetitions must be positive")
    device = torch.device("cuda", torch.cuda.current_device())
    samples = []
    with torch.inference_mode(inference_mode):
        for _ in range(warmup):
            operation()
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        for _ in range(repetitions):
            torch.cuda.synchronize(device)
            start = time.perf_counter()
            operation()
            torch.cuda.synchronize(device)
            samples.append((time.perf_counter() - start) * 1000)
    ordered = sorted(samples)
    return BenchmarkResult(statistics.median(samples), ordered[0],
                           ordered[min(len(ordered) - 1, int(len(ordered) * 0.95))], repetitions, str(device),
                           torch.cuda.max_memory_allocated(device))


def benchmark_model(model: Model | nn.Module, batch: Any, **options: Any) -> BenchmarkResult:
    wrapped = model if isinstance(model, Model) else Model(model)

    def run() -> Any:
        if isinstance(batch, dict):
            return wrapped(**batch)
        if isinstance(batch, (tuple, list)):
            return wrapped(*batch)
        return wrapped(batch)

    return benchmark(run, **options)
