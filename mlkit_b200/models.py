"""Model wrappers the packed-inference API is expressed in.

Minimal counterparts of ``src/mlkit/models/model.py:18-166``: ``Model`` places a module on CUDA and
forwards calls to it; ``QModel`` additionally carries the ``Q`` of every quantised layer, which is what
``optimize`` substitutes packed layers from and what checkpoints serialise.  Architecture adapters,
calibration and reports beyond a plain record are outside the packed-inference path.
"""

from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

import torch
from torch import Tensor, nn
from torch.utils._pytree import tree_map

from mlkit_b200.quantization import Q


def weight_name(module_name: str) -> str:
    return f"{module_name}.weight" if module_name else "weight"


@dataclass
class LayerReport:
    """One quantised layer: its name, shape, total stored bits, relative error and seconds spent."""

    name: str
    shape: tuple
    bits: float | None
    loss: float
    seconds: float

    @property
    def elements(self) -> int:
        return int(self.shape[0]) * int(self.shape[1])

    @property
    def bpw(self) -> float | None:
        return None if self.bits is None else self.bits / self.elements


class _Architecture:
    def __init__(self, model: nn.Module) -> None:
        self.model = model


class Model(nn.Module):
    def __init__(self, module: nn.Module, tokenizer: Any = None, *, name: str | None = None) -> None:
        super().__init__()
        self.module = module.cuda()
        self.tokenizer = tokenizer
        self.name = name or type(module).__name__
        self.architecture = _Architecture(module)
        self.execution_backend = "dense"
        first = next(module.parameters(), None)
        self._initial_dtype = torch.float32 if first is None else first.dtype
        self._parameter_accounting: tuple[int, int] | None = None

    def _to_device(self, args: tuple, kwargs: dict) -> tuple[tuple, dict]:
        device = self.device
        return tree_map(lambda value: value.to(device) if isinstance(value, Tensor) else value, (args, kwargs))

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        args, kwargs = self._to_device(args, kwargs)
        return self.module(*args, **kwargs)

    def generate(self, *args: Any, **kwargs: Any) -> Any:
        args, kwargs = self._to_device(args, kwargs)
        return self.module.generate(*args, **kwargs)

    @property
    def device(self) -> torch.device:
        tensor = next(self.module.parameters(), None)
        if tensor is None:
            tensor = next(self.module.buffers(), None)
        return torch.device("cuda") if tensor is None else tensor.device

    @property
    def dtype(self) -> torch.dtype:
        tensor = next(self.module.parameters(), None)
        return self._initial_dtype if tensor is None else tensor.dtype

    @property
    def config(self) -> Any:
        return self.module.config

    @property
    def storage_bytes(self) -> int:
        """Bytes held by distinct parameter and buffer storages."""
        seen: dict[tuple, int] = {}
        for tensor in (*self.module.parameters(), *self.module.buffers()):
            storage = tensor.untyped_storage()
            seen[(tensor.device, storage.data_ptr())] = storage.nbytes()
        return sum(seen.values())


class QModel(Model):
    """A converted model: ``quantized`` maps layer names to their ``Q``; ``tied_weights`` maps a
    parameter that shares a quantised weight (a tied embedding) to the layer that owns the codes."""

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self.quantized: dict[str, Q] = {}
        self.layer_reports: list[LayerReport] = []
        self.stability_reports: dict[str, Any] = {}
        self.pass_reports: list[Any] = []
        self.activation_specs: dict[str, Any] = {}
        self.kv_spec: Any = None
        self.tied_weights: dict[str, str] = {}

    @property
    def bpw(self) -> float | None:
        if not self.layer_reports or any(record.bits is None for record in self.layer_reports):
            return None
        return sum(record.bits for record in self.layer_reports) / sum(r.elements for r in self.layer_reports)

    @property
    def model_bpw(self) -> float | None:
        """Bits per weight over every parameter, untouched ones at their storage width."""
        if self.bpw is None:
            return None
        if self._parameter_accounting is None:
            quantised = {weight_name(record.name) for record in self.layer_reports} | set(self.tied_weights)
            elements = bits = 0
            for name, parameter in self.module.named_parameters():
                elements += parameter.numel()
                if name not in quantised:
                    bits += parameter.numel() * parameter.element_size() * 8
            self._parameter_accounting = (elements, bits)
        elements, untouched_bits = self._parameter_accounting
        return (untouched_bits + sum(record.bits for record in self.layer_reports)) / elements

    def report(self, *, print_table: bool = True) -> list[dict[str, Any]]:
        records = [asdict(record) | {"bpw": record.bpw} for record in self.layer_reports]
        if print_table:
            for record in self.layer_reports:
                width = "?" if record.bpw is None else f"{record.bpw:.3f}"
                print(f"{record.name:58} {width:>7} {record.loss:12.5g} {record.seconds:9.3f}")
        return records

    def save(self, path: str | Path, **options: Any) -> None:
        from mlkit_b200.checkpoints import save

        save(self, path, **options)
