"""Conversion entry points the packed path needs: round-to-nearest ``quantize`` and the online
input transforms that ride on a layer as forward pre-hooks.

``install_transform`` / ``record_transform`` keep the descriptor format of
``src/mlkit/conversion/model_transforms.py:179-209`` (``{"kind": "rotation", "name", "seed"}`` and
``{"kind": "smooth", "name"}``), so transforms written into a checkpoint manifest by the reference
are re-installed here, with the rotation body replaced by the fused transform kernel.
``quantize`` covers the calibration-free case of ``src/mlkit/conversion/model_conversion.py``
(``calib=None``): every ``nn.Linear`` is rounded with the given format.
"""

import time
from collections.abc import Callable, Iterable
from typing import Any

import torch
from torch import Tensor, nn

from mlkit_b200 import transforms
from mlkit_b200.models import LayerReport, Model, QModel
from mlkit_b200.quantization import Ctx, Q, as_q, layer_seed


def record_transform(model: nn.Module, descriptor: dict[str, Any]) -> None:
    descriptors = getattr(model, "_mlkit_transforms", [])
    descriptors.append(descriptor)
    model.__dict__["_mlkit_transforms"] = descriptors


class _RotateInputs:
    """Pre-hook: ``x -> S(x * signs)`` in the activation dtype, one fused launch.

    The sign vector is drawn once per device with the reference's recipe (a torch generator on the
    activation's device seeded with the descriptor's seed) and cached as int8.
    """

    def __init__(self, seed: int) -> None:
        self.seed = seed
        self._signs: dict[tuple[torch.device, int], Tensor] = {}

    def signs_for(self, width: int, device: torch.device) -> Tensor:
        key = (device, width)
        if key not in self._signs:
            self._signs[key] = transforms.sign_vector(width, self.seed, device)
        return self._signs[key]

    def __call__(self, layer: nn.Module, arguments: tuple) -> tuple:
        inputs = arguments[0]
        if not inputs.is_cuda:
            raise ValueError("the online rotation runs on CUDA activations only")
        signs = self.signs_for(inputs.shape[-1], inputs.device)
        take = getattr(layer, "take_rotation", None)
        last = next(reversed(layer._forward_pre_hooks.values()), None) is self   # nothing edits the input after this hook
        if take is not None and last and take(inputs, signs):
            return None     # the layer rotates while it loads its activations (one launch instead of two)
        rotated = transforms.structured_transform(inputs, signs=signs)
        return (rotated, *arguments[1:])

    def __deepcopy__(self, memo: dict) -> "_RotateInputs":
        return _RotateInputs(self.seed)


def _balance_inputs(layer: nn.Module, arguments: tuple) -> tuple:
    inputs = arguments[0]
    return ((inputs.float() / layer._mlkit_input_scale).to(inputs.dtype), *arguments[1:])


def install_transform(model: nn.Module, descriptor: dict[str, Any], state: dict[str, Tensor] | None = None) -> None:
    """Attach the online transform a descriptor names to its layer."""
    module = model.get_submodule(descriptor["name"])
    if descriptor["kind"] == "rotation":
        module.register_forward_pre_hook(_RotateInputs(int(descriptor["seed"])))
    elif descriptor["kind"] == "smooth":
        if state is not None:
            module.register_buffer("_mlkit_input_scale", state[f"{descriptor['name']}._mlkit_input_scale"])
        module.register_forward_pre_hook(_balance_inputs)
    else:
        raise ValueError(f"unknown model transform {descriptor['kind']!r}")


def rotate_inputs(model: Model | nn.Module, names: Iterable[str] | None = None, *, seed: int = 0) -> None:
    """Online Hadamard rotation of the inputs of the named linears (default: every ``o_proj`` and
    ``down_proj``): the weight is rotated along its input axis with a per-layer seed and a pre-hook
    rotates the activations to match, so the layer's function is preserved."""
    root = model.module if isinstance(model, Model) else model
    chosen = set(names) if names is not None else None
    with torch.no_grad():
        for name, module in root.named_modules():
            if not isinstance(module, nn.Linear):
                continue
            if chosen is None and name.split(".")[-1] not in {"o_proj", "down_proj"}:
                continue
            if chosen is not None and name not in chosen:
                continue
            seed_of_layer = layer_seed(name, seed)
            signs = transforms.sign_vector(module.in_features, seed_of_layer, module.weight.device)
            rotated = transforms.structured_transform(module.weight.float().contiguous(), signs=signs)
            module.weight.copy_(rotated.to(module.weight.dtype))
            descriptor = {"kind": "rotation", "name": name, "seed": seed_of_layer}
            install_transform(root, descriptor)
            record_transform(root, descriptor)


def quantize(model: Model | nn.Module, format: Callable[[Tensor, Ctx], Q | Tensor], calib: Any = None,
             *, skip: Iterable[str] = (), seed: int = 0, **unused: Any) -> QModel:
    """Round every ``nn.Linear`` weight with ``format`` (calibration-free) and return a ``QModel``
    whose module holds the reconstructions."""
    if calib is not None:
        raise NotImplementedError("mlkit_b200.quantize covers calibration-free (round-to-nearest) formats")
    source = model.module if isinstance(model, Model) else model
    converted = QModel(source, getattr(model, "tokenizer", None), name=getattr(model, "name", None))
    skipped = set(skip)
    with torch.no_grad():
        for name, module in converted.module.named_modules():
            if not isinstance(module, nn.Linear) or name in skipped:
                continue
            started = time.perf_counter()
            weight = module.weight.detach()
            result = as_q(format(weight.float(), Ctx(name, module, seed=seed, device=weight.device)))
            reconstruction = result.w
            module.weight.copy_(reconstruction.to(weight.dtype))
            error = (reconstruction - weight.float()).square().sum() / weight.float().square().sum().clamp_min(1e-30)
            converted.quantized[name] = result.to("cpu", detach=True)
            converted.layer_reports.append(LayerReport(name, tuple(weight.shape), result.bits, float(error),
                                                       time.perf_counter() - started))
    return converted
