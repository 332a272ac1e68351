"""mlkit checkpoints: a versioned JSON manifest (``mlkit.json``) beside one ``weights.safetensors``.

Same on-disk format as ``src/mlkit/checkpoints/saving.py:23-157`` and ``loading.py:36-180``
(format version 1), so a checkpoint written by the reference restores here and the restored
``QModel`` routes through ``optimize`` to the packed kernels:

* per codec layer: ``"<layer>.codes"`` (the bit stream at ``code_bits``), ``"<layer>.params.<p>"``
  (scales and offsets at their storage format; identical tensors are stored once and later
  descriptors point at the first copy), a manifest entry with ``codec``, ``shape``, ``code_bits``,
  ``bits``, ``params`` descriptors and JSON-able ``metadata``;
* ``"state.<name>"`` for every other state entry, except quantised weights, tied weights and the
  packed layer's own ``packed/scales/values/zeros`` buffers (codes are re-packed from the model);
* writes go to a temporary directory that replaces the destination atomically.
"""

import hashlib
import json
import os
import shutil
import tempfile
from collections.abc import Callable
from dataclasses import asdict
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import load_file, save_file
from torch import Tensor, nn

from mlkit_b200.conversion import install_transform, record_transform
from mlkit_b200.models import LayerReport, QModel, weight_name
from mlkit_b200.quantization import Q, decoder, pack, registered, unpack

FORMAT_VERSION = 1
MANIFEST_FILE = "mlkit.json"
WEIGHTS_FILE = "weights.safetensors"
# parameter tensors stored in these dtypes are widened to fp32 on load (src/mlkit/checkpoints/loading.py:33,180)
_HALF_STORAGE = {torch.float16, torch.bfloat16, torch.float8_e4m3fn}
_JSON_TYPES = (str, int, float, bool, list, dict, type(None))


def _store_parameter(name: str, parameter: str, value: Tensor, metadata: dict, tensors: dict,
                     seen: dict) -> dict[str, Any]:
    """Descriptor of one tensor parameter; the tensor goes into ``tensors`` unless an equal one exists."""
    identifier = f"{name}.params.{parameter}"
    descriptor: dict[str, Any] = {"tensor": identifier, "encoding": None}
    bits = metadata.get("parameter_bits", {}).get(parameter)
    if bits is not None:
        descriptor.update(encoding="packed", bits=bits, shape=list(value.shape))
        value = pack(value, bits)
    else:
        storage = metadata.get("parameter_formats", {}).get(parameter)
        if parameter in {"scales", "zero"}:
            storage = metadata.get("scale_fmt", "fp32")
        if storage == "fp16":
            value = value.half()
        elif storage == "bf16":
            value = value.bfloat16()
    stored = value.detach().cpu().contiguous()
    key = (str(stored.dtype), tuple(stored.shape),
           hashlib.sha256(stored.reshape(-1).view(torch.uint8).numpy().tobytes()).digest())
    if key in seen:
        descriptor["tensor"] = seen[key]
    else:
        tensors[identifier] = stored.clone()
        seen[key] = identifier
    return descriptor


def save(model: QModel, path: str | Path, *, overwrite: bool = False) -> None:
    destination = Path(path).resolve()
    if destination.exists() and not overwrite:
        raise FileExistsError(f"checkpoint destination already exists: {destination}")
    destination.parent.mkdir(parents=True, exist_ok=True)
    staging = Path(tempfile.mkdtemp(prefix="mlkit_checkpoint_", dir=destination.parent))
    try:
        tensors: dict[str, Tensor] = {}
        seen: dict[tuple, str] = {}
        layers: dict[str, Any] = {}
        for name, quantized in model.quantized.items():
            if not (registered(quantized.codec) and quantized.codes is not None):
                tensors[f"{name}.reconstruction"] = quantized.w.detach().cpu().contiguous()
                layers[name] = {"codec": None, "bits": quantized.bits}
                continue
            code_bits = quantized.metadata.get("code_bits")
            if code_bits is None:
                code_bits = max(1, int(quantized.codes.max()).bit_length())
            tensors[f"{name}.codes"] = pack(quantized.codes.cpu(), code_bits)
            parameters = {
                key: (_store_parameter(name, key, value, quantized.metadata, tensors, seen)
                      if isinstance(value, Tensor) else {"value": value})
                for key, value in quantized.params.items()
            }
            layers[name] = {
                "codec": quantized.codec, "shape": list(quantized.codes.shape), "code_bits": code_bits,
                "bits": quantized.bits, "params": parameters,
                "metadata": {k: v for k, v in quantized.metadata.items() if isinstance(v, _JSON_TYPES)},
            }
        omitted = {weight_name(name) for name in model.quantized} | set(model.tied_weights)
        storages: dict[tuple, str] = {}
        aliases: dict[str, str] = {}
        for name, value in model.module.state_dict().items():
            owner, _, field = name.rpartition(".")
            if owner in model.quantized and field in {"packed", "scales", "values", "zeros"}:
                continue
            if name in omitted:
                continue
            identity = (value.device, value.data_ptr(), value.dtype, tuple(value.shape), tuple(value.stride()))
            if identity in storages:
                aliases[name] = storages[identity]
            else:
                tensors[f"state.{name}"] = value.detach().cpu().contiguous().clone()
                storages[identity] = name
        save_file(tensors, str(staging / WEIGHTS_FILE))
        configuration = getattr(model.module, "config", None)
        if configuration is not None:
            configuration.save_pretrained(staging)
        if model.tokenizer is not None:
            model.tokenizer.save_pretrained(staging)
        manifest = {
            "format_version": FORMAT_VERSION, "name": model.name,
            "architecture": "transformers" if configuration is not None else "external",
            "dtype": str(model.dtype).removeprefix("torch."), "layers": layers,
            "reports": [asdict(record) for record in model.layer_reports], "pass_reports": [],
            "stability_reports": model.stability_reports, "logical_bpw": model.bpw, "model_bpw": model.model_bpw,
            "parameter_accounting": model._parameter_accounting,
            "transforms": getattr(model.module, "_mlkit_transforms", []),
            "activations": model.activation_specs, "kv": model.kv_spec, "state_aliases": aliases,
            "tied_weights": model.tied_weights,
            "tensor_bytes": sum(value.numel() * value.element_size() for value in tensors.values()),
        }
        (staging / MANIFEST_FILE).write_text(json.dumps(manifest, indent=2) + "\n")
        if destination.exists():
            backup = destination.with_name(f"{destination.name}.previous")
            if backup.exists():
                raise FileExistsError(f"checkpoint backup already exists: {backup}")
            os.replace(destination, backup)
            try:
                os.replace(staging, destination)
            except BaseException:
                os.replace(backup, destination)
                raise
            shutil.rmtree(backup)
        else:
            os.replace(staging, destination)
    finally:
        if staging.exists():
            shutil.rmtree(staging)


def _load_parameter(tensors: dict[str, Tensor], descriptor: dict[str, Any]) -> Tensor:
    value = tensors[descriptor["tensor"]]
    if descriptor.get("encoding") == "e8m0":
        return torch.pow(2.0, value.float() - 127)
    if descriptor.get("encoding") == "packed":
        return unpack(value, descriptor["bits"], tuple(descriptor["shape"]))
    return value.float() if value.dtype in _HALF_STORAGE else value


def restore_layer(tensors: dict[str, Tensor], name: str, layer: dict[str, Any]) -> Q:
    """Rebuild one layer's ``Q`` on the device its tensors live on."""
    if layer["codec"] is None:
        return Q(tensors[f"{name}.reconstruction"], bits=layer["bits"])
    codes = unpack(tensors[f"{name}.codes"], layer["code_bits"], tuple(layer["shape"]))
    parameters = {key: (_load_parameter(tensors, value) if "tensor" in value else value["value"])
                  for key, value in layer["params"].items()}
    return Q(codes=codes, params=parameters, decode=decoder(layer["codec"]), codec=layer["codec"],
             bits=layer["bits"], metadata=layer.get("metadata", {}) | {"code_bits": layer["code_bits"]})


def load_checkpoint(path: str | Path, *, model: nn.Module | Callable[[], nn.Module] | None = None) -> QModel:
    """Restore a ``QModel`` on CUDA: codes are unpacked and decoded on the device (bit-exact kernel),
    dense reconstructions fill the module, online transforms are re-installed."""
    directory = Path(path)
    manifest = json.loads((directory / MANIFEST_FILE).read_text())
    if manifest.get("format_version") != FORMAT_VERSION:
        raise ValueError("unsupported mlkit checkpoint format version")
    if manifest.get("activations") or manifest.get("kv") is not None:
        # the reference installs online activation / KV quantisers for these entries
        # (src/mlkit/checkpoints/loading.py:86-100); loading without them would run different numerics
        raise NotImplementedError("this checkpoint asks for online activation or KV-cache quantisation, "
                                  "which mlkit_b200 does not implement")
    dtype = getattr(torch, manifest["dtype"])
    tokenizer = None
    if model is None:
        if manifest["architecture"] != "transformers":
            raise ValueError("external architecture checkpoints require model=module or model=factory")
        from transformers import AutoConfig, AutoModelForCausalLM, AutoTokenizer

        configuration = AutoConfig.from_pretrained(directory, trust_remote_code=False)
        module = AutoModelForCausalLM.from_config(configuration, trust_remote_code=False, dtype=dtype)
        if (directory / "tokenizer_config.json").exists():
            tokenizer = AutoTokenizer.from_pretrained(directory, trust_remote_code=False)
    else:
        module = model if isinstance(model, nn.Module) else model()
        module.to(dtype=dtype)
    tensors = load_file(str(directory / WEIGHTS_FILE), device="cuda")
    state = {name.removeprefix("state."): value for name, value in tensors.items() if name.startswith("state.")}
    for alias, canonical in manifest.get("state_aliases", {}).items():
        state[alias] = state[canonical]
    quantized: dict[str, Q] = {}
    for name, layer in manifest["layers"].items():
        restored = restore_layer(tensors, name, layer)
        with torch.no_grad():
            state[weight_name(name)] = restored.w.to(dtype)
        quantized[name] = restored.to("cpu", detach=True)
    tied = manifest.get("tied_weights", {})
    for parameter_name, layer_name in tied.items():
        state[parameter_name] = state[weight_name(layer_name)]
    del tensors
    for descriptor in manifest.get("transforms", []):
        install_transform(module, descriptor, state)
        record_transform(module, descriptor)
    for name, value in state.items():  # biases that conversion introduced on bias-free projections
        owner, _, field = name.rpartition(".")
        if field == "bias":
            target = module.get_submodule(owner)
            if isinstance(target, nn.Linear) and target.bias is None:
                target.bias = nn.Parameter(value.detach().clone())
    module.load_state_dict(state, strict=True)
    module.cuda().eval()
    converted = QModel(module, tokenizer, name=manifest["name"])
    converted.quantized = quantized
    converted.tied_weights = dict(tied)
    converted.stability_reports = manifest.get("stability_reports", {})
    converted.activation_specs = {}
    converted.kv_spec = None
    converted.layer_reports = [
        LayerReport(record["name"], tuple(record["shape"]), record.get("bits"), record.get("loss", 0.0),
                    record.get("seconds", 0.0))
        for record in manifest.get("reports", [])
    ]
    if manifest.get("parameter_accounting") is not None:
        converted._parameter_accounting = tuple(manifest["parameter_accounting"])
    return converted


def load(name: str | Path, **options: Any) -> QModel:
    """``mk.load`` for checkpoint directories (``src/mlkit/models/loading.py:12-21``)."""
    path = Path(name)
    if not (path / MANIFEST_FILE).is_file():
        raise ValueError(f"{path} is not an mlkit checkpoint directory")
    return load_checkpoint(path, **options)
