"""Regenerate the golden vectors under ``tests/golden`` from the reference library itself.

Run once, in a container where the reference checkout is importable on CPU:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

It imports mlkit (the reference), drives its CPU tensor paths on seeded inputs
and stores inputs and outputs as compressed ``.npz`` files.  The tests never
import the reference; they read these files.  Nothing here runs on a GPU.
"""

import json
import math
import sys
from pathlib import Path

import numpy as np
import torch

import mlkit as mk  # the reference library, not this repository's package
from mlkit.kernels.packed_linear import layout_for
from mlkit.inference.packed_linear import packed_compatible
from mlkit.quantization.codecs import decode_scaled
from mlkit.quantization.context import Ctx, layer_seed
from mlkit.quantization.operations.orthogonal_transforms import (
    hadamard,
    paley_matrix,
    randomized_transform,
    structured_transform,
    transform_factor,
)

HERE = Path(__file__).resolve().parent


def bitstream_vectors() -> dict:
    out = {}
    generator = torch.Generator().manual_seed(1234)
    for bits in range(1, 17):
        for count in (0, 1, 7, 17, 64, 200):
            codes = torch.randint(2**bits, (count,), dtype=torch.int32, generator=generator)
            packed = mk.pack(codes, bits)
            assert torch.equal(mk.unpack(packed, bits, codes.shape).int(), codes)
            out[f"b{bits}_n{count}_codes"] = codes.numpy()
            out[f"b{bits}_n{count}_packed"] = packed.numpy()
    return out


CODEC_CASES = {
    # name: (format factory, out rows, in width, input rows)
    "int2_g128": (lambda: mk.int(2, group=128), 24, 256, 1),
    "int3_g128": (lambda: mk.int(3, group=128), 24, 256, 8),
    "int4_g128": (lambda: mk.int(4, group=128), 24, 256, 1),
    "int4_g128_qwen": (lambda: mk.int(4, group=128), 16, 896, 1),
    "int5_g64": (lambda: mk.int(5, group=64), 24, 256, 3),
    "int6_g32": (lambda: mk.int(6, group=32), 24, 256, 3),
    "int7_g64": (lambda: mk.int(7, group=64), 24, 256, 3),
    "int8_g128": (lambda: mk.int(8, group=128), 24, 256, 8),
    "nf4_g64": (lambda: mk.nf4(group=64), 24, 256, 8),
    "codebook3_g64_mse": (
        lambda: mk.scaled(
            mk.grid.values(torch.tensor([-1, -0.5, -0.25, 0, 0.25, 0.5, 1.0]), bits=3),
            group=64, scale="mse"),
        24, 256, 8),
    "int4_g64_asym": (lambda: mk.int(4, group=64, asym=True), 24, 256, 3),
    "int3_g64_asym": (lambda: mk.int(3, group=64, asym=True), 24, 256, 3),
    "e4m3_g64": (lambda: mk.scaled(mk.grid.fp("e4m3"), group=64), 24, 256, 3),
    "int4_g32_ragged": (lambda: mk.int(4, group=32), 71, 130, 7),
    "nf4_g32_ragged": (lambda: mk.nf4(group=32), 71, 130, 3),
    "int4_g64_mse": (lambda: mk.int(4, group=64, scale="mse"), 16, 192, 2),
}


def codec_vectors() -> tuple[dict, dict]:
    arrays, meta = {}, {}
    for index, (name, (factory, rows, width, samples)) in enumerate(CODEC_CASES.items()):
        generator = torch.Generator().manual_seed(100 + index)
        weight = (torch.randn(rows, width, generator=generator) * 0.02).half().float()
        x = torch.randn(samples, width, generator=generator).half()
        q = factory()(weight, Ctx(device="cpu"))
        bits = int(q.metadata["code_bits"])
        group = int(q.params["group"])
        zero = q.params.get("zero")
        packed = mk.pack(q.codes, bits)
        decoded = decode_scaled(q.codes, scales=q.params["scales"], values=q.params["values"],
                                group=group, zero=zero)
        assert torch.equal(decoded, q.w)
        scales16 = q.params["scales"].half()
        assert torch.equal(scales16.float(), q.params["scales"])
        zero16 = None if zero is None else zero.half()
        dense16 = decode_scaled(q.codes, scales=scales16.float(), values=q.params["values"],
                                group=group, zero=None if zero16 is None else zero16.float()
                                ).to(torch.float16)
        y = torch.nn.functional.linear(x.float(), dense16.float())
        layout = layout_for(bits, width, group)
        arrays[f"{name}.weight"] = weight.numpy()
        arrays[f"{name}.x"] = x.numpy()
        arrays[f"{name}.codes"] = q.codes.numpy()
        arrays[f"{name}.packed"] = packed.numpy()
        arrays[f"{name}.scales"] = q.params["scales"].numpy()
        arrays[f"{name}.values"] = q.params["values"].numpy()
        if zero is not None:
            arrays[f"{name}.zero"] = zero.numpy()
            arrays[f"{name}.zero16"] = zero16.numpy()
        arrays[f"{name}.decoded"] = decoded.numpy()
        arrays[f"{name}.dense16"] = dense16.numpy()
        arrays[f"{name}.y"] = y.numpy()
        meta[name] = {
            "bits": bits, "group": group, "rows": rows, "width": width, "samples": samples,
            "integer": bool(name.startswith("int")), "asym": zero is not None,
            "scale": "mse" if name.endswith("mse") else "absmax",
            "codec": q.codec, "metadata": {k: v for k, v in q.metadata.items()},
            "layout": None if layout is None else
            [layout.bits, layout.bytes_per_word, layout.codes_per_word, layout.tile_words],
            "compatible": bool(packed_compatible(q)), "total_bits": q.bits,
        }
    return arrays, meta


def transform_vectors() -> tuple[dict, dict]:
    arrays, meta = {}, {"factors": {}, "seeds": {}}
    generator = torch.Generator().manual_seed(77)
    for width in (1, 2, 4, 8, 16, 32, 64, 128, 512, 2048, 4096):
        value = torch.randn(3, width, generator=generator)
        arrays[f"fwht{width}.x"] = value.numpy()
        arrays[f"fwht{width}.y"] = hadamard(value).numpy()
        arrays[f"fwht{width}.raw"] = hadamard(value, normalize=False).numpy()
    for order in (12, 20, 28, 44, 76):
        arrays[f"paley{order}"] = paley_matrix(order).numpy()
    for width in (7, 12, 20, 28, 96, 896, 4096, 4864, 8192, 14336, 28672, 11008, 13824, 5120):
        factor, power, basis = transform_factor(width)
        meta["factors"][str(width)] = [factor, power, basis is not None]
        if basis is not None and f"basis{factor}" not in arrays:
            arrays[f"basis{factor}"] = basis.numpy()
    for width in (7, 12, 20, 28, 96, 896, 4864, 14336):
        value = torch.randn(2, width, generator=generator)
        arrays[f"structured{width}.x"] = value.numpy()
        arrays[f"structured{width}.y"] = structured_transform(value).numpy()
        arrays[f"structured{width}.inverse"] = structured_transform(value, inverse=True).numpy()
    for width, seed in ((4096, 5), (14336, 9), (896, 3)):
        value = torch.randn(2, width, generator=generator)
        outliers = torch.randperm(width, generator=generator)[: max(1, width // 100)]
        value[:, outliers] *= 50
        value = value.half().float()
        sign_generator = torch.Generator(device="cpu").manual_seed(seed)
        signs = torch.randint(2, (width,), generator=sign_generator) * 2 - 1
        arrays[f"rht{width}.x"] = value.numpy()
        arrays[f"rht{width}.signs"] = signs.to(torch.int8).numpy()
        arrays[f"rht{width}.y"] = randomized_transform(value, seed=seed).numpy()
        arrays[f"rht{width}.inverse"] = randomized_transform(value, seed=seed, inverse=True).numpy()
        meta["seeds"][str(width)] = seed
    meta["layer_seed"] = {
        name: [seed, layer_seed(name, seed)]
        for name, seed in (("model.layers.0.self_attn.o_proj", 0),
                           ("model.layers.17.mlp.down_proj", 3), ("", 0))
    }
    return arrays, meta


def layout_table() -> dict:
    table = {}
    for bits in range(1, 10):
        for width in (16, 64, 130, 250, 255, 256, 896, 4096, 14336):
            for group in (5, 8, 16, 20, 32, 50, 64, 96, 128, 256):
                layout = layout_for(bits, width, group)
                table[f"{bits},{width},{group}"] = None if layout is None else [
                    layout.bits, layout.bytes_per_word, layout.codes_per_word, layout.tile_words]
    return table


def main() -> None:
    torch.manual_seed(0)
    np.savez_compressed(HERE / "bitstream.npz", **bitstream_vectors())
    arrays, codec_meta = codec_vectors()
    np.savez_compressed(HERE / "codecs.npz", **arrays)
    arrays, transform_meta = transform_vectors()
    np.savez_compressed(HERE / "transforms.npz", **arrays)
    meta = {
        "reference": {"package": "mlkit", "version": mk.__version__},
        "torch": torch.__version__, "python": sys.version.split()[0],
        "codecs": codec_meta, "transforms": transform_meta, "layouts": layout_table(),
        "linspace_0p5_1_20": [float(v) for v in torch.linspace(0.5, 1.0, 20)],
        "reciprocal_sqrt": {str(w): float(torch.tensor(1.0) / torch.tensor(math.sqrt(w)))
                            for w in (512, 1024, 4096, 8192)},
    }
    (HERE / "golden.json").write_text(json.dumps(meta, indent=1, sort_keys=True) + "\n")
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
