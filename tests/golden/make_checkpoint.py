"""Write the reference-made checkpoint fixture under ``tests/golden/ckpt`` with the reference's own ``save``.

Run once, in a container where the reference checkout is importable on CPU:

    PYTHONPATH=<reference>/src python tests/golden/make_checkpoint.py

The reference moves every model to CUDA when it wraps it (``src/mlkit/models/model.py:28``); inside
this script only, ``nn.Module.cuda`` is replaced by the identity so that conversion and ``save`` run on
the CPU.  Two checkpoints are written:

* ``tied``: an embedding tied to the output head around two projections, INT4 with groups of 8 and
  fp16 scales (the model of the reference's own checkpoint test,
  ``tests/checkpoints/test_checkpoints.py:60-80``), with its inputs and the reference's outputs;
* ``rotated``: one ``o_proj`` with an online rotation descriptor recorded by the reference's
  ``record_transform`` (``src/mlkit/conversion/model_transforms.py:179-183``).  The sign vector of a
  rotation comes from the generator of the device the model runs on, so a CPU-made file cannot carry
  outputs that a CUDA load reproduces; the fixture pins the manifest and tensor layout only.
"""

import json
import shutil
from pathlib import Path

import numpy as np
import torch
from torch import nn

nn.Module.cuda = lambda self, *args, **kwargs: self  # CPU only, in this script only

import mlkit as mk  # noqa: E402  (the reference library, not this repository's package)
from mlkit.conversion.model_transforms import install_transform, record_transform  # noqa: E402
from mlkit.quantization.context import layer_seed  # noqa: E402
from mlkit.quantization.operations.orthogonal_transforms import rht  # noqa: E402

HERE = Path(__file__).resolve().parent / "ckpt"


class TiedLanguageModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.embedding = nn.Embedding(32, 16)
        self.projections = nn.Sequential(nn.Linear(16, 16), nn.Linear(16, 16))
        self.lm_head = nn.Linear(16, 32, bias=False)
        self.lm_head.weight = self.embedding.weight

    def forward(self, tokens):
        return self.lm_head(self.projections(self.embedding(tokens)))


class Attention(nn.Module):
    def __init__(self):
        super().__init__()
        self.o_proj = nn.Linear(64, 24, bias=False)

    def forward(self, x):
        return self.o_proj(x)


def main() -> None:
    torch.manual_seed(2024)
    if HERE.exists():
        shutil.rmtree(HERE)
    HERE.mkdir(parents=True)
    record = {}

    converted = mk.quantize(TiedLanguageModel(), mk.int(4, group=8), calib=None)
    converted.save(HERE / "tied")
    tokens = torch.randint(32, (2, 7), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        logits = converted(tokens)
    np.savez_compressed(HERE / "tied_io.npz", tokens=tokens.numpy(), logits=logits.float().numpy())
    record["tied"] = {"bpw": converted.bpw, "model_bpw": converted.model_bpw}

    module = Attention()
    seed = layer_seed("o_proj", 7)
    with torch.no_grad():
        module.o_proj.weight.copy_(rht(module.o_proj.weight.float(), seed=seed))
    descriptor = {"kind": "rotation", "name": "o_proj", "seed": seed}
    install_transform(module, descriptor)
    record_transform(module, descriptor)
    rotated = mk.quantize(module, mk.int(4, group=32), calib=None)
    rotated.save(HERE / "rotated")
    record["rotated"] = {"seed": seed, "bpw": rotated.bpw}

    (HERE / "fixture.json").write_text(json.dumps(record, indent=1))
    for path in sorted(HERE.rglob("*")):
        if path.is_file():
            print(path.relative_to(HERE), path.stat().st_size)


if __name__ == "__main__":
    main()
