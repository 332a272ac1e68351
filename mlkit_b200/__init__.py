"""mlkit_b200: B200-native packed-weight inference behind mlkit's module API.

The names below mirror the facade of the reference (``src/mlkit/__init__.py``) for the packed
inference path, so ``import mlkit_b200 as mk`` keeps code written against ``mk.optimize``,
``mk.PackedLinear``, ``mk.int`` / ``mk.nf4`` / ``mk.scaled``, ``mk.codec``, ``mk.pack``, ``mk.rht``,
``mk.load`` ... working, with every device computation done by hand-written sm_100a kernels in
``libmlkit_b200.so``.  There is no CPU fallback: operations raise without a CUDA device or library.
"""

from mlkit_b200.checkpoints import load, load_checkpoint, save
from mlkit_b200.conversion import install_transform, quantize, record_transform, rotate_inputs
from mlkit_b200.inference import (
    BenchmarkResult,
    PackedEmbedding,
    PackedLayout,
    PackedLinear,
    benchmark,
    benchmark_model,
    CapturedCall,
    capture,
    fuse_siblings,
    layout_for,
    optimize,
    packed_compatible,
)
from mlkit_b200.models import LayerReport, Model, QModel
from mlkit_b200.quantization import (
    Ctx,
    Grid,
    Q,
    Scaled,
    as_q,
    codec,
    decode_feedback,
    decode_scaled,
    decoder,
    grid,
    int,
    layer_seed,
    nf4,
    pack,
    registered,
    scaled,
    unpack,
)
from mlkit_b200.transforms import hadamard, randomized_transform, rht, structured_transform, transform_factor

__version__ = "0.1.0"

__all__ = [
    "BenchmarkResult", "Ctx", "Grid", "LayerReport", "Model", "PackedEmbedding", "PackedLayout", "PackedLinear",
    "Q", "QModel", "Scaled", "as_q", "benchmark", "benchmark_model", "codec", "decode_feedback", "decode_scaled",
    "CapturedCall", "capture", "decoder", "fuse_siblings", "grid", "hadamard", "install_transform", "int", "layer_seed", "layout_for", "load",
    "load_checkpoint", "nf4", "optimize", "pack", "packed_compatible", "quantize", "randomized_transform",
    "record_transform", "registered", "rht", "rotate_inputs", "save", "scaled", "structured_transform",
    "transform_factor", "unpack",
]
