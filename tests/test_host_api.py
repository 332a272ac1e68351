"""Host-side API (no GPU): bit streams, formats, registry, layouts, factor bases, C ABI surface."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import mlkit_b200 as mk
from mlkit_b200 import _native, transforms
from mlkit_b200 import build as native_build

ROOT = Path(__file__).resolve().parent.parent


def test_bitstream_matches_reference_vectors(golden_bitstream):
    for bits in range(1, 17):
        for count in (0, 1, 7, 17, 64, 200):
            codes = torch.from_numpy(golden_bitstream[f"b{bits}_n{count}_codes"])
            packed = torch.from_numpy(golden_bitstream[f"b{bits}_n{count}_packed"])
            assert torch.equal(mk.pack(codes, bits), packed)
            assert packed.numel() == (count * bits + 7) // 8
            assert torch.equal(mk.unpack(packed, bits, codes.shape).int(), codes)


def test_bitstream_validation_errors():
    with pytest.raises(ValueError, match="capacity"):
        mk.pack(torch.tensor([16]), 4)
    with pytest.raises(ValueError, match="byte count"):
        mk.unpack(torch.zeros(1, dtype=torch.uint8), 4, (4,))
    with pytest.raises(ValueError, match="sixteen"):
        mk.pack(torch.tensor([1]), 17)
    with pytest.raises(TypeError):
        mk.pack(torch.tensor([1.0]), 4)
    with pytest.raises(ValueError, match="uint8"):
        mk.unpack(torch.zeros(1, dtype=torch.int32), 4, (2,))


def build_format(name: str, info: dict, values: np.ndarray):
    if name.startswith("int"):
        return mk.int(info["bits"], group=info["group"], asym=info["asym"], scale=info["scale"])
    if name.startswith("nf4"):
        return mk.nf4(group=info["group"])
    return mk.scaled(mk.grid.values(torch.from_numpy(values), bits=info["bits"]), group=info["group"],
                     scale=info["scale"])


def test_formats_reproduce_reference_codes_and_scales(golden_meta, golden_codecs):
    for name, info in golden_meta["codecs"].items():
        g = lambda field: golden_codecs.get(f"{name}.{field}")
        if name.startswith("e4m3"):
            fmt = mk.scaled(mk.grid.fp("e4m3"), group=info["group"])
        else:
            fmt = build_format(name, info, g("values"))
        q = fmt(torch.from_numpy(g("weight")), mk.Ctx(device="cpu"))
        assert torch.equal(q.params["values"], torch.from_numpy(g("values"))), name
        assert torch.equal(q.params["scales"], torch.from_numpy(g("scales"))), name
        assert torch.equal(q.codes, torch.from_numpy(g("codes"))), name
        if info["asym"]:
            assert torch.equal(q.params["zero"], torch.from_numpy(g("zero"))), name
        assert q.codec == info["codec"] and q.metadata["code_bits"] == info["bits"]
        assert q.metadata["scale_fmt"] == info["metadata"]["scale_fmt"]
        assert q.bits == info["total_bits"], name
        assert torch.equal(q.w, torch.from_numpy(g("decoded"))), name
        assert mk.packed_compatible(q) == info["compatible"]
        assert torch.equal(mk.pack(q.codes, info["bits"]), torch.from_numpy(g("packed")))


def test_layout_table_matches_reference(golden_meta):
    for key, expected in golden_meta["layouts"].items():
        bits, width, group = (int(v) for v in key.split(","))
        layout = mk.layout_for(bits, width, group)
        got = None if layout is None else [layout.bits, layout.bytes_per_word, layout.codes_per_word, layout.tile_words]
        assert got == expected, key
    layout = mk.layout_for(3, 4096, 128)
    assert (layout.tile_codes, layout.row_bytes(4096), layout.tiles_per_row(4096)) == (128, 1536, 32)


def test_packed_compatible_rules():
    q = mk.int(4, group=32)(torch.randn(4, 64))
    assert mk.packed_compatible(q)
    for change in ({"codec": "vector_scaled"}, {"offset": 8}, {"permutation": torch.arange(64)}, {"refit": 48}):
        other = mk.Q(codes=q.codes, params=dict(q.params), decode=q.decode, codec=q.codec, metadata=q.metadata)
        for key, value in change.items():
            if key == "codec":
                other.codec = value
            else:
                other.params[key] = value
        assert not mk.packed_compatible(other)
    wide = mk.int(12, group=32)(torch.randn(4, 64))
    assert not mk.packed_compatible(wide)
    assert mk.packed_compatible(mk.Q(codes=q.codes, params=q.params | {"refit": 64}, decode=q.decode,
                                     codec="feedback", metadata=q.metadata))


def test_codec_registry_contract():
    assert mk.registered("scaled") and mk.registered("feedback") and not mk.registered("nope")
    with pytest.raises(ValueError, match="requires registered codec"):
        mk.decoder("nope")
    with pytest.raises(ValueError, match="already registered"):
        mk.codec("scaled")(lambda codes: codes)
    with pytest.raises(ValueError, match="empty"):
        mk.codec("")(lambda codes: codes)

    @mk.codec("test_identity_codec")
    def identity(codes, **params):
        return codes.float()

    assert mk.decoder("test_identity_codec") is identity


def test_q_contract():
    with pytest.raises(ValueError, match="reconstruction or codes"):
        mk.Q()
    with pytest.raises(ValueError, match="nonnegative"):
        mk.Q(torch.zeros(2, 2), bits=-1)
    q = mk.nf4(group=32)(torch.randn(6, 64))
    moved = q.to("cpu", detach=True)
    assert torch.equal(moved.w, q.w) and moved.codec == "scaled" and q.bpw == q.bits / 384
    with pytest.raises(TypeError):
        mk.as_q(3)


def test_layer_seed_matches_reference(golden_meta):
    for name, (seed, expected) in golden_meta["transforms"]["layer_seed"].items():
        assert mk.layer_seed(name, seed) == expected


def test_factor_bases_match_reference(golden_meta, golden_transforms):
    for order in (12, 20, 28, 44, 76):
        assert torch.equal(transforms.paley_matrix(order), torch.from_numpy(golden_transforms[f"paley{order}"]))
    for width, (factor, power, has_basis) in golden_meta["transforms"]["factors"].items():
        got_factor, got_power, basis = mk.transform_factor(int(width))
        assert (got_factor, got_power, basis is not None) == (factor, power, has_basis), width
        if basis is not None:
            torch.testing.assert_close(basis, torch.from_numpy(golden_transforms[f"basis{factor}"]), rtol=0, atol=1e-7)
    with pytest.raises(ValueError, match="power-of-two"):
        mk.hadamard(torch.randn(3, 12))


def test_restore_layer_widens_fp8_scales_and_refuses_online_quantisers(tmp_path):
    """A layer as the reference's ``save`` writes it with ``scale_fmt="fp8"`` (scales stored as
    float8_e4m3fn, src/mlkit/checkpoints/saving.py:60-69): the loader widens them to fp32 and the
    reconstruction equals the oracle's.  A manifest that asks for online activation or KV-cache
    quantisation is refused instead of being loaded without its quantisers."""
    import json

    from mlkit_b200 import checkpoints
    from oracle import bitstream, codec

    rng = np.random.default_rng(4)
    rows, width, group, bits = 6, 64, 32, 4
    codes = rng.integers(0, 16, size=(rows, width), dtype=np.uint8)
    scales8 = torch.from_numpy((rng.random((rows, width // group), dtype=np.float32) * 0.05 + 0.01)).to(torch.float8_e4m3fn)
    values = codec.int_values(bits)
    tensors = {"layer.codes": torch.from_numpy(bitstream.pack(codes, bits)), "layer.params.scales": scales8,
               "layer.params.values": torch.from_numpy(values)}
    layer = {"codec": "scaled", "shape": [rows, width], "code_bits": bits, "bits": 4.5,
             "params": {"scales": {"tensor": "layer.params.scales", "encoding": None},
                        "values": {"tensor": "layer.params.values", "encoding": None}, "group": {"value": group},
                        "offset": {"value": 0}},
             "metadata": {"scale_fmt": "fp8"}}
    restored = checkpoints.restore_layer(tensors, "layer", layer)
    assert restored.params["scales"].dtype == torch.float32
    expected = codec.decode_scaled(codes, scales8.float().numpy(), values, group)
    assert np.array_equal(restored.w.numpy(), expected)

    manifest = {"format_version": 1, "name": "m", "architecture": "external", "dtype": "float16", "layers": {},
                "activations": {"layer": {"bits": 8}}, "kv": None}
    (tmp_path / "mlkit.json").write_text(json.dumps(manifest))
    with pytest.raises(NotImplementedError, match="online activation"):
        checkpoints.load_checkpoint(tmp_path, model=torch.nn.Linear(4, 4))


def test_hot_path_refuses_cpu_tensors():
    linear = torch.nn.Linear(64, 8)
    q = mk.int(4, group=32)(linear.weight.detach())
    with pytest.raises(ValueError, match="CUDA weights"):
        mk.PackedLinear(linear, q)
    with pytest.raises(ValueError, match="CUDA"):
        mk.rht(torch.randn(2, 64), seed=1)
    with pytest.raises(ValueError, match="backend must be"):
        mk.optimize(linear, backend="fast")


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "mlkit_b200.h").read_text()
    declared = set(re.findall(r"\b(mkb_[a-z_0-9]+)\s*\(", header))
    assert {"mkb_gemv", "mkb_gemv_ex", "mkb_dequant", "mkb_dequant_rows", "mkb_hadamard", "mkb_version",
            "mkb_last_error"} <= declared
    library = ctypes.CDLL(str(native_build.build()))
    for symbol in declared:
        assert hasattr(library, symbol), symbol
    assert set(_native.SIGNATURES) == declared
    assert _native.library().mkb_version() >= 100
    # argument validation runs before any CUDA call, so it is testable without a GPU
    status = _native.library().mkb_gemv_ex(None, None, None, None, None, None, None, 9, 1, 128, 128, 4, 16, 0, 0,
                                           64, 1, 0, 0.0, 0, None)
    assert status == -2 and b"outside 1..8" in _native.library().mkb_last_error()


def test_size_queries_need_no_gpu():
    library = _native.library()
    assert library.mkb_gemm_workspace_bytes(64, 14336, 4096) > 0
    assert library.mkb_gemm_workspace_bytes(129, 14336, 4096) == 0      # more rows than one launch takes
    assert library.mkb_gemm_workspace_bytes(64, 14336, 4100) == 0       # K not a multiple of the group
    # flagged packets: four bytes of flags per four bytes of data, two parities, behind a fixed header
    small, large = library.mkb_peer_buffer_bytes(1, 8192, 8), library.mkb_peer_buffer_bytes(8, 8192, 8)
    assert small > 0 and large - small == 2 * 8 * 7 * 8192 * 4
    assert library.mkb_peer_buffer_bytes(9, 8192, 8) == 0 and library.mkb_peer_buffer_bytes(8, 8192, 17) == 0
    assert library.mkb_gemv_static_scratch_bytes() == 8 << 20
    assert library.mkb_gemv_workspace_bytes(8, 14336, 4096, 4) > 0


def test_route_rules_of_the_wrappers():
    from mlkit_b200 import kernels

    scales = torch.empty(0, dtype=torch.float16)
    layer = dict(width=4096, group=128, bits=4, dtype=torch.float16, scales=scales, zeros=None, integer_grid=True,
                 grid_minimum=-8.0, levels=16)
    assert kernels.gemm_supported(17, **layer) and kernels.gemm_supported(128, **layer)
    assert not kernels.gemm_supported(129, **layer)
    assert not kernels.gemm_supported(17, **{**layer, "bits": 3})
    assert not kernels.gemm_supported(17, **{**layer, "group": 64})
    assert not kernels.gemm_supported(17, **{**layer, "dtype": torch.bfloat16})
    assert not kernels.gemm_supported(17, **{**layer, "zeros": scales})
    assert not kernels.gemm_supported(17, **{**layer, "grid_minimum": 0.0})
    # profitable against reconstruct + library GEMM: always up to 32 rows, above that for large weights only
    assert kernels.gemm_supported(32, outputs=1024, **layer)
    assert not kernels.gemm_supported(64, outputs=1024, **layer)
    assert kernels.gemm_supported(64, outputs=8192, **layer)
    # rotation on load: power-of-two widths of at least one warp's span, activations that fit shared memory
    assert kernels.rotated_matvec_supported(1, 4096, torch.float16)
    assert kernels.rotated_matvec_supported(4, 4096, torch.float16)
    assert not kernels.rotated_matvec_supported(4, 4096, torch.float16, profitable=True)
    assert kernels.rotated_matvec_supported(1, 4096, torch.float16, profitable=True)
    assert not kernels.rotated_matvec_supported(1, 14336, torch.float16)      # factor width
    assert not kernels.rotated_matvec_supported(1, 256, torch.float16)
    assert not kernels.rotated_matvec_supported(8, 4096, torch.float16)       # 128 KB of fp32 activations
    assert not kernels.rotated_matvec_supported(1, 4096, torch.bfloat16)
    assert not kernels.rotated_matvec_supported(9, 512, torch.float16)
