"""The numpy oracle against vectors produced by the reference library itself (CPU)."""

import numpy as np
import pytest

from oracle import bitstream, codec, matvec, transforms


def test_bitstream_matches_reference(golden_bitstream):
    for bits in range(1, 17):
        for count in (0, 1, 7, 17, 64, 200):
            codes = golden_bitstream[f"b{bits}_n{count}_codes"]
            packed = golden_bitstream[f"b{bits}_n{count}_packed"]
            assert np.array_equal(bitstream.pack(codes, bits), packed)
            assert np.array_equal(bitstream.unpack(packed, bits, codes.shape).astype(np.int32), codes)


def test_bitstream_validation():
    with pytest.raises(ValueError, match="capacity"):
        bitstream.pack(np.array([16]), 4)
    with pytest.raises(ValueError, match="byte count"):
        bitstream.unpack(np.zeros(1, dtype=np.uint8), 4, (4,))
    with pytest.raises(TypeError):
        bitstream.pack(np.array([1.0]), 4)


def test_layout_table_matches_reference(golden_meta):
    for key, expected in golden_meta["layouts"].items():
        bits, width, group = (int(v) for v in key.split(","))
        got = bitstream.fused_layout(bits, width, group)
        assert (None if got is None else list(got)) == expected, key


def test_decode_and_matvec_match_reference(golden_meta, golden_codecs):
    for name, info in golden_meta["codecs"].items():
        g = lambda field: golden_codecs.get(f"{name}.{field}")
        codes = bitstream.unpack(g("packed"), info["bits"], (info["rows"], info["width"]))
        assert np.array_equal(codes, g("codes")), name
        decoded = codec.decode_scaled(codes, g("scales"), g("values"), info["group"], g("zero"))
        assert np.array_equal(decoded, g("decoded")), name
        dense16 = codec.reconstruct_weight(codes, g("scales").astype(np.float16), g("values"),
                                           info["group"], g("zero16"))
        assert np.array_equal(dense16, g("dense16")), name
        y = matvec.reconstruct_then_matmul(g("x"), g("packed"), g("scales").astype(np.float16),
                                           g("values"), info["group"], info["bits"],
                                           (info["rows"], info["width"]), zero16=g("zero16"))
        assert matvec.relative_l2(y, g("y")) < 1e-6, name


def test_rtn_encode_matches_reference(golden_meta, golden_codecs):
    for name, info in golden_meta["codecs"].items():
        g = lambda field: golden_codecs.get(f"{name}.{field}")
        codes, scales, zero = codec.rtn_encode(
            g("weight"), g("values"), info["group"], integer=info["integer"],
            scale=info["scale"], asym=info["asym"])
        assert np.array_equal(scales, g("scales")), name
        assert np.array_equal(codes, g("codes")), name
        if info["asym"]:
            assert np.array_equal(zero, g("zero")), name


def test_linspace_restatement(golden_meta):
    expected = np.array(golden_meta["linspace_0p5_1_20"], dtype=np.float32)
    assert np.array_equal(codec.torch_like_linspace(0.5, 1.0, 20), expected)


def test_fwht_bit_exact(golden_transforms):
    for width in (1, 2, 4, 8, 16, 32, 64, 128, 512, 2048, 4096):
        x = golden_transforms[f"fwht{width}.x"]
        assert np.array_equal(transforms.hadamard(x, normalize=False), golden_transforms[f"fwht{width}.raw"])
        assert np.array_equal(transforms.hadamard(x), golden_transforms[f"fwht{width}.y"])
    with pytest.raises(ValueError, match="power-of-two"):
        transforms.hadamard(np.zeros((3, 12), dtype=np.float32))


def test_factor_bases(golden_meta, golden_transforms):
    for order in (12, 20, 28, 44, 76):
        assert np.array_equal(transforms.paley_matrix(order), golden_transforms[f"paley{order}"])
    for width, (factor, power, has_basis) in golden_meta["transforms"]["factors"].items():
        got_factor, got_power, basis = transforms.transform_factor(int(width))
        assert (got_factor, got_power, basis is not None) == (factor, power, has_basis), width
        if basis is not None:
            np.testing.assert_allclose(basis, golden_transforms[f"basis{factor}"], rtol=0, atol=1e-7)


def test_structured_and_randomized_transforms(golden_meta, golden_transforms):
    for width in (7, 12, 20, 28, 96, 896, 4864, 14336):
        x = golden_transforms[f"structured{width}.x"]
        np.testing.assert_allclose(transforms.structured_transform(x),
                                   golden_transforms[f"structured{width}.y"], rtol=0, atol=2e-6)
        np.testing.assert_allclose(transforms.structured_transform(x, inverse=True),
                                   golden_transforms[f"structured{width}.inverse"], rtol=0, atol=2e-6)
    for width in golden_meta["transforms"]["seeds"]:
        x = golden_transforms[f"rht{width}.x"]
        signs = golden_transforms[f"rht{width}.signs"]
        scale = np.abs(golden_transforms[f"rht{width}.y"]).max()
        np.testing.assert_allclose(transforms.randomized_transform(x, signs),
                                   golden_transforms[f"rht{width}.y"], rtol=0, atol=2e-6 * scale)
        np.testing.assert_allclose(transforms.randomized_transform(x, signs, inverse=True),
                                   golden_transforms[f"rht{width}.inverse"], rtol=0, atol=2e-6 * scale)
