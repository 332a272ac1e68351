"""GPU parity: every kernel, called through the C ABI, against the numpy oracle and the golden vectors.

Bit-exact for codes and dequantised weights; relative L2 <= 2e-3 for the matvec and the transforms
(the tolerance the hot-path specification states); tighter where the arithmetic allows it.
"""

import numpy as np
import pytest
import torch

from oracle import bitstream, codec, matvec, transforms
from tests import helpers

pytestmark = pytest.mark.gpu
TOLERANCE = 2e-3


def dev(array, dtype=None):
    if array is None:
        return None
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    return tensor.cuda() if dtype is None else tensor.to(dtype).cuda()


def run_matvec(layer, x, kernel="auto", bias=None):
    from mlkit_b200 import kernels

    values = dev(layer["values"])
    integer, low = kernels.integer_grid_of(values)
    out = torch.empty((x.shape[0], layer["rows"]), dtype=torch.float16, device="cuda")
    kernels.packed_matvec(dev(x), dev(layer["packed"]), dev(layer["scales16"]), values, dev(layer["zero16"]),
                          dev(bias), out, group=layer["group"], bits=layer["bits"], integer_grid=integer,
                          grid_minimum=low, kernel=kernel)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def oracle_matvec(layer, x, bias=None):
    return matvec.reconstruct_then_matmul(x, layer["packed"], layer["scales16"], layer["values"], layer["group"],
                                          layer["bits"], (layer["rows"], layer["width"]), zero16=layer["zero16"],
                                          bias=bias)


# ---------------------------------------------------------------- dequantisation (bit-exact)
def test_dequant_matches_golden_vectors(golden_meta, golden_codecs):
    from mlkit_b200 import kernels

    for name, info in golden_meta["codecs"].items():
        g = lambda field: golden_codecs.get(f"{name}.{field}")
        zero16 = g("zero16")
        weight, codes = kernels.dequantize(
            dev(g("packed")), dev(g("scales").astype(np.float16)), dev(g("values")), dev(zero16),
            shape=(info["rows"], info["width"]), group=info["group"], bits=info["bits"],
            dtype=torch.float16, codes=True)
        assert np.array_equal(codes.cpu().numpy(), g("codes")), name
        assert np.array_equal(weight.cpu().numpy(), g("dense16")), name
        full, _ = kernels.dequantize(
            dev(g("packed")), dev(g("scales")), dev(g("values")), dev(g("zero")),
            shape=(info["rows"], info["width"]), group=info["group"], bits=info["bits"], dtype=torch.float32)
        assert np.array_equal(full.cpu().numpy(), g("decoded")), name


@pytest.mark.parametrize("bits", range(1, 9))
@pytest.mark.parametrize("shape,group", [((7, 37), 5), ((1, 1), 1), ((33, 130), 32), ((5, 8), 8), ((64, 256), 96)])
@pytest.mark.parametrize("zeros", [False, True])
def test_dequant_every_width_and_ragged_shape(bits, shape, group, zeros):
    from mlkit_b200 import kernels

    layer = helpers.random_layer(*shape, bits, group, seed=bits, zeros=zeros)
    expected = codec.reconstruct_weight(layer["codes"], layer["scales16"], layer["values"], group, layer["zero16"])
    for dtype, storage in ((torch.float16, np.float16), (torch.float32, np.float32)):
        weight, codes = kernels.dequantize(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]),
                                           dev(layer["zero16"]), shape=shape, group=group, bits=bits, dtype=dtype,
                                           codes=True)
        assert np.array_equal(codes.cpu().numpy(), layer["codes"])
        reference = codec.reconstruct_weight(layer["codes"], layer["scales16"], layer["values"], group,
                                             layer["zero16"], storage=storage)
        assert np.array_equal(weight.cpu().numpy(), reference)
    assert expected.dtype == np.float16
    bf16, _ = kernels.dequantize(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]),
                                 dev(layer["zero16"]), shape=shape, group=group, bits=bits, dtype=torch.bfloat16)
    full = codec.decode_scaled(layer["codes"], layer["scales16"].astype(np.float32), layer["values"], group,
                               None if layer["zero16"] is None else layer["zero16"].astype(np.float32))
    assert torch.equal(bf16.cpu(), torch.from_numpy(full).to(torch.bfloat16))


def test_dequant_empty_and_codes_only():
    from mlkit_b200 import kernels

    weight, codes = kernels.dequantize(torch.empty(0, dtype=torch.uint8, device="cuda"),
                                       torch.empty((0, 0), dtype=torch.float16, device="cuda"),
                                       torch.zeros(16, device="cuda"), None, shape=(0, 64), group=32, bits=4,
                                       codes=True)
    assert weight.shape == (0, 64) and codes.shape == (0, 64)
    layer = helpers.random_layer(9, 21, 3, 7, seed=4)
    _, codes = kernels.dequantize(dev(layer["packed"]), None, None, None, shape=(9, 21), group=7, bits=3,
                                  dtype=None, codes=True)
    assert np.array_equal(codes.cpu().numpy(), layer["codes"])


def test_dequant_rows_gathers_like_an_embedding():
    from mlkit_b200 import kernels

    for bits, width, group in ((4, 130, 32), (3, 64, 32), (8, 96, 32), (4, 4096, 128)):
        layer = helpers.random_layer(50, width, bits, group, seed=bits, zeros=bits == 3)
        dense = codec.reconstruct_weight(layer["codes"], layer["scales16"], layer["values"], group, layer["zero16"])
        rows = np.array([3, 3, 49, 0, 17], dtype=np.int64)
        out = kernels.dequantize_rows(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]),
                                      dev(layer["zero16"]), dev(rows), shape=(50, width), group=group, bits=bits,
                                      dtype=torch.float16)
        assert np.array_equal(out.cpu().numpy(), dense[rows])


# ---------------------------------------------------------------- encoding on the device (bit-exact)
def test_device_rtn_encode_matches_the_reference_vectors(golden_meta, golden_codecs):
    """``mkb_rtn_encode`` through the format objects: codes, scales and the packed stream of every
    symmetric absolute-maximum case of the golden set equal what the reference produced."""
    import mlkit_b200 as mk
    from tests.test_host_api import build_format

    checked = 0
    for name, info in golden_meta["codecs"].items():
        if info["asym"] or info["scale"] != "absmax":
            continue
        if name.startswith("e4m3"):
            fmt = mk.scaled(mk.grid.fp("e4m3"), group=info["group"])
        else:
            fmt = build_format(name, info, golden_codecs[f"{name}.values"])
        weight = torch.from_numpy(golden_codecs[f"{name}.weight"]).cuda()
        q = fmt(weight.float(), mk.Ctx(name, device="cuda"))
        assert q.codes.is_cuda and q.codes.dtype == torch.uint8
        assert np.array_equal(q.codes.cpu().numpy(), golden_codecs[f"{name}.codes"]), name
        assert np.array_equal(q.params["scales"].cpu().numpy(), golden_codecs[f"{name}.scales"]), name
        assert np.array_equal(mk.pack(q.codes, info["bits"]).cpu().numpy(), golden_codecs[f"{name}.packed"]), name
        checked += 1
    assert checked >= 8


@pytest.mark.parametrize("kind,bits,group,width", [("int", 4, 128, 4096), ("int", 3, 128, 1024), ("int", 8, 128, 512),
                                                    ("int", 2, 64, 320), ("nf4", 4, 64, 4096), ("codebook3", 3, 64, 1000),
                                                    ("int", 4, 128, 200), ("int", 5, 64, 256)])
def test_device_rtn_encode_equals_the_tensor_route(kind, bits, group, width):
    """The kernel against the torch-op route of the same format on the same device: codes, scales and
    the packed stream, including a trailing partial group (1000 = 15 x 64 + 40, 200 = 128 + 72)."""
    import mlkit_b200 as mk
    from mlkit_b200 import kernels

    values, integer = helpers.grid_values(kind, bits)
    grid = mk.grid.int(bits) if integer else mk.grid.values(torch.from_numpy(values), bits=bits)
    fmt = mk.scaled(grid, group=group)
    weight = (torch.randn(300, width, device="cuda") * 0.02).half()
    weight[5, :group] = 0                       # an all-zero group: the scale floor
    weight[7, 3] = 30.0                         # a large outlier
    levels = grid.values.cuda()
    packed, scales16, codes = kernels.rtn_encode(weight, levels, group=group, bits=bits, integer_grid=integer,
                                                 low=fmt._low, high=fmt._high, reciprocal=fmt._reciprocal, codes=True)
    expected = fmt(weight.float().cpu())        # the tensor route (CPU tensors never take the kernel)
    assert torch.equal(codes.cpu(), expected.codes)
    assert torch.equal(scales16.float().cpu(), expected.params["scales"])
    assert torch.equal(packed.cpu(), mk.pack(expected.codes, bits))


# ---------------------------------------------------------------- matvec (<= 2e-3 relative L2)
def test_matvec_matches_golden_vectors(golden_meta, golden_codecs):
    for name, info in golden_meta["codecs"].items():
        g = lambda field: golden_codecs.get(f"{name}.{field}")
        layer = {"rows": info["rows"], "width": info["width"], "bits": info["bits"], "group": info["group"],
                 "values": g("values"), "packed": g("packed"), "scales16": g("scales").astype(np.float16),
                 "zero16": g("zero16")}
        kernels_to_try = ["scalar", "auto"]
        if info["width"] % 128 == 0 and info["group"] % 32 == 0:
            kernels_to_try.append("tiled")
        for kernel in kernels_to_try:
            y = run_matvec(layer, g("x"), kernel)
            assert matvec.relative_l2(y, g("y")) < TOLERANCE, (name, kernel)


@pytest.mark.parametrize("rows_in", [1, 2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("kernel", ["scalar", "tiled", "tmem", "bulk", "stream"])
def test_matvec_int4_g128_every_row_count(rows_in, kernel):
    layer = helpers.make_layer(1000, 1024, 4, 128, seed=3)   # 1000 rows: a ragged last row tile
    x = helpers.activations(rows_in, 1024, seed=rows_in)
    bias = (np.random.default_rng(5).standard_normal(1000) * 0.1).astype(np.float16)
    for b in (None, bias):
        error = matvec.relative_l2(run_matvec(layer, x, kernel, b), oracle_matvec(layer, x, b))
        assert error < TOLERANCE, error
        assert error < 5e-4   # fp32 accumulation leaves only the fp16 rounding of the output


TILED_CODECS = [
    ("int", 2, 128), ("int", 4, 128), ("int", 8, 128), ("int", 3, 128), ("int", 5, 64), ("int", 6, 32),
    ("int", 7, 64), ("int", 4, 32), ("int", 4, 64), ("int", 2, 64), ("int", 8, 32), ("int", 4, 256),
    ("nf4", 4, 64), ("codebook3", 3, 64), ("nf4", 4, 128),
]


@pytest.mark.parametrize("kind,bits,group", TILED_CODECS)
@pytest.mark.parametrize("rows_in", [1, 8])
@pytest.mark.parametrize("asym", [False, True])
def test_matvec_tiled_every_codec(kind, bits, group, rows_in, asym):
    if asym and kind != "int":
        pytest.skip("offsets are an integer-grid feature of the formats")
    layer = helpers.make_layer(272, 768, bits, group, kind, seed=bits + group, asym=asym)
    x = helpers.activations(rows_in, 768, seed=2)
    expected = oracle_matvec(layer, x)
    for kernel in ("tiled", "scalar"):
        assert matvec.relative_l2(run_matvec(layer, x, kernel), expected) < TOLERANCE, kernel
    # the streaming kernel: integer grids of 2, 4, 8 bits with groups of 128; tables of 3- and 4-bit
    # codes with groups of 64 or 128; nothing with offsets
    streams = not asym and ((kind == "int" and bits in (2, 4, 8) and group == 128) or (bits in (3, 4) and group in (64, 128)))
    if streams:
        got = run_matvec(layer, x, "stream")
        assert matvec.relative_l2(got, expected) < TOLERANCE
        assert np.array_equal(got, run_matvec(layer, x, "stream"))
    else:
        with pytest.raises(ValueError, match="streaming kernel"):
            run_matvec(layer, x, "stream")


@pytest.mark.parametrize("bits,width,group", [(1, 64, 16), (3, 40, 8), (5, 72, 24), (7, 64, 64), (4, 130, 32),
                                              (6, 36, 12), (2, 20, 4), (8, 19, 19)])
def test_matvec_scalar_covers_odd_layouts(bits, width, group):
    if bitstream.fused_layout(bits, width, group) is None and (width % bitstream.word_geometry(bits)[1]
                                                               or group % bitstream.word_geometry(bits)[1]):
        pytest.skip("layout splits a packing word: the module routes it to the dense path")
    layer = helpers.random_layer(23, width, bits, group, seed=width, zeros=bool(bits & 1))
    x = helpers.activations(3, width, seed=9)
    assert matvec.relative_l2(run_matvec(layer, x, "scalar"), oracle_matvec(layer, x)) < TOLERANCE


def test_matvec_other_dtypes_use_the_scalar_kernel():
    """fp32 / bf16 activations and scales: the weight is used unrounded, as the reference kernel does
    (kernels/packed_linear.py:162-166), so the yardstick is the fp32 reconstruction."""
    from mlkit_b200 import kernels

    layer = helpers.make_layer(100, 256, 4, 64, seed=8)
    x32 = helpers.activations(5, 256, seed=3).astype(np.float32)
    dense32 = codec.decode_scaled(layer["codes"], layer["scales16"].astype(np.float32), layer["values"], 64)
    expected = x32 @ dense32.T
    values = dev(layer["values"])
    for x_dtype, scale_dtype, bound in ((torch.float32, torch.float32, 1e-5), (torch.float32, torch.float16, 1e-5),
                                        (torch.bfloat16, torch.bfloat16, 8e-3)):
        x = torch.from_numpy(x32).to(x_dtype).cuda()
        scales = torch.from_numpy(layer["scales16"]).to(scale_dtype).cuda()
        out = torch.empty((5, 100), dtype=x_dtype, device="cuda")
        kernels.packed_matvec(x, dev(layer["packed"]), scales, values, None, None, out, group=64, bits=4)
        assert matvec.relative_l2(out.float().cpu().numpy(), expected) < bound


@pytest.mark.parametrize("group", [128, 256, 512])
def test_matvec_tmem_groups_bias_and_ragged_rows(group):
    layer = helpers.make_layer(300, 1536, 4, group, seed=group)
    bias = (np.random.default_rng(2).standard_normal(300) * 0.1).astype(np.float16)
    for rows_in in (1, 5, 8):
        x = helpers.activations(rows_in, 1536, seed=rows_in, outliers=True)
        expected = oracle_matvec(layer, x, bias)
        assert matvec.relative_l2(run_matvec(layer, x, "tmem", bias), expected) < TOLERANCE


@pytest.mark.parametrize("group", [128, 256, 512])
@pytest.mark.parametrize("width", [1536, 2304, 5120, 11008 - 11008 % 256])
def test_matvec_bulk_groups_bias_ragged_rows_and_splits(group, width):
    """The TMA-fed kernel: widths that need 1, 2 or 3 K slabs, a last slab that is partly empty, a
    ragged last row tile, a bias, and scale groups wider than a chunk."""
    layer = helpers.make_layer(300, width, 4, group, seed=group + width)
    bias = (np.random.default_rng(2).standard_normal(300) * 0.1).astype(np.float16)
    for rows_in in (1, 3, 8):
        x = helpers.activations(rows_in, width, seed=rows_in, outliers=True)
        expected = oracle_matvec(layer, x, bias)
        first = run_matvec(layer, x, "bulk", bias)
        assert matvec.relative_l2(first, expected) < TOLERANCE
        assert np.array_equal(first, run_matvec(layer, x, "bulk", bias))   # fixed summation order


STREAM_SHAPES = [(300, 1536), (4864, 896), (272, 768), (1000, 1024), (48, 14336), (2368, 8192), (16, 128), (10, 384),
                 (8192, 1024), (8192, 3584), (1280, 8192), (7168, 8192)]


@pytest.mark.parametrize("rows,width", STREAM_SHAPES)
def test_matvec_stream_shapes_bias_ragged_rows_and_splits(rows, width):
    """The streaming kernel: one and two k-tiles per warp (odd and even K / 128), K split over one to
    eight CTAs of a cluster, several row tiles per visit, a partial last row tile, a bias; the
    tensor-parallel shard shapes of the 70B-shaped decoder are among them."""
    layer = helpers.make_layer(rows, width, 4, 128, seed=rows + width)
    bias = (np.random.default_rng(2).standard_normal(rows) * 0.1).astype(np.float16)
    for rows_in in (1, 3, 8):
        x = helpers.activations(rows_in, width, seed=rows_in, outliers=True)
        expected = oracle_matvec(layer, x, bias)
        first = run_matvec(layer, x, "stream", bias)
        assert matvec.relative_l2(first, expected) < TOLERANCE
        assert np.array_equal(first, run_matvec(layer, x, "stream", bias))   # fixed summation order


@pytest.mark.parametrize("kind,bits,group", [("int", 2, 128), ("int", 8, 128), ("int", 3, 128), ("nf4", 4, 64),
                                             ("nf4", 4, 128), ("codebook3", 3, 64), ("int", 4, 64), ("int", 5, 128),
                                             ("int", 6, 128), ("int", 7, 128)])
@pytest.mark.parametrize("rows,width", [(300, 1536), (4864, 896), (48, 8192), (1000, 1024)])
def test_matvec_stream_every_codec_bias_ragged_rows_and_splits(kind, bits, group, rows, width):
    """Every codec of the streaming kernel on shapes with one and two k-tiles per warp, K split over a
    cluster, a partial last row tile and a bias."""
    layer = helpers.make_layer(rows, width, bits, group, kind, seed=bits + group + rows)
    bias = (np.random.default_rng(2).standard_normal(rows) * 0.1).astype(np.float16)
    for rows_in in (1, 8):
        x = helpers.activations(rows_in, width, seed=rows_in, outliers=True)
        expected = oracle_matvec(layer, x, bias)
        first = run_matvec(layer, x, "stream", bias)
        assert matvec.relative_l2(first, expected) < TOLERANCE
        assert np.array_equal(first, run_matvec(layer, x, "stream", bias))


def test_matvec_stream_refuses_what_it_does_not_cover():
    layer = helpers.make_layer(64, 512, 4, 32, seed=1)    # groups narrower than 64 codes
    with pytest.raises(ValueError, match="streaming kernel"):
        run_matvec(layer, helpers.activations(1, 512), "stream")
    layer = helpers.make_layer(64, 512, 4, 128, seed=1, asym=True)   # offsets
    with pytest.raises(ValueError, match="streaming kernel"):
        run_matvec(layer, helpers.activations(1, 512), "stream")


def test_matvec_bulk_refuses_what_it_does_not_cover():
    layer = helpers.make_layer(64, 640, 4, 128, seed=1)   # 640 codes: not a whole number of 256-code chunks
    with pytest.raises(ValueError, match="TMA-fed kernel"):
        run_matvec(layer, helpers.activations(1, 640), "bulk")
    layer = helpers.make_layer(64, 512, 4, 64, seed=1)    # groups narrower than 128 codes
    with pytest.raises(ValueError, match="TMA-fed kernel"):
        run_matvec(layer, helpers.activations(1, 512), "bulk")


def test_matvec_tmem_refuses_what_it_does_not_cover():
    layer = helpers.make_layer(64, 640, 4, 128, seed=1)   # 640 codes: not a whole number of 512-code slabs
    with pytest.raises(ValueError, match="tensor-memory kernel"):
        run_matvec(layer, helpers.activations(1, 640), "tmem")


def test_matvec_rejects_bad_arguments():
    from mlkit_b200 import kernels

    layer = helpers.random_layer(16, 256, 4, 128)
    x = dev(helpers.activations(9, 256))
    out = torch.empty((9, 16), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="outside 1..8"):
        kernels.packed_matvec(x, dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None, None,
                              out, group=128, bits=4)
    with pytest.raises(ValueError, match="packing word"):
        kernels.packed_matvec(x[:1, :255].contiguous(), dev(layer["packed"]), dev(layer["scales16"]),
                              dev(layer["values"])[:8].contiguous(), None, None, out[:1].contiguous(), group=128,
                              bits=3)


FULL_SIZE_CODECS = [("int", 2, 128), ("int", 3, 128), ("int", 8, 128), ("nf4", 4, 64), ("codebook3", 3, 64)]


@pytest.mark.parametrize("kind,bits,group", FULL_SIZE_CODECS)
def test_matvec_codec_sweep_full_size(kind, bits, group):
    """The codec sweep of the baseline at its own size, one 4096 -> 14336 linear, one and eight rows:
    bit-exact dequantisation and the matvec within 2e-3 of reconstruct-then-matmul.  (Scales by absolute
    maximum here; the MSE-fitted codebook scales are covered at a smaller size, the search being slow
    on the host and the kernels blind to how a scale was chosen.)"""
    from mlkit_b200 import kernels

    rows, width = 14336, 4096
    layer = helpers.make_layer(rows, width, bits, group, kind, seed=bits + group)
    dense, codes = kernels.dequantize(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None,
                                      shape=(rows, width), group=group, bits=bits, codes=True)
    assert np.array_equal(codes.cpu().numpy(), layer["codes"])
    reference = codec.reconstruct_weight(layer["codes"], layer["scales16"], layer["values"], group)
    assert np.array_equal(dense.cpu().numpy(), reference)
    for rows_in in (1, 8):
        x = helpers.activations(rows_in, width, seed=rows_in)
        expected = x.astype(np.float32) @ reference.astype(np.float32).T
        y = run_matvec(layer, x, "auto")
        assert matvec.relative_l2(y, expected) < TOLERANCE
        assert np.array_equal(y, run_matvec(layer, x, "auto"))


def test_matvec_codebook_with_fitted_scales():
    layer = helpers.make_layer(512, 4096, 3, 64, "codebook3", seed=9, scale="mse")
    for rows_in in (1, 8):
        x = helpers.activations(rows_in, 4096, seed=rows_in)
        assert matvec.relative_l2(run_matvec(layer, x, "auto"), oracle_matvec(layer, x)) < TOLERANCE


def test_matvec_auto_falls_back_when_the_tiled_kernel_does_not_fit():
    """A 256-entry table codec at K = 28672 and eight rows needs more shared memory than an SM has in
    the tiled kernel: AUTO must take the scalar kernel instead of refusing the call."""
    layer = helpers.random_layer(64, 28672, 8, 128, seed=2)
    x = helpers.activations(8, 28672, seed=3)
    assert matvec.relative_l2(run_matvec(layer, x, "auto"), oracle_matvec(layer, x)) < TOLERANCE


LLAMA8B = {"q": (4096, 4096), "k": (1024, 4096), "o": (4096, 4096), "gate": (14336, 4096), "down": (4096, 14336)}


@pytest.mark.parametrize("name", list(LLAMA8B))
def test_matvec_llama8b_shapes_full_size(name):
    rows, width = LLAMA8B[name]
    layer = helpers.make_layer(rows, width, 4, 128, seed=len(name))
    from mlkit_b200 import kernels

    dense, codes = kernels.dequantize(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None,
                                      shape=(rows, width), group=128, bits=4, codes=True)
    assert np.array_equal(codes.cpu().numpy(), layer["codes"])
    reference = codec.reconstruct_weight(layer["codes"], layer["scales16"], layer["values"], 128)
    assert np.array_equal(dense.cpu().numpy(), reference)
    for rows_in in (1, 2, 4, 8):
        x = helpers.activations(rows_in, width, seed=rows_in)
        expected = x.astype(np.float32) @ reference.astype(np.float32).T
        y = run_matvec(layer, x, "auto")
        assert matvec.relative_l2(y, expected) < TOLERANCE
        again = run_matvec(layer, x, "auto")
        assert np.array_equal(y, again)   # fixed summation order: run-to-run identical
        through_tmem = run_matvec(layer, x, "tmem")   # the tcgen05 kernel on the same inputs
        assert matvec.relative_l2(through_tmem, expected) < TOLERANCE
        assert np.array_equal(through_tmem, run_matvec(layer, x, "tmem"))
        through_stream = run_matvec(layer, x, "stream")   # the streaming kernel (what "auto" takes here)
        assert matvec.relative_l2(through_stream, expected) < TOLERANCE
        assert np.array_equal(through_stream, run_matvec(layer, x, "stream"))
        through_bulk = run_matvec(layer, x, "bulk")   # the TMA-fed kernel on the same inputs
        assert matvec.relative_l2(through_bulk, expected) < TOLERANCE
        assert np.array_equal(through_bulk, run_matvec(layer, x, "bulk"))
        # linearity, a size-independent property: f(2x) == 2 f(x) exactly in binary floating point
        # (products and fp32 sums scale by two without rounding)
        # (outputs in the fp16 subnormal range are excluded: their rounding step does not scale)
        doubled = run_matvec(layer, (x * np.float16(2)).astype(np.float16), "auto")
        normal = np.abs(y.astype(np.float32)) >= 2.0**-13
        assert np.array_equal(doubled[normal], (y * np.float16(2)).astype(np.float16)[normal])
        # tiny activations keep their precision (no operand is pushed into the fp16 subnormal range)
        tiny = run_matvec(layer, (x * np.float16(2.0**-10)).astype(np.float16), "auto")
        assert matvec.relative_l2(tiny.astype(np.float32) * 1024, expected) < TOLERANCE


# ---------------------------------------------------------------- transforms
def run_transform(x, signs, dtype, inverse=False):
    from mlkit_b200 import kernels

    width = x.shape[-1]
    factor, power, basis = transforms.transform_factor(width)
    out = kernels.structured_transform(dev(x, dtype), factor=factor, power=power, basis=dev(basis),
                                       signs=dev(signs), inverse=inverse)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


def test_fwht_bit_exact_against_stagewise_golden(golden_transforms):
    from mlkit_b200 import kernels

    for width in (1, 2, 4, 8, 16, 32, 64, 128, 512, 2048, 4096):
        x = golden_transforms[f"fwht{width}.x"]
        raw = kernels.structured_transform(dev(x), factor=1, power=width, normalize=False)
        assert np.array_equal(raw.cpu().numpy(), golden_transforms[f"fwht{width}.raw"]), width
        scaled = kernels.structured_transform(dev(x), factor=1, power=width)
        assert np.array_equal(scaled.cpu().numpy(), transforms.hadamard(x, by_multiply=True)), width
        np.testing.assert_allclose(scaled.cpu().numpy(), golden_transforms[f"fwht{width}.y"], rtol=2e-7, atol=0)


def test_structured_and_randomized_transform_golden(golden_meta, golden_transforms):
    for width in (7, 12, 20, 28, 96, 896, 4864, 14336):
        x = golden_transforms[f"structured{width}.x"]
        for inverse, key in ((False, "y"), (True, "inverse")):
            got = run_transform(x, None, torch.float32, inverse)
            assert matvec.relative_l2(got, golden_transforms[f"structured{width}.{key}"]) < 1e-6, width
    for width in golden_meta["transforms"]["seeds"]:
        x, signs = golden_transforms[f"rht{width}.x"], golden_transforms[f"rht{width}.signs"]
        for inverse, key in ((False, "y"), (True, "inverse")):
            expected = golden_transforms[f"rht{width}.{key}"]
            assert matvec.relative_l2(run_transform(x, signs, torch.float32, inverse), expected) < 1e-6
            half = run_transform(x, signs, torch.float16, inverse)
            assert matvec.relative_l2(half, expected) < TOLERANCE
            assert np.array_equal(half, run_transform(x, signs, torch.float32, inverse).astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("width", [4096, 14336, 8192, 28672])
@pytest.mark.parametrize("rows", [1, 8])
def test_rotated_matvec_path(width, rows):
    """Outlier activations, sign flip + transform, then the packed matvec of a pre-rotated weight."""
    rng = np.random.default_rng(width)
    signs = (rng.integers(0, 2, width) * 2 - 1).astype(np.int8)
    x = helpers.activations(rows, width, seed=width, outliers=True)
    rotated = run_transform(x, signs, torch.float16)
    expected = transforms.randomized_transform(x.astype(np.float32), signs, by_multiply=True)
    assert matvec.relative_l2(rotated, expected) < TOLERANCE
    out_rows = 256
    weight = (rng.standard_normal((out_rows, width), dtype=np.float32) * np.float32(0.02))
    turned = transforms.randomized_transform(weight, signs).astype(np.float16).astype(np.float32)
    values = codec.int_values(4)
    codes, scales, _ = codec.rtn_encode(turned, values, 128, integer=True)
    layer = {"rows": out_rows, "width": width, "bits": 4, "group": 128, "values": values,
             "packed": bitstream.pack(codes, 4), "scales16": scales.astype(np.float16), "zero16": None}
    y = run_matvec(layer, rotated.astype(np.float16), "auto")
    expected_y = oracle_matvec(layer, expected.astype(np.float16))
    assert matvec.relative_l2(y, expected_y) < TOLERANCE
    # the rotation is function preserving: (W R^T)(R x) ~ W x up to quantisation error of W
    plain = x.astype(np.float32) @ weight.T
    assert matvec.relative_l2(y, plain) < 0.2


@pytest.mark.parametrize("kernel", ["tiled", "stream", "auto"])
@pytest.mark.parametrize("rows_in", [1, 5, 8])
def test_matvec_gated_input_equals_swiglu_then_matvec(kernel, rows_in):
    """MKB_GEMV_GATED: x = gate | up, the kernel forms silu(gate) * up on load with the rounding points
    of the separate operator, so the result equals silu_mul followed by the plain matvec bit for bit."""
    from mlkit_b200 import kernels

    width, outputs = 4096, 304
    layer = helpers.make_layer(outputs, width, 4, 128, seed=9)
    gate_up = dev((np.random.default_rng(rows_in).standard_normal((rows_in, 2 * width)) * 1.5).astype(np.float16))
    act = torch.empty((rows_in, width), dtype=torch.float16, device="cuda")
    kernels.silu_mul(gate_up, act)
    packed, scales, values = dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"])
    plain = torch.empty((rows_in, outputs), dtype=torch.float16, device="cuda")
    fused = torch.empty_like(plain)
    options = dict(group=128, bits=4, integer_grid=True, grid_minimum=-8.0, kernel=kernel)
    kernels.packed_matvec(act, packed, scales, values, None, None, plain, **options)
    kernels.packed_matvec(gate_up, packed, scales, values, None, None, fused, gated=True, **options)
    assert torch.equal(plain, fused)
    with pytest.raises(ValueError, match="gated"):
        kernels.packed_matvec(gate_up, packed, scales, values, None, None, fused, gated=True, group=128, bits=4,
                              integer_grid=True, grid_minimum=-8.0, kernel="scalar")


def test_zz_no_bounded_wait_expired_in_this_session():
    """The split-K kernels report an expired wait through the workspace's status word: after all the
    matvec tests of this module it must still be clear."""
    from mlkit_b200 import kernels

    layer = helpers.make_layer(512, 8192, 4, 128, seed=2)   # K split over slabs: uses the workspace
    x = helpers.activations(8, 8192, seed=1)
    assert matvec.relative_l2(run_matvec(layer, x, "bulk"), oracle_matvec(layer, x)) < TOLERANCE
    assert kernels.workspace_status() == 0


# ---------------------------------------------------------------- rotation fused into the matvec
@pytest.mark.parametrize("case", [("int4", 4096, 4, 128), ("int4", 8192, 2, 128), ("int4", 1024, 8, 128),
                                  ("int4", 512, 3, 128), ("nf4", 4096, 2, 64), ("int8", 2048, 4, 128),
                                  ("int2", 4096, 1, 128)])
def test_matvec_with_rotation_on_load_equals_transform_then_matvec(case):
    """``mkb_gemv_hadamard``: every CTA rotates the activations in shared memory with the butterflies of the
    transform kernel and rounds them to fp16 as that kernel stores them, so the result equals the two
    launches bit for bit, with and without a sign vector, for every row count up to the limit."""
    from mlkit_b200 import kernels

    kind, width, most_rows, group = case
    bits = {"int4": 4, "nf4": 4, "int8": 8, "int2": 2}[kind]
    outputs = 272
    layer = helpers.make_layer(outputs, width, bits, group, kind="nf4" if kind == "nf4" else "int", seed=width)
    packed, scales, values = dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"])
    integer, low = kernels.integer_grid_of(values)
    rng = np.random.default_rng(width + bits)
    signs = dev((rng.integers(0, 2, width) * 2 - 1).astype(np.int8))
    for rows in range(1, most_rows + 1):
        x = dev(helpers.activations(rows, width, seed=rows, outliers=True))
        for sign_vector in (signs, None):
            rotated = kernels.structured_transform(x, factor=1, power=width, signs=sign_vector)
            expected = torch.empty((rows, outputs), dtype=torch.float16, device="cuda")
            kernels.packed_matvec(rotated, packed, scales, values, None, None, expected, group=group, bits=bits,
                                  integer_grid=integer, grid_minimum=low, kernel="stream")
            fused = torch.empty_like(expected)
            kernels.packed_matvec_rotated(x, sign_vector, packed, scales, values, None, fused, group=group, bits=bits,
                                          integer_grid=integer, grid_minimum=low)
            assert torch.equal(fused, expected), (case, rows, sign_vector is None)
    # and against the oracle, end to end
    x = helpers.activations(1, width, seed=3, outliers=True)
    turned = transforms.randomized_transform(x.astype(np.float32), signs.cpu().numpy(), by_multiply=True)
    got = torch.empty((1, outputs), dtype=torch.float16, device="cuda")
    kernels.packed_matvec_rotated(dev(x), signs, packed, scales, values, None, got, group=group, bits=bits,
                                  integer_grid=integer, grid_minimum=low)
    assert matvec.relative_l2(got.cpu().numpy(), oracle_matvec(layer, turned.astype(np.float16))) < TOLERANCE


def test_matvec_with_rotation_on_load_refuses_what_it_does_not_cover():
    from mlkit_b200 import kernels

    for width, rows in ((4096, 5), (14336, 1), (256, 1)):
        layer = helpers.random_layer(64, width, 4, 128, seed=1, lut_len=16)
        layer["values"] = codec.int_values(4)
        out = torch.empty((rows, 64), dtype=torch.float16, device="cuda")
        x = torch.zeros((rows, width), dtype=torch.float16, device="cuda")
        assert not kernels.rotated_matvec_supported(rows, width, torch.float16)
        with pytest.raises(ValueError, match="gemv_hadamard"):
            kernels.packed_matvec_rotated(x, None, dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]),
                                          None, out, group=128, bits=4, integer_grid=True, grid_minimum=-8.0)
