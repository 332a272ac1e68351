"""GPU parity of the fused dequantise + GEMM (``mkb_gemm``, 9..128 activation rows) against the oracle's
reconstruct-then-matmul, which is the dense route of the reference above eight rows
(``src/mlkit/inference/packed_linear.py:153-154``)."""

import numpy as np
import pytest
import torch

from oracle import bitstream, codec, matvec
from tests import helpers

pytestmark = pytest.mark.gpu
TOLERANCE = 2e-3


def dev(array):
    return None if array is None else torch.from_numpy(np.ascontiguousarray(array)).cuda()


def int4_layer(rows, width, seed):
    """Uniform random INT4 codes on the integer grid with random fp16 scales per 128 codes."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(rows, width), dtype=np.uint8)
    scales = (rng.random((rows, width // 128), dtype=np.float32) * 0.01 + 0.001).astype(np.float16)
    return {"rows": rows, "width": width, "bits": 4, "group": 128, "values": codec.int_values(4), "codes": codes,
            "packed": bitstream.pack(codes, 4), "scales16": scales, "zero16": None}


def run_gemm(layer, x, bias=None):
    from mlkit_b200 import kernels

    out = torch.empty((x.shape[0], layer["rows"]), dtype=torch.float16, device="cuda")
    kernels.packed_gemm(dev(x), dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), dev(bias), out,
                        group=128, bits=4, integer_grid=True, grid_minimum=-8.0)
    torch.cuda.synchronize()
    assert kernels.gemm_status() == 0
    return out.cpu().numpy()


def oracle(layer, x, bias=None):
    return matvec.reconstruct_then_matmul(x, layer["packed"], layer["scales16"], layer["values"], 128, 4,
                                          (layer["rows"], layer["width"]), bias=bias)


def test_one_hot_rows_return_the_reconstructed_weight_bit_for_bit():
    """x = unit vectors: y[m, n] is the fp16 weight W[n, k(m)] itself, so the decode (rounding of
    (c - 8) * scale to fp16), the K order of both operands and the row mapping are checked exactly."""
    from mlkit_b200 import kernels

    rows, width = 200, 512
    layer = int4_layer(rows, width, seed=1)
    dense, _ = kernels.dequantize(dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None,
                                  shape=(rows, width), group=128, bits=4, dtype=torch.float16)
    dense = dense.cpu().numpy()
    assert np.array_equal(dense, codec.decode_scaled(layer["codes"], layer["scales16"].astype(np.float32),
                                                     layer["values"], 128).astype(np.float16))
    for start in range(0, width, 128):
        x = np.zeros((128, width), dtype=np.float16)
        x[np.arange(128), start + np.arange(128)] = 1.0
        assert np.array_equal(run_gemm(layer, x), dense[:, start:start + 128].T)


@pytest.mark.parametrize("rows_in", [9, 16, 17, 48, 100, 128])
@pytest.mark.parametrize("shape", [(128, 128), (300, 1024), (4096, 4096), (1024, 14336), (14336, 4096)])
def test_gemm_matches_reconstruct_then_matmul(shape, rows_in):
    out_rows, width = shape
    layer = int4_layer(out_rows, width, seed=out_rows + width)
    x = helpers.activations(rows_in, width, seed=rows_in)
    bias = (np.random.default_rng(3).standard_normal(out_rows) * 0.1).astype(np.float16) if rows_in % 2 else None
    got = run_gemm(layer, x, bias)
    assert matvec.relative_l2(got, oracle(layer, x, bias)) < TOLERANCE
    # a second call reuses the workspace the first one left behind: same bits
    assert np.array_equal(got, run_gemm(layer, x, bias))


def test_gemm_agrees_with_the_matvec_kernels_on_eight_rows():
    layer = helpers.make_layer(512, 2048, 4, 128, seed=5)
    x = helpers.activations(8, 2048, seed=2)
    from mlkit_b200 import kernels

    out = torch.empty((8, 512), dtype=torch.float16, device="cuda")
    kernels.packed_matvec(dev(x), dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None, None, out,
                          group=128, bits=4, integer_grid=True, grid_minimum=-8.0, kernel="auto")
    assert matvec.relative_l2(run_gemm(layer, x), out.cpu().numpy().astype(np.float32)) < TOLERANCE


def test_gemm_refuses_what_it_does_not_cover():
    from mlkit_b200 import kernels

    layer = int4_layer(256, 512, seed=2)
    out = torch.empty((129, 256), dtype=torch.float16, device="cuda")
    x = torch.zeros((129, 512), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        kernels.packed_gemm(x, dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None, out,
                            group=128, bits=4, integer_grid=True, grid_minimum=-8.0)
    with pytest.raises(ValueError, match="gemm"):
        kernels.packed_gemm(x[:16], dev(layer["packed"]), dev(layer["scales16"]), dev(layer["values"]), None, out[:16],
                            group=64, bits=4, integer_grid=True, grid_minimum=-8.0)


def test_packed_linear_takes_the_fused_gemm_between_nine_and_128_rows():
    import mlkit_b200 as mk

    torch.manual_seed(0)
    linear = torch.nn.Linear(1024, 768, bias=True).half().cuda()
    q = mk.int(4, group=128)(linear.weight.detach().float(), mk.Ctx("layer", device="cuda"))
    packed = mk.PackedLinear(linear, q)
    with torch.inference_mode():
        for rows in (9, 32):
            x = torch.randn(2, rows // 2 if rows % 2 == 0 else rows, 1024, device="cuda").half()
            x = x[:1] if rows % 2 else x
            dense = torch.nn.functional.linear(x, packed.weight, packed.bias)
            got = packed(x)
            assert got.shape == dense.shape
            error = (got.float() - dense.float()).norm() / dense.float().norm()
            assert float(error) < TOLERANCE
        from mlkit_b200 import kernels

        assert not kernels.gemm_supported(64, width=1024, group=128, bits=4, dtype=torch.float16, scales=packed.scales,
                                          zeros=None, integer_grid=True, grid_minimum=-8.0, levels=16, outputs=768)
        assert kernels.gemm_supported(128, width=8192, group=128, bits=4, dtype=torch.float16, scales=packed.scales,
                                      zeros=None, integer_grid=True, grid_minimum=-8.0, levels=16, outputs=4096)
        wide = torch.randn(200, 1024, device="cuda").half()        # above 128 rows: the dense route
        assert torch.equal(packed(wide), torch.nn.functional.linear(wide, packed.weight, packed.bias))


def test_packed_linear_runs_nine_to_sixteen_rows_as_matvec_chunks():
    """Up to 16 rows (32 for layers the fused GEMM does not cover) the module runs the matvec on chunks of
    eight rows: every output row equals the row the matvec gives for it alone or in any other batch."""
    import mlkit_b200 as mk

    torch.manual_seed(1)
    for fmt, most in ((mk.int(4, group=128), 16), (mk.nf4(group=64), 32)):
        linear = torch.nn.Linear(1024, 512, bias=True).half().cuda()
        packed = mk.PackedLinear(linear, fmt(linear.weight.detach().float(), mk.Ctx("layer", device="cuda")))
        with torch.inference_mode():
            x = torch.randn(most, 1024, device="cuda").half()
            whole = packed(x)
            pieces = torch.cat([packed(x[start:start + 8]) for start in range(0, most, 8)])
            assert torch.equal(whole, pieces)
            odd = packed(x[:most - 3])
            assert torch.equal(odd, whole[:most - 3])
            dense = torch.nn.functional.linear(x, packed.weight, packed.bias)
            assert float((whole.float() - dense.float()).norm() / dense.float().norm()) < TOLERANCE
