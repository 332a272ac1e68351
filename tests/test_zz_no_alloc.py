"""The allocation-free matvec entry point, ``mkb_gemv_static``.

Some programs that embed the library cannot give it scratch memory: a server that handed every spare
byte of HBM to its KV cache when it started, a plugin that must not call the CUDA allocator, code
that runs while a stream is being captured.  For them the tensor-memory matvec keeps its split-K
scratch in an 8 MiB array inside the library.  This file checks, through the C ABI, that it returns
the same numbers as the workspace-taking entry point on two calls in a row, and that a shape whose
scratch would not fit is refused.  The file name sorts last so that it runs after every other test.
"""

import numpy as np
import pytest
import torch

from oracle import matvec
from tests import helpers

pytestmark = pytest.mark.gpu
TOLERANCE = 2e-3


def _device(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def _run_both(layer, x, bias=None):
    from mlkit_b200 import _native

    lib = _native.library()
    rows_in, width = x.shape
    outputs = layer["rows"]
    packed, scales, values = _device(layer["packed"]), _device(layer["scales16"]), _device(layer["values"])
    x_dev = _device(x)
    bias_dev = None if bias is None else _device(bias)
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.mkb_gemv_workspace_bytes(rows_in, outputs, width, 4)
    workspace = torch.zeros(need, dtype=torch.uint8, device="cuda")
    expected = torch.empty((rows_in, outputs), dtype=torch.float16, device="cuda")
    status = lib.mkb_gemv_ws(x_dev.data_ptr(), packed.data_ptr(), scales.data_ptr(), values.data_ptr(), None,
                             None if bias_dev is None else bias_dev.data_ptr(), expected.data_ptr(), rows_in, outputs,
                             width, layer["group"], 4, 16, _native.F16, _native.F16, width // 2, scales.stride(0), 1,
                             -8.0, _native.GEMV_TMEM, workspace.data_ptr(), workspace.numel(), stream)
    _native.check(status, "mkb_gemv_ws")
    results = []
    for _ in range(2):   # two calls in a row share the built-in scratch
        out = torch.full((rows_in, outputs), float("nan"), dtype=torch.float16, device="cuda")
        status = lib.mkb_gemv_static(x_dev.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                     None if bias_dev is None else bias_dev.data_ptr(), out.data_ptr(), rows_in,
                                     outputs, width, layer["group"], width // 2, scales.stride(0), -8.0, stream)
        _native.check(status, "mkb_gemv_static")
        results.append(out)
    torch.cuda.synchronize()
    import ctypes

    expired = ctypes.c_int(-1)   # no bounded wait ran out in the calls above
    _native.check(lib.mkb_gemv_static_status(ctypes.byref(expired)), "mkb_gemv_static_status")
    assert expired.value == 0
    return expected.cpu().numpy(), [r.cpu().numpy() for r in results]


@pytest.mark.parametrize("shape,rows_in", [((300, 1024), 1), ((1000, 1536), 5), ((4096, 4096), 8)])
def test_static_scratch_entry_matches_the_workspace_entry(shape, rows_in):
    layer = helpers.make_layer(shape[0], shape[1], 4, 128, seed=shape[0])
    x = helpers.activations(rows_in, shape[1], seed=rows_in)
    bias = (np.random.default_rng(3).standard_normal(shape[0]) * 0.1).astype(np.float16)
    expected, results = _run_both(layer, x, bias)
    for got in results:
        assert matvec.relative_l2(got, expected) < TOLERANCE
        assert np.array_equal(got, expected)   # same kernel, same summation order
    reference = matvec.reconstruct_then_matmul(x, layer["packed"], layer["scales16"], layer["values"], 128, 4, shape,
                                               bias=bias)
    assert matvec.relative_l2(results[1], reference) < TOLERANCE


def test_static_scratch_entry_at_the_limit_of_the_scratch():
    """254 row blocks x 8 slabs x 8 rows need exactly the 8 MiB the library holds; one row block more is
    refused.  Random codes (the arithmetic is value-blind); the yardstick is the workspace entry.  On
    a machine with a second GPU the same call runs there too: every device has its own array."""
    from mlkit_b200 import _native
    from oracle import bitstream

    rows, width = 254 * 128, 4096
    rng = np.random.default_rng(8)
    layer = {"rows": rows, "group": 128, "values": np.arange(-8, 8, dtype=np.float32),
             "packed": rng.integers(0, 256, size=rows * width // 2, dtype=np.uint8),
             "scales16": (rng.random((rows, width // 128), dtype=np.float32) * 0.01 + 0.001).astype(np.float16)}
    x = helpers.activations(8, width, seed=4)
    assert _native.library().mkb_gemv_workspace_bytes(8, rows, width, 4) >= 8 << 20
    for device in range(min(2, torch.cuda.device_count())):
        with torch.cuda.device(device):
            expected, results = _run_both(layer, x)
            for got in results:
                assert np.array_equal(got, expected)
    lib = _native.library()
    big = torch.zeros(8, width, dtype=torch.float16, device="cuda")
    status = lib.mkb_gemv_static(big.data_ptr(), big.data_ptr(), big.data_ptr(), None, big.data_ptr(), 8, rows + 128,
                                 width, 128, width // 2, width // 128, -8.0, torch.cuda.current_stream().cuda_stream)
    assert status == -2 and b"built-in scratch holds" in lib.mkb_last_error()


def test_static_scratch_entry_refuses_what_does_not_fit():
    from mlkit_b200 import _native

    lib = _native.library()
    assert lib.mkb_gemv_static_scratch_bytes() == 8 << 20
    x = torch.zeros(8, 8192, dtype=torch.float16, device="cuda")
    packed = torch.zeros(16, dtype=torch.uint8, device="cuda")
    # 28672 x 8192 at eight rows would need ~58 MB of scratch: refused before anything is launched or read
    status = lib.mkb_gemv_static(x.data_ptr(), packed.data_ptr(), x.data_ptr(), None, x.data_ptr(), 8, 28672, 8192, 128,
                                 4096, 64, -8.0, torch.cuda.current_stream().cuda_stream)
    assert status == -2
    assert b"built-in scratch holds" in lib.mkb_last_error()
    status = lib.mkb_gemv_static(x.data_ptr(), packed.data_ptr(), x.data_ptr(), None, x.data_ptr(), 1, 128, 640, 128,
                                 320, 5, -8.0, torch.cuda.current_stream().cuda_stream)
    assert status == -2 and b"multiple of 512" in lib.mkb_last_error()
