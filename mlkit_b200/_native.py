"""ctypes binding of libmlkit_b200.so (the C ABI of ``include/mlkit_b200.h``).

There is no CPU or pure-PyTorch fallback: when the library cannot be loaded, every operation
raises.  The library is built in-tree by ``mlkit_b200.build``; a missing or stale library is
rebuilt on first use when nvcc is present.
"""

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

from mlkit_b200 import build as _build

F16, BF16, F32 = 0, 1, 2
GEMV_AUTO, GEMV_SCALAR, GEMV_TILED, GEMV_TMEM, GEMV_BULK, GEMV_STREAM = 0, 1, 2, 3, 4, 5
GEMV_GATED = 0x100

SIGNATURES = {
    "mkb_version": (c_int, []),
    "mkb_last_error": (c_char_p, []),
    "mkb_gemv": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_int64, c_int64, c_int, c_float, c_void_p]),
    "mkb_gemv_ex": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_int64, c_int64, c_int, c_float, c_int, c_void_p]),
    "mkb_gemv_workspace_bytes": (c_int64, [c_int] * 4),
    "mkb_gemv_workspace_status": (c_int, [c_void_p, c_int64, c_void_p]),
    "mkb_gemv_hadamard": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_int64, c_int64, c_int, c_float, c_int, c_void_p]),
    "mkb_gemm_workspace_bytes": (c_int64, [c_int] * 3),
    "mkb_gemm": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_int64, c_int64, c_int, c_float, c_void_p, c_int64, c_void_p]),
    "mkb_gemm_status": (c_int, [c_void_p, c_void_p]),
    "mkb_gemv_ws": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_int64, c_int64, c_int, c_float, c_int, c_void_p, c_int64,
                            c_void_p]),
    "mkb_gemv_static_scratch_bytes": (c_int64, []),
    "mkb_gemv_static": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_int64, c_int64, c_float, c_void_p]),
    "mkb_gemv_static_status": (c_int, [c_void_p]),
    "mkb_dequant": (c_int, [c_void_p] * 6 + [c_int64, c_int64] + [c_int] * 5 + [c_int64, c_void_p]),
    "mkb_dequant_rows": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int] * 5 + [c_int64, c_void_p]),
    "mkb_rtn_encode": (c_int, [c_void_p] * 5 + [c_int64] + [c_int] * 5 + [c_float] * 3 + [c_int, c_void_p]),
    "mkb_hadamard": (c_int, [c_void_p] * 4 + [c_int64] + [c_int] * 6 + [c_void_p]),
    "mkb_add_rmsnorm": (c_int, [c_void_p] * 4 + [c_int, c_int, c_float, c_void_p]),
    "mkb_rope_append": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_float, c_void_p]),
    "mkb_attention_decode": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_float, c_void_p]),
    "mkb_rope_attention_decode": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_float, c_float, c_void_p]),
    "mkb_argmax": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "mkb_decode_status": (c_int, [c_void_p]),
    "mkb_silu_mul": (c_int, [c_void_p] * 2 + [c_int, c_int, c_void_p]),
    "mkb_peer_buffer_bytes": (c_int64, [c_int] * 3),
    "mkb_peer_alloc": (c_int, [c_int64, c_void_p]),
    "mkb_peer_free": (c_int, [c_void_p]),
    "mkb_peer_export": (c_int, [c_void_p, c_void_p]),
    "mkb_peer_open": (c_int, [c_void_p, c_void_p]),
    "mkb_peer_close": (c_int, [c_void_p]),
    "mkb_peer_reduce_add_rmsnorm": (c_int, [c_void_p] * 7 + [c_int] * 5 + [c_float, c_void_p]),
    "mkb_peer_status": (c_int, [c_void_p, c_void_p]),
    "mkb_peer_set_poll_limit": (c_int, [c_void_p, c_int64]),
    "mkb_peer_set_split": (c_int, [c_void_p, c_int]),
}

_library = None


class NativeError(RuntimeError):
    """A call into libmlkit_b200 was rejected or the library is unavailable."""


def library() -> ctypes.CDLL:
    global _library
    if _library is not None:
        return _library
    try:
        path = _build.build()
    except Exception as error:  # no nvcc and no prebuilt library
        if not _build.OUTPUT.exists():
            raise NativeError(
                "libmlkit_b200.so is not built and cannot be built here "
                f"({error}); run `python -m mlkit_b200.build` where nvcc is available"
            ) from error
        path = _build.OUTPUT
    try:
        handle = ctypes.CDLL(str(path))
    except OSError as error:
        raise NativeError(f"cannot load {path}: {error}") from error
    for name, (result, arguments) in SIGNATURES.items():
        function = getattr(handle, name)
        function.restype = result
        function.argtypes = arguments
    _library = handle
    return handle


def check(status: int, what: str) -> None:
    if status == 0:
        return
    message = library().mkb_last_error().decode(errors="replace")
    if status in (-1, -2, -3):
        raise ValueError(f"{what}: {message}")
    raise NativeError(f"{what}: {message} (code {status})")
