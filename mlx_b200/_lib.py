"""ctypes binding of libb200q.so (the C-ABI declared in include/b200q.h).

The library is the product: there is no Python or CPU fallback.  Importing this module
fails loudly when the shared library has not been built (python -m mlx_b200.build).
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")

F32, F16, BF16 = 0, 1, 2
OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_WORKSPACE = -4
ERR_DEVICE = -5

# name -> (restype, argtypes); every symbol include/b200q.h declares.
_vp, _i, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
SIGNATURES = {
    "b200q_version": (_i, []),
    "b200q_last_error": (ctypes.c_char_p, []),
    "b200q_quantize": (_i, [_vp, _i, _i64, _i64, _i, _i, _vp, _vp, _vp, _vp]),
    "b200q_dequantize": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _i, _vp, _vp]),
    "b200q_dequantize_rows": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i64, _i64, _i, _i, _vp, _vp]),
    "b200q_qmm_workspace_bytes": (_sz, [_i, _i64, _i64, _i64, _i64, _i, _i, _i]),
    "b200q_qmm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i64, _i, _i, _i, _i64, _vp, _sz, _vp]),
    "b200q_gather_qmm_workspace_bytes": (_sz, [_i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i]),
    "b200q_gather_qmm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _i64, _i64, _i64, _i64, _i64,
                              _i, _i, _i, _i, _vp, _sz, _vp]),
    "b200q_gather_qmm_chain_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "b200q_gather_qmm_chain": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _i64, _i64, _i64, _i64, _i64,
                                    _i64, _i, _i, _vp, _sz, _vp]),
    "b200q_gather_qmm_swiglu_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "b200q_gather_qmm_swiglu": (_i, [_vp] * 12 + [_i64, _vp, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _vp, _sz, _vp]),
    "b200q_workspace_init": (_i, [_vp, _sz, _vp]),
    "b200q_read_status": (_i, [_vp, _sz, _vp, ctypes.POINTER(ctypes.c_uint32)]),
    "b200q_qmm_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i, _i, _i, _vp, _sz, _vp]),
    "b200q_qmm_decode_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i, _i, _vp]),
    "b200q_qmm_sharded": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _i64, _i64, _i64, _i, _i, _vp, _sz, _vp]),
    "b200q_gather_qmm_sharded": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _i, _i, _i64, _i64, _i64, _i64, _i64,
                                      _i64, _i64, _i, _i, _vp, _sz, _vp]),
    "b200q_qmm_sharded_signal": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _i64, _i64, _i64, _i, _i, _vp, _vp, _vp,
                                      _vp, _i, _i, _vp, _sz, _vp]),
    "b200q_gather_qmm_sharded_signal": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _i, _i, _i64, _i64, _i64, _i64,
                                             _i64, _i64, _i64, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200q_set_peer_wait_limit_ms": (None, [_i]),
    "b200q_peer_signal": (_i, [_vp, _i, _vp, _vp]),
    "b200q_peer_wait": (_i, [_vp, _vp, _vp, _vp]),
    "b200q_peer_reduce": (_i, [_vp, _i, _i64, _i64, _vp, _i, _vp]),
    "b200q_ipc_alloc": (_i, [_sz, _vp, _vp]),
    "b200q_ipc_open": (_i, [_vp, _vp]),
    "b200q_ipc_close": (_i, [_vp]),
    "b200q_ipc_free": (_i, [_vp]),
    "b200q_gguf_repack": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp]),
    "b200q_qmm_kernel_name": (ctypes.c_char_p, [_i, _i64, _i64, _i64, _i64, _i, _i, _i]),
    "b200q_launch_count": (ctypes.c_uint64, []),
    "b200q_set_weights_constant": (None, [_i]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build the CUDA library first (python -m mlx_b200.build). "
                "There is no CPU fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().b200q_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Map a status code to the exception type the reference front-end raises."""
    if rc == OK:
        return
    msg = last_error()
    if rc == ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(f"b200q error {rc}: {msg}")
