"""The C-ABI library loads without a GPU, exports every symbol include/b200q.h declares,
and rejects invalid arguments on the host before touching CUDA."""
import ctypes
import os
import re

import pytest

from mlx_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    syms = declared_symbols()
    assert syms, "no declarations parsed"
    assert sorted(_lib.SIGNATURES) == syms


def test_library_exports_all_symbols():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(lib, s), s
    assert _lib.load().b200q_version() == 1


@pytest.mark.parametrize("group,bits,K,code", [
    (48, 4, 256, _lib.ERR_INVALID_ARGUMENT),
    (64, 7, 256, _lib.ERR_INVALID_ARGUMENT),
    (64, 1, 256, _lib.ERR_INVALID_ARGUMENT),
    (64, 4, 96, _lib.ERR_INVALID_ARGUMENT),
])
def test_quantize_rejects_on_host(group, bits, K, code):
    lib = _lib.load()
    rc = lib.b200q_quantize(None, _lib.BF16, 4, K, group, bits, None, None, None, None)
    assert rc == code
    assert _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)


def test_qmm_rejects_on_host():
    lib = _lib.load()
    bad = [
        dict(dtype=7), dict(group=16), dict(bits=7), dict(K=100), dict(M=-1),
    ]
    for kw in bad:
        a = dict(dtype=_lib.BF16, M=4, N=64, K=256, group=64, bits=4)
        a.update(kw)
        rc = lib.b200q_qmm(None, None, None, None, None, a["dtype"], 1, a["M"], a["N"], a["K"], a["group"],
                           a["bits"], 1, 0, None, 0, None)
        assert rc == _lib.ERR_INVALID_ARGUMENT, kw
    # empty problems succeed without touching the device
    assert lib.b200q_qmm(None, None, None, None, None, _lib.BF16, 1, 0, 64, 256, 64, 4, 1, 0, None, 0, None) == 0
    assert lib.b200q_quantize(None, _lib.F32, 0, 256, 64, 4, None, None, None, None) == 0


def test_kernel_selection_names():
    lib = _lib.load()
    name = lambda M, N, K, dt=_lib.BF16, tr=1, bits=4, g=64: lib.b200q_qmm_kernel_name(dt, 1, M, N, K, g, bits, tr).decode()
    assert name(1, 4096, 4096) == "qmv_rows"
    assert name(16, 14336, 4096) == "qmv_rows"
    assert name(16, 14336, 4096, bits=3) == "qmv_mma"
    assert name(17, 14336, 4096) == "qmv_rows" and name(32, 14336, 4096) == "qmv_rows"   # two passes of up to 16 rows
    assert name(33, 14336, 4096) == "qmm_tcgen05" and name(17, 14336, 4096, bits=3) == "qmm_tcgen05"
    assert name(16, 14336, 4096, dt=_lib.F32) == "qmm_generic"
    assert name(16, 4096, 4096, tr=0) == "qmm_generic"
    assert name(1, 4096, 4096, tr=0) == "qvm" and name(4, 4096, 4096, tr=0, bits=8) == "qvm"
    assert name(2, 4096, 4096, tr=0, bits=3) == "qmm_generic"
    assert name(4, 100, 96, g=32) == "qmm_generic"
    assert lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, 16, 14336, 4096, 64, 4, 1) > 14336 * 64


def test_sharded_rejects_on_host():
    """b200q_qmm_sharded validates its output description before any CUDA call."""
    lib = _lib.load()
    dummy = ctypes.c_void_p(4096)
    one = (ctypes.c_void_p * 1)(4096)
    nine = (ctypes.c_void_p * 9)(*([4096] * 9))
    call = lambda ys, n, ld, col0, nl=128: lib.b200q_qmm_sharded(dummy, dummy, dummy, dummy, ys, n, ld, col0, _lib.BF16, 4, nl,
                                                                  256, 64, 4, dummy, 1 << 20, None)
    assert call(one, 0, 256, 0) == _lib.ERR_INVALID_ARGUMENT           # no output buffer
    assert call(nine, 9, 256, 0) == _lib.ERR_INVALID_ARGUMENT          # more than 8 ranks
    assert call(one, 1, 64, 0) == _lib.ERR_INVALID_ARGUMENT            # row pitch below the local width
    assert call(one, 1, 256, 192) == _lib.ERR_INVALID_ARGUMENT         # columns [192, 320) outside a pitch of 256
    assert b"fit a row pitch" in lib.b200q_last_error()
    assert lib.b200q_peer_signal(None, 2, dummy, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.b200q_peer_wait(None, dummy, dummy, None) == _lib.ERR_INVALID_ARGUMENT


def test_gather_sharded_rejects_on_host():
    lib = _lib.load()
    dummy = ctypes.c_void_p(4096)
    two = (ctypes.c_void_p * 2)(4096, 8192)
    call = lambda n_peers, self_, e_lo, e_loc, K=256: lib.b200q_gather_qmm_sharded(
        dummy, dummy, dummy, dummy, dummy, dummy, 8, two, n_peers, self_, _lib.BF16, 4, 8, e_lo, e_loc, 1, 128, K, 64, 4,
        dummy, 1 << 24, None)
    assert call(2, 2, 0, 4) == _lib.ERR_INVALID_ARGUMENT        # self outside the buffer list
    assert call(2, 0, 6, 4) == _lib.ERR_INVALID_ARGUMENT        # experts [6, 10) of 8
    assert call(2, 0, 0, 4, K=96) == _lib.ERR_INVALID_ARGUMENT  # K not a multiple of the group


def test_embedding_and_gated_mlp_reject_on_host():
    lib = _lib.load()
    d = ctypes.c_void_p(4096)
    rows_call = lambda **kw: lib.b200q_dequantize_rows(
        d, d, d, d, kw.get("n", 4), kw.get("dtype", _lib.BF16), 16, kw.get("K", 256), kw.get("group", 64),
        kw.get("bits", 4), d, None)
    assert rows_call(group=48) == _lib.ERR_INVALID_ARGUMENT
    assert rows_call(bits=7) == _lib.ERR_INVALID_ARGUMENT
    assert rows_call(K=100) == _lib.ERR_INVALID_ARGUMENT
    assert rows_call(dtype=9) == _lib.ERR_INVALID_ARGUMENT
    assert rows_call(n=-1) == _lib.ERR_INVALID_ARGUMENT
    assert rows_call(n=0) == 0                                   # nothing to look up
    glu = lambda **kw: lib.b200q_gather_qmm_swiglu(
        d, d, d, d, d, d, d, d, d, d, d, d, kw.get("n", 8), d, kw.get("dtype", _lib.BF16), 8, 4, 1, kw.get("H", 256),
        kw.get("K1", 256), 128, kw.get("group", 64), kw.get("bits", 4), d, kw.get("ws", 1 << 24), None)
    assert glu(group=16) == _lib.ERR_INVALID_ARGUMENT
    assert glu(H=96) == _lib.ERR_INVALID_ARGUMENT               # hidden width not a multiple of the group
    assert glu(n=0) == 0
    assert glu(dtype=_lib.F32) == _lib.ERR_UNSUPPORTED          # bfloat16 only
    assert glu(ws=256) == _lib.ERR_WORKSPACE
    assert lib.b200q_gather_qmm_swiglu_workspace_bytes(8, 4, 1, 256, 256) > lib.b200q_gather_qmm_workspace_bytes(
        _lib.BF16, 8, 8, 4, 1, 256, 256, 64, 4, 1)


def test_weights_constant_promise_toggles_on_the_host():
    """b200q_set_weights_constant is host state only; the Python wrapper mirrors it so that
    quantized_matmul can suspend the promise around a call whose weights it has just copied."""
    import mlx_b200 as mb
    from mlx_b200 import ops

    mb.set_weights_constant(True)
    assert ops._weights_constant is True
    mb.set_weights_constant(False)
    assert ops._weights_constant is False
