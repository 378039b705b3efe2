"""GPU parity of gather_qmm against the reference gather loop
(mlx/backend/cpu/quantized.cpp:700-747), shapes after python/tests/test_quantized.py:1127-1266."""
import os

import numpy as np
import pytest
import torch

import mlx_b200 as mb
import oracle as O
from util import from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "affine_golden.npz")


def test_gather_golden():
    gold = np.load(GOLDEN)
    a = {k: gold[f"gather/{k}"] for k in ("wq", "s", "b", "x", "lhs", "rhs", "y")}
    y = mb.gather_qmm(to_torch(a["x"], "f32"), u32_to_torch(a["wq"]), to_torch(a["s"], "f32"), to_torch(a["b"], "f32"),
                      lhs_indices=torch.from_numpy(a["lhs"].astype(np.int64)), rhs_indices=torch.from_numpy(a["rhs"].astype(np.int64)))
    ok, rel = qmm_close(from_torch(y), a["y"], 1e-4)
    assert ok, rel


@pytest.mark.parametrize("dtype", ("f32", "bf16"))
@pytest.mark.parametrize("transpose", (True, False))
def test_gather_index_patterns(dtype, transpose):
    E, M, N, K, g, bits = 5, 3, 64, 128, 32, 4
    wshape = (E, N, K) if transpose else (E, K, N)
    w = make_w(11, wshape, dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    x = make_x(12, (4, M, K), dtype)
    rng = np.random.default_rng(3)
    cases = [
        (rng.integers(0, 4, (7,)), rng.integers(0, E, (7,))),
        (None, rng.integers(0, E, (4,))),
        (rng.integers(0, 4, (E,)), None),
        (rng.integers(0, 4, (2, 3)), rng.integers(0, E, (2, 3))),
        (rng.integers(0, 4, (2, 1)), rng.integers(0, E, (1, 3))),
    ]
    args = (u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    for lhs, rhs in cases:
        tl = None if lhs is None else torch.from_numpy(lhs)
        tr = None if rhs is None else torch.from_numpy(rhs)
        y = mb.gather_qmm(to_torch(x, dtype), *args, lhs_indices=tl, rhs_indices=tr, transpose=transpose,
                          group_size=g, bits=bits)
        l = np.arange(4) if lhs is None else lhs
        r = np.arange(E) if rhs is None else rhs
        l, r = np.broadcast_arrays(l, r)
        assert tuple(y.shape) == l.shape + (M, N)
        ref = O.gather_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), l.ravel(), r.ravel(),
                           transpose, g, bits, "f32")
        ok, rel = qmm_close(O.to_f32(from_torch(y), dtype).reshape(ref.shape), ref, 1e-4 if dtype == "f32" else 1e-2)
        assert ok, rel


def test_gather_bad_index_is_flagged_not_faulted():
    from mlx_b200 import _lib, ops
    import ctypes
    E, M, N, K = 2, 1, 32, 128
    w = make_w(13, (E, N, K), "f32")
    wq, s, b = O.quantize(w, 64, 4, "f32")
    x = to_torch(make_x(14, (3, M, K), "f32"), "f32")
    y = mb.gather_qmm(x, u32_to_torch(wq), to_torch(s, "f32"), to_torch(b, "f32"),
                      lhs_indices=torch.tensor([0, 1, 2]), rhs_indices=torch.tensor([0, 9, 1]))
    torch.cuda.synchronize()
    assert bool((y[1] == 0).all()) and bool((y[0] != 0).any()) and bool((y[2] != 0).any())
    ws = ops._workspaces.get(x.device, 0)
    st = (ctypes.c_uint32 * 4)()
    rc = _lib.load().b200q_read_status(ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), st)
    assert rc == 0 and st[0] == 1 and st[1] == 1
