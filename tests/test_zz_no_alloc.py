"""The allocation-free decode entry point (b200q_qmm_decode_static).

Some callers may not allocate device memory where they run the operator (a plugin under a
host framework's allocator or capture rules, a serving loop that bans allocator calls after
start-up), so they cannot hand b200q_qmm a workspace.  This entry point keeps its scratch in
a fixed array inside the library.  The test calls it through the C ABI twice in a row (the
array is shared and keeps the previous call's contents) and compares with b200q_qmm on the
same inputs, within the tolerance of the other matmul tests; it also checks the size limit.
This file sorts last so a run that stops at the first failure has run everything else."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from mlx_b200 import _lib
from util import from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("M,N,K,g,bits", [(16, 14336, 4096, 64, 4), (1, 4096, 4096, 64, 4), (7, 1000, 1024, 32, 3),
                                          (3, 32768, 1024, 64, 4)])  # the last case sits exactly at the built-in array's limit
def test_static_scratch_matches_workspace_entry_point(M, N, K, g, bits):
    lib = _lib.load()
    dtype = "bf16"
    wq_np, s_np, b_np = O.quantize(make_w(31, (N, K), dtype), g, bits, dtype)
    wq, s, b = u32_to_torch(wq_np), to_torch(s_np, dtype), to_torch(b_np, dtype)
    x_np = make_x(32, (M, K), dtype)
    x = to_torch(x_np, dtype)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # existing entry point with a caller workspace
    need = lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M, N, K, g, bits, 1)
    ws = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
    y_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200q_qmm(P(x), P(wq), P(s), P(b), P(y_ref), _lib.BF16, 1, M, N, K, g, bits, 1, 0, P(ws), ws.numel(), stream)
    assert rc == 0, _lib.last_error()

    # the allocation-free entry point, two calls in a row on the shared array
    before = torch.cuda.memory_allocated()
    outs = []
    for _ in range(2):
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.b200q_qmm_decode_static(P(x), P(wq), P(s), P(b), P(y), _lib.BF16, M, N, K, g, bits, stream)
        assert rc == 0, _lib.last_error()
        outs.append(y)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() - before <= 2 * M * N * 2 + 1024  # only the two outputs made here

    ref = O.to_f32(from_torch(y_ref), dtype)
    oracle = O.qmm_f32_from(x_np, wq_np, s_np, b_np, dtype, transpose=True, group_size=g, bits=bits)
    for y in outs:
        got = O.to_f32(from_torch(y), dtype)
        ok, rel = qmm_close(got, ref)
        assert ok, rel
        ok, rel = qmm_close(got, oracle)
        assert ok, rel


def test_static_scratch_rejects_oversize_and_bad_arguments():
    lib = _lib.load()
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    args = lambda M, N, K, dt=_lib.BF16, g=64, bits=4: lib.b200q_qmm_decode_static(
        P(dummy), P(dummy), P(dummy), P(dummy), P(dummy), dt, M, N, K, g, bits, None)
    assert args(1, 32768 + 16, 4096) == _lib.ERR_UNSUPPORTED
    assert "exceeds the built-in scratch" in _lib.last_error()
    assert args(17, 4096, 4096) == _lib.ERR_UNSUPPORTED
    assert args(16, 4096, 8192) == _lib.ERR_UNSUPPORTED   # 16 rows of 8192 activations exceed shared memory
    assert "do not fit in shared memory" in _lib.last_error()
    assert args(4, 4096, 4096, dt=_lib.F32) == _lib.ERR_UNSUPPORTED
    assert args(4, 4096, 4096, g=48) == _lib.ERR_INVALID_ARGUMENT
