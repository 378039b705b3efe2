"""N-sharded linear with the all_gather fused into the matmul epilogue (peer stores), 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one machine")
def test_sharded_matmul_allgather_two_ranks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541",
                          os.path.join(root, "tests", "peer_worker.py")], cwd=root, env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.count("PEER-OK") == 2, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one machine")
def test_sharded_matmul_through_the_copy_kernel_two_ranks():
    """The same worker with B200Q_PUSH=1: prefill-size products store their block locally and
    peer_push_kernel moves it to the other rank and signals (the form chosen by default above four
    ranks); every gathered result is checked against the oracle as before."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200Q_PUSH="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29543",
                          os.path.join(root, "tests", "peer_worker.py")], cwd=root, env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.count("PEER-OK") == 2, res.stdout[-3000:] + res.stderr[-3000:]


def test_bounded_wait_runs_out_and_is_reported():
    """A rank that never signals: the bounded wait of the exchange gives up after its limit (set to
    50 ms here), stores code 6 in the status word and lets the stream go on; the host-side check
    turns that into an exception and hands back a zeroed workspace.  Nothing is made to fault: the
    flag is simply never raised."""
    import ctypes
    import time

    from mlx_b200 import _lib, ops

    lib = _lib.load()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    sync = torch.zeros(64, dtype=torch.int32, device="cuda")     # flag at word 0 (stays 0), epoch at word 32
    sync[32] = 2                                                 # two signals expected, none will come
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    ws[100] = 7                                                  # stale scratch that a later kernel would trip over
    status = ctypes.c_void_p(ws.data_ptr() + ws.numel() - 16)
    stream = torch.cuda.current_stream().cuda_stream
    lib.b200q_set_peer_wait_limit_ms(50)
    try:
        t0 = time.perf_counter()
        rc = lib.b200q_peer_wait(P(sync), ctypes.c_void_p(sync.data_ptr() + 128), status, ctypes.c_void_p(stream))
        assert rc == 0, _lib.last_error()
        with pytest.raises(ops.DeviceStatusError) as ei:
            ops.read_workspace_status(ws, stream, "peer exchange")
        waited = time.perf_counter() - t0
    finally:
        lib.b200q_set_peer_wait_limit_ms(0)
    assert ei.value.code == 6 and "peer" in str(ei.value)
    assert 0.02 < waited < 5.0, waited
    assert int(ws.to(torch.int32).sum()) == 0          # the check re-zeroed the workspace
    ops.read_workspace_status(ws, stream, "peer exchange")   # and the status is clear again
    # a wait whose flag is already there returns at once and reports nothing
    sync[0] = 2
    rc = lib.b200q_peer_wait(P(sync), ctypes.c_void_p(sync.data_ptr() + 128), status, ctypes.c_void_p(stream))
    assert rc == 0
    ops.read_workspace_status(ws, stream, "peer exchange")
