"""Worker of tests/test_peer_gpu.py: one process per GPU (launched with torch.distributed.run).
Checks the matmul with the all_gather fused into its epilogue against the oracle on every rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import mlx_b200 as mb  # noqa: E402
import oracle as O  # noqa: E402
from mlx_b200 import _lib, ops  # noqa: E402
from mlx_b200.distributed import (PeerOutput, QuantizedAllToShardedLinear, QuantizedShardedToAllLinear,  # noqa: E402
                                  expert_bounds, sharded_gather_qmm, sharded_matmul_allgather, sharded_matmul_allreduce)
from util import from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")   # plumbing only: exchanges the 64-byte IPC handles
    N, K, g = 1024, 512, 64
    wq, s, b = O.quantize(make_w(5, (N, K), "bf16"), g, 4, "bf16")
    layer = QuantizedAllToShardedLinear(u32_to_torch(wq), to_torch(s, "bf16"), to_torch(b, "bf16"), g, 4,
                                        rank=rank, world=world)
    out = PeerOutput(96, N)
    ok = True
    for step, M in enumerate((16, 1, 96, 7, 16)):   # decode kernel (M <= 16) and tensor-core kernel
        x = make_x(20 + step, (M, K), "bf16")
        y = sharded_matmul_allgather(layer, to_torch(x, "bf16"), out)
        torch.cuda.synchronize()
        ref = O.qmm_f32_from(x, wq, s, b, "bf16", transpose=True, group_size=g, bits=4)
        good, rel = qmm_close(O.to_f32(from_torch(y.contiguous()), "bf16"), ref)
        st = (__import__("ctypes").c_uint32 * 4)()
        ws = ops._workspaces.get(y.device, 0, "qmm")
        _lib.load().b200q_read_status(__import__("ctypes").c_void_p(ws.data_ptr()), ws.numel(), None, st)
        print(f"rank {rank} step {step} M={M} ok={good} rel={rel:.4f} status={st[0]}", flush=True)
        ok = ok and good and st[0] == 0
        dist.barrier()
    out.close()

    # ---- a chain of sharded layers on the row-owning decode kernel (K a multiple of 16 groups): every
    # call's x is the gathered output of the previous one, the wait for it runs inside the consuming
    # kernel, the host waits once at the end.  Checked against the oracle applied layer by layer.
    Nc = Kc = 2048
    wqc, sc_, bc_ = O.quantize(make_w(6, (Nc, Kc), "bf16", std=0.03), g, 4, "bf16")
    chain = QuantizedAllToShardedLinear(u32_to_torch(wqc), to_torch(sc_, "bf16"), to_torch(bc_, "bf16"), g, 4,
                                        rank=rank, world=world)
    assert mb.qmm_kernel_name(torch.bfloat16, 16, Nc // world, Kc, g, 4) == "qmv_rows"
    outc = PeerOutput(16, Nc)
    for trial, M in enumerate((16, 5)):
        x0 = make_x(60 + trial, (M, Kc), "bf16")
        depth = 4
        h = to_torch(x0, "bf16")
        for _ in range(depth):
            h = sharded_matmul_allgather(chain, h, outc, chained=True)
        outc.wait()
        torch.cuda.synchronize()
        outc.check()
        ref_h = x0
        for _ in range(depth):
            ref_h = O.to_dtype(O.qmm_f32_from(ref_h, wqc, sc_, bc_, "bf16", transpose=True, group_size=g, bits=4), "bf16")
        good, rel = qmm_close(O.to_f32(from_torch(h.contiguous()), "bf16"), O.to_f32(ref_h, "bf16"), 3e-2)
        print(f"rank {rank} chain M={M} depth={depth} ok={good} rel={rel:.4f}", flush=True)
        ok = ok and good
        dist.barrier()
    outc.close()

    # ---- expert-parallel gather_qmm: 8 experts over the ranks, 40 tokens, top-2
    E, tokens, topk, N2, K2 = 8, 40, 2, 256, 512
    wq2, s2, b2 = O.quantize(make_w(7, (E, N2, K2), "bf16"), g, 4, "bf16")
    x2 = make_x(8, (tokens, 1, K2), "bf16")
    rng = np.random.default_rng(3)
    rhs = rng.permuted(np.tile(np.arange(E), (tokens, 1)), axis=1)[:, :topk].astype(np.uint32)
    lhs = np.broadcast_to(np.arange(tokens, dtype=np.uint32)[:, None], rhs.shape).copy()
    lo, hi = expert_bounds(E, rank, world)
    out2 = PeerOutput(tokens * topk, N2)
    ref2 = O.gather_qmm(O.to_f32(x2, "bf16"), wq2, O.to_f32(s2, "bf16"), O.to_f32(b2, "bf16"), lhs.ravel(), rhs.ravel(),
                        True, g, 4, "f32")
    for step in range(3):
        y2 = sharded_gather_qmm(to_torch(x2, "bf16"), u32_to_torch(wq2[lo:hi]), to_torch(s2[lo:hi], "bf16"),
                                to_torch(b2[lo:hi], "bf16"), torch.from_numpy(lhs.astype(np.int64)),
                                torch.from_numpy(rhs.astype(np.int64)), lo, E, out2, g, 4)
        torch.cuda.synchronize()
        good, rel = qmm_close(O.to_f32(from_torch(y2.contiguous()), "bf16").reshape(ref2.shape), ref2)
        print(f"rank {rank} gather step {step} ok={good} rel={rel:.4f}", flush=True)
        ok = ok and good
        dist.barrier()
    out2.close()

    # ---- K-sharded linear: partial products summed over the ranks (fused exchange)
    N3, K3 = 512, 2048
    wq3, s3, b3 = O.quantize(make_w(9, (N3, K3), "bf16"), g, 4, "bf16")
    down = QuantizedShardedToAllLinear(u32_to_torch(wq3), to_torch(s3, "bf16"), to_torch(b3, "bf16"), g, 4, rank=rank, world=world)
    out3 = PeerOutput(world * 40, N3)
    for step, M in enumerate((16, 40, 3)):
        x3 = make_x(30 + step, (M, K3), "bf16")
        y3 = sharded_matmul_allreduce(down, to_torch(x3, "bf16"), out3)
        torch.cuda.synchronize()
        ref3 = O.qmm_f32_from(x3, wq3, s3, b3, "bf16", transpose=True, group_size=g, bits=4)
        good, rel = qmm_close(O.to_f32(from_torch(y3), "bf16"), ref3)
        # every rank must hold bit-identical results (same slots, same order of additions)
        mine = y3.view(torch.int16).cpu().to(torch.int32)   # gloo has no int16 collectives
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        same = all(torch.equal(both[0], t) for t in both)
        print(f"rank {rank} allreduce step {step} M={M} ok={good} rel={rel:.4f} identical={same}", flush=True)
        ok = ok and good and same
        dist.barrier()
    out3.close()
    dist.destroy_process_group()
    print(f"rank {rank} {'PEER-OK' if ok else 'PEER-FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
