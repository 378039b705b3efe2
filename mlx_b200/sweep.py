"""Measures every configuration the reference benchmark description names, through the C ABI.

    python -m mlx_b200.sweep [--quick]

One JSON line per case: kernel-only time (CUDA events around a CUDA graph of repeated calls,
weights rotated over enough copies to exceed the 126 MB L2), algorithmic bytes / flops, and
the fraction of the measured HBM and bf16 tensor peaks (MEASURED_PEAKS.json next to the repo
root when present, else 6650 GB/s / 1590 TFLOP/s).

Cases: C1 decode GEMV (M=1, 4096x4096), C2 small-batch decode (M=16, 14336x4096), C3 prefill
(M=4096), C4 bit-width / group sweep on the 70B-MLP shape (K=8192, N=28672; bits 3/6/8 x group
32/128 at M 1 and 512) plus quantize / dequantize of that matrix, C5 Mixtral-style gather_qmm
(8 experts, 512 tokens, top-2), T0 the non-transposed decode form.  Inputs are seeded synthetic draws (x ~ N(0,1), W ~ N(0,0.02)).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import numpy as np
import torch

from . import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = lambda t: ctypes.c_void_p(t.data_ptr())


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def graph_time(fn, iters, stream):
    """Seconds per call of fn(i): `iters` calls captured in one CUDA graph, replayed twice."""
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        g.replay()
        e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / iters


def make_weights(N, K, bits, group, copies, seed=2):
    out = []
    for c in range(copies):
        g = torch.Generator(device="cuda").manual_seed(seed + c)
        w = (0.02 * torch.randn(N, K, device="cuda", generator=g)).to(torch.bfloat16)
        out.append(ops.quantize(w, group, bits))
        del w
    return out


def qmm_case(tag, M, N, K, bits, group, iters, transpose=True):
    lib = _lib.load()
    hbm, tf, src = peaks()
    wbytes = N * K * bits // 8 + 4 * N * K // group
    copies = max(1, min(16, int(np.ceil(2 * 126e6 / wbytes)))) if M <= 64 else 1
    ws_list = make_weights(N, K, bits, group, copies) if transpose else make_weights(K, N, bits, group, copies)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    tr = 1 if transpose else 0
    need = max(int(lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M, N, K, group, bits, tr)), 256)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    st = torch.cuda.Stream()
    sp = ctypes.c_void_p(st.cuda_stream)

    def call(i):
        q, s, b = ws_list[i % copies]
        rc = lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M, N, K, group, bits, tr, 0, P(ws), ws.numel(), sp)
        if rc:
            raise RuntimeError(_lib.last_error())

    t = graph_time(call, iters, st)
    B = wbytes + M * K * 2 + M * N * 2
    F = 2.0 * M * N * K
    rec = {"case": tag, "op": "quantized_matmul" if transpose else "quantized_matmul(transpose=False)", "M": M, "N": N, "K": K, "bits": bits, "group": group,
           "kernel": lib.b200q_qmm_kernel_name(_lib.BF16, 1, M, N, K, group, bits, tr).decode(), "us": t * 1e6,
           "GBps": B / t / 1e9, "TFLOPs": F / t / 1e12, "frac_hbm": B / t / 1e9 / hbm, "frac_tensor": F / t / 1e12 / tf,
           "weight_copies": copies, "peaks": src}
    print(json.dumps(rec), flush=True)
    del ws_list


def quant_case(tag, N, K, bits, group, iters):
    lib = _lib.load()
    hbm, _, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(2)
    w = (0.02 * torch.randn(N, K, device="cuda", generator=g)).to(torch.bfloat16)
    wq = torch.empty(N, K * bits // 32, dtype=torch.int32, device="cuda")
    s = torch.empty(N, K // group, dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(s)
    out = torch.empty_like(w)
    st = torch.cuda.Stream()
    sp = ctypes.c_void_p(st.cuda_stream)
    tq = graph_time(lambda i: lib.b200q_quantize(P(w), _lib.BF16, N, K, group, bits, P(wq), P(s), P(b), sp), iters, st)
    td = graph_time(lambda i: lib.b200q_dequantize(P(wq), P(s), P(b), _lib.BF16, N, K, group, bits, P(out), sp), iters, st)
    B = N * K * 2 + N * K * bits // 8 + 4 * N * K // group
    for op, t in (("quantize", tq), ("dequantize", td)):
        print(json.dumps({"case": tag, "op": op, "N": N, "K": K, "bits": bits, "group": group, "us": t * 1e6,
                          "GBps": B / t / 1e9, "frac_hbm": B / t / 1e9 / hbm, "peaks": src}), flush=True)


def gather_case(tag, E, tokens, topk, N, K, bits, group, iters):
    lib = _lib.load()
    hbm, tf, src = peaks()
    ws_list = make_weights(N, K, bits, group, E, seed=100)
    wq = torch.stack([w[0].view(torch.int32) for w in ws_list])
    s = torch.stack([w[1] for w in ws_list])
    b = torch.stack([w[2] for w in ws_list])
    del ws_list
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(tokens, K, device="cuda", generator=g).to(torch.bfloat16)
    rng = np.random.default_rng(3)
    rhs = rng.permuted(np.tile(np.arange(E), (tokens, 1)), axis=1)[:, :topk].astype(np.int32)
    lhs = np.broadcast_to(np.arange(tokens, dtype=np.int32)[:, None], rhs.shape).copy()
    rhs_t, lhs_t = torch.from_numpy(rhs.ravel()).cuda(), torch.from_numpy(lhs.ravel()).cuda()
    n_idx = tokens * topk
    y = torch.empty(n_idx, N, device="cuda", dtype=torch.bfloat16)
    need = int(lib.b200q_gather_qmm_workspace_bytes(_lib.BF16, n_idx, tokens, E, 1, N, K, group, bits, 1))
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    st = torch.cuda.Stream()
    sp = ctypes.c_void_p(st.cuda_stream)

    def call(i):
        rc = lib.b200q_gather_qmm(P(x), P(wq), P(s), P(b), P(lhs_t), P(rhs_t), n_idx, P(y), _lib.BF16, tokens, E, 1, N, K,
                                  group, bits, 1, 0, P(ws), ws.numel(), sp)
        if rc:
            raise RuntimeError(_lib.last_error())

    t = graph_time(call, iters, st)
    B = E * (N * K * bits // 8 + 4 * N * K // group) + tokens * K * 2 + n_idx * N * 2 + 8 * n_idx
    F = 2.0 * n_idx * N * K
    print(json.dumps({"case": tag, "op": "gather_qmm", "experts": E, "tokens": tokens, "top_k": topk, "N": N, "K": K,
                      "bits": bits, "group": group, "us": t * 1e6, "GBps": B / t / 1e9, "TFLOPs": F / t / 1e12,
                      "frac_hbm": B / t / 1e9 / hbm, "frac_tensor": F / t / 1e12 / tf, "peaks": src}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="fewer iterations and no 70B-shape sweep")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: there is no CPU fallback")
    it = 10 if a.quick else 40
    qmm_case("C1", 1, 4096, 4096, 4, 64, it)
    qmm_case("C2", 16, 14336, 4096, 4, 64, it)
    qmm_case("C3", 4096, 14336, 4096, 4, 64, max(it // 4, 3))
    if not a.quick:
        for bits in (3, 6, 8):
            for group in (32, 128):
                qmm_case("C4", 1, 28672, 8192, bits, group, 10)
                qmm_case("C4", 512, 28672, 8192, bits, group, 4)
        for bits, group in ((3, 32), (6, 128), (8, 32), (4, 64)):
            quant_case("C4", 28672, 8192, bits, group, 4)
    gather_case("C5", 8, 512, 2, 14336, 4096, 4, 64, max(it // 4, 3))
    if not a.quick:
        # the non-transposed form (vector-Jacobian product of the decode matmul)
        qmm_case("T0", 1, 4096, 4096, 4, 64, it, transpose=False)
        qmm_case("T0", 1, 28672, 8192, 4, 64, 10, transpose=False)
        qmm_case("T0", 4, 4096, 14336, 8, 64, 10, transpose=False)


if __name__ == "__main__":
    main()
