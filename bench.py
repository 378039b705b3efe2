#!/usr/bin/env python
"""Benchmark of the affine quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--gather fused|nccl] [--config headline|all] [--no-prefill] [--no-moe] [--no-cpu]

Headline workload: the small-batch decode configuration - x [16, 4096] bf16 ~ N(0,1),
W [14336, 4096] ~ N(0, 0.02) quantized at 4 bits / group 64 (Llama-3-8B MLP up-projection),
`quantized_matmul(transpose=True)`.  A step is one call on one batch; successive steps use
different weight copies (enough of them to exceed twice the 126 MB L2 per rank) so every step
streams from HBM.  With N > 1 ranks the weight rows are split evenly across ranks (strong
scaling of the same matrix) and a step ends with the all_gather of the per-rank outputs, fused
into the matmul epilogue (peer stores + completion flags) or, with --gather nccl, by NCCL.

One JSON line is printed by rank 0 (last line of stdout).  `value` is the device-timed
throughput in algorithmic GB/s with inputs resident in HBM; `e2e` is the same metric through
the host-buffer path (pinned host x in, the full gathered y out, copies and a synchronise per
step inside the timed region); `roofline` relates the decode kernel to the measured HBM peak;
`prefill` reports the tensor-core path on the M = 4096 configuration, exchange included at
N > 1; `moe` the Mixtral-style gather_qmm configuration (experts split over the ranks);
`parity` says whether sampled outputs of each leg - taken from rank 0's GATHERED result, columns
from every rank's block - agree with the CPU checker; `cpu_baseline` times the reference
project's own CPU code.  `--config all` first prints one line per case of the other named
configurations (GEMV, bit-width / group sweep with quantize / dequantize, non-transposed
decode), each with its own parity result.  `--impl reference` times only the reference CPU
code (all host cores) and prints its own line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "4-bit g64 qmm: decode GB/s & prefill TFLOPS at 1/2/4/8 B200 vs roofline"
M_DEC, N_DEC, K_DEC, GROUP, BITS = 16, 14336, 4096, 64, 4
M_PRE = 4096
E_MOE, TOK_MOE, TOPK_MOE = 8, 512, 2
L2_BYTES = 126e6
WORKLOAD = (f"decode quantized_matmul M={M_DEC} N={N_DEC} K={K_DEC} bits={BITS} group={GROUP} transpose=True "
            "(Llama-3-8B MLP up-projection)")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel on the one-GPU
# workload, from an ncu capture of that kernel (a constant, not measured in this run; with the
# matrix split over R ranks the per-rank traffic is this divided by R: it is all weight stream)
TRAFFIC_FROM_PROFILE = {"qmv_rows": 33222400, "qmv_mma": 33494784}


def algorithmic_bytes(M, N, K, bits=BITS, group=GROUP):
    return N * K * bits // 8 + 2 * (N * K // group) * 2 + M * K * 2 + M * N * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        top = sorted(sm)[len(sm) // 2:]  # the upper half: samples taken under load
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------ CPU reference arm
def cpu_reference_run(cores: int, reps: int):
    """Times the reference project's CPU quantized_matmul (oracle/_ref/ref_oracle when it was
    compiled, else the C restatement) on the decode workload: `cores` processes, each on an
    independent slice of the weight rows, wall time = slowest process."""
    import oracle as O

    rng = np.random.default_rng(2)
    n_per = N_DEC // cores // 16 * 16
    w = (0.02 * rng.standard_normal((n_per, K_DEC))).astype(np.float32)
    wq, s, b = O.quantize(O.to_f32(O.to_dtype(w, "bf16"), "bf16"), GROUP, BITS, "f32")
    x = O.to_f32(O.to_dtype(np.random.default_rng(1).standard_normal((M_DEC, K_DEC)).astype(np.float32), "bf16"), "bf16")
    kind = "reference" if O.have_reference() else "port"
    t0 = time.perf_counter()
    if kind == "reference":
        with tempfile.TemporaryDirectory() as d:
            files = {}
            for name, arr in (("x", x), ("wq", wq), ("s", s), ("b", b)):
                files[name] = os.path.join(d, name + ".bin")
                np.ascontiguousarray(arr).tofile(files[name])
            procs = [subprocess.Popen(
                [O.REF_BIN, "qmm", "f32", str(M_DEC), str(n_per), str(K_DEC), str(GROUP), str(BITS), "1",
                 files["x"], files["wq"], files["s"], files["b"], os.path.join(d, f"y{i}.bin"), str(reps)],
                stdout=subprocess.PIPE, text=True) for i in range(cores)]
            secs = []
            for p in procs:
                out, _ = p.communicate()
                secs.append(float(out.split()[-1]))
        per_call = max(secs)
    else:
        best = 1e30
        for _ in range(reps):
            t = time.perf_counter()
            O.qmm(x, wq, s, b, True, GROUP, BITS, "f32")
            best = min(best, time.perf_counter() - t)
        per_call, cores = best, 1
    wall = time.perf_counter() - t0
    rows = n_per * cores
    gbs = algorithmic_bytes(M_DEC, rows, K_DEC) / per_call / 1e9
    sample = (f"{kind} CPU _qmm_t<float,4,64>: x [{M_DEC},{K_DEC}] against {rows} of {N_DEC} weight rows "
              f"({cores} process(es) x {n_per} rows), best of {reps} calls, {wall:.1f} s of wall time")
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample}, per_call


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    reps = max(1, min(args.steps, 5))
    for _ in range(min(args.warmup, 1)):
        cpu_reference_run(cores, 1)
    base, per_call = cpu_reference_run(cores, reps)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_call * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "arm": "the reference project's CPU code on the host cores, a bounded sample "
                                                "of the workload (see cpu_baseline.sample)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------ helpers of the GPU arm
def carrier(t):
    """bf16 torch tensor -> the checker's uint16 carrier array."""
    import torch
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def close_enough(got: np.ndarray, ref: np.ndarray, rel=1e-2):
    """|y - y_ref| <= rel |y_ref| + rel rms(y_ref), the tolerance of the parity tests."""
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref ** 2))) if ref.size else 0.0
    return bool(np.all(np.abs(got - ref) <= rel * np.abs(ref) + rel * rms + 1e-30))


def oracle_columns(w_rows_bf16: np.ndarray, x_bf16: np.ndarray, bits=BITS, group=GROUP):
    """Checker result for the given weight rows (uint16 carrier of the bf16 weights BEFORE
    quantization): quantize and multiply on the CPU with the reference's arithmetic."""
    import oracle as O
    wq, s, b = O.quantize(w_rows_bf16, group, bits, "bf16")
    return O.qmm_f32_from(x_bf16, wq, s, b, "bf16", transpose=True, group_size=group, bits=bits)


def queue_delay(torch, stream):
    """About 100 us of spinning queued on `stream` ahead of a start event: the work that follows is
    already enqueued when the event's time is taken, so the interval holds device time only, not the
    host's launch latency (which is as long as several steps of this workload)."""
    with torch.cuda.stream(stream):
        torch.cuda._sleep(200000)


def graph_time(fn, iters, stream, torch):
    """Seconds per call of fn(i): `iters` calls captured in one CUDA graph, best of three replays."""
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
    best = 1e30
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        queue_delay(torch, stream)
        with torch.cuda.stream(stream):
            e0.record(stream)
            g.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3 / iters)
    return best


# ------------------------------------------------------------------------ other named configurations
def sweep_cases(lib, _lib, mb, torch, dev, quick=False):
    """One JSON line per case of the configurations other than the headline one, each with a
    parity result against the CPU checker (one GPU; run by --config all on rank 0)."""
    import oracle as O
    hbm, tf, src = measured_peaks()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = torch.cuda.Stream(device=dev)
    sp = ctypes.c_void_p(stream.cuda_stream)

    def qmm_case(tag, M, N, K, bits, group, iters, transpose=True):
        wbytes = N * K * bits // 8 + 4 * N * K // group
        copies = max(1, min(16, int(math.ceil(2 * L2_BYTES / wbytes)))) if M <= 64 else 1
        ws_list, w0 = [], None
        for c in range(copies):
            g = torch.Generator(device=dev).manual_seed(2 + c)
            shape = (N, K) if transpose else (K, N)
            w = (0.02 * torch.randn(*shape, device=dev, generator=g)).to(torch.bfloat16)
            ws_list.append(mb.quantize(w, group, bits))
            if c == 0:
                w0 = w
            else:
                del w
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        tr = 1 if transpose else 0
        need = max(int(lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M, N, K, group, bits, tr)), 256)
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)

        def call(i):
            q, s, b = ws_list[i % copies]
            rc = lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M, N, K, group, bits, tr, 0, P(ws), ws.numel(), sp)
            if rc:
                raise RuntimeError(_lib.last_error())
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            call(0)
        torch.cuda.synchronize()
        # parity on sampled token rows (all outputs of those rows)
        rows = np.unique(np.concatenate([[0, M - 1], np.random.default_rng(5).integers(0, M, 4)]))[:6]
        q0, s0, b0 = ws_list[0]
        q0_np = q0.view(torch.int32).cpu().numpy().view(np.uint32)
        ref = O.qmm_f32_from(carrier(x)[rows], q0_np, carrier(s0), carrier(b0), "bf16", transpose=transpose,
                             group_size=group, bits=bits)
        got = O.to_f32(carrier(y)[rows], "bf16")
        ok = close_enough(got, ref)
        del w0
        t = graph_time(call, iters, stream, torch)
        B = wbytes + M * K * 2 + M * N * 2
        F = 2.0 * M * N * K
        print(json.dumps({"case": tag, "op": "quantized_matmul" if transpose else "quantized_matmul(transpose=False)",
                          "M": M, "N": N, "K": K, "bits": bits, "group": group,
                          "kernel": lib.b200q_qmm_kernel_name(_lib.BF16, 1, M, N, K, group, bits, tr).decode(),
                          "us": t * 1e6, "GBps": B / t / 1e9, "TFLOPs": F / t / 1e12, "frac_hbm": B / t / 1e9 / hbm,
                          "frac_tensor": F / t / 1e12 / tf, "weight_copies": copies, "matches_oracle": ok, "peaks": src}),
              flush=True)
        del ws_list

    def quant_case(tag, N, K, bits, group, iters):
        g = torch.Generator(device=dev).manual_seed(2)
        w = (0.02 * torch.randn(N, K, device=dev, generator=g)).to(torch.bfloat16)
        wq = torch.empty(N, K * bits // 32, dtype=torch.int32, device=dev)
        s = torch.empty(N, K // group, dtype=torch.bfloat16, device=dev)
        b = torch.empty_like(s)
        out = torch.empty_like(w)
        tq = graph_time(lambda i: lib.b200q_quantize(P(w), _lib.BF16, N, K, group, bits, P(wq), P(s), P(b), sp), iters, stream, torch)
        td = graph_time(lambda i: lib.b200q_dequantize(P(wq), P(s), P(b), _lib.BF16, N, K, group, bits, P(out), sp), iters, stream, torch)
        # bit-exactness on a band of rows
        rows = slice(0, 256)
        rq, rs, rb = O.quantize(carrier(w[rows]), group, bits, "bf16")
        ok_q = (np.array_equal(wq[rows].cpu().numpy().view(np.uint32), rq) and np.array_equal(carrier(s[rows]), rs)
                and np.array_equal(carrier(b[rows]), rb))
        ok_d = np.array_equal(carrier(out[rows]), O.dequantize(rq, rs, rb, group, bits, "bf16"))
        B = N * K * 2 + N * K * bits // 8 + 4 * N * K // group
        for op, t, ok in (("quantize", tq, ok_q), ("dequantize", td, ok_d)):
            print(json.dumps({"case": tag, "op": op, "N": N, "K": K, "bits": bits, "group": group, "us": t * 1e6,
                              "GBps": B / t / 1e9, "frac_hbm": B / t / 1e9 / hbm, "bit_exact_vs_oracle": bool(ok), "peaks": src}),
                  flush=True)

    it = 10 if quick else 40
    qmm_case("C1", 1, 4096, 4096, 4, 64, it)
    for bits in (3, 6, 8):
        for group in (32, 128):
            qmm_case("C4", 1, 28672, 8192, bits, group, 10)
            qmm_case("C4", 512, 28672, 8192, bits, group, 4)
    for bits, group in ((3, 32), (6, 128), (8, 32), (4, 64)):
        quant_case("C4", 28672, 8192, bits, group, 4)
    # decode shapes around the headline one: the down projection, larger batches, the 70B shape
    for (M, N, K, bits) in ((1, 4096, 14336, 4), (16, 4096, 14336, 4), (1, 28672, 8192, 4), (16, 28672, 8192, 4),
                            (32, 14336, 4096, 4), (64, 14336, 4096, 4), (1, 8192, 28672, 4), (16, 28672, 8192, 8)):
        qmm_case("D", M, N, K, bits, 64, 10)
    # the non-transposed form (vector-Jacobian product of the decode matmul)
    qmm_case("T0", 1, 4096, 4096, 4, 64, it, transpose=False)
    qmm_case("T0", 1, 28672, 8192, 4, 64, 10, transpose=False)
    qmm_case("T0", 4, 4096, 14336, 8, 64, 10, transpose=False)


# ------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200q")
    ap.add_argument("--gather", default="fused", choices=("fused", "nccl"),
                    help="N > 1: all_gather fused into the matmul epilogue (peer stores) or the NCCL collective")
    ap.add_argument("--config", default="headline", choices=("headline", "all"))
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-moe", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    import mlx_b200 as mb
    from mlx_b200 import _lib
    from mlx_b200.distributed import (PeerOutput, QuantizedAllToShardedLinear, all_gather_columns, expert_bounds,
                                      shard_bounds, sharded_gather_qmm, sharded_matmul_allgather)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    # The weights of this benchmark are constants (as in inference): the decode kernel may request
    # them while the previous kernel of the stream is still finishing.
    mb.set_weights_constant(True)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    hbm_peak, tf_peak, peak_src = measured_peaks()

    if args.config == "all" and rank == 0:
        sweep_cases(lib, _lib, mb, torch, dev)
    if world > 1:
        dist.barrier()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def align_ranks():
        """N > 1: a one-element all_reduce on the timing stream right before a timed interval.  The host
        barrier lets the ranks go hundreds of microseconds apart, and a rank that starts late keeps the
        others waiting for its flags inside their interval; after the collective all streams continue
        within a few microseconds of each other."""
        if world > 1:
            with torch.cuda.stream(stream):
                dist.all_reduce(torch.zeros(1, device=dev))

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- synthetic inputs: this rank's row shard of enough weight copies to exceed 2 x L2
    lo, hi = shard_bounds(N_DEC, rank, world)
    n_loc = hi - lo
    shard_bytes = algorithmic_bytes(0, n_loc, K_DEC)
    copies = max(8, min(96, int(math.ceil(2 * L2_BYTES / shard_bytes))))
    weights, w0_full = [], None
    for c in range(copies):
        g = torch.Generator(device=dev).manual_seed(100 + c)
        w = (0.02 * torch.randn(N_DEC, K_DEC, device=dev, generator=g)).to(torch.bfloat16)
        weights.append(mb.quantize(w[lo:hi].contiguous(), GROUP, BITS))
        if c == 0 and rank == 0:
            w0_full = w      # kept for the parity check against the CPU checker
        else:
            del w
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(M_DEC, K_DEC, device=dev, generator=g).to(torch.bfloat16)
    y = torch.empty(M_DEC, n_loc, device=dev, dtype=torch.bfloat16)
    ws_bytes = max(int(lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1)), 256)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    kernel = lib.b200q_qmm_kernel_name(_lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1).decode()

    class Gather:  # cache holder for the all_gather staging buffer
        _gather_buf = None

    # N > 1: by default the all_gather is fused into the matmul epilogue (peer stores into every
    # rank's output buffer, flags raised by the kernel's last thread block, one bounded wait);
    # --gather nccl runs the collective instead.
    fused = world > 1 and args.gather == "fused"
    peer_out = None
    if fused:
        try:
            peer_out = PeerOutput(M_DEC, N_DEC)
        except RuntimeError as e:   # raised on every rank together: fall back to the collective
            if rank == 0:
                print(f"bench: fused gather unavailable ({e}); using NCCL", file=sys.stderr)
            fused = False
    layers = [QuantizedAllToShardedLinear(q, s, b, GROUP, BITS, rank=rank, world=world, already_sharded=True)
              for (q, s, b) in weights] if world > 1 else None

    def step(i, chained=False):
        """One step: the matmul on this rank's rows and, at N > 1, the exchange; returns the full [M, N].
        chained: the wait for a step's exchange sits in the next step's kernel; the chain is closed by
        peer_out.wait().  "buffers" (x is a replicated input, as in the workload): only the stores into
        the exchange buffers wait; True (x would be the previous step's gathered output): the loads wait too."""
        if fused:
            return sharded_matmul_allgather(layers[i % copies], x, peer_out, chained=chained)
        q, s, b = weights[i % copies]
        rc = lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1, 0,
                           P(ws), ws.numel(), sp)
        if rc != 0:
            raise RuntimeError(_lib.last_error())
        if world > 1:
            return all_gather_columns(y, None, world, cache=Gather)
        return y

    # ---- parity of the (gathered) result against the CPU checker, sampled columns of every rank's block
    parity = {}
    barrier()
    with torch.cuda.stream(stream):
        y_full = step(0)
    barrier()
    if fused:
        peer_out.check()
    if rank == 0:
        rng = np.random.default_rng(11)
        per = N_DEC // world
        cols = np.concatenate([r * per + np.sort(rng.choice(per, 8, replace=False)) for r in range(world)])
        ref = oracle_columns(carrier(w0_full[torch.from_numpy(cols).to(dev)]), carrier(x))
        import oracle as O
        got = O.to_f32(carrier(y_full[:, torch.from_numpy(cols).to(dev)]), "bf16")
        parity["decode_gathered_matches_oracle"] = close_enough(got, ref)
        parity["decode_columns_checked"] = int(cols.size)
    del w0_full

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
    barrier()

    # ---- device-timed region: exactly `steps` steps on the launching stream, replayed from a CUDA
    # graph (no host launch gaps); with the NCCL collective in the step they run eagerly.
    sampler = ClockSampler(local_rank)
    launches0 = lib.b200q_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graphed = world == 1 or fused
    if graphed:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(args.steps):
                step(i, chained="buffers")
            if fused:
                peer_out.wait()   # closes the chain: every step's result is complete on every rank
        launches = int(lib.b200q_launch_count() - launches0)
        graph.replay()  # one untimed replay to settle the instantiated graph
        barrier()
        sampler.start()
        time.sleep(0.3)
        barrier()
        align_ranks()
        queue_delay(torch, stream)
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        barrier()
    else:
        sampler.start()
        time.sleep(0.3)
        barrier()
        align_ranks()
        queue_delay(torch, stream)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(args.steps):
                step(i)
            e1.record(stream)
        barrier()
        launches = int(lib.b200q_launch_count() - launches0)
    clocks = sampler.stop()
    ms_per_step = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    total_bytes = algorithmic_bytes(M_DEC, N_DEC, K_DEC)
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    if fused:
        peer_out.check()
    # the same steps as a dependent chain (every kernel also holds its x loads until all ranks have
    # finished the previous step, as if x were that step's gathered output): reported beside the headline
    ms_dependent = None
    if fused:
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=stream):
            for i in range(args.steps):
                step(i, chained=True)
            peer_out.wait()
        g2.replay()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        align_ranks()
        queue_delay(torch, stream)
        with torch.cuda.stream(stream):
            f0.record(stream)
            g2.replay()
            f1.record(stream)
        barrier()
        ms_dependent = max_over_ranks(f0.elapsed_time(f1)) / args.steps
        peer_out.check()

    # ---- kernel-only duration for the roofline (same stream, events around kernel launches only)
    def kernel_only(i):
        q, s, b = weights[i % copies]
        lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1, 0, P(ws), ws.numel(), sp)
    kernel_s = graph_time(kernel_only, args.steps, stream, torch)
    achieved = algorithmic_bytes(M_DEC, n_loc, K_DEC) / kernel_s / 1e9
    traffic = TRAFFIC_FROM_PROFILE.get(kernel)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": (traffic // world if traffic else None),
                "traffic_source": "constant from an ncu capture of this kernel on the one-GPU workload, divided by the rank count "
                                  "(not measured in this run)",
                "kernel": kernel, "kernel_us": kernel_s * 1e6, "peak_source": peak_src}

    # ---- end to end: pinned host x in, the FULL [M, N] result out, synchronised every step
    x_host = torch.empty(M_DEC, K_DEC, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    y_host = torch.empty(M_DEC, N_DEC, dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(x)
    if world == 1:
        def e2e_step(i):
            q, s, b = weights[i % copies]
            rc = lib.b200q_qmm_host(P(x_host), P(x_dev), P(q), P(s), P(b), P(y), P(y_host), _lib.BF16, M_DEC, N_DEC, K_DEC,
                                    GROUP, BITS, 1, P(ws), ws.numel(), sp)
            if rc != 0:
                raise RuntimeError(_lib.last_error())
        e2e_note = "b200q_qmm_host: pinned x -> device, kernel, y -> pinned host, synchronised every step"
    else:
        def e2e_step(i):
            with torch.cuda.stream(stream):
                x_dev.copy_(x_host, non_blocking=True)
                if fused:
                    full = sharded_matmul_allgather(layers[i % copies], x_dev, peer_out)
                else:
                    q, s, b = weights[i % copies]
                    lib.b200q_qmm(P(x_dev), P(q), P(s), P(b), P(y), _lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1, 0,
                                  P(ws), ws.numel(), sp)
                    full = all_gather_columns(y, None, world, cache=Gather)
                y_host.copy_(full, non_blocking=True)
        e2e_note = ("pinned x -> device, sharded matmul with the gather (" + ("fused" if fused else "NCCL") +
                    "), the full gathered [M, N] -> pinned host on every rank, synchronised every step")
    for i in range(args.warmup):
        e2e_step(i)
        stream.synchronize()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
        stream.synchronize()  # the caller reads y_host after every step
    e2e_s = max_over_ranks((time.perf_counter() - t0) / args.steps)
    e2e = {"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": M_DEC * K_DEC * 2,
           "d2h_bytes_per_step": M_DEC * N_DEC * 2, "ms_per_step": e2e_s * 1e3,
           "note": e2e_note + "; weights stay resident in HBM"}
    # the host copy of the last e2e step against the device result of the same weights
    with torch.cuda.stream(stream):
        y_dev_last = step(args.steps - 1)
        y_dev_last = y_dev_last.float().cpu()
    torch.cuda.synchronize(dev)
    barrier()
    e2e_gap = float((y_host.float() - y_dev_last).abs().max())
    parity["e2e_matches_device"] = bool(e2e_gap == 0.0)

    # ---- prefill configuration on the tensor-core path; at N > 1 through the sharded operator, the
    # exchange inside the timed region (fused peer stores + flags, and the NCCL collective beside it)
    prefill = None
    if not args.no_prefill:
        xp = torch.randn(M_PRE, K_DEC, device=dev, generator=g).to(torch.bfloat16)
        yp = torch.empty(M_PRE, n_loc, device=dev, dtype=torch.bfloat16)
        reps = 10
        peer_pre = None
        if world > 1:
            try:
                peer_pre = PeerOutput(M_PRE, N_DEC)
            except RuntimeError:
                peer_pre = None

        def pre_local(i):
            q, s, b = weights[i % copies]
            rc = lib.b200q_qmm(P(xp), P(q), P(s), P(b), P(yp), _lib.BF16, 1, M_PRE, n_loc, K_DEC, GROUP, BITS, 1, 0,
                               P(ws), ws.numel(), sp)
            if rc != 0:
                raise RuntimeError(_lib.last_error())
            return yp

        def timed(fn):
            with torch.cuda.stream(stream):
                for i in range(3):
                    fn(i)
            barrier()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                p0.record(stream)
                for i in range(reps):
                    out = fn(i)
                p1.record(stream)
            barrier()
            return max_over_ranks(p0.elapsed_time(p1)) / reps, out

        flops = 2.0 * M_PRE * N_DEC * K_DEC
        if world == 1:
            ms_f, full = timed(pre_local)
            ms_n = None
        else:
            ms_n, full_n = timed(lambda i: all_gather_columns(pre_local(i), None, world, cache=Gather))
            if peer_pre is not None:
                ms_f, full = timed(lambda i: sharded_matmul_allgather(layers[i % copies], xp, peer_pre))
                peer_pre.check()
            else:
                ms_f, full = None, full_n
        ms_local, _ = timed(pre_local)
        # parity: sampled token rows of the gathered result, sampled columns of every rank's block
        if rank == 0:
            gw = torch.Generator(device=dev).manual_seed(100 + (reps - 1) % copies)
            wl = (0.02 * torch.randn(N_DEC, K_DEC, device=dev, generator=gw)).to(torch.bfloat16)
            rng = np.random.default_rng(12)
            per = N_DEC // world
            cols = np.concatenate([r * per + np.sort(rng.choice(per, 8, replace=False)) for r in range(world)])
            rows = np.array([0, 255, 256, 1023, 2048, M_PRE - 1])
            ref = oracle_columns(carrier(wl[torch.from_numpy(cols).to(dev)]), carrier(xp)[rows])
            import oracle as O
            got = O.to_f32(carrier(full[torch.from_numpy(rows).to(dev)][:, torch.from_numpy(cols).to(dev)]), "bf16")
            parity["prefill_gathered_matches_oracle"] = close_enough(got, ref)
            del wl
        best_ms = ms_f if ms_f is not None else ms_n
        prefill = {"workload": f"prefill quantized_matmul M={M_PRE} N={N_DEC} K={K_DEC} bits={BITS} group={GROUP}, N-sharded over the "
                               "ranks" + (", all_gather of the outputs inside the timed region" if world > 1 else ""),
                   "value": flops / (best_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": best_ms,
                   "ms_fused_gather": ms_f if world > 1 else None, "ms_nccl_gather": ms_n, "ms_local_matmul_only": ms_local,
                   "kernel": lib.b200q_qmm_kernel_name(_lib.BF16, 1, M_PRE, n_loc, K_DEC, GROUP, BITS, 1).decode(),
                   "roofline": {"bound": "tensor", "achieved": flops / world / (ms_local * 1e-3) / 1e12, "peak": tf_peak,
                                "unit": "TFLOP/s", "frac": flops / world / (ms_local * 1e-3) / 1e12 / tf_peak,
                                "note": "per GPU, matmul kernel alone", "peak_source": peak_src}}
        if peer_pre is not None:
            peer_pre.close()
        del xp, yp

    # ---- Mixtral-style MoE layer: 8 experts [14336, 4096], 512 tokens, top-2; experts split over the ranks
    moe = None
    if not args.no_moe and E_MOE % world == 0:
        import oracle as O
        elo, ehi = expert_bounds(E_MOE, rank, world)
        wq_e, s_e, b_e, w_keep = [], [], [], {}
        for e in range(elo, ehi):
            ge = torch.Generator(device=dev).manual_seed(1000 + e)
            w = (0.02 * torch.randn(N_DEC, K_DEC, device=dev, generator=ge)).to(torch.bfloat16)
            q, s, b = mb.quantize(w, GROUP, BITS)
            wq_e.append(q.view(torch.int32)); s_e.append(s); b_e.append(b)
            del w
        wq_l = torch.stack(wq_e).view(torch.uint32)
        s_l, b_l = torch.stack(s_e), torch.stack(b_e)
        del wq_e, s_e, b_e
        gx = torch.Generator(device=dev).manual_seed(3)
        xm = torch.randn(TOK_MOE, 1, K_DEC, device=dev, generator=gx).to(torch.bfloat16)
        rng = np.random.default_rng(3)
        rhs = rng.permuted(np.tile(np.arange(E_MOE), (TOK_MOE, 1)), axis=1)[:, :TOPK_MOE].astype(np.int64)
        lhs = np.broadcast_to(np.arange(TOK_MOE, dtype=np.int64)[:, None], rhs.shape).copy()
        rhs_t, lhs_t = torch.from_numpy(rhs).to(dev), torch.from_numpy(lhs).to(dev)
        n_idx = TOK_MOE * TOPK_MOE
        peer_moe = None
        if world > 1:
            try:
                peer_moe = PeerOutput(n_idx, N_DEC)
            except RuntimeError:
                peer_moe = None
        if world == 1:
            moe_fn = lambda i: mb.gather_qmm(xm, wq_l, s_l, b_l, lhs_indices=lhs_t, rhs_indices=rhs_t, group_size=GROUP, bits=BITS)
        elif peer_moe is not None:
            moe_fn = lambda i: sharded_gather_qmm(xm, wq_l, s_l, b_l, lhs_t, rhs_t, elo, E_MOE, peer_moe, GROUP, BITS)
        else:
            moe_fn = None
        if moe_fn is not None:
            reps = 10
            with torch.cuda.stream(stream):
                for i in range(3):
                    ym = moe_fn(i)
            barrier()
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                m0.record(stream)
                for i in range(reps):
                    ym = moe_fn(i)
                m1.record(stream)
            barrier()
            moe_ms = max_over_ranks(m0.elapsed_time(m1)) / reps
            if peer_moe is not None:
                peer_moe.check()
            if rank == 0:   # sampled index pairs, experts of every rank among them, sampled output columns
                ym2 = ym.reshape(n_idx, N_DEC)
                picks = []
                for r in range(world):
                    l2, h2 = expert_bounds(E_MOE, r, world)
                    own = np.nonzero((rhs.ravel() >= l2) & (rhs.ravel() < h2))[0]
                    picks.extend(own[:3].tolist())
                cols = np.sort(rng.choice(N_DEC, 16, replace=False))
                ok = True
                for pidx in picks:
                    e, tok = int(rhs.ravel()[pidx]), int(lhs.ravel()[pidx])
                    ge = torch.Generator(device=dev).manual_seed(1000 + e)
                    w = (0.02 * torch.randn(N_DEC, K_DEC, device=dev, generator=ge)).to(torch.bfloat16)
                    ref = oracle_columns(carrier(w[torch.from_numpy(cols).to(dev)]), carrier(xm[tok]))
                    got = O.to_f32(carrier(ym2[pidx:pidx + 1][:, torch.from_numpy(cols).to(dev)]), "bf16")
                    ok = ok and close_enough(got, ref)
                    del w
                parity["moe_gathered_matches_oracle"] = bool(ok)
                parity["moe_pairs_checked"] = len(picks)
            Bm = E_MOE * algorithmic_bytes(0, N_DEC, K_DEC) + TOK_MOE * K_DEC * 2 + n_idx * N_DEC * 2 + 8 * n_idx
            Fm = 2.0 * n_idx * N_DEC * K_DEC
            moe = {"workload": f"gather_qmm {E_MOE} experts [{N_DEC},{K_DEC}] bits={BITS} group={GROUP}, {TOK_MOE} tokens top-{TOPK_MOE}, "
                               f"experts split over {world} rank(s)" + (", rows exchanged by peer stores inside the timed region" if world > 1 else ""),
                   "ms": moe_ms, "TFLOPs": Fm / (moe_ms * 1e-3) / 1e12, "GBps": Bm / (moe_ms * 1e-3) / 1e9,
                   "frac_tensor_per_gpu": Fm / world / (moe_ms * 1e-3) / 1e12 / tf_peak,
                   "frac_hbm_per_gpu": Bm / world / (moe_ms * 1e-3) / 1e9 / hbm_peak}
        if peer_moe is not None:
            peer_moe.close()

    status = (ctypes.c_uint32 * 4)()
    lib.b200q_read_status(P(ws), ws.numel(), sp, status)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_baseline, _ = cpu_reference_run(1, 10)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "arm": "N-sharded over the ranks" + ((", all_gather of outputs per step " + ("fused into the kernel epilogue (peer stores over NVLink, "
                              "flags raised by the kernel's last thread block; x is a replicated input, so every kernel holds only its "
                              "stores into the exchange buffers until all ranks have finished the previous step, one bounded wait closes "
                              "the chain; ms_per_step_dependent_chain holds the loads back as well)" if fused else "by NCCL")) if world > 1 else ""),
                       "l2": f"weights rotated over {copies} distinct copies ({copies * shard_bytes / 1e6:.0f} MB per rank, "
                             f"more than twice the {L2_BYTES / 1e6:.0f} MB L2) so every step reads HBM",
                       "weights": "declared constant (b200q_set_weights_constant): requested before the previous kernel has finished",
                       "timing": "CUDA events on the launching stream" + (", steps replayed from one CUDA graph" if graphed else "")
                                 + "; a 100 us delay kernel is queued ahead of the start event, so the interval holds device time only",
                       "parallelism": f"n-shard x{world}"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "prefill": prefill, "moe": moe,
            "parity": parity, "cpu_baseline": cpu_baseline, "device_status": list(status), "e2e_max_abs_gap": e2e_gap,
            "ms_per_step_dependent_chain": ms_dependent,
        }
        print(json.dumps(line))
    if world > 1:
        if peer_out is not None:
            peer_out.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
