#!/usr/bin/env python
"""Benchmark of the affine quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the small-batch decode configuration - x [16, 4096] bf16 ~ N(0,1),
W [14336, 4096] ~ N(0, 0.02) quantized at 4 bits / group 64 (Llama-3-8B MLP up-projection),
`quantized_matmul(transpose=True)`.  A step is one call on one batch; successive steps use
different weight copies (8 x 33 MB > the 126 MB L2) so every step streams from HBM.  With
N > 1 ranks the weight rows are split evenly across ranks (strong scaling of the same
matrix) and a step ends with the all_gather of the per-rank outputs.

One JSON line is printed by rank 0.  `value` is the device-timed throughput in algorithmic
GB/s with inputs resident in HBM; `e2e` is the same metric through the host-buffer C-ABI
call with the host<->device copies inside the timed region; `roofline` relates the decode
kernel to the measured HBM peak; `prefill` reports the tensor-core path on the
M = 4096 configuration; `cpu_baseline` times the reference project's own CPU code.
`--impl reference` times only that CPU code (all host cores) and prints its own line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
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
WEIGHT_COPIES = 8
# dram__bytes_read.sum + dram__bytes_write.sum per launch of qmv_mma_kernel on the one-GPU decode
# workload (profiles/qmv_mma_kernel_decode_M16_N14336_K4096.md); with the matrix split over R
# ranks the per-rank traffic is this divided by R (it is all weight stream)
NCU_TRAFFIC_BYTES = 33494784


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
        "config": {"workload": f"decode quantized_matmul M={M_DEC} N={N_DEC} K={K_DEC} bits={BITS} group={GROUP} "
                               "on host cores (bounded sample, see cpu_baseline.sample)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200q")
    ap.add_argument("--gather", default="fused", choices=("fused", "nccl"),
                    help="N > 1: all_gather fused into the matmul epilogue (peer stores) or the NCCL collective")
    ap.add_argument("--no-prefill", action="store_true")
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
    from mlx_b200.distributed import all_gather_columns, shard_bounds

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
    P = lambda t: ctypes.c_void_p(t.data_ptr())

    # ---- synthetic inputs: this rank's row shard of WEIGHT_COPIES weight matrices
    lo, hi = shard_bounds(N_DEC, rank, world)
    n_loc = hi - lo
    weights = []
    for c in range(WEIGHT_COPIES):
        g = torch.Generator(device=dev).manual_seed(100 + c)
        w = (0.02 * torch.randn(N_DEC, K_DEC, device=dev, generator=g)).to(torch.bfloat16)[lo:hi].contiguous()
        weights.append(mb.quantize(w, GROUP, BITS))
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
    # rank's output buffer, flag signal + bounded wait); --gather nccl runs the collective instead.
    fused = world > 1 and args.gather == "fused"
    if fused:
        from mlx_b200.distributed import PeerOutput, QuantizedAllToShardedLinear, sharded_matmul_allgather
        try:
            peer_out = PeerOutput(M_DEC, N_DEC)
        except RuntimeError as e:   # raised on every rank together: fall back to the collective
            if rank == 0:
                print(f"bench: fused gather unavailable ({e}); using NCCL", file=sys.stderr)
            fused = False
    if fused:
        layers = [QuantizedAllToShardedLinear(q, s, b, GROUP, BITS, rank=rank, world=world, already_sharded=True)
                  for (q, s, b) in weights]

    def step(i):
        if fused:
            return sharded_matmul_allgather(layers[i % WEIGHT_COPIES], x, peer_out)
        q, s, b = weights[i % WEIGHT_COPIES]
        rc = lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1, 0,
                           P(ws), ws.numel(), sp)
        if rc != 0:
            raise RuntimeError(_lib.last_error())
        if world > 1:
            return all_gather_columns(y, None, world, cache=Gather)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
    barrier()

    # ---- device-timed region: exactly `steps` steps on the launching stream, replayed from a CUDA
    # graph (no host launch gaps); with the NCCL collective in the step they run eagerly.
    sampler = ClockSampler(local_rank)
    launches0 = lib.b200q_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world == 1 or fused:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(args.steps):
                step(i)
        launches = int(lib.b200q_launch_count() - launches0)
        graph.replay()  # one untimed replay to settle the instantiated graph
        barrier()
        sampler.start()
        time.sleep(0.3)
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        barrier()
    else:
        sampler.start()
        time.sleep(0.3)
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(args.steps):
                step(i)
            e1.record(stream)
        barrier()
        launches = int(lib.b200q_launch_count() - launches0)
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    total_bytes = algorithmic_bytes(M_DEC, N_DEC, K_DEC)
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- kernel-only duration for the roofline (same stream, events around kernel launches only)
    with torch.cuda.stream(stream):
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kg, stream=stream):
            for i in range(args.steps):
                q, s, b = weights[i % WEIGHT_COPIES]
                lib.b200q_qmm(P(x), P(q), P(s), P(b), P(y), _lib.BF16, 1, M_DEC, n_loc, K_DEC, GROUP, BITS, 1, 0,
                              P(ws), ws.numel(), sp)
        kg.replay()
        torch.cuda.synchronize(dev)
        k0.record(stream)
        kg.replay()
        k1.record(stream)
    torch.cuda.synchronize(dev)
    kernel_ms = k0.elapsed_time(k1) / args.steps
    hbm_peak, tf_peak, peak_src = measured_peaks()
    achieved = algorithmic_bytes(M_DEC, n_loc, K_DEC) / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": (NCU_TRAFFIC_BYTES // world if kernel == "qmv_mma" else None), "kernel": kernel, "kernel_us": kernel_ms * 1e3, "peak_source": peak_src}

    # ---- end to end through the host-buffer C-ABI call (pinned host x and y, copies timed)
    x_host = torch.empty(M_DEC, K_DEC, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    y_host = torch.empty(M_DEC, n_loc, dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(x)

    def e2e_step(i):
        q, s, b = weights[i % WEIGHT_COPIES]
        rc = lib.b200q_qmm_host(P(x_host), P(x_dev), P(q), P(s), P(b), P(y), P(y_host), _lib.BF16, M_DEC, n_loc, K_DEC,
                                GROUP, BITS, 1, P(ws), ws.numel(), sp)
        if rc != 0:
            raise RuntimeError(_lib.last_error())

    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
        stream.synchronize()  # the caller reads y_host after every step
    e2e_s = (time.perf_counter() - t0) / args.steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": M_DEC * K_DEC * 2,
           "d2h_bytes_per_step": M_DEC * n_loc * 2, "ms_per_step": e2e_s * 1e3,
           "note": "b200q_qmm_host: pinned x -> device, kernel, y -> pinned host, synchronised every step; "
                   "weights stay resident in HBM"}
    # y holds the last kernel-only step on the same weights; partial sums combine in arrival order, so the
    # two runs may differ in the last bfloat16 bit: compare within the matmul tolerance and report the gap
    y_d, y_h = y.float().cpu(), y_host.float()
    e2e_gap = float((y_h - y_d).abs().max())
    ok_check = bool(torch.allclose(y_h, y_d, rtol=1e-2, atol=1e-2 * float(y_d.pow(2).mean().sqrt())))

    # ---- prefill configuration on the tensor-core path (rank-local shard)
    prefill = None
    if not args.no_prefill:
        xp = torch.randn(M_PRE, K_DEC, device=dev, generator=g).to(torch.bfloat16)
        yp = torch.empty(M_PRE, n_loc, device=dev, dtype=torch.bfloat16)
        reps = 10
        with torch.cuda.stream(stream):
            for i in range(3):
                q, s, b = weights[i % WEIGHT_COPIES]
                lib.b200q_qmm(P(xp), P(q), P(s), P(b), P(yp), _lib.BF16, 1, M_PRE, n_loc, K_DEC, GROUP, BITS, 1, 0,
                              P(ws), ws.numel(), sp)
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(stream)
            for i in range(reps):
                q, s, b = weights[i % WEIGHT_COPIES]
                lib.b200q_qmm(P(xp), P(q), P(s), P(b), P(yp), _lib.BF16, 1, M_PRE, n_loc, K_DEC, GROUP, BITS, 1, 0,
                              P(ws), ws.numel(), sp)
            p1.record(stream)
        torch.cuda.synchronize(dev)
        pms = p0.elapsed_time(p1) / reps
        if world > 1:
            t = torch.tensor([pms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            pms = float(t.item())
        tflops = 2.0 * M_PRE * N_DEC * K_DEC / (pms * 1e-3) / 1e12
        prefill = {"workload": f"prefill M={M_PRE} N={N_DEC} K={K_DEC} (rank-local N shard, outputs not gathered)",
                   "value": tflops, "unit": "TFLOP/s", "ms": pms,
                   "kernel": lib.b200q_qmm_kernel_name(_lib.BF16, 1, M_PRE, n_loc, K_DEC, GROUP, BITS, 1).decode(),
                   "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": tf_peak, "unit": "TFLOP/s",
                                "frac": tflops / world / tf_peak, "peak_source": peak_src}}
        del xp, yp

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
            "config": {"workload": f"decode quantized_matmul M={M_DEC} N={N_DEC} K={K_DEC} bits={BITS} group={GROUP} "
                                   "transpose=True (Llama-3-8B MLP up-projection), N-sharded over the ranks"
                                   + ((", all_gather of outputs per step " + ("fused into the kernel epilogue (peer stores over NVLink)" if fused else "by NCCL")) if world > 1 else ""),
                       "l2": f"weights rotated over {WEIGHT_COPIES} distinct copies "
                             f"({WEIGHT_COPIES * algorithmic_bytes(0, n_loc, K_DEC) / 1e6:.0f} MB per rank) so reads "
                             "come from HBM",
                       "timing": "CUDA events on the launching stream" + (", steps replayed from one CUDA graph" if (world == 1 or fused) else ""),
                       "parallelism": f"n-shard x{world}"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "prefill": prefill,
            "cpu_baseline": cpu_baseline, "device_status": list(status), "e2e_matches_device": ok_check, "e2e_max_abs_gap": e2e_gap,
        }
        print(json.dumps(line))
    if world > 1:
        if fused:
            peer_out.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
