"""N-sharded quantized linear over one process per GPU (NCCL through torch.distributed).

Mirrors the reference's tensor-parallel layer for quantized weights
(python/mlx/nn/layers/distributed.py:40-93 `_shard`/`_all_to_sharded`, :357-455
`QuantizedAllToShardedLinear`) and its all_gather primitive
(mlx/distributed/ops.cpp:62-84, mlx/distributed/nccl/nccl.cpp:346-358):

* rank r keeps rows [r*N/R, (r+1)*N/R) of `weight`, `scales` and `biases`; the packed
  layout is row-major, so a shard is a contiguous slice and is never repacked;
* x is replicated; every rank computes y_r [.., M, N/R] with its local rows;
* `all_gather` concatenates the shards.  The reference gathers on axis 0; `gather_output`
  returns the row-major [.., M, N] a caller of an unsharded layer would see.

torch.distributed only carries the collective; the matmul is libb200q.so.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Row range of `rank` when n rows are split evenly (n must divide: the reference
    raises for uneven splits, nn/layers/distributed.py:75-83)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if n % world != 0:
        raise ValueError(f"cannot shard {n} rows evenly across {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of a [.., N, C] tensor owned by `rank` (axis max(ndim-2, 0))."""
    axis = max(t.ndim - 2, 0)
    lo, hi = shard_bounds(t.shape[axis], rank, world)
    return t.narrow(axis, lo, hi - lo).contiguous()


class QuantizedAllToShardedLinear:
    """y_r = x @ dequant(W_r)^T with the rows of W split across the ranks of `group`."""

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                 group_size: int = 64, bits: int = 4, group: Optional[dist.ProcessGroup] = None,
                 rank: Optional[int] = None, world: Optional[int] = None, already_sharded: bool = False):
        if rank is None or world is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group, self.rank, self.world = group, rank, world
        self.group_size, self.bits = group_size, bits
        if already_sharded:
            self.weight, self.scales, self.biases = weight, scales, biases
        else:
            self.weight = shard_rows(weight, rank, world)
            self.scales = shard_rows(scales, rank, world)
            self.biases = shard_rows(biases, rank, world)
        self.n_local = self.weight.shape[-2]
        self._gather_buf = None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                    group_size=self.group_size, bits=self.bits)

    def gather_output(self, y_local: torch.Tensor) -> torch.Tensor:
        """all_gather of the per-rank outputs -> [.., M, N] row-major."""
        return all_gather_columns(y_local, self.group, self.world, cache=self)


def all_gather_columns(y_local: torch.Tensor, group=None, world: Optional[int] = None, cache=None) -> torch.Tensor:
    """Concatenate per-rank [.., M, n] blocks along the last axis."""
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    shape = (world,) + tuple(y_local.shape)
    buf = getattr(cache, "_gather_buf", None) if cache is not None else None
    if buf is None or tuple(buf.shape) != shape or buf.dtype != y_local.dtype or buf.device != y_local.device:
        buf = torch.empty(shape, dtype=y_local.dtype, device=y_local.device)
        if cache is not None:
            cache._gather_buf = buf
    # axis-0 gather, exactly the reference's AllGather ([R*d0, ...] == [R, d0, ...])
    if y_local.is_cuda:
        dist.all_gather_into_tensor(buf, y_local, group=group)
    else:  # CPU process groups (gloo) gather into a list of views of the same buffer
        dist.all_gather([buf[r] for r in range(world)], y_local, group=group)
    # [R, .., M, n] -> [.., M, R*n]
    nd = buf.ndim
    perm = tuple(range(1, nd - 1)) + (0, nd - 1)
    out = buf.permute(perm)
    return out.reshape(tuple(y_local.shape[:-1]) + (world * y_local.shape[-1],))


def expert_bounds(n_experts: int, rank: int, world: int) -> Tuple[int, int]:
    """Experts owned by `rank` in the expert-parallel layout (contiguous blocks)."""
    return shard_bounds(n_experts, rank, world)


# ---------------------------------------------------------------------------------------------
# all_gather fused into the matmul epilogue: every rank's kernel stores its [M, N/R] block
# straight into the [M, N] output buffer of every rank (peer stores over NVLink), so no
# collective runs after the kernel; a per-rank flag word says when all blocks have landed.
# ---------------------------------------------------------------------------------------------
import ctypes

from . import _lib


class _DevMem:
    """Exposes a raw device pointer to torch through __cuda_array_interface__ (as uint16)."""

    def __init__(self, ptr: int, n_u16: int):
        self.__cuda_array_interface__ = {"shape": (n_u16,), "typestr": "<u2", "data": (ptr, False), "version": 2}


class PeerOutput:
    """Two alternating [m_max, n_total] bf16 output buffers per rank, mapped into every rank of
    `group` with CUDA IPC, plus one arrival flag per rank.  Collective constructor (all ranks of
    the group call it).  Ranks must be processes on one machine, one GPU each."""

    N_BUF = 2

    def __init__(self, m_max: int, n_total: int, group=None):
        self.lib = _lib.load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks can share output buffers")
        self.m_max, self.n_total = m_max, n_total
        self.buf_bytes = (m_max * n_total * 2 + 255) // 256 * 256
        total = self.N_BUF * self.buf_bytes + 256          # outputs, then the flag word, the epoch (+128), the block counter (+192)
        # Every rank walks the same sequence of collectives even when a local step fails; the failure
        # is agreed on at the end, so that all ranks raise together instead of some of them hanging.
        err = None
        ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        self._own = None
        try:
            _lib.check(self.lib.b200q_ipc_alloc(total, ctypes.byref(ptr), handle))
            self._own = ptr.value
        except Exception as e:  # noqa: BLE001
            err = e
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle) if err is None else None, group=group)
        self.base = []
        if err is None and all(h is not None for h in handles):
            try:
                for q in range(self.world):
                    if q == self.rank:
                        self.base.append(self._own)
                    else:
                        p = ctypes.c_void_p()
                        h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[q])
                        _lib.check(self.lib.b200q_ipc_open(h, ctypes.byref(p)))
                        self.base.append(p.value)
            except Exception as e:  # noqa: BLE001
                err = e
        elif err is None:
            err = RuntimeError("another rank could not allocate its buffer")
        oks = [None] * self.world
        dist.all_gather_object(oks, err is None, group=group)
        if not all(oks):
            for q, b in enumerate(self.base):
                if q != self.rank:
                    self.lib.b200q_ipc_close(ctypes.c_void_p(b))
            if self._own is not None:
                self.lib.b200q_ipc_free(ctypes.c_void_p(self._own))
                self._own = None
            raise RuntimeError(f"[PeerOutput] peer-mapped output buffers are not available on every rank: {err}")
        self.flag = [b + self.N_BUF * self.buf_bytes for b in self.base]
        self.epoch = self._own + self.N_BUF * self.buf_bytes + 128
        self.counter = self._own + self.N_BUF * self.buf_bytes + 192
        self.step = 0
        self._ws = None   # workspace of the last call: its status word says whether a wait ran out
        # torch views of the local buffers, made once (nothing is created during stream capture)
        self._views = [torch.as_tensor(_DevMem(self._own + i * self.buf_bytes, m_max * n_total), device="cuda")
                       .view(torch.bfloat16).view(m_max, n_total) for i in range(self.N_BUF)]
        dist.barrier(group=group)   # nobody stores into a buffer that is not mapped yet

    def y_ptrs(self, buf: int):
        return (ctypes.c_void_p * self.world)(*[b + buf * self.buf_bytes for b in self.base])

    def flag_ptrs(self):
        return (ctypes.c_void_p * self.world)(*self.flag)

    def local(self, buf: int, m: int) -> torch.Tensor:
        """This rank's copy of the gathered [m, n_total] result in buffer `buf`."""
        return self._views[buf][:m]

    def wait(self) -> None:
        """Makes the current stream wait (bounded) until every rank's part of the last exchange step
        has landed in this rank's buffer."""
        if self._ws is None:
            return
        status = ctypes.c_void_p(self._ws.data_ptr() + self._ws.numel() - 16)
        st = ctypes.c_void_p(torch.cuda.current_stream(self._ws.device).cuda_stream)
        _lib.check(self.lib.b200q_peer_wait(ctypes.c_void_p(self.flag[self.rank]), ctypes.c_void_p(self.epoch), status, st))

    def check(self) -> None:
        """Synchronises the current stream and raises ops.DeviceStatusError if the last exchange
        did not complete (a peer lagged behind the bounded wait, code 6) or a kernel gave up on one
        of its own waits.  The exchange functions below never synchronise: call this before results
        are consumed where a rank may stall for longer than the wait's bound."""
        if self._ws is not None:
            ops.read_workspace_status(self._ws, torch.cuda.current_stream(self._ws.device).cuda_stream, "peer exchange")

    def close(self):
        if self._own is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # no rank may still be storing into a buffer that goes away
        for q, b in enumerate(self.base):
            if q != self.rank:
                self.lib.b200q_ipc_close(ctypes.c_void_p(b))
        self.lib.b200q_ipc_free(ctypes.c_void_p(self._own))
        self._own = None


def sharded_matmul_allgather(layer: "QuantizedAllToShardedLinear", x: torch.Tensor, out: PeerOutput,
                             chained=False) -> torch.Tensor:
    """y = x @ dequant(W)^T for the full W, every rank holding only its rows: one matmul launch
    whose epilogue stores to all ranks and whose last thread block updates the flags, and one
    bounded wait (`out.check()` tells whether it ran out).

    chained=True is for a chain of sharded layers on one stream whose x is the previous call's
    gathered output: the call waits, before it reads x or stores its result, until every rank has
    finished the PREVIOUS call's exchange (inside the decode kernel, whose weight stream starts
    meanwhile) and does not wait for its own; the caller ends the chain with `out.wait()` before
    the last result is used.  chained="buffers" is the same for calls whose x comes from elsewhere
    (a replicated input, another exchange that was waited for): only the stores into the exchange
    buffers wait, so loads and products overlap the previous exchange.  x: [M, K] bf16 CUDA,
    the same on every rank.  Returns this rank's [M, N] view (valid until the buffer is used again
    two calls later)."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_cuda:
        raise ValueError("[sharded_matmul_allgather] x must be a 2-D bfloat16 CUDA tensor")
    M, K = x.shape
    if M > out.m_max or layer.n_local * out.world != out.n_total:
        raise ValueError("[sharded_matmul_allgather] output buffers do not match the layer")
    lib = out.lib
    x = x.contiguous()
    dt = _lib.BF16
    need = max(int(lib.b200q_qmm_workspace_bytes(dt, 1, M, layer.n_local, K, layer.group_size, layer.bits, 1)), 256)
    ws = ops._workspaces.get(x.device, need, "qmm")
    st = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    buf = out.step % out.N_BUF
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(lib.b200q_qmm_sharded_signal(vp(x), vp(layer.weight), vp(layer.scales), vp(layer.biases), out.y_ptrs(buf),
                                            out.world, out.n_total, out.rank * layer.n_local, dt, M, layer.n_local, K,
                                            layer.group_size, layer.bits, out.flag_ptrs(), ctypes.c_void_p(out.epoch),
                                            ctypes.c_void_p(out.counter),
                                            ctypes.c_void_p(out.flag[out.rank] if (chained and out.step > 0) else 0),
                                            0 if chained == "buffers" else 1, out.rank, vp(ws), ws.numel(), st))
    out.step += 1
    out._ws = ws
    if not chained:
        out.wait()
    return out.local(buf, M)


def sharded_gather_qmm(x: torch.Tensor, w_local: torch.Tensor, scales_local: torch.Tensor, biases_local: torch.Tensor,
                       lhs_indices: torch.Tensor, rhs_indices: torch.Tensor, e_lo: int, n_experts: int,
                       out: PeerOutput, group_size: int = 64, bits: int = 4) -> torch.Tensor:
    """Expert-parallel gather_qmm: this rank holds experts [e_lo, e_lo + E_local) of `n_experts`
    (`expert_bounds`), x [B, M, K] bf16 and the flat index pairs are the same on every rank.  Every
    rank multiplies the pairs of its own experts and stores the rows into every rank's buffer;
    returns this rank's complete [n_idx, M, N] (valid until the buffer is used again two calls later)."""
    if x.dtype != torch.bfloat16 or x.dim() != 3 or not x.is_cuda:
        raise ValueError("[sharded_gather_qmm] x must be a [B, M, K] bfloat16 CUDA tensor")
    B, M, K = x.shape
    E_local, N = w_local.shape[0], w_local.shape[1]
    lhs32 = lhs_indices.reshape(-1).to(device=x.device, dtype=torch.int32).contiguous()
    rhs32 = rhs_indices.reshape(-1).to(device=x.device, dtype=torch.int32).contiguous()
    n_idx = rhs32.numel()
    if lhs32.numel() != n_idx or n_idx * M > out.m_max or N != out.n_total:
        raise ValueError("[sharded_gather_qmm] index arrays / output buffers do not match the problem")
    lib = out.lib
    x = x.contiguous()
    dt = _lib.BF16
    need = max(int(lib.b200q_gather_qmm_workspace_bytes(dt, n_idx, B, n_experts, M, N, K, group_size, bits, 1)), 256)
    ws = ops._workspaces.get(x.device, need, "gather")
    st = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    buf = out.step % out.N_BUF
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(lib.b200q_gather_qmm_sharded_signal(vp(x), vp(w_local), vp(scales_local), vp(biases_local), vp(lhs32),
                                                   vp(rhs32), n_idx, out.y_ptrs(buf), out.world, out.rank, dt, B, n_experts,
                                                   e_lo, E_local, M, N, K, group_size, bits, out.flag_ptrs(),
                                                   ctypes.c_void_p(out.epoch), ctypes.c_void_p(out.counter), vp(ws),
                                                   ws.numel(), st))
    out.step += 1
    out._ws = ws
    status = ctypes.c_void_p(ws.data_ptr() + ws.numel() - 16)
    _lib.check(lib.b200q_peer_wait(ctypes.c_void_p(out.flag[out.rank]), ctypes.c_void_p(out.epoch), status, st))
    return out.local(buf, n_idx * M).view(n_idx, M, N)


# ---------------------------------------------------------------------------------------------
# K-sharded linear (QuantizedShardedToAllLinear of the reference,
# python/mlx/nn/layers/distributed.py:490-588): rank r multiplies its slice of the input
# dimension, then the partial outputs are summed over the ranks (all_sum).
# ---------------------------------------------------------------------------------------------
def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of the last axis owned by `rank` (packed weight words or scale groups)."""
    lo, hi = shard_bounds(t.shape[-1], rank, world)
    if t.dtype == torch.uint32:   # torch has no strided copy for uint32: go through the int32 view
        return t.view(torch.int32).narrow(-1, lo, hi - lo).contiguous().view(torch.uint32)
    return t.narrow(-1, lo, hi - lo).contiguous()


class QuantizedShardedToAllLinear:
    """y = sum over ranks of x[..., k-slice] @ dequant(W[:, k-slice])^T."""

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
                 bits: int = 4, group: Optional[dist.ProcessGroup] = None, rank: Optional[int] = None,
                 world: Optional[int] = None, already_sharded: bool = False):
        if rank is None or world is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group, self.rank, self.world = group, rank, world
        self.group_size, self.bits = group_size, bits
        if already_sharded:
            self.weight, self.scales, self.biases = weight, scales, biases
        else:
            if scales.shape[-1] % world != 0:
                raise ValueError(f"cannot shard {scales.shape[-1]} quantization groups evenly across {world} ranks")
            self.weight = shard_cols(weight, rank, world)
            self.scales = shard_cols(scales, rank, world)
            self.biases = shard_cols(biases, rank, world)
        self.n_out = self.weight.shape[-2]
        self.k_local = self.scales.shape[-1] * group_size

    def x_slice(self, x: torch.Tensor) -> torch.Tensor:
        return x[..., self.rank * self.k_local:(self.rank + 1) * self.k_local].contiguous()

    def partial(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(self.x_slice(x), self.weight, self.scales, self.biases, transpose=True,
                                    group_size=self.group_size, bits=self.bits)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """Partial matmul + all_reduce through the process group (the reference's formulation)."""
        y = self.partial(x)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        return y


def sharded_matmul_allreduce(layer: QuantizedShardedToAllLinear, x: torch.Tensor, out: PeerOutput) -> torch.Tensor:
    """The same result with the exchange fused into the matmul: every rank's kernel stores its
    partial [M, N] into slot `rank` of every rank's buffer (peer stores), then one flag update, one
    bounded wait and a local fp32 sum over the slots.  `out` must hold world * M rows of N columns
    (`PeerOutput(world * m_max, N)`).  x: [M, K] bf16 CUDA, the same on every rank."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_cuda:
        raise ValueError("[sharded_matmul_allreduce] x must be a 2-D bfloat16 CUDA tensor")
    M = x.shape[0]
    N, R = layer.n_out, out.world
    if N != out.n_total or R * M > out.m_max:
        raise ValueError("[sharded_matmul_allreduce] output buffers do not match the layer")
    lib = out.lib
    xs = layer.x_slice(x)
    K = xs.shape[1]
    dt = _lib.BF16
    need = max(int(lib.b200q_qmm_workspace_bytes(dt, 1, M, N, K, layer.group_size, layer.bits, 1)), 256)
    ws = ops._workspaces.get(x.device, need, "qmm")
    st = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    buf = out.step % out.N_BUF
    slot_bytes = M * N * 2
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    ys = (ctypes.c_void_p * R)(*[b + buf * out.buf_bytes + out.rank * slot_bytes for b in out.base])
    _lib.check(lib.b200q_qmm_sharded_signal(vp(xs), vp(layer.weight), vp(layer.scales), vp(layer.biases), ys, R, N, 0, dt, M,
                                            N, K, layer.group_size, layer.bits, out.flag_ptrs(), ctypes.c_void_p(out.epoch),
                                            ctypes.c_void_p(out.counter), ctypes.c_void_p(0), 0, -1, vp(ws), ws.numel(), st))
    out.step += 1
    out._ws = ws
    status = ctypes.c_void_p(ws.data_ptr() + ws.numel() - 16)
    _lib.check(lib.b200q_peer_wait(ctypes.c_void_p(out.flag[out.rank]), ctypes.c_void_p(out.epoch), status, st))
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.b200q_peer_reduce(ctypes.c_void_p(out._own + buf * out.buf_bytes), R, M * N, M * N, vp(y), dt, st))
    return y
