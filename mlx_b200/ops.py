"""Host-side mirror of the reference operator front-end for the affine quantized path.

Same names, argument meaning and error behaviour as ``mlx.core.quantize``,
``dequantize``, ``quantized_matmul`` and ``gather_qmm`` (reference: mlx/ops.cpp:4784-4834
quantized_matmul, :5208-5245 quantize, :5465-5517 dequantize, :5553-5629 gather_qmm;
validation helpers :110-181, :4704-4754).  Arrays are ``torch`` CUDA tensors: torch only
supplies device memory and streams, every computation is a call into libb200q.so.
Invalid arguments raise ``ValueError`` (the reference's std::invalid_argument).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_MODES = ("affine", "mxfp4", "mxfp8", "nvfp4")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(tag: str, *ts: torch.Tensor) -> torch.device:
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError(f"[{tag}] tensors must live on a CUDA device: there is no CPU fallback")
        if t.device != dev:
            raise ValueError(f"[{tag}] all tensors must be on the same device")
    return dev


def _as_u32(w: torch.Tensor, tag: str) -> torch.Tensor:
    if w.dtype == torch.uint32:
        return w
    raise ValueError(f"[{tag}] The weight matrix should be uint32 but received {w.dtype}")


class _Workspaces:
    """One zero-initialised scratch buffer per (device, stream, operator); it only grows.

    quantized_matmul and gather_qmm keep separate buffers: the matmul kernels rely on
    counters that start at zero and are left at zero, while gather_qmm uses its buffer as
    plain scratch (sorted indices, tile table, gathered rows)."""

    def __init__(self):
        self._bufs = {}

    def get(self, dev: torch.device, nbytes: int, op: str) -> torch.Tensor:
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream, op)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            with torch.cuda.device(dev):
                buf = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=dev)
            self._bufs[key] = buf
        return buf


_workspaces = _Workspaces()

_STATUS_TEXT = {
    1: "gather index out of range (that output was zeroed)",
    2: "bounded wait expired in the bulk-copy ring of a decode kernel",
    3: "bounded wait expired in the tcgen05 prefill kernel",
    4: "bounded wait expired in the tcgen05 decode kernel",
    5: "bounded wait expired in the TMA ring of the stream decode kernel",
    6: "bounded wait for a peer GPU's completion flag expired: the gathered output is incomplete",
    7: "bounded wait expired in the row-owning decode kernel",
}


class DeviceStatusError(RuntimeError):
    """A kernel of this library gave up on a bounded wait (or met a bad gather index) and said so
    in the status word of its workspace: the outputs of that call are not valid."""

    def __init__(self, code: int, words, where: str):
        self.code, self.words = int(code), tuple(int(w) for w in words)
        super().__init__(f"b200q device status {self.code} ({_STATUS_TEXT.get(self.code, 'unknown')}) in the "
                         f"{where} workspace; status words {self.words}")


def read_workspace_status(ws: torch.Tensor, stream_ptr: int, where: str = "caller") -> None:
    """Synchronises the stream, reads and clears the status word at the end of `ws`, and raises
    DeviceStatusError if it is non-zero, after zeroing the whole workspace again (an aborted
    kernel leaves counters and partial sums behind that would corrupt every later call)."""
    lib = _lib.load()
    st = (ctypes.c_uint32 * 4)()
    sp = ctypes.c_void_p(stream_ptr)
    with torch.cuda.device(ws.device):
        _lib.check(lib.b200q_read_status(ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp, st))
        if st[0] != 0:
            _lib.check(lib.b200q_workspace_init(ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp))
            raise DeviceStatusError(st[0], list(st), where)


def check_status(device: Optional[torch.device] = None) -> None:
    """Checked mode on request: synchronises every stream this module has launched on (for
    `device`, or all devices) and raises DeviceStatusError if any kernel reported a failure since
    the last check.  The operators themselves never synchronise; call this where the results are
    about to be consumed on the host, or set B200Q_CHECK_STATUS=1 to have every operator call do
    it before it returns (debugging: it serialises host and device)."""
    for (dev_index, stream_ptr, op), ws in list(_workspaces._bufs.items()):
        if device is not None and torch.device(device).index not in (None, dev_index):
            continue
        read_workspace_status(ws, stream_ptr, op)


def _checked() -> bool:
    import os
    return os.environ.get("B200Q_CHECK_STATUS", "0") == "1"


def _mode_params(mode: str, group_size, bits, tag: str) -> Tuple[int, int]:
    if mode not in _MODES:
        raise ValueError(f"[{tag}] Invalid quantization mode '{mode}'.")
    if mode != "affine":
        raise NotImplementedError(f"[{tag}] only the affine mode is built; '{mode}' is out of scope")
    return (64 if group_size is None else int(group_size), 4 if bits is None else int(bits))


def _validate_mode_with_type(tag, scales, biases, out_type):
    # mlx/ops.cpp:4704-4754
    if out_type is not None and not out_type.is_floating_point:
        raise ValueError(f"[{tag}] Only real floating types are supported but output dtype == {out_type}.")
    if biases is None:
        raise ValueError(f"[{tag}] Biases must be provided for affine quantization.")
    dtype = torch.promote_types(scales.dtype, biases.dtype)
    if not dtype.is_floating_point:
        raise ValueError(
            f"[{tag}] Only real floating types are supported but scales.dtype() == {scales.dtype} "
            f"and biases.dtype() == {biases.dtype}."
        )
    return out_type if out_type is not None else dtype


def _validate_quantized_input(tag, w, scales, group_size, bits, biases):
    # mlx/ops.cpp:110-150
    _as_u32(w, tag)
    if biases is not None and scales.shape != biases.shape:
        raise ValueError(
            f"[{tag}] Scales and biases should have the same shape. Received scales with shape "
            f"{tuple(scales.shape)} and biases with {tuple(biases.shape)}"
        )
    if w.ndim < 2 or scales.ndim != w.ndim or tuple(w.shape[:-2]) != tuple(scales.shape[:-2]):
        raise ValueError(
            f"[{tag}] Weight and scales should have the same batch shape. Received weight with shape "
            f"{tuple(w.shape)}, scales with {tuple(scales.shape)}."
        )
    if w.shape[-1] * 32 // bits != scales.shape[-1] * group_size:
        raise ValueError(
            f"[{tag}] The shapes of the weight and scales are incompatible based on bits and group_size. "
            f"w.shape() == {tuple(w.shape)} and scales.shape() == {tuple(scales.shape)} "
            f"with group_size={group_size} and bits={bits}"
        )


def _extract_dims(tag, x, w, scales, biases, transpose, group_size, bits):
    # mlx/ops.cpp:152-181
    _validate_quantized_input(tag, w, scales, group_size, bits, biases)
    if x.ndim < 1:
        raise ValueError(f"[{tag}] x must have at least one dimension")
    x_inner = x.shape[-1]
    w_inner = w.shape[-1] * 32 // bits if transpose else w.shape[-2]
    w_outer = w.shape[-2] if transpose else w.shape[-1] * 32 // bits
    if w_inner != x_inner:
        raise ValueError(
            f"[{tag}] Last dimension of first input with shape (..., {x_inner}) does not match the expanded "
            f"quantized matrix ({w_inner}, {w_outer}) computed from shape {tuple(w.shape)} with "
            f"group_size={group_size}, bits={bits} and transpose={transpose}"
        )
    return w_inner, w_outer


# --------------------------------------------------------------------------- quantize
def quantize(w: torch.Tensor, group_size: Optional[int] = None, bits: Optional[int] = None,
             mode: str = "affine"):
    """-> (w_q uint32 [..., K*bits/32], scales [..., K/g], biases [..., K/g]); mlx/ops.cpp:5208."""
    group_size, bits = _mode_params(mode, group_size, bits, "quantize")
    if not w.dtype.is_floating_point or w.dtype not in _DT:
        raise ValueError(f"[quantize] Only real floating types can be quantized but w has type {w.dtype}.")
    if w.ndim < 2:
        raise ValueError(
            f"[quantize] The matrix to be quantized must have at least 2 dimension but it has only {w.ndim}."
        )
    if group_size not in (32, 64, 128):
        raise ValueError(
            f"[quantize] The requested group size {group_size} is not supported. "
            "The supported group sizes are 32, 64, and 128."
        )
    if bits < 2 or bits > 8 or bits == 7:
        raise ValueError(
            f"[quantize] The requested number of bits {bits} is not supported. "
            "The supported bits are 2, 3, 4, 5, 6 and 8."
        )
    if w.shape[-1] % group_size != 0:
        raise ValueError(
            f"[quantize] The last dimension of the matrix needs to be divisible by the quantization group "
            f"size {group_size}. However the provided matrix has shape {tuple(w.shape)}"
        )
    dev = _require_cuda("quantize", w)
    w = w.contiguous()
    K = w.shape[-1]
    rows = w.numel() // K if K else 0
    lead = tuple(w.shape[:-1])
    with torch.cuda.device(dev):
        wq = torch.empty(lead + (K * bits // 32,), dtype=torch.uint32, device=dev)
        scales = torch.empty(lead + (K // group_size,), dtype=w.dtype, device=dev)
        biases = torch.empty_like(scales)
        rc = _lib.load().b200q_quantize(_ptr(w), _DT[w.dtype], rows, K, group_size, bits, _ptr(wq),
                                        _ptr(scales), _ptr(biases), _stream(w))
    _lib.check(rc)
    return wq, scales, biases


def dequantize(w: torch.Tensor, scales: torch.Tensor, biases: Optional[torch.Tensor] = None,
               group_size: Optional[int] = None, bits: Optional[int] = None, mode: str = "affine",
               dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """mlx/ops.cpp:5465-5517 (+ affine_dequantize :5258-5340)."""
    group_size, bits = _mode_params(mode, group_size, bits, "dequantize")
    out_type = _validate_mode_with_type("dequantize", scales, biases, dtype)
    if bits <= 0:
        raise ValueError(f"[dequantize] Invalid value for bits: {bits}")
    if group_size <= 0:
        raise ValueError(f"[dequantize] Invalid value for group_size: {group_size}")
    if w.dtype != torch.uint32:
        raise ValueError("[dequantize] The matrix should be given as a uint32")
    if w.ndim < 2:
        raise ValueError(
            f"[dequantize] The matrix to be dequantized must have at least 2 dimension but it has only {w.ndim}."
        )
    if (w.ndim != scales.ndim or w.ndim != biases.ndim or tuple(w.shape[:-1]) != tuple(scales.shape[:-1])
            or tuple(w.shape[:-1]) != tuple(biases.shape[:-1])):
        raise ValueError("[dequantize] Shape of scales and biases does not match the matrix")
    K = w.shape[-1] * 32 // bits
    if K != scales.shape[-1] * group_size or scales.shape != biases.shape:
        raise ValueError(
            "[dequantize] Shape of scales and biases does not match the matrix given the quantization "
            f"parameters. Provided matrix of shape {tuple(w.shape)} and scales/biases of shape "
            f"{tuple(scales.shape)} with group_size={group_size} and bits={bits}."
        )
    if scales.dtype not in _DT or scales.dtype != biases.dtype:
        ct = torch.promote_types(scales.dtype, biases.dtype)
        scales, biases = scales.to(ct), biases.to(ct)
    dev = _require_cuda("dequantize", w, scales, biases)
    w, scales, biases = w.contiguous(), scales.contiguous(), biases.contiguous()
    rows = w.numel() // w.shape[-1] if w.shape[-1] else 0
    with torch.cuda.device(dev):
        out = torch.empty(tuple(w.shape[:-1]) + (K,), dtype=scales.dtype, device=dev)
        rc = _lib.load().b200q_dequantize(_ptr(w), _ptr(scales), _ptr(biases), _DT[scales.dtype], rows, K,
                                          group_size, bits, _ptr(out), _stream(w))
    _lib.check(rc)
    return out if out.dtype == out_type else out.to(out_type)


def quantized_embedding(ids: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                        group_size: Optional[int] = None, bits: Optional[int] = None,
                        mode: str = "affine") -> torch.Tensor:
    """QuantizedEmbedding.__call__ (python/mlx/nn/layers/quantized.py:149-158):
    dequantize(w[ids], scales[ids], biases[ids]) as one kernel.  ids: any integer tensor;
    out: ids.shape + [K] in the dtype of scales."""
    group_size, bits = _mode_params(mode, group_size, bits, "quantized_embedding")
    _validate_mode_with_type("quantized_embedding", scales, biases, None)
    if w.dtype != torch.uint32:
        raise ValueError("[quantized_embedding] The matrix should be given as a uint32")
    if w.ndim != 2 or scales.ndim != 2 or biases.shape != scales.shape or scales.shape[0] != w.shape[0]:
        raise ValueError("[quantized_embedding] Shape of scales and biases does not match the matrix")
    K = w.shape[-1] * 32 // bits
    if K != scales.shape[-1] * group_size:
        raise ValueError(
            "[quantized_embedding] Shape of scales and biases does not match the matrix given the quantization "
            f"parameters. Provided matrix of shape {tuple(w.shape)} and scales/biases of shape "
            f"{tuple(scales.shape)} with group_size={group_size} and bits={bits}."
        )
    if ids.dtype.is_floating_point or ids.dtype == torch.bool:
        raise ValueError("[quantized_embedding] ids must be integral.")
    if scales.dtype not in _DT or scales.dtype != biases.dtype:
        ct = torch.promote_types(scales.dtype, biases.dtype)
        scales, biases = scales.to(ct), biases.to(ct)
    dev = _require_cuda("quantized_embedding", w, scales, biases)
    w, scales, biases = w.contiguous(), scales.contiguous(), biases.contiguous()
    ids64 = ids.to(device=dev, dtype=torch.int64).contiguous().reshape(-1)
    ids64 = torch.where(ids64 < 0, ids64 + w.shape[0], ids64)  # negative ids count from the end, as indexing does
    ids32 = ids64.to(torch.int32)  # uint32 bit pattern
    with torch.cuda.device(dev):
        out = torch.empty(tuple(ids.shape) + (K,), dtype=scales.dtype, device=dev)
        rc = _lib.load().b200q_dequantize_rows(_ptr(w), _ptr(scales), _ptr(biases), _ptr(ids32), ids32.numel(),
                                               _DT[scales.dtype], w.shape[0], K, group_size, bits, _ptr(out),
                                               _stream(w))
    _lib.check(rc)
    return out


# ------------------------------------------------------------------- quantized_matmul
_weights_constant = os.environ.get("B200Q_WEIGHTS_CONSTANT", "") == "1"


def set_weights_constant(on: bool) -> None:
    """The caller's promise that packed weights, scales and biases are not written by whatever
    precedes a matmul on its stream (b200q_set_weights_constant): the decode kernel may then request
    them before the previous kernel has finished.  quantized_matmul suspends the promise for a call
    in which it had to cast or copy one of the three itself (that copy IS the preceding kernel)."""
    global _weights_constant
    _weights_constant = bool(on)
    _lib.load().b200q_set_weights_constant(int(_weights_constant))


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor,
                     biases: Optional[torch.Tensor] = None, transpose: bool = True,
                     group_size: Optional[int] = None, bits: Optional[int] = None,
                     mode: str = "affine") -> torch.Tensor:
    """mlx/ops.cpp:4784-4834.  x [..., M, K] (or [K]); w [..., N, K*bits/32] when transposed."""
    group_size, bits = _mode_params(mode, group_size, bits, "quantized_matmul")
    dtype = _validate_mode_with_type("quantized_matmul", scales, biases, None)
    _, w_outer = _extract_dims("quantized_matmul", x, w, scales, biases, transpose, group_size, bits)
    dtype = torch.promote_types(x.dtype, dtype)
    if not dtype.is_floating_point or dtype not in _DT:
        raise ValueError(f"[quantized_matmul] Only real floating types are supported but x.dtype() == {x.dtype}.")
    dev = _require_cuda("quantized_matmul", x, w, scales, biases)
    given = (w, scales, biases)
    x, scales, biases = x.to(dtype), scales.to(dtype), biases.to(dtype)

    vector = x.ndim == 1
    if vector:
        x = x.unsqueeze(0)
    K = x.shape[-1]
    M = x.shape[-2]
    if x.ndim > 2 and w.ndim > 2:
        # both batched: broadcast the batch dimensions (mlx/ops.cpp:4823-4825)
        bshape = torch.broadcast_shapes(x.shape[:-2], w.shape[:-2])
        x = x.expand(bshape + x.shape[-2:]).contiguous()
        w = w.expand(bshape + w.shape[-2:]).contiguous()
        scales = scales.expand(bshape + scales.shape[-2:]).contiguous()
        biases = biases.expand(bshape + biases.shape[-2:]).contiguous()
        batch, w_stride, out_lead = x.numel() // max(M * K, 1), 1, tuple(bshape)
    elif w.ndim > 2:
        # 2-D x against a stack of matrices
        bshape = tuple(w.shape[:-2])
        x = x.expand(bshape + x.shape[-2:]).contiguous()
        w, scales, biases = w.contiguous(), scales.contiguous(), biases.contiguous()
        batch, w_stride, out_lead = w.numel() // max(w.shape[-1] * w.shape[-2], 1), 1, bshape
    else:
        x, w, scales, biases = x.contiguous(), w.contiguous(), scales.contiguous(), biases.contiguous()
        out_lead = tuple(x.shape[:-2])
        batch, w_stride = (x.numel() // max(M * K, 1) if M * K else 0), 0
        if M * K == 0:
            batch = 1
            for d in out_lead:
                batch *= d
    N = w_outer
    lib = _lib.load()
    with torch.cuda.device(dev):
        y = torch.empty(out_lead + (M, N), dtype=dtype, device=dev)
        need = lib.b200q_qmm_workspace_bytes(_DT[dtype], batch, M, N, K, group_size, bits, int(transpose))
        ws = _workspaces.get(dev, need, "qmm")
        # a weight operand this function has just cast or copied was written by the kernel right
        # before the matmul on this stream: no early weight loads for this call
        fresh = _weights_constant and any(a.data_ptr() != b.data_ptr() for a, b in zip((w, scales, biases), given))
        if fresh:
            lib.b200q_set_weights_constant(0)
        try:
            rc = lib.b200q_qmm(_ptr(x), _ptr(w), _ptr(scales), _ptr(biases), _ptr(y), _DT[dtype], batch, M, N, K,
                               group_size, bits, int(transpose), w_stride, _ptr(ws), ws.numel(), _stream(x))
        finally:
            if fresh:
                lib.b200q_set_weights_constant(1)
    _lib.check(rc)
    if _checked():
        read_workspace_status(ws, torch.cuda.current_stream(dev).cuda_stream, "qmm")
    return y.squeeze(-2) if vector else y


# -------------------------------------------------------------------------- gather_qmm
def gather_qmm(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: Optional[torch.Tensor] = None,
               lhs_indices: Optional[torch.Tensor] = None, rhs_indices: Optional[torch.Tensor] = None,
               transpose: bool = True, group_size: Optional[int] = None, bits: Optional[int] = None,
               mode: str = "affine", sorted_indices: bool = False) -> torch.Tensor:
    """mlx/ops.cpp:5553-5629.  out shape = broadcast(lhs, rhs).shape + [M, N]."""
    if lhs_indices is None and rhs_indices is None:
        return quantized_matmul(x, w, scales, biases, transpose, group_size, bits, mode)
    group_size, bits = _mode_params(mode, group_size, bits, "gather_qmm")
    out_type = _validate_mode_with_type("gather_qmm", scales, biases, None)
    _, w_outer = _extract_dims("gather_qmm", x, w, scales, biases, transpose, group_size, bits)
    out_type = torch.promote_types(x.dtype, out_type)
    if not out_type.is_floating_point or out_type not in _DT:
        raise ValueError(f"[gather_qmm] Only real floating types are supported but x.dtype() == {x.dtype}.")
    if x.ndim < 2:
        raise ValueError("[gather_qmm] x must have at least two dimensions")
    for idx, name in ((lhs_indices, "lhs_indices"), (rhs_indices, "rhs_indices")):
        if idx is not None and (idx.dtype.is_floating_point or idx.dtype == torch.bool):
            raise ValueError(f"[gather_qmm] Got {name} with invalid dtype. Indices must be integral.")
    dev = _require_cuda("gather_qmm", x, w, scales, biases)

    def default_idx(t):  # indices_or_default, mlx/ops.cpp:79-108
        shape = tuple(t.shape[:-2])
        n = 1
        for d in shape:
            n *= d
        return torch.arange(n, dtype=torch.int64, device=dev).reshape(shape)

    lhs = default_idx(x) if lhs_indices is None else lhs_indices.to(device=dev, dtype=torch.int64)
    rhs = default_idx(w) if rhs_indices is None else rhs_indices.to(device=dev, dtype=torch.int64)
    lhs, rhs = torch.broadcast_tensors(lhs, rhs)
    idx_shape = tuple(lhs.shape)
    lhs32 = lhs.contiguous().reshape(-1).to(torch.int32)  # bit pattern of uint32 indices
    rhs32 = rhs.contiguous().reshape(-1).to(torch.int32)

    x, scales, biases = x.to(out_type).contiguous(), scales.to(out_type).contiguous(), biases.to(out_type).contiguous()
    w = w.contiguous()
    M, K = x.shape[-2], x.shape[-1]
    x_batch = x.numel() // max(M * K, 1) if M * K else 0
    E = w.numel() // max(w.shape[-1] * w.shape[-2], 1) if w.shape[-1] * w.shape[-2] else 0
    N = w_outer
    n_idx = lhs32.numel()
    flags = (1 if (sorted_indices and rhs_indices is None) else 0) | (2 if (sorted_indices and lhs_indices is None) else 0)
    lib = _lib.load()
    with torch.cuda.device(dev):
        y = torch.empty(idx_shape + (M, N), dtype=out_type, device=dev)
        need = lib.b200q_gather_qmm_workspace_bytes(_DT[out_type], n_idx, x_batch, E, M, N, K, group_size, bits,
                                                    int(transpose))
        ws = _workspaces.get(dev, need, "gather")
        rc = lib.b200q_gather_qmm(_ptr(x), _ptr(w), _ptr(scales), _ptr(biases), _ptr(lhs32), _ptr(rhs32), n_idx,
                                  _ptr(y), _DT[out_type], x_batch, E, M, N, K, group_size, bits, int(transpose),
                                  flags, _ptr(ws), ws.numel(), _stream(x))
    _lib.check(rc)
    if _checked():
        read_workspace_status(ws, torch.cuda.current_stream(dev).cuda_stream, "gather")
    return y


def qmm_kernel_name(dtype: torch.dtype, M: int, N: int, K: int, group_size: int = 64, bits: int = 4,
                    transpose: bool = True, batch: int = 1) -> str:
    """Which kernel family quantized_matmul launches for this problem."""
    return _lib.load().b200q_qmm_kernel_name(_DT[dtype], batch, M, N, K, group_size, bits, int(transpose)).decode()


def gather_qmm_chain(x: torch.Tensor, w1: torch.Tensor, scales1: torch.Tensor, biases1: torch.Tensor,
                     w2: torch.Tensor, scales2: torch.Tensor, biases2: torch.Tensor,
                     rhs_indices: torch.Tensor, lhs_indices: Optional[torch.Tensor] = None,
                     group_size: Optional[int] = None, bits: Optional[int] = None) -> torch.Tensor:
    """gather_qmm(gather_qmm(x, w1, ...), w2, ...) over the same index pairs with one sort by expert
    (the reference composes the two calls, benchmarks/python/gather_qmm_bench.py:52-63).
    x [B, M, K1] bf16; w1 [E, N1, K1*bits/32]; w2 [E, N2, N1*bits/32]; out: idx_shape + [M, N2]."""
    group_size, bits = _mode_params("affine", group_size, bits, "gather_qmm_chain")
    _validate_quantized_input("gather_qmm_chain", w1, scales1, group_size, bits, biases1)
    _validate_quantized_input("gather_qmm_chain", w2, scales2, group_size, bits, biases2)
    if x.dtype != torch.bfloat16 or x.ndim < 2:
        raise ValueError("[gather_qmm_chain] x must be bfloat16 with at least two dimensions")
    dev = _require_cuda("gather_qmm_chain", x, w1, scales1, biases1, w2, scales2, biases2)
    M, K1 = x.shape[-2], x.shape[-1]
    N1, N2 = w1.shape[-2], w2.shape[-2]
    if w1.shape[-1] * 32 // bits != K1 or w2.shape[-1] * 32 // bits != N1 or w1.shape[:-2] != w2.shape[:-2]:
        raise ValueError("[gather_qmm_chain] w1 must map K1 -> N1 and w2 N1 -> N2 for the same experts")
    x_batch = x.numel() // max(M * K1, 1)
    E = w1.numel() // max(w1.shape[-1] * N1, 1)
    rhs = rhs_indices.to(device=dev, dtype=torch.int64)
    lhs = (torch.arange(x_batch, device=dev).reshape(tuple(x.shape[:-2])) if lhs_indices is None
           else lhs_indices.to(device=dev, dtype=torch.int64))
    lhs, rhs = torch.broadcast_tensors(lhs, rhs)
    idx_shape = tuple(lhs.shape)
    lhs32, rhs32 = lhs.contiguous().reshape(-1).to(torch.int32), rhs.contiguous().reshape(-1).to(torch.int32)
    n_idx = lhs32.numel()
    x = x.contiguous()
    c = lambda t: t.to(torch.bfloat16).contiguous()
    scales1, biases1, scales2, biases2 = c(scales1), c(biases1), c(scales2), c(biases2)
    w1, w2 = w1.contiguous(), w2.contiguous()
    lib = _lib.load()
    with torch.cuda.device(dev):
        y = torch.empty(idx_shape + (M, N2), dtype=torch.bfloat16, device=dev)
        need = lib.b200q_gather_qmm_chain_workspace_bytes(n_idx, E, M, N1, K1)
        ws = _workspaces.get(dev, need, "gather")
        rc = lib.b200q_gather_qmm_chain(_ptr(x), _ptr(w1), _ptr(scales1), _ptr(biases1), _ptr(w2), _ptr(scales2),
                                        _ptr(biases2), _ptr(lhs32), _ptr(rhs32), n_idx, _ptr(y), _lib.BF16, x_batch, E, M,
                                        N1, K1, N2, group_size, bits, _ptr(ws), ws.numel(), _stream(x))
    _lib.check(rc)
    return y


def gather_qmm_swiglu(x: torch.Tensor, gate, up, down, rhs_indices: torch.Tensor,
                      lhs_indices: Optional[torch.Tensor] = None, group_size: Optional[int] = None,
                      bits: Optional[int] = None) -> torch.Tensor:
    """Gated expert MLP: gather_qmm(silu(gather_qmm(x, *gate)) * gather_qmm(x, *up), *down) over the same
    index pairs with one sort (three mlx/ops.cpp:5553-5629 calls and the activation in the reference).
    gate, up, down: (w, scales, biases) triples; gate/up [E, H, K1*bits/32], down [E, N2, H*bits/32];
    x [B, M, K1] bf16; out: idx_shape + [M, N2]."""
    group_size, bits = _mode_params("affine", group_size, bits, "gather_qmm_swiglu")
    for t in (gate, up, down):
        _validate_quantized_input("gather_qmm_swiglu", t[0], t[1], group_size, bits, t[2])
    if x.dtype != torch.bfloat16 or x.ndim < 2:
        raise ValueError("[gather_qmm_swiglu] x must be bfloat16 with at least two dimensions")
    M, K1 = x.shape[-2], x.shape[-1]
    H, N2 = gate[0].shape[-2], down[0].shape[-2]
    if (gate[0].shape != up[0].shape or gate[0].shape[-1] * 32 // bits != K1 or down[0].shape[-1] * 32 // bits != H
            or gate[0].shape[:-2] != down[0].shape[:-2]):
        raise ValueError("[gather_qmm_swiglu] gate and up must map K1 -> H and down H -> N2 for the same experts")
    dev = _require_cuda("gather_qmm_swiglu", x, *gate, *up, *down)
    x_batch = x.numel() // max(M * K1, 1)
    E = gate[0].numel() // max(gate[0].shape[-1] * H, 1)
    rhs = rhs_indices.to(device=dev, dtype=torch.int64)
    lhs = (torch.arange(x_batch, device=dev).reshape(tuple(x.shape[:-2])) if lhs_indices is None
           else lhs_indices.to(device=dev, dtype=torch.int64))
    lhs, rhs = torch.broadcast_tensors(lhs, rhs)
    idx_shape = tuple(lhs.shape)
    lhs32, rhs32 = lhs.contiguous().reshape(-1).to(torch.int32), rhs.contiguous().reshape(-1).to(torch.int32)
    n_idx = lhs32.numel()
    x = x.contiguous()
    trip = lambda t: (t[0].contiguous(), t[1].to(torch.bfloat16).contiguous(), t[2].to(torch.bfloat16).contiguous())
    gate, up, down = trip(gate), trip(up), trip(down)
    lib = _lib.load()
    with torch.cuda.device(dev):
        y = torch.empty(idx_shape + (M, N2), dtype=torch.bfloat16, device=dev)
        need = lib.b200q_gather_qmm_swiglu_workspace_bytes(n_idx, E, M, H, K1)
        ws = _workspaces.get(dev, need, "gather")
        rc = lib.b200q_gather_qmm_swiglu(_ptr(x), *[_ptr(t) for t in gate], *[_ptr(t) for t in up], *[_ptr(t) for t in down],
                                         _ptr(lhs32), _ptr(rhs32), n_idx, _ptr(y), _lib.BF16, x_batch, E, M, H, K1, N2,
                                         group_size, bits, _ptr(ws), ws.numel(), _stream(x))
    _lib.check(rc)
    return y
