"""Gradients of quantized_matmul, stated with the same identities as the reference's
QuantizedMatmul::vjp (mlx/primitives.cpp:3532-3598):

  d x      = quantized_matmul(cotangent, w, scales, biases, transpose = not transpose)
  d biases = sum over each group of  dW            (dW = cotangent^T x, or x^T cotangent)
  d scales = sum over each group of  dW * q        (q = dequantize(w, ones, zeros))
  d w      : none ("no gradient wrt the quantized weights")

The product for d x runs on this library's kernels (the non-transposed form of the forward);
dW is a plain dense product (torch.matmul, a library GEMM) followed by group sums.
"""
from typing import Optional

import torch

from . import ops


class _QuantizedMatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, scales, biases, transpose, group_size, bits):
        ctx.save_for_backward(x, w, scales, biases)
        ctx.cfg = (bool(transpose), group_size, bits)
        return ops.quantized_matmul(x, w, scales, biases, transpose, group_size, bits)

    @staticmethod
    def backward(ctx, cotangent):
        x, w, scales, biases = ctx.saved_tensors
        transpose, group_size, bits = ctx.cfg
        dx = ds = db = None
        if ctx.needs_input_grad[0]:
            dx = ops.quantized_matmul(cotangent.contiguous(), w, scales, biases, not transpose, group_size, bits)
            dx = dx.to(x.dtype)
        if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
            if w.ndim != 2:
                raise RuntimeError("[quantized_matmul] gradients wrt scales and biases need a 2-D weight")
            fc = cotangent.reshape(-1, cotangent.shape[-1])
            fx = x.reshape(-1, x.shape[-1]).to(fc.dtype)
            dw = fc.transpose(0, 1) @ fx if transpose else fx.transpose(0, 1) @ fc
            dsb = dw.unflatten(-1, (-1, group_size))
            if ctx.needs_input_grad[3]:
                db = dsb.sum(-1).to(biases.dtype)
            if ctx.needs_input_grad[2]:
                q = ops.dequantize(w, torch.ones_like(scales), torch.zeros_like(biases), group_size, bits)
                ds = (dsb * q.unflatten(-1, (-1, group_size)).to(dsb.dtype)).sum(-1).to(scales.dtype)
        return dx, None, ds, db, None, None, None


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                     transpose: bool = True, group_size: Optional[int] = None, bits: Optional[int] = None,
                     mode: str = "affine") -> torch.Tensor:
    """ops.quantized_matmul with autograd support for x, scales and biases."""
    group_size, bits = ops._mode_params(mode, group_size, bits, "quantized_matmul")
    return _QuantizedMatmulFn.apply(x, w, scales, biases, transpose, group_size, bits)


def jvp(x_tangent: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
        transpose: bool = True, group_size: Optional[int] = None, bits: Optional[int] = None) -> torch.Tensor:
    """QuantizedMatmul::jvp (mlx/primitives.cpp:3600-3619): the same product applied to the tangent of x."""
    return ops.quantized_matmul(x_tangent, w, scales, biases, transpose, group_size, bits)


class _GatherQmmFn(torch.autograd.Function):
    """GatherQMM::vjp (mlx/primitives.cpp:3718-3837).  d x: the cotangent goes through gather_qmm with
    the transposition flipped and the same rhs_indices, then its rows are added into x at lhs_indices.
    d scales / d biases: the per-pair dense products cotangent_i^T x[lhs_i] (or x[lhs_i]^T cotangent_i)
    are added into the matrix of the expert rhs_i names (the reference's gather_mm_grad), then summed
    over each group exactly as in the dense case."""

    @staticmethod
    def forward(ctx, x, w, scales, biases, lhs_indices, rhs_indices, transpose, group_size, bits):
        ctx.save_for_backward(w, scales, biases, lhs_indices, rhs_indices, x)
        ctx.cfg = (bool(transpose), group_size, bits, tuple(x.shape), x.dtype)
        return ops.gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, transpose, group_size, bits)

    @staticmethod
    def backward(ctx, cotangent):
        w, scales, biases, lhs_indices, rhs_indices, x = ctx.saved_tensors
        transpose, group_size, bits, x_shape, x_dtype = ctx.cfg
        idx_shape = tuple(cotangent.shape[:-2])
        M = cotangent.shape[-2]
        rhs = torch.broadcast_to(rhs_indices, idx_shape).reshape(-1)
        lhs = torch.broadcast_to(lhs_indices, idx_shape).reshape(-1).to(torch.int64)
        fc = cotangent.reshape((-1, M, cotangent.shape[-1])).contiguous()
        dx = ds = db = None
        if ctx.needs_input_grad[0]:
            g = ops.gather_qmm(fc, w, scales, biases, None, rhs, not transpose, group_size, bits)   # [n_idx, M, K]
            dx = torch.zeros((max(1, torch.Size(x_shape[:-2]).numel()),) + tuple(x_shape[-2:]), dtype=torch.float32,
                             device=g.device)
            dx.index_add_(0, lhs, g.float())
            dx = dx.to(x_dtype).reshape(x_shape)
        if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
            xs = x.reshape((-1,) + tuple(x_shape[-2:]))[lhs].float()                # [n_idx, M, K]
            cf = fc.float()
            pair = cf.transpose(1, 2) @ xs if transpose else xs.transpose(1, 2) @ cf
            n_mat = max(1, torch.Size(w.shape[:-2]).numel())
            dw = torch.zeros((n_mat,) + tuple(pair.shape[-2:]), dtype=torch.float32, device=pair.device)
            dw.index_add_(0, rhs.to(torch.int64), pair)
            dsb = dw.reshape(tuple(w.shape[:-2]) + tuple(pair.shape[-2:])).unflatten(-1, (-1, group_size))
            if ctx.needs_input_grad[3]:
                db = dsb.sum(-1).to(biases.dtype)
            if ctx.needs_input_grad[2]:
                q = ops.dequantize(w, torch.ones_like(scales), torch.zeros_like(biases), group_size, bits)
                ds = (dsb * q.unflatten(-1, (-1, group_size)).float()).sum(-1).to(scales.dtype)
        return dx, None, ds, db, None, None, None, None, None


def gather_qmm(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
               lhs_indices: Optional[torch.Tensor] = None, rhs_indices: Optional[torch.Tensor] = None,
               transpose: bool = True, group_size: Optional[int] = None, bits: Optional[int] = None,
               mode: str = "affine") -> torch.Tensor:
    """ops.gather_qmm with autograd support for x, scales and biases."""
    group_size, bits = ops._mode_params(mode, group_size, bits, "gather_qmm")
    if lhs_indices is None and rhs_indices is None:
        return quantized_matmul(x, w, scales, biases, transpose, group_size, bits)
    dev = x.device
    if lhs_indices is None:
        lhs_indices = torch.arange(max(1, torch.Size(x.shape[:-2]).numel()), device=dev).reshape(tuple(x.shape[:-2]))
    if rhs_indices is None:
        rhs_indices = torch.arange(max(1, torch.Size(w.shape[:-2]).numel()), device=dev).reshape(tuple(w.shape[:-2]))
    lhs_indices, rhs_indices = torch.broadcast_tensors(lhs_indices.to(dev), rhs_indices.to(dev))
    return _GatherQmmFn.apply(x, w, scales, biases, lhs_indices.contiguous(), rhs_indices.contiguous(), transpose,
                              group_size, bits)
