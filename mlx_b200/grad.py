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
