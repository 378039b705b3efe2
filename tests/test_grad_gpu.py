"""Gradients of quantized_matmul against a dense fp64 torch reference of the same operator
(the vjp/jvp identities of mlx/primitives.cpp:3532-3619, tested there by
python/tests/test_quantized.py:480-538)."""
import pytest
import torch

import mlx_b200 as mb
from mlx_b200 import grad

pytestmark = pytest.mark.gpu


def dense_reference(x, q, scales, biases, transpose, g):
    w = (q.unflatten(-1, (-1, g)) * scales.unsqueeze(-1) + biases.unsqueeze(-1)).flatten(-2)
    return x @ (w.transpose(0, 1) if transpose else w)


@pytest.mark.parametrize("transpose", [True, False])
@pytest.mark.parametrize("bits,g", [(8, 64), (4, 32), (3, 128)])
def test_qmm_vjp_matches_dense_autograd(transpose, bits, g):
    torch.manual_seed(bits * 10 + g)
    M, N, K = 8, 1024, 512
    w = torch.randn((N, K) if transpose else (K, N), device="cuda")
    wq, s, b = mb.quantize(w, g, bits)
    x = torch.randn(2, M, K, device="cuda", requires_grad=True)
    s.requires_grad_(True)
    b.requires_grad_(True)
    c = torch.randn(2, M, N, device="cuda")
    y = grad.quantized_matmul(x, wq, s, b, transpose, g, bits)
    dx, ds, db = torch.autograd.grad(y, (x, s, b), c)
    # the vjp wrt x is the operator with the transposition flipped (test_quantized.py:505-509)
    flipped = mb.quantized_matmul(c, wq, s.detach(), b.detach(), not transpose, g, bits)
    assert float((dx - flipped).abs().max()) <= 1e-5 * float(flipped.abs().max())
    q = mb.dequantize(wq, torch.ones_like(s), torch.zeros_like(b), g, bits).double()
    x64, s64, b64 = (t.detach().double().requires_grad_(True) for t in (x, s, b))
    y64 = dense_reference(x64, q, s64, b64, transpose, g)
    rx, rs, rb = torch.autograd.grad(y64, (x64, s64, b64), c.double())
    for got, ref in ((y.detach(), y64.detach()), (dx, rx), (ds, rs), (db, rb)):
        tol = 2e-3 * float(ref.abs().max())          # fp32 sums (TF32 allowed in the dense dW product)
        assert got.shape == ref.shape and float((got.double() - ref).abs().max()) <= tol


def test_qmm_jvp_and_bf16_vector():
    torch.manual_seed(3)
    N, K, g, bits = 512, 256, 64, 4
    wq, s, b = mb.quantize(torch.randn(N, K, device="cuda").to(torch.bfloat16), g, bits)
    t = torch.randn(4, K, device="cuda", dtype=torch.bfloat16)
    y_t, y_o = grad.jvp(t, wq, s, b, True, g, bits), mb.quantized_matmul(t, wq, s, b, True, g, bits)
    assert float((y_t.float() - y_o.float()).abs().max()) <= 1e-2 * float(y_o.float().abs().max())
    x = torch.randn(K, device="cuda", dtype=torch.bfloat16, requires_grad=True)   # vector input
    y = grad.quantized_matmul(x, wq, s, b, True, g, bits)
    (dx,) = torch.autograd.grad(y, (x,), torch.ones_like(y))
    assert dx.shape == x.shape and dx.dtype == x.dtype
    ref = mb.dequantize(wq, s, b, g, bits).float().sum(0)
    assert float((dx.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max()) + 1e-2


def test_no_gradient_wrt_packed_weights():
    wq, s, b = mb.quantize(torch.randn(64, 256, device="cuda"), 64, 4)
    x = torch.randn(2, 256, device="cuda", requires_grad=True)
    y = grad.quantized_matmul(x, wq, s, b)
    assert y.requires_grad and not wq.requires_grad


@pytest.mark.parametrize("transpose", [True, False])
def test_gather_qmm_vjp_matches_dense_autograd(transpose):
    """d x of gather_qmm (mlx/primitives.cpp:3718-3772; python/tests/test_quantized.py:755-842 checks
    the same identity): rows of the flipped product added back at lhs_indices."""
    torch.manual_seed(11)
    E, B, M, N, K, g, bits = 4, 6, 2, 256, 128, 64, 4
    w = torch.randn((E, N, K) if transpose else (E, K, N), device="cuda")
    wq, s, b = mb.quantize(w, g, bits)
    x = torch.randn(B, M, K, device="cuda", requires_grad=True)
    s.requires_grad_(True)
    b.requires_grad_(True)
    lhs = torch.tensor([0, 0, 3, 5, 5, 5, 2], device="cuda")
    rhs = torch.tensor([1, 3, 0, 1, 1, 1, 3], device="cuda")        # expert 2 is never used
    y = grad.gather_qmm(x, wq, s, b, lhs, rhs, transpose, g, bits)
    assert tuple(y.shape) == (7, M, N)
    c = torch.randn_like(y)
    dx, ds, db = torch.autograd.grad(y, (x, s, b), c)
    q = mb.dequantize(wq, torch.ones_like(s), torch.zeros_like(b), g, bits).double()
    x64, s64, b64 = (t.detach().double().requires_grad_(True) for t in (x, s, b))
    wd = (q.unflatten(-1, (-1, g)) * s64.unsqueeze(-1) + b64.unsqueeze(-1)).flatten(-2)
    y64 = torch.stack([x64[l] @ (wd[r].transpose(0, 1) if transpose else wd[r]) for l, r in zip(lhs.tolist(), rhs.tolist())])
    rx, rs, rb = torch.autograd.grad(y64, (x64, s64, b64), c.double())
    assert float((y.detach().double() - y64.detach()).abs().max()) <= 1e-3 * float(y64.detach().abs().max())
    assert dx.shape == x.shape and float((dx.double() - rx).abs().max()) <= 1e-3 * float(rx.abs().max())
    assert not dx[1].any() and not dx[4].any()       # rows no index pair reads get no gradient
    # d scales / d biases (mlx/primitives.cpp:3780-3834): fp32 sums, TF32 allowed in the dense products
    for got, ref in ((ds, rs), (db, rb)):
        assert got.shape == ref.shape and float((got.double() - ref).abs().max()) <= 2e-3 * float(ref.abs().max())
    assert not ds[2].any() and not db[2].any()       # an expert no pair names gets no gradient
