"""Error behaviour of the operator front-end (mirrors the reference's
python/tests/test_quantized.py:877-956 test_mode_error_cases / test_throw): every case
must raise ValueError before any device work, so CPU tensors suffice here."""
import pytest
import torch

import mlx_b200 as mb


def u32(*shape):
    return torch.zeros(shape, dtype=torch.int32).view(torch.uint32)


def test_quantize_errors():
    w = torch.zeros(4, 256)
    with pytest.raises(ValueError):
        mb.quantize(w, group_size=48)
    with pytest.raises(ValueError):
        mb.quantize(w, bits=7)
    with pytest.raises(ValueError):
        mb.quantize(torch.zeros(256))
    with pytest.raises(ValueError):
        mb.quantize(torch.zeros(4, 100), group_size=64)
    with pytest.raises(ValueError):
        mb.quantize(torch.zeros(4, 256, dtype=torch.int32))
    with pytest.raises(ValueError):
        mb.quantize(w, mode="xyz")


def test_quantized_matmul_errors():
    x = torch.zeros(2, 256)
    w, s, b = u32(8, 32), torch.zeros(8, 4), torch.zeros(8, 4)
    with pytest.raises(ValueError):  # biases required for affine
        mb.quantized_matmul(x, w, s, None)
    with pytest.raises(ValueError):  # weight must be uint32
        mb.quantized_matmul(x, w.view(torch.int32), s, b)
    with pytest.raises(ValueError):  # scales / biases shapes differ
        mb.quantized_matmul(x, w, s, torch.zeros(8, 2))
    with pytest.raises(ValueError):  # w/scales incompatible with bits
        mb.quantized_matmul(x, w, s, b, bits=8)
    with pytest.raises(ValueError):  # x inner dim mismatch
        mb.quantized_matmul(torch.zeros(2, 128), w, s, b)
    with pytest.raises(ValueError):  # batch shape mismatch between w and scales
        mb.quantized_matmul(x, u32(2, 8, 32), torch.zeros(3, 8, 4), torch.zeros(3, 8, 4))
    with pytest.raises(ValueError):  # non floating scales
        mb.quantized_matmul(x, w, s.int(), b.int())
    with pytest.raises(ValueError):  # transpose=False: x inner must equal w rows
        mb.quantized_matmul(torch.zeros(2, 9), w, s, b, transpose=False)


def test_dequantize_errors():
    w, s, b = u32(8, 32), torch.zeros(8, 4), torch.zeros(8, 4)
    with pytest.raises(ValueError):
        mb.dequantize(w, s, None)
    with pytest.raises(ValueError):
        mb.dequantize(w.view(torch.int32), s, b)
    with pytest.raises(ValueError):
        mb.dequantize(u32(32), torch.zeros(4), torch.zeros(4))
    with pytest.raises(ValueError):
        mb.dequantize(w, s, b, group_size=32)
    with pytest.raises(ValueError):
        mb.dequantize(w, s, b, dtype=torch.int32)


def test_gather_qmm_errors():
    x = torch.zeros(3, 2, 256)
    w, s, b = u32(4, 8, 32), torch.zeros(4, 8, 4), torch.zeros(4, 8, 4)
    idx = torch.zeros(5, dtype=torch.int64)
    with pytest.raises(ValueError):
        mb.gather_qmm(x, w, s, None, rhs_indices=idx)
    with pytest.raises(ValueError):
        mb.gather_qmm(torch.zeros(3, 2, 128), w, s, b, rhs_indices=idx)
    with pytest.raises(ValueError):
        mb.gather_qmm(x, w, s, b, rhs_indices=torch.zeros(5))


def test_no_cpu_fallback():
    x = torch.zeros(2, 256)
    w, s, b = u32(8, 32), torch.zeros(8, 4), torch.zeros(8, 4)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.quantized_matmul(x, w, s, b)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.quantize(torch.zeros(4, 256))


def test_quantized_embedding_and_swiglu_errors():
    w, s = u32(8, 32), torch.zeros(8, 4, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="integral"):
        mb.quantized_embedding(torch.zeros(3), w, s, s, 64, 4)
    with pytest.raises(ValueError, match="does not match"):
        mb.quantized_embedding(torch.zeros(3, dtype=torch.int64), w, s[:, :2], s[:, :2], 64, 4)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.quantized_embedding(torch.zeros(3, dtype=torch.int64), w, s, s, 64, 4)
    x = torch.zeros(4, 1, 256, dtype=torch.bfloat16)
    gate = (u32(2, 128, 32), torch.zeros(2, 128, 4, dtype=torch.bfloat16), torch.zeros(2, 128, 4, dtype=torch.bfloat16))
    down = (u32(2, 256, 16), torch.zeros(2, 256, 2, dtype=torch.bfloat16), torch.zeros(2, 256, 2, dtype=torch.bfloat16))
    idx = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(ValueError, match="bfloat16"):
        mb.gather_qmm_swiglu(x.float(), gate, gate, down, rhs_indices=idx)
    with pytest.raises(ValueError, match="same experts"):
        mb.gather_qmm_swiglu(x, gate, down, down, rhs_indices=idx)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.gather_qmm_swiglu(x, gate, gate, down, rhs_indices=idx)


def test_grad_wrapper_has_no_cpu_fallback():
    from mlx_b200 import grad
    x = torch.zeros(2, 256, requires_grad=True)
    w, s, b = u32(8, 32), torch.zeros(8, 4), torch.zeros(8, 4)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        grad.quantized_matmul(x, w, s, b)
    with pytest.raises(ValueError):
        grad.quantized_matmul(x, w, s, b, group_size=48)
