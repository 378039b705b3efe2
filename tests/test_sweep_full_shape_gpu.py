"""Parity at the full size of the bit-width / group sweep configuration: W [28672, 8192]
(the 70B MLP shape), bits {3, 6, 8} x group {32, 128}, M in {1, 512}, bf16.

* quantize and dequantize of the WHOLE matrix are compared bit for bit with the CPU checker
  (all 235 M elements, not a sample);
* the M = 1 product is compared with the checker's float result over all 28672 outputs;
* the M = 512 product is compared on sampled token rows over all outputs (the checker needs
  about 0.3 s per row at this size), the other rows through finiteness, and the first 16 rows
  through linearity across kernels: the decode kernel's result for 2 x must equal twice the
  prefill kernel's rows within the bf16 tolerance.
Tolerance for the products: |y - y_ref| <= 1e-2 |y_ref| + 1e-2 rms(y_ref)."""
import numpy as np
import pytest
import torch

import mlx_b200 as mb
import oracle as O
from util import from_torch, make_w, make_x, qmm_close, to_torch

pytestmark = pytest.mark.gpu
N, K = 28672, 8192


@pytest.fixture(scope="module")
def weights():
    return make_w(2, (N, K), "bf16")


@pytest.mark.parametrize("g", (32, 128))
@pytest.mark.parametrize("bits", (3, 6, 8))
def test_full_shape_round_trip_and_products(weights, bits, g):
    dtype = "bf16"
    wq_ref, s_ref, b_ref = O.quantize(weights, g, bits, dtype)
    w_dev = to_torch(weights, dtype)
    wq, s, b = mb.quantize(w_dev, g, bits)
    del w_dev
    assert np.array_equal(from_torch(wq), wq_ref), "packed weights differ"
    assert np.array_equal(from_torch(s), s_ref), "scales differ"
    assert np.array_equal(from_torch(b), b_ref), "biases differ"
    # dequantize: every element
    w_hat = mb.dequantize(wq, s, b, g, bits)
    ref_hat = O.dequantize(wq_ref, s_ref, b_ref, g, bits, dtype)
    assert np.array_equal(from_torch(w_hat), ref_hat), "dequantized weights differ"
    del w_hat, ref_hat

    # M = 1: all outputs
    x1 = make_x(1, (1, K), dtype)
    y1 = mb.quantized_matmul(to_torch(x1, dtype), wq, s, b, group_size=g, bits=bits)
    ref1 = O.qmm_f32_from(x1, wq_ref, s_ref, b_ref, dtype, transpose=True, group_size=g, bits=bits)
    ok, rel = qmm_close(O.to_f32(from_torch(y1), dtype), ref1)
    assert ok, f"M=1 bits={bits} g={g}: {rel:.3e}"

    # M = 512: sampled rows (tile seams included) against the checker
    M = 512
    x = make_x(3, (M, K), dtype)
    y = mb.quantized_matmul(to_torch(x, dtype), wq, s, b, group_size=g, bits=bits)
    assert mb.qmm_kernel_name(torch.bfloat16, M, N, K, g, bits) == "qmm_tcgen05"
    rows = np.array([0, 127, 128, 255, 256, 511])
    ref = O.qmm_f32_from(x[rows], wq_ref, s_ref, b_ref, dtype, transpose=True, group_size=g, bits=bits)
    got = O.to_f32(from_torch(y[torch.from_numpy(rows).cuda()]), dtype)
    ok, rel = qmm_close(got, ref)
    assert ok, f"M=512 bits={bits} g={g}: {rel:.3e}"
    yf = y.float()
    assert bool(torch.isfinite(yf).all())
    # linearity: y(2 x_r) = 2 y(x_r) up to output rounding; the 16-row call runs on the decode kernel
    x2 = to_torch(x, dtype)[:16] * 2
    y2 = mb.quantized_matmul(x2, wq, s, b, group_size=g, bits=bits)
    ok, rel = qmm_close(y2.float().cpu().numpy(), 2.0 * yf[:16].cpu().numpy())
    assert ok, f"linearity bits={bits} g={g}: {rel:.3e}"
