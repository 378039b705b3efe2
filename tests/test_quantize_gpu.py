"""GPU parity: quantize must be bit-exact with the reference CPU quantize (through the
pinned restatement and the golden vectors); dequantize must reproduce the op-composed
reference (multiply, then add, each rounded to T)."""
import os

import numpy as np
import pytest
import torch

import mlx_b200 as mb
import oracle as O
from util import from_torch, make_w, to_torch, u32_to_torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "affine_golden.npz")
DTYPES = ("f32", "f16", "bf16")
GROUPS = (32, 64, 128)
BITS = (2, 3, 4, 5, 6, 8)


def same(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g", GROUPS)
@pytest.mark.parametrize("bits", BITS)
def test_quantize_golden(dtype, g, bits):
    gold = np.load(GOLDEN)
    t = f"{dtype}_g{g}_b{bits}"
    wq, s, b = mb.quantize(to_torch(gold[f"{t}/w"], dtype), g, bits)
    assert same(from_torch(wq), gold[f"{t}/wq"])
    assert same(from_torch(s), gold[f"{t}/s"])
    assert same(from_torch(b), gold[f"{t}/b"])


def edge_matrix(rng, rows, K, g):
    w = (0.02 * rng.standard_normal((rows, K))).astype(np.float32)
    w[0, :g] = 0.0
    w[1, :g] = 0.375
    w[2, :g] = -np.abs(w[2, :g])
    w[3, :g] = np.abs(w[3, :g])
    w[4, 0], w[4, 1:g] = 1.0, -1.0
    w[5, :g] = (np.arange(g) - g // 2) * 0.5
    w[6, :g] = 1e-9 * rng.standard_normal(g)  # scale clamps to eps
    w[7, :g] = 3e3 * rng.standard_normal(g)   # large magnitudes (finite in float16)
    return w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g", GROUPS)
@pytest.mark.parametrize("bits", BITS)
def test_quantize_bit_exact_vs_oracle(dtype, g, bits):
    rng = np.random.default_rng(1000 + g + bits)
    w = O.to_dtype(edge_matrix(rng, 67, 1536, g), dtype)
    ref = O.quantize(w, g, bits, dtype)
    got = mb.quantize(to_torch(w, dtype), g, bits)
    for r, t in zip(ref, got):
        assert same(r, from_torch(t))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g", GROUPS)
@pytest.mark.parametrize("bits", BITS)
def test_dequantize_bit_exact_vs_oracle(dtype, g, bits):
    rng = np.random.default_rng(2000 + g + bits)
    w = O.to_dtype(edge_matrix(rng, 33, 1024, g), dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    ref = O.dequantize(wq, s, b, g, bits, dtype)
    got = mb.dequantize(u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype), g, bits)
    assert same(ref, from_torch(got))


def test_quantize_batched_shape_and_empty():
    w = torch.randn(3, 5, 256, device="cuda", dtype=torch.bfloat16)
    wq, s, b = mb.quantize(w, 64, 4)
    assert wq.shape == (3, 5, 32) and s.shape == (3, 5, 4) and wq.dtype == torch.uint32
    ref = O.quantize(from_torch(w).reshape(15, 256), 64, 4, "bf16")
    assert same(ref[0], from_torch(wq).reshape(15, 32))
    e = mb.quantize(torch.zeros(0, 128, device="cuda"), 64, 4)
    assert e[0].shape == (0, 16) and e[1].shape == (0, 2)


def test_round_trip_large_matrix_properties():
    """Size-independent properties on a full-size weight (70B-MLP shape rows subsampled to keep
    the run short): quantize(dequantize(quantize(w))) is idempotent on the codes, and the
    reconstruction error is bounded by |scale| per group (python/tests/test_quantized.py:22-39)."""
    torch.manual_seed(0)
    w = (0.02 * torch.randn(2048, 8192, device="cuda")).to(torch.bfloat16)
    for bits, g in ((3, 32), (6, 128), (8, 32), (4, 64)):
        wq, s, b = mb.quantize(w, g, bits)
        wh = mb.dequantize(wq, s, b, g, bits)
        err = (w.float() - wh.float()).abs().reshape(2048, -1, g)
        bound = s.float().abs().unsqueeze(-1) * 1.01 + 2.0 ** -7 * (b.float().abs().unsqueeze(-1) + 2 ** bits * s.float().abs().unsqueeze(-1))
        assert bool((err <= bound + 1e-6).all())
        # spot rows against the oracle, bit-exact
        rows = [0, 1, 777, 2047]
        ref = O.quantize(from_torch(w[rows]), g, bits, "bf16")
        wq_rows = wq.view(torch.int32)[rows].view(torch.uint32)  # torch cannot index uint32 directly
        assert same(ref[0], from_torch(wq_rows)) and same(ref[1], from_torch(s[rows])) and same(ref[2], from_torch(b[rows]))


@pytest.mark.parametrize("dtype", ("f32", "bf16", "f16"))
@pytest.mark.parametrize("g,bits", [(32, 2), (64, 3), (64, 4), (128, 5), (32, 6), (128, 8)])
def test_quantize_rounding_ties_and_extremes(dtype, g, bits):
    """The kernel replaces most divisions by a multiplication with 1/scale and redoes the exact
    division only near rounding ties: inputs that sit ON the ties (k + 1/2 steps of the grid),
    huge and tiny magnitudes and groups with zeros must still be bit-exact."""
    rng = np.random.default_rng(bits * 100 + g)
    rows, K = 48, 1024
    nb = (1 << bits) - 1
    base = rng.standard_normal((rows, K)).astype(np.float32)
    grid = rng.integers(0, 2 * nb + 1, size=(rows, K)).astype(np.float32) * 0.5   # 0, 0.5, ..., nb
    grid[:, ::g] = 0.0
    grid[:, 1::g] = nb
    zeros = base.copy()
    zeros[::7, ::5] = 0.0
    cases = [grid, -grid, grid * 0.125 + 3.0, base * (1e30 if dtype != "f16" else 1e3),
             base * (1e-30 if dtype == "f32" else 1e-6), zeros]
    for ci, w in enumerate(cases):
        wd = O.to_dtype(w, dtype)
        rq, rs, rb = O.quantize(wd, g, bits, dtype)
        q, s, b = mb.quantize(to_torch(wd, dtype), g, bits)
        assert np.array_equal(from_torch(q).view(np.uint32), rq.view(np.uint32)), (ci, "wq")
        assert np.array_equal(from_torch(s), rs) and np.array_equal(from_torch(b), rb), (ci, "scales/biases")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g,bits", [(32, 3), (64, 4), (128, 6), (64, 8), (32, 2), (128, 5)])
def test_quantized_embedding_bit_exact_vs_oracle(dtype, g, bits):
    """QuantizedEmbedding look-up (python/mlx/nn/layers/quantized.py:149-158) = the oracle's
    dequantize of the indexed rows; negative ids count from the end, out-of-range ids give zeros."""
    rng = np.random.default_rng(2500 + g + bits)
    rows, K = 211, 768
    w = O.to_dtype(edge_matrix(rng, rows, K, g), dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    ids = rng.integers(0, rows, size=(5, 37))
    ids[0, 0], ids[1, 1], ids[2, 2] = -1, -rows, rows - 1
    pos = np.where(ids < 0, ids + rows, ids).reshape(-1)
    ref = O.dequantize(wq[pos], s[pos], b[pos], g, bits, dtype).reshape(5, 37, K)
    got = mb.quantized_embedding(torch.from_numpy(ids).cuda(), u32_to_torch(wq), to_torch(s, dtype),
                                 to_torch(b, dtype), g, bits)
    assert got.shape == (5, 37, K) and same(ref, from_torch(got))
    bad = mb.quantized_embedding(torch.tensor([rows, 3, 2 ** 31 - 1], device="cuda"), u32_to_torch(wq),
                                 to_torch(s, dtype), to_torch(b, dtype), g, bits)
    assert not bad[0].any() and not bad[2].any()
    assert same(from_torch(bad[1]), O.dequantize(wq[3:4], s[3:4], b[3:4], g, bits, dtype)[0])
    empty = mb.quantized_embedding(torch.zeros(0, dtype=torch.int64, device="cuda"), u32_to_torch(wq),
                                   to_torch(s, dtype), to_torch(b, dtype), g, bits)
    assert empty.shape == (0, K)


def test_quantized_embedding_rejects():
    wq = torch.zeros(4, 32, dtype=torch.int32, device="cuda").view(torch.uint32)
    s = torch.zeros(4, 4, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="integral"):
        mb.quantized_embedding(torch.zeros(2, device="cuda"), wq, s, s, 64, 4)
    with pytest.raises(ValueError, match="does not match"):
        mb.quantized_embedding(torch.zeros(2, dtype=torch.int64, device="cuda"), wq, s[:, :2], s[:, :2], 64, 4)
