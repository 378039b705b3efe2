"""GPU parity of gather_qmm against the reference gather loop
(mlx/backend/cpu/quantized.cpp:700-747), shapes after python/tests/test_quantized.py:1127-1266."""
import os

import numpy as np
import pytest
import torch

import mlx_b200 as mb
import oracle as O
from util import from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "affine_golden.npz")


def test_gather_golden():
    gold = np.load(GOLDEN)
    a = {k: gold[f"gather/{k}"] for k in ("wq", "s", "b", "x", "lhs", "rhs", "y")}
    y = mb.gather_qmm(to_torch(a["x"], "f32"), u32_to_torch(a["wq"]), to_torch(a["s"], "f32"), to_torch(a["b"], "f32"),
                      lhs_indices=torch.from_numpy(a["lhs"].astype(np.int64)), rhs_indices=torch.from_numpy(a["rhs"].astype(np.int64)))
    ok, rel = qmm_close(from_torch(y), a["y"], 1e-4)
    assert ok, rel


@pytest.mark.parametrize("dtype", ("f32", "bf16"))
@pytest.mark.parametrize("transpose", (True, False))
def test_gather_index_patterns(dtype, transpose):
    E, M, N, K, g, bits = 5, 3, 64, 128, 32, 4
    wshape = (E, N, K) if transpose else (E, K, N)
    w = make_w(11, wshape, dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    x = make_x(12, (4, M, K), dtype)
    rng = np.random.default_rng(3)
    cases = [
        (rng.integers(0, 4, (7,)), rng.integers(0, E, (7,))),
        (None, rng.integers(0, E, (4,))),
        (rng.integers(0, 4, (E,)), None),
        (rng.integers(0, 4, (2, 3)), rng.integers(0, E, (2, 3))),
        (rng.integers(0, 4, (2, 1)), rng.integers(0, E, (1, 3))),
    ]
    args = (u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    for lhs, rhs in cases:
        tl = None if lhs is None else torch.from_numpy(lhs)
        tr = None if rhs is None else torch.from_numpy(rhs)
        y = mb.gather_qmm(to_torch(x, dtype), *args, lhs_indices=tl, rhs_indices=tr, transpose=transpose,
                          group_size=g, bits=bits)
        l = np.arange(4) if lhs is None else lhs
        r = np.arange(E) if rhs is None else rhs
        l, r = np.broadcast_arrays(l, r)
        assert tuple(y.shape) == l.shape + (M, N)
        ref = O.gather_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), l.ravel(), r.ravel(),
                           transpose, g, bits, "f32")
        ok, rel = qmm_close(O.to_f32(from_torch(y), dtype).reshape(ref.shape), ref, 1e-4 if dtype == "f32" else 1e-2)
        assert ok, rel


def test_gather_bad_index_is_flagged_not_faulted():
    from mlx_b200 import _lib, ops
    import ctypes
    E, M, N, K = 2, 1, 32, 128
    w = make_w(13, (E, N, K), "f32")
    wq, s, b = O.quantize(w, 64, 4, "f32")
    x = to_torch(make_x(14, (3, M, K), "f32"), "f32")
    y = mb.gather_qmm(x, u32_to_torch(wq), to_torch(s, "f32"), to_torch(b, "f32"),
                      lhs_indices=torch.tensor([0, 1, 2]), rhs_indices=torch.tensor([0, 9, 1]))
    torch.cuda.synchronize()
    assert bool((y[1] == 0).all()) and bool((y[0] != 0).any()) and bool((y[2] != 0).any())
    ws = ops._workspaces.get(x.device, 0, "gather")
    st = (ctypes.c_uint32 * 4)()
    rc = _lib.load().b200q_read_status(ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), st)
    assert rc == 0 and st[0] == 1 and st[1] == 1


# ---- sort-by-expert grouped path (bf16, 4-bit, transpose) -------------------------------
def _moe_case(E, tokens, topk, N, K, M=1, g=64, seed=0, bits=4):
    dtype = "bf16"
    wq, s, b = O.quantize(make_w(100 + seed, (E, N, K), dtype), g, bits, dtype)
    x = make_x(1 + seed, (tokens, M, K), dtype)
    rng = np.random.default_rng(3 + seed)
    rhs = rng.permuted(np.tile(np.arange(E), (tokens, 1)), axis=1)[:, :topk].astype(np.uint32)
    lhs = np.broadcast_to(np.arange(tokens, dtype=np.uint32)[:, None], rhs.shape).copy()
    return dtype, wq, s, b, x, lhs, rhs


@pytest.mark.parametrize("E,tokens,topk,N,K,M,g", [(8, 64, 2, 256, 512, 1, 64), (4, 33, 2, 200, 256, 1, 32),
                                                    (8, 512, 2, 1024, 4096, 1, 64), (3, 10, 1, 128, 128, 3, 128),
                                                    (16, 7, 4, 384, 1024, 2, 64)])
def test_gather_grouped_vs_oracle(E, tokens, topk, N, K, M, g):
    dtype, wq, s, b, x, lhs, rhs = _moe_case(E, tokens, topk, N, K, M, g)
    y = mb.gather_qmm(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype),
                      lhs_indices=torch.from_numpy(lhs.astype(np.int64)), rhs_indices=torch.from_numpy(rhs.astype(np.int64)),
                      group_size=g, bits=4)
    assert tuple(y.shape) == (tokens, topk, M, N)
    ref = O.gather_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), lhs.ravel(), rhs.ravel(), True,
                       g, 4, "f32")
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype).reshape(ref.shape), ref)
    assert ok, rel


@pytest.mark.parametrize("bits", (3, 6, 8))
def test_gather_grouped_other_bit_widths(bits):
    E, tokens, topk, N, K, g = 4, 40, 2, 256, 512, 64
    dtype, wq, s, b, x, lhs, rhs = _moe_case(E, tokens, topk, N, K, 1, g, bits=bits)
    y = mb.gather_qmm(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype),
                      lhs_indices=torch.from_numpy(lhs.astype(np.int64)), rhs_indices=torch.from_numpy(rhs.astype(np.int64)),
                      group_size=g, bits=bits)
    ref = O.gather_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), lhs.ravel(), rhs.ravel(), True,
                       g, bits, "f32")
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype).reshape(ref.shape), ref)
    assert ok, rel


def test_gather_grouped_full_size_moe_layer():
    """Mixtral-style layer: 8 experts [14336, 4096], 512 tokens, top-2.  Every output slot must equal
    the plain quantized_matmul of its token with its expert (the kernels share no code path for the
    gather), and sampled slots are checked against the oracle."""
    E, tokens, topk, N, K = 8, 512, 2, 14336, 4096
    dtype, wq, s, b, x, lhs, rhs = _moe_case(E, tokens, topk, N, K)
    wq_t, s_t, b_t = u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype)
    x_t = to_torch(x, dtype)
    y = mb.gather_qmm(x_t, wq_t, s_t, b_t, rhs_indices=torch.from_numpy(rhs.astype(np.int64)),
                      lhs_indices=torch.from_numpy(lhs.astype(np.int64)))
    assert tuple(y.shape) == (tokens, topk, 1, N)
    rhs_t = torch.from_numpy(rhs.astype(np.int64)).cuda()
    for e in range(E):
        tok, slot = torch.nonzero(rhs_t == e, as_tuple=True)
        ye = mb.quantized_matmul(x_t[tok, 0], wq_t.view(torch.int32)[e].view(torch.uint32), s_t[e], b_t[e])
        got = y[tok, slot, 0]
        assert torch.allclose(got.float(), ye.float(), rtol=2e-2, atol=2e-2), e
    idx = [(0, 0), (17, 1), (511, 1), (300, 0)]
    for t, k in idx:
        e = int(rhs[t, k])
        ref = O.qmm_f32_from(x[t], wq[e], s[e], b[e], dtype, transpose=True, group_size=64, bits=4)
        ok, rel = qmm_close(O.to_f32(from_torch(y[t, k]), dtype), ref)
        assert ok, rel


def test_gather_grouped_bad_index_flagged():
    from mlx_b200 import _lib, ops
    import ctypes
    dtype, wq, s, b, x, lhs, rhs = _moe_case(4, 16, 2, 128, 256)
    rhs[5, 1] = 77  # out of range expert
    y = mb.gather_qmm(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype),
                      lhs_indices=torch.from_numpy(lhs.astype(np.int64)), rhs_indices=torch.from_numpy(rhs.astype(np.int64)))
    torch.cuda.synchronize()
    assert bool((y[5, 1] == 0).all()) and bool((y[5, 0] != 0).any())
    ws = ops._workspaces.get(y.device, 0, "gather")
    st = (ctypes.c_uint32 * 4)()
    rc = _lib.load().b200q_read_status(ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), st)
    assert rc == 0 and st[0] == 1 and st[1] == 5 * 2 + 1
    good = np.ones(rhs.shape, bool); good[5, 1] = False
    ref = O.gather_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), lhs[good], rhs[good], True, 64, 4, "f32")
    got = O.to_f32(from_torch(y), dtype)[good]
    ok, rel = qmm_close(got.reshape(ref.shape), ref)
    assert ok, rel


def test_gather_then_decode_on_one_stream():
    """A grouped gather_qmm followed by a decode-sized quantized_matmul on the same stream: the
    gather's scratch (sorted indices, tile table, gathered rows) must not leak into the counters
    the decode kernel expects to find at zero."""
    E, tokens, topk, N, K, g = 4, 48, 2, 256, 512, 64
    dtype, wq, s, b, x, lhs, rhs = _moe_case(E, tokens, topk, N, K, 1, g)
    wq_t, s_t, b_t, x_t = u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype), to_torch(x, dtype)
    for _ in range(2):
        mb.gather_qmm(x_t, wq_t, s_t, b_t, lhs_indices=torch.from_numpy(lhs.astype(np.int64)),
                      rhs_indices=torch.from_numpy(rhs.astype(np.int64)), group_size=g, bits=4)
        y = mb.quantized_matmul(x_t[:3, 0], wq_t.view(torch.int32)[1].view(torch.uint32), s_t[1], b_t[1], group_size=g, bits=4)
        ref = O.qmm_f32_from(x[:3, 0], wq[1], s[1], b[1], dtype, transpose=True, group_size=g, bits=4)
        ok, rel = qmm_close(O.to_f32(from_torch(y), dtype), ref)
        assert ok, rel


@pytest.mark.parametrize("E,tokens,topk,K1,N1,N2", [(8, 96, 2, 512, 384, 256), (4, 33, 4, 1024, 1024, 128)])
def test_gather_chain_vs_two_calls_and_oracle(E, tokens, topk, K1, N1, N2):
    """Two chained gather_qmm with one sort: identical to calling gather_qmm twice (the kernels and
    the rounding of the intermediate are the same) and close to the oracle."""
    g, dtype = 64, "bf16"
    wq1, s1, b1 = O.quantize(make_w(50, (E, N1, K1), dtype), g, 4, dtype)
    wq2, s2, b2 = O.quantize(make_w(51, (E, N2, N1), dtype), g, 4, dtype)
    x = make_x(52, (tokens, 1, K1), dtype)
    rng = np.random.default_rng(9)
    rhs = rng.integers(0, E, size=(tokens, topk)).astype(np.int64)
    t = lambda a: to_torch(a, dtype)
    args1 = (u32_to_torch(wq1), t(s1), t(b1))
    args2 = (u32_to_torch(wq2), t(s2), t(b2))
    lhs = torch.arange(tokens).reshape(tokens, 1).expand(tokens, topk)
    y = mb.gather_qmm_chain(t(x), *args1, *args2, rhs_indices=torch.from_numpy(rhs), lhs_indices=lhs)
    assert tuple(y.shape) == (tokens, topk, 1, N2)
    h = mb.gather_qmm(t(x), *args1, lhs_indices=lhs, rhs_indices=torch.from_numpy(rhs))           # [tokens, topk, 1, N1]
    y2 = mb.gather_qmm(h.reshape(tokens * topk, 1, N1), *args2, rhs_indices=torch.from_numpy(rhs.reshape(-1)))
    assert torch.equal(y.reshape(-1, N2).view(torch.int16), y2.reshape(-1, N2).view(torch.int16))
    hq = from_torch(h.reshape(tokens * topk, 1, N1).contiguous())
    ref = O.gather_qmm(O.to_f32(hq, dtype), wq2, O.to_f32(s2, dtype), O.to_f32(b2, dtype),
                       np.arange(tokens * topk, dtype=np.uint32), rhs.reshape(-1).astype(np.uint32), True, g, 4, "f32")
    ok, rel = qmm_close(O.to_f32(from_torch(y.contiguous()), dtype).reshape(ref.shape), ref)
    assert ok, rel


@pytest.mark.parametrize("E,tokens,topk,K1,H,N2", [(4, 48, 2, 256, 384, 256), (8, 160, 2, 512, 1024, 512)])
def test_gather_swiglu_vs_three_calls_and_oracle(E, tokens, topk, K1, H, N2):
    """Gated expert MLP with one sort: the same as three gather_qmm calls with the activation
    between them (fp32 silu(g)*u of the bfloat16 products, one rounding), and its last product
    close to the oracle's on the same activations."""
    g, dtype = 64, "bf16"
    trip = lambda seed, shape: O.quantize(make_w(seed, shape, dtype), g, 4, dtype)
    gate, up, down = trip(60, (E, H, K1)), trip(61, (E, H, K1)), trip(62, (E, N2, H))
    x = make_x(63, (tokens, 1, K1), dtype)
    rng = np.random.default_rng(10)
    rhs = rng.integers(0, E, size=(tokens, topk)).astype(np.int64)
    t = lambda a: to_torch(a, dtype)
    dev = lambda q: (u32_to_torch(q[0]), t(q[1]), t(q[2]))
    lhs = torch.arange(tokens).reshape(tokens, 1).expand(tokens, topk)
    rhs_t = torch.from_numpy(rhs)
    y = mb.gather_qmm_swiglu(t(x), dev(gate), dev(up), dev(down), rhs_indices=rhs_t, lhs_indices=lhs)
    assert tuple(y.shape) == (tokens, topk, 1, N2)
    hg = mb.gather_qmm(t(x), *dev(gate), lhs_indices=lhs, rhs_indices=rhs_t).float()
    hu = mb.gather_qmm(t(x), *dev(up), lhs_indices=lhs, rhs_indices=rhs_t).float()
    h = (hg / (1.0 + torch.exp(-hg)) * hu).to(torch.bfloat16).reshape(tokens * topk, 1, H)
    y3 = mb.gather_qmm(h, *dev(down), rhs_indices=rhs_t.reshape(-1))
    # the device's fast exp/divide may move an activation by one bfloat16 step: compare within tolerance
    ok, rel = qmm_close(y.float().cpu().numpy().reshape(-1, N2), y3.float().cpu().numpy().reshape(-1, N2))
    assert ok, rel
    ref = O.gather_qmm(O.to_f32(from_torch(h.contiguous()), dtype), down[0], O.to_f32(down[1], dtype), O.to_f32(down[2], dtype),
                       np.arange(tokens * topk, dtype=np.uint32), rhs.reshape(-1).astype(np.uint32), True, g, 4, "f32")
    ok, rel = qmm_close(O.to_f32(from_torch(y.contiguous()), dtype).reshape(ref.shape), ref)
    assert ok, rel
