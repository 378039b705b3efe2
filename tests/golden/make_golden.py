"""Generates tests/golden/affine_golden.npz and tests/golden/gguf_unpack_golden.npz by running
the reference project's own CPU code (oracle/_ref/ref_oracle and oracle/_ref/ref_gguf, compiled
from the reference checkout by oracle/Makefile).

    python tests/golden/make_golden.py

Only runs where the reference checkout is available; the produced file is committed
so that the pin tests can run anywhere.  Inputs are seeded numpy draws; every case
stores inputs and the reference outputs.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "affine_golden.npz")
OUT_GGUF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gguf_unpack_golden.npz")


def special_rows(w, g):
    """Edge groups the reference arithmetic treats specially."""
    w[0, :g] = 0.0                      # all-zero group
    w[1, :g] = 0.375                    # constant group
    w[2, :g] = -np.abs(w[2, :g])        # all-negative group
    w[3, :g] = np.abs(w[3, :g])         # all-positive group
    w[4, 0] = 1.0                       # |min| == |max|
    w[4, 1:g] = -1.0
    w[5, :g] = (np.arange(g) - g // 2) * 0.5  # values that land on .5 rounding ties
    return w


def main():
    O.build(with_reference=True)
    assert O.have_reference(), "reference binary missing"
    data = {}
    rng = np.random.default_rng(20240229)
    for dtype in ("f32", "f16", "bf16"):
        for g in (32, 64, 128):
            for bits in (2, 3, 4, 5, 6, 8):
                tag = f"{dtype}_g{g}_b{bits}"
                K = 256
                w = (0.02 * rng.standard_normal((8, K))).astype(np.float32)
                w = O.to_dtype(special_rows(w, g), dtype)
                wq, s, b = O.ref_quantize(w, g, bits, dtype)
                x = O.to_dtype(rng.standard_normal((3, K)).astype(np.float32), dtype)
                y, _ = O.ref_qmm(x, wq, s, b, True, g, bits, dtype)
                # float instantiation fed the same (exactly representable) inputs
                y32, _ = O.ref_qmm(O.to_f32(x, dtype), wq, O.to_f32(s, dtype), O.to_f32(b, dtype), True, g, bits, "f32")
                # no-transpose: the same packed array read as W[K=8, N=256]
                xn = O.to_dtype(rng.standard_normal((2, 8)).astype(np.float32), dtype)
                yn, _ = O.ref_qmm(xn, wq, s, b, False, g, bits, dtype)
                for k, v in dict(w=w, wq=wq, s=s, b=b, x=x, y=y, y32=y32, xn=xn, yn=yn).items():
                    data[f"{tag}/{k}"] = v
    # gather: 4 experts, 6 index pairs, M=2
    g, bits, dtype, K, N, E = 64, 4, "f32", 128, 16, 4
    w = (0.02 * rng.standard_normal((E, N, K))).astype(np.float32)
    wq, s, b = O.ref_quantize(w, g, bits, dtype)
    x = rng.standard_normal((5, 2, K)).astype(np.float32)
    lhs = np.array([4, 0, 3, 3, 1, 2], dtype=np.uint32)
    rhs = np.array([1, 3, 0, 2, 2, 1], dtype=np.uint32)
    y = O.ref_gather_qmm(x, wq, s, b, lhs, rhs, True, g, bits, dtype)
    for k, v in dict(wq=wq, s=s, b=b, x=x, lhs=lhs, rhs=rhs, y=y).items():
        data[f"gather/{k}"] = v
    np.savez_compressed(OUT, **data)
    print(OUT, os.path.getsize(OUT), "bytes,", len(data), "arrays")
    # GGUF: the reference's nibble re-ordering of Q4 blocks (oracle/_ref/ref_gguf)
    assert O.have_reference_gguf(), "reference GGUF binary missing"
    quants = np.random.default_rng(20240301).integers(0, 256, (64, 16), dtype=np.uint8)
    quants[0] = np.arange(16) | (np.arange(16, 32) % 16) << 4     # weight j -> j % 16, readable by eye
    np.savez_compressed(OUT_GGUF, quants=quants, unpacked=O.ref_gguf_unpack(quants))
    print(OUT_GGUF, os.path.getsize(OUT_GGUF), "bytes")


if __name__ == "__main__":
    main()
