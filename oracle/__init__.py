"""TEST INFRASTRUCTURE ONLY - the CPU checker for the affine quantized-matmul path.

Nothing in the product package imports this module.  It is used by ``tests/``, by the
smoke test and by the CPU-baseline legs of ``bench.py``.

Two back ends, same numpy-level API:

* ``qref``  - ``oracle/qref.c``, a plain-C restatement of the reference CPU code
  (loaded with ctypes from ``oracle/_build/libqref.so``);
* ``ref``   - ``oracle/_ref/ref_oracle``, the reference project's own CPU translation
  unit compiled from the reference checkout (file driven, run as a subprocess).

bfloat16 arrays are carried as ``numpy.uint16`` bit patterns, float16 as
``numpy.float16`` and float32 as ``numpy.float32``; every function takes the element
type as the string ``"f32"``, ``"f16"`` or ``"bf16"``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_QREF_SO = os.path.join(_HERE, "_build", "libqref.so")
REF_BIN = os.path.join(_HERE, "_ref", "ref_oracle")
_DT = {"f32": 0, "f16": 1, "bf16": 2}
_NP = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}

_lib = None


def reference_root() -> str | None:
    """Checkout of the reference project: $REF_ROOT, else a directory named `reference` next to
    this repository.  None when neither holds the CPU translation unit."""
    cands = [os.environ.get("REF_ROOT"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "mlx", "backend", "cpu", "quantized.cpp")):
            return c
    return None


def build(with_reference: bool | None = None) -> None:
    """Compile the C restatement and, when the reference checkout is present, the
    reference-driven binary.  Building the checker is not using it."""
    ref_root = reference_root()
    targets = ["qref"]
    if with_reference is None:
        with_reference = ref_root is not None
    cmd = ["make", "-s", "-C", _HERE]
    if with_reference:
        if ref_root is None:
            raise RuntimeError("the reference checkout was not found: set REF_ROOT")
        targets.append("ref")
        cmd.append(f"REF_ROOT={ref_root}")
    subprocess.run(cmd + targets, check=True)


def have_reference() -> bool:
    return os.path.isfile(REF_BIN) and os.access(REF_BIN, os.X_OK)


def _load():
    global _lib
    if _lib is None:
        if not os.path.isfile(_QREF_SO):
            build(with_reference=False)
        lib = ctypes.CDLL(_QREF_SO)
        vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        lib.qref_quantize.argtypes = [vp, i32, sz, i32, i32, vp, vp, vp]
        lib.qref_dequantize.argtypes = [vp, vp, vp, i32, sz, i32, i32, vp]
        lib.qref_qmm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32]
        lib.qref_gather_qmm.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, i32, i32, i32, i32, i32, i32, i32]
        lib.qref_gguf_repack.argtypes = [vp, i32, sz, vp, vp, vp]
        for f in (lib.qref_quantize, lib.qref_dequantize, lib.qref_qmm, lib.qref_gather_qmm, lib.qref_gguf_repack):
            f.restype = i32
        _lib = lib
    return _lib


# ----------------------------------------------------------------------------- dtypes
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest even); returns uint16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_dtype(a_f32: np.ndarray, dtype: str) -> np.ndarray:
    """float32 values -> array in the carrier type of `dtype` (rounded to nearest even)."""
    if dtype == "f32":
        return np.ascontiguousarray(a_f32, dtype=np.float32)
    if dtype == "f16":
        return np.ascontiguousarray(a_f32, dtype=np.float32).astype(np.float16)
    return f32_to_bf16_bits(a_f32)


def to_f32(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return bf16_bits_to_f32(a)
    return np.ascontiguousarray(a).astype(np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _chk(a, dtype):
    a = np.ascontiguousarray(a)
    if a.dtype != _NP[dtype]:
        raise TypeError(f"expected carrier {_NP[dtype]} for {dtype}, got {a.dtype}")
    return a


# ------------------------------------------------------------------------ C restatement
def quantize(w, group_size=64, bits=4, dtype="f32"):
    """-> (wq uint32 [.., K*bits/32], scales [.., K/g], biases [.., K/g])."""
    w = _chk(w, dtype)
    K = w.shape[-1]
    lead = w.shape[:-1]
    wq = np.zeros(lead + (K * bits // 32,), dtype=np.uint32)
    s = np.zeros(lead + (K // group_size,), dtype=_NP[dtype])
    b = np.zeros_like(s)
    rc = _load().qref_quantize(_p(w), _DT[dtype], w.size, group_size, bits, _p(wq), _p(s), _p(b))
    if rc:
        raise ValueError(f"qref_quantize failed rc={rc}")
    return wq, s, b


def dequantize(wq, scales, biases, group_size=64, bits=4, dtype="f32"):
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    scales, biases = _chk(scales, dtype), _chk(biases, dtype)
    K = wq.shape[-1] * 32 // bits
    out = np.zeros(wq.shape[:-1] + (K,), dtype=_NP[dtype])
    rc = _load().qref_dequantize(_p(wq), _p(scales), _p(biases), _DT[dtype], out.size, group_size, bits, _p(out))
    if rc:
        raise ValueError(f"qref_dequantize failed rc={rc}")
    return out


def qmm(x, wq, scales, biases, transpose=True, group_size=64, bits=4, dtype="f32"):
    """2-D quantized matmul in element type `dtype` (the reference accumulates in T)."""
    x = _chk(x, dtype)
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    scales, biases = _chk(scales, dtype), _chk(biases, dtype)
    M, K = x.shape
    N = wq.shape[0] if transpose else wq.shape[1] * 32 // bits
    y = np.zeros((M, N), dtype=_NP[dtype])
    rc = _load().qref_qmm(_p(y), _p(x), _p(wq), _p(scales), _p(biases), _DT[dtype], M, N, K,
                          group_size, bits, int(transpose))
    if rc:
        raise ValueError(f"qref_qmm failed rc={rc}")
    return y


def gather_qmm(x, wq, scales, biases, lhs, rhs, transpose=True, group_size=64, bits=4, dtype="f32"):
    """x [Bx, M, K], wq [E, ., .], lhs/rhs flat uint32 [n] -> y [n, M, N]."""
    x = _chk(x, dtype)
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    scales, biases = _chk(scales, dtype), _chk(biases, dtype)
    lhs = np.ascontiguousarray(lhs, dtype=np.uint32).ravel()
    rhs = np.ascontiguousarray(rhs, dtype=np.uint32).ravel()
    _, M, K = x.shape
    N = wq.shape[1] if transpose else wq.shape[2] * 32 // bits
    y = np.zeros((lhs.size, M, N), dtype=_NP[dtype])
    rc = _load().qref_gather_qmm(_p(y), _p(x), _p(wq), _p(scales), _p(biases), _p(lhs), _p(rhs), lhs.size,
                                 _DT[dtype], M, N, K, group_size, bits, int(transpose))
    if rc:
        raise ValueError(f"qref_gather_qmm failed rc={rc}")
    return y


def qmm_f32_from(x, wq, scales, biases, dtype, **kw):
    """The parity oracle for matmul outputs: the reference's float instantiation fed the
    (exactly representable) low-precision inputs upcast to float32."""
    return qmm(to_f32(x, dtype), wq, to_f32(scales, dtype), to_f32(biases, dtype), dtype="f32", **kw)


# ------------------------------------------------------------- reference-compiled binary
def _run_ref(args, inputs, outputs):
    """inputs: {name: array}; outputs: {name: (dtype, shape)}.  `args` holds the names."""
    if not have_reference():
        raise FileNotFoundError(REF_BIN)
    with tempfile.TemporaryDirectory() as d:
        argv = [REF_BIN]
        for a in args:
            if a in inputs:
                path = os.path.join(d, a + ".bin")
                np.ascontiguousarray(inputs[a]).tofile(path)
                argv.append(path)
            elif a in outputs:
                argv.append(os.path.join(d, a + ".bin"))
            else:
                argv.append(str(a))
        res = subprocess.run(argv, check=True, capture_output=True, text=True)
        outs = {}
        for name, (dt, shape) in outputs.items():
            outs[name] = np.fromfile(os.path.join(d, name + ".bin"), dtype=dt).reshape(shape)
        return outs, res.stdout


def ref_quantize(w, group_size=64, bits=4, dtype="f32"):
    w = _chk(w, dtype)
    K = w.shape[-1]
    rows = w.size // K
    lead = w.shape[:-1]
    outs, _ = _run_ref(
        ["quantize", dtype, rows, K, group_size, bits, "w", "wq", "s", "b"],
        {"w": w},
        {"wq": (np.uint8, (rows, K * bits // 8)), "s": (_NP[dtype], lead + (K // group_size,)),
         "b": (_NP[dtype], lead + (K // group_size,))},
    )
    wq = outs["wq"].view(np.uint32).reshape(lead + (K * bits // 32,))
    return wq, outs["s"], outs["b"]


def ref_qmm(x, wq, scales, biases, transpose=True, group_size=64, bits=4, dtype="f32", reps=1):
    """Returns (y, seconds_per_call)."""
    x = _chk(x, dtype)
    M, K = x.shape
    N = wq.shape[0] if transpose else wq.shape[1] * 32 // bits
    outs, stdout = _run_ref(
        ["qmm", dtype, M, N, K, group_size, bits, int(transpose), "x", "wq", "s", "b", "y", reps],
        {"x": x, "wq": np.ascontiguousarray(wq, dtype=np.uint32), "s": _chk(scales, dtype), "b": _chk(biases, dtype)},
        {"y": (_NP[dtype], (M, N))},
    )
    secs = float(stdout.split()[-1])
    return outs["y"], secs


def ref_gather_qmm(x, wq, scales, biases, lhs, rhs, transpose=True, group_size=64, bits=4, dtype="f32"):
    x = _chk(x, dtype)
    _, M, K = x.shape
    N = wq.shape[1] if transpose else wq.shape[2] * 32 // bits
    lhs = np.ascontiguousarray(lhs, dtype=np.uint32).ravel()
    rhs = np.ascontiguousarray(rhs, dtype=np.uint32).ravel()
    outs, _ = _run_ref(
        ["gather", dtype, M, N, K, group_size, bits, int(transpose), lhs.size, "x", "wq", "s", "b", "lhs", "rhs", "y"],
        {"x": x, "wq": np.ascontiguousarray(wq, dtype=np.uint32), "s": _chk(scales, dtype),
         "b": _chk(biases, dtype), "lhs": lhs, "rhs": rhs},
        {"y": (_NP[dtype], (lhs.size, M, N))},
    )
    return outs["y"]


# ----------------------------------------------------------------------------- GGUF repack
GGUF_BLOCK_BYTES = {2: 18, 3: 20, 8: 34}   # Q4_0, Q4_1, Q8_0
REF_GGUF_BIN = os.path.join(_HERE, "_ref", "ref_gguf")


def have_reference_gguf() -> bool:
    return os.path.isfile(REF_GGUF_BIN) and os.access(REF_GGUF_BIN, os.X_OK)


def ref_gguf_unpack(quants: np.ndarray) -> np.ndarray:
    """The reference's own unpack_32_4 (mlx/io/gguf_quants.cpp:13-31) on uint8 [n, 16] quant
    bytes of Q4 blocks -> uint8 [n, 16] in the affine layout's nibble order."""
    quants = np.ascontiguousarray(quants, dtype=np.uint8).reshape(-1, 16)
    with tempfile.TemporaryDirectory() as d:
        fi, fo = os.path.join(d, "i.bin"), os.path.join(d, "o.bin")
        quants.tofile(fi)
        subprocess.run([REF_GGUF_BIN, "unpack", str(quants.shape[0]), fi, fo], check=True)
        return np.fromfile(fo, dtype=np.uint8).reshape(-1, 16)


def gguf_repack(blocks: np.ndarray, gguf_type: int):
    """blocks uint8 [n_blocks, block_bytes] -> (wq uint8 [n_blocks, 16 or 32], scales, biases as
    float16 bit patterns uint16 [n_blocks]); restates mlx/io/gguf_quants.cpp:11-102."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    n = blocks.shape[0]
    per = 16 if gguf_type in (2, 3) else 32
    wq = np.zeros((n, per), dtype=np.uint8)
    s = np.zeros(n, dtype=np.uint16)
    b = np.zeros(n, dtype=np.uint16)
    rc = _load().qref_gguf_repack(_p(blocks), gguf_type, n, _p(wq), _p(s), _p(b))
    if rc != 0:
        raise ValueError(f"qref_gguf_repack: unsupported type {gguf_type}")
    return wq, s, b
