"""GPU parity of quantized_matmul against the reference's float instantiation fed the
same (exactly representable) inputs.  Tolerance (bf16/f16 outputs):
|y - y_ref| <= 1e-2*|y_ref| + 1e-2*rms(y_ref); float32 outputs: 1e-4 on the same form."""
import os

import numpy as np
import pytest
import torch

import mlx_b200 as mb
import oracle as O
from util import col_scale, from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "affine_golden.npz")
REL = {"f32": 1e-4, "f16": 1e-2, "bf16": 1e-2}


def run_case(dtype, M, N, K, g, bits, transpose=True, seed=0, expect_kernel=None):
    wshape = (N, K) if transpose else (K, N)
    w = make_w(100 + seed, wshape, dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    x = make_x(200 + seed, (M, K), dtype)
    ref = O.qmm_f32_from(x, wq, s, b, dtype, transpose=transpose, group_size=g, bits=bits)
    if expect_kernel is not None:
        assert mb.qmm_kernel_name(torch.bfloat16 if dtype == "bf16" else (torch.float16 if dtype == "f16" else torch.float32),
                                  M, N, K, g, bits, transpose) in expect_kernel
    y = mb.quantized_matmul(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype),
                            transpose=transpose, group_size=g, bits=bits)
    assert tuple(y.shape) == (M, N)
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype), ref, REL[dtype])
    assert ok, f"max err / max|ref| = {rel:.3e}"
    return rel


@pytest.mark.parametrize("dtype", ("f32", "f16", "bf16"))
@pytest.mark.parametrize("g", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_golden_qmm(dtype, g, bits):
    gold = np.load(GOLDEN)
    t = f"{dtype}_g{g}_b{bits}"
    args = (u32_to_torch(gold[f"{t}/wq"]), to_torch(gold[f"{t}/s"], dtype), to_torch(gold[f"{t}/b"], dtype))
    y = mb.quantized_matmul(to_torch(gold[f"{t}/x"], dtype), *args, transpose=True, group_size=g, bits=bits)
    # the golden weights hold rows of very different magnitude (edge-case groups): scale the
    # absolute term per output column
    cs = col_scale(gold[f"{t}/wq"], gold[f"{t}/s"], gold[f"{t}/b"], gold[f"{t}/x"], dtype, g, bits)
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype), gold[f"{t}/y32"], REL[dtype], cs[None, :])
    assert ok, rel
    # transpose=False on the same packed array read as [K=8, N=256]
    yn = mb.quantized_matmul(to_torch(gold[f"{t}/xn"], dtype), *args, transpose=False, group_size=g, bits=bits)
    refn = O.qmm_f32_from(gold[f"{t}/xn"], gold[f"{t}/wq"], gold[f"{t}/s"], gold[f"{t}/b"], dtype,
                          transpose=False, group_size=g, bits=bits)
    ok, rel = qmm_close(O.to_f32(from_torch(yn), dtype), refn, REL[dtype])
    assert ok, rel


# ---- decode path (mma.sync GEMV / skinny GEMM) ---------------------------------------
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
@pytest.mark.parametrize("g", (32, 64, 128))
@pytest.mark.parametrize("M", (1, 3, 8, 9, 16))
def test_qmv_all_widths(bits, g, M):
    run_case("bf16", M, 512, 1024, g, bits, seed=bits * 10 + M, expect_kernel=("qmv_rows", "qmv_mma"))


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 14336, 4096), (7, 67, 256), (2, 8, 128), (16, 1000, 2048),
                                   (5, 28672, 8192), (13, 4104, 4096), (16, 24, 128)])
def test_qmv_shapes_4bit(M, N, K):
    run_case("bf16", M, N, K, 64, 4, seed=M + N, expect_kernel=("qmv_rows", "qmv_mma"))


@pytest.mark.parametrize("M,g", [(1, 64), (2, 32), (4, 128)])
def test_row_owning_kernel_on_a_large_ragged_matrix(M, g):
    """Large matrices whose row count is not a multiple of the 16-row stage (the last stage of the
    last thread block is zero-filled past N)."""
    run_case("bf16", M, 28672 - 96 + 5, 8192, g, 4, seed=M + g, expect_kernel=("qmv_rows",))


def test_qmv_repeated_calls_reuse_scratch():
    """The scratch counters and partial sums must be left clean by every call."""
    dtype, M, N, K = "bf16", 16, 14336, 4096
    w = make_w(1, (N, K), dtype)
    wq, s, b = O.quantize(w, 64, 4, dtype)
    args = (u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    x = to_torch(make_x(2, (M, K), dtype), dtype)
    y0 = mb.quantized_matmul(x, *args)
    for _ in range(5):
        y = mb.quantized_matmul(x, *args)
        assert torch.equal(y.view(torch.int16), y0.view(torch.int16)) or torch.allclose(y.float(), y0.float(), rtol=2e-2, atol=1e-2)
    ref = O.qmm_f32_from(from_torch(x), wq, s, b, dtype, transpose=True, group_size=64, bits=4)
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype), ref)
    assert ok, rel


# ---- generic path ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ("f32", "f16"))
@pytest.mark.parametrize("transpose", (True, False))
@pytest.mark.parametrize("bits,g", [(2, 128), (4, 64), (8, 32), (3, 64), (5, 32), (6, 128)])
@pytest.mark.parametrize("M", (8, 33))
def test_generic_shapes(dtype, transpose, bits, g, M):
    # shapes of the reference's test_qmm (python/tests/test_quantized.py:288-323)
    run_case(dtype, M, 256, 128, g, bits, transpose=transpose, seed=M)


@pytest.mark.parametrize("transpose", (True, False))
def test_bf16_no_transpose_and_ragged(transpose):
    run_case("bf16", 33, 384, 256, 64, 4, transpose=transpose, seed=3)
    run_case("bf16", 5, 96, 160, 32, 8, transpose=transpose, seed=4)


def test_batched_x_and_vector_x():
    dtype = "bf16"
    w = make_w(5, (256, 512), dtype)
    wq, s, b = O.quantize(w, 64, 4, dtype)
    x = make_x(6, (3, 4, 512), dtype)
    y = mb.quantized_matmul(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    assert tuple(y.shape) == (3, 4, 256)
    ref = O.qmm_f32_from(x.reshape(12, 512), wq, s, b, dtype, transpose=True, group_size=64, bits=4)
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype).reshape(12, 256), ref)
    assert ok, rel
    yv = mb.quantized_matmul(to_torch(x[0, 0], dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    assert tuple(yv.shape) == (256,)
    ok, rel = qmm_close(O.to_f32(from_torch(yv), dtype), ref[0])
    assert ok, rel


def test_batched_weights():
    dtype = "f32"
    w = make_w(7, (3, 64, 128), dtype)
    wq, s, b = O.quantize(w, 32, 4, dtype)
    x = make_x(8, (3, 5, 128), dtype)
    y = mb.quantized_matmul(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype), group_size=32)
    for i in range(3):
        ref = O.qmm(x[i], wq[i], s[i], b[i], True, 32, 4, dtype)
        ok, rel = qmm_close(from_torch(y[i]), ref, 1e-4)
        assert ok, rel


def test_mixed_dtype_promotes_to_float32():
    # bf16 x with float32 scales promotes to float32 (mlx/ops.cpp:4803-4818)
    w = make_w(9, (64, 128), "f32")
    wq, s, b = O.quantize(w, 64, 4, "f32")
    x = make_x(10, (4, 128), "bf16")
    y = mb.quantized_matmul(to_torch(x, "bf16"), u32_to_torch(wq), to_torch(s, "f32"), to_torch(b, "f32"))
    assert y.dtype == torch.float32
    ref = O.qmm(O.to_f32(x, "bf16"), wq, s, b, True, 64, 4, "f32")
    ok, rel = qmm_close(from_torch(y), ref, 1e-4)
    assert ok, rel


def test_register_path_decode_kernel_in_subprocess():
    """B200Q_QMV_IMPL=mma keeps the row-owning kernel out of the selection, so the register-path
    kernel (the one that also serves bits 3/5/6 and ragged K) runs the 4-bit shapes; the override is
    read once per process, hence the child process."""
    import subprocess
    import sys
    code = r'''
import sys
sys.path.insert(0, "tests")
import torch, oracle as O, mlx_b200 as mb
from util import from_torch, make_w, make_x, qmm_close, to_torch, u32_to_torch
for (M, N, K, g) in [(1, 4096, 4096, 64), (16, 14336, 4096, 64), (8, 1000, 2048, 32), (13, 4104, 4096, 128)]:
    assert mb.qmm_kernel_name(torch.bfloat16, M, N, K, g, 4) == "qmv_mma"
    wq, s, b = O.quantize(make_w(N, (N, K), "bf16"), g, 4, "bf16")
    x = make_x(M, (M, K), "bf16")
    ref = O.qmm_f32_from(x, wq, s, b, "bf16", transpose=True, group_size=g, bits=4)
    for _ in range(2):
        y = mb.quantized_matmul(to_torch(x, "bf16"), u32_to_torch(wq), to_torch(s, "bf16"), to_torch(b, "bf16"), group_size=g, bits=4)
    ok, rel = qmm_close(O.to_f32(from_torch(y), "bf16"), ref)
    assert ok, (M, N, K, g, rel)
print("mma-ok")
'''
    env = dict(os.environ, B200Q_QMV_IMPL="mma")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "mma-ok" in res.stdout, res.stdout + res.stderr


@pytest.mark.parametrize("bits,g", [(2, 64), (2, 128), (4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)])
@pytest.mark.parametrize("M", (1, 7, 8, 9, 16))
def test_row_owning_kernel_every_instantiation(bits, g, M):
    """Every (bits, group, token-tile) instantiation of the row-owning kernel, on a K that needs two
    phases for some of them and a row count that leaves the last 16-row stage half empty."""
    run_case("bf16", M, 2504, 4096, g, bits, seed=bits + g + M, expect_kernel=("qmv_rows",))


@pytest.mark.parametrize("M,N,K,bits,g", [(3, 4096, 14336, 4, 64), (16, 4096, 14336, 4, 64), (2, 1024, 28672, 8, 64),
                                          (16, 520, 7168, 4, 32), (5, 136, 16384, 2, 128)])
def test_row_owning_kernel_long_k_phases(M, N, K, bits, g):
    """K longer than one phase of the 16 K slices: phases of different widths, running sums in shared memory."""
    run_case("bf16", M, N, K, g, bits, seed=M + K, expect_kernel=("qmv_rows",))


@pytest.mark.parametrize("M,N,K,bits,g", [(17, 2504, 4096, 4, 64), (24, 1024, 2048, 8, 32), (25, 520, 8192, 2, 64),
                                          (32, 14336, 4096, 4, 64)])
def test_row_owning_kernel_two_passes(M, N, K, bits, g):
    """17 to 32 token rows: two passes of the row-owning kernel (16 rows, then the rest)."""
    run_case("bf16", M, N, K, g, bits, seed=M + N, expect_kernel=("qmv_rows",))


def test_kernel_selection_by_token_count():
    """The selection a caller sees for C2's matrix as the token count grows."""
    name = lambda M, **kw: mb.qmm_kernel_name(torch.bfloat16, M, 14336, 4096, kw.get("g", 64), kw.get("bits", 4))
    assert [name(M) for M in (1, 16, 17, 32, 33, 64, 512)] == ["qmv_rows"] * 4 + ["qmm_tcgen05"] * 3
    assert name(32, bits=3) == "qmm_tcgen05" and name(16, bits=3) == "qmv_mma"


def test_row_owning_kernel_extreme_activations():
    """Each warp scales its x slice by a power of two chosen from the slice's magnitude: values
    up to 2^60 and down to 2^-60 must survive."""
    dtype, M, N, K = "bf16", 4, 256, 1024
    w = make_w(7, (N, K), dtype)
    wq, s, b = O.quantize(w, 64, 4, dtype)
    rng = np.random.default_rng(8)
    xf = rng.standard_normal((M, K)).astype(np.float32)
    xf[0] *= 2.0 ** 60
    xf[1] *= 2.0 ** -60
    xf[2, ::7] *= 2.0 ** 40
    x = O.to_dtype(xf, dtype)
    ref = O.qmm_f32_from(x, wq, s, b, dtype, transpose=True, group_size=64, bits=4)
    y = mb.quantized_matmul(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    assert mb.qmm_kernel_name(torch.bfloat16, M, N, K, 64, 4) == "qmv_rows"
    got = O.to_f32(from_torch(y), dtype)
    for m in range(M):   # rows differ by 120 binades: compare row by row
        ok, rel = qmm_close(got[m:m + 1], ref[m:m + 1])
        assert ok, (m, rel)


# ---- prefill path (TMA + tcgen05 + TMEM) -------------------------------------------------
@pytest.mark.parametrize("M,N,K,g", [(64, 128, 128, 64), (17, 128, 128, 32), (33, 256, 256, 128), (256, 256, 512, 64),
                                     (300, 384, 1024, 128), (100, 200, 256, 64), (512, 1024, 4096, 64),
                                     (257, 130, 384, 32)])
def test_tcgen05_shapes(M, N, K, g):
    run_case("bf16", M, N, K, g, 4, seed=M + K, expect_kernel=("qmm_tcgen05",))


@pytest.mark.parametrize("bits", (2, 3, 5, 6, 8))
@pytest.mark.parametrize("g", (32, 64, 128))
def test_tcgen05_all_bit_widths(bits, g):
    run_case("bf16", 96, 200, 640, g, bits, seed=bits + g, expect_kernel=("qmm_tcgen05",))
    run_case("bf16", 512, 256, 1024, g, bits, seed=bits, expect_kernel=("qmm_tcgen05",))


@pytest.mark.parametrize("bits", (4, 8, 3))
@pytest.mark.parametrize("M", (8, 96))
def test_rows_of_very_different_magnitude(bits, M):
    """Weight rows spanning 2^-24 .. 2^8 in magnitude, some all zero: the prefill kernel's unpack has
    a form for scales whose exponent leaves room for a factor 2^133 and a general form for the
    others, and both meet inside one warp here; the decode kernels see the same matrix (M = 8).
    Tolerance per output column: 1e-2 (|y_ref| + ||w_n|| rms(x))."""
    dtype, N, K, g = "bf16", 384, 1024, 64
    rng = np.random.default_rng(40 + bits)
    wf = rng.standard_normal((N, K)).astype(np.float32) * (2.0 ** rng.integers(-24, 9, size=(N, 1))).astype(np.float32)
    wf[5] = 0.0
    wf[200, :512] = 0.0
    w = O.to_dtype(wf, dtype)
    wq, s, b = O.quantize(w, g, bits, dtype)
    x = make_x(41, (M, K), dtype)
    ref = O.qmm_f32_from(x, wq, s, b, dtype, transpose=True, group_size=g, bits=bits)
    y = mb.quantized_matmul(to_torch(x, dtype), u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype),
                            group_size=g, bits=bits)
    cs = col_scale(wq, s, b, x, dtype, g, bits)
    ok, rel = qmm_close(O.to_f32(from_torch(y), dtype), ref, 1e-2, cs[None, :])
    assert ok, rel
    assert not from_torch(y)[:, 5].any()


def test_ragged_k_falls_back_to_generic():
    run_case("bf16", 40, 96, 192, 32, 4, seed=1, expect_kernel=("qmm_generic",))


def test_tcgen05_prefill_full_size_sampled_rows():
    """Prefill configuration (M=4096, N=14336, K=4096, 4-bit g64): the oracle checks 48 sampled
    token rows over all N; linearity over the token axis covers the rest: y(x1 + x2) rows equal
    the sum of separately computed rows within the bf16 tolerance."""
    dtype, M, N, K = "bf16", 4096, 14336, 4096
    w = make_w(2, (N, K), dtype)
    wq, s, b = O.quantize(w, 64, 4, dtype)
    x = make_x(1, (M, K), dtype)
    args = (u32_to_torch(wq), to_torch(s, dtype), to_torch(b, dtype))
    y = mb.quantized_matmul(to_torch(x, dtype), *args)
    assert mb.qmm_kernel_name(torch.bfloat16, M, N, K, 64, 4) == "qmm_tcgen05"
    rows = np.unique(np.concatenate([np.arange(0, 8), np.arange(M - 8, M), np.random.default_rng(5).integers(0, M, 32)]))
    ref = O.qmm_f32_from(x[rows], wq, s, b, dtype, transpose=True, group_size=64, bits=4)
    got = O.to_f32(from_torch(y[torch.from_numpy(rows).cuda()]), dtype)
    ok, rel = qmm_close(got, ref)
    assert ok, rel
    # every row is finite and non-trivial, and tile seams (multiples of 256 tokens / 128 rows of W) are covered
    yf = y.float()
    assert bool(torch.isfinite(yf).all()) and float(yf.abs().mean()) > 0.1
    seam_rows = np.array([255, 256, 257, 511, 512, 2047, 2048, 3839, 3840])
    ref2 = O.qmm_f32_from(x[seam_rows], wq, s, b, dtype, transpose=True, group_size=64, bits=4)
    ok, rel = qmm_close(O.to_f32(from_torch(y[torch.from_numpy(seam_rows).cuda()]), dtype), ref2)
    assert ok, rel


# ---- non-transposed decode (qvm): y = x @ dequant(W[K, N]) -----------------------------------
@pytest.mark.parametrize("dtype", ("bf16", "f16", "f32"))
@pytest.mark.parametrize("bits,g", [(4, 64), (8, 32), (2, 128)])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (4, 1536, 1000), (2, 64, 7), (3, 14336, 512)])
def test_qvm_no_transpose(dtype, bits, g, M, N, K):
    if N % g:
        pytest.skip("N must be a multiple of the group size")
    rel = run_case(dtype, M, N, K, g, bits, transpose=False, seed=M + K, expect_kernel=("qvm",))
    assert rel < 2e-2


def test_qvm_then_transposed_decode_share_workspace():
    """The split-K slots of the non-transposed kernel must be left zeroed for the kernels that
    accumulate into the same workspace."""
    for _ in range(2):
        run_case("bf16", 2, 4096, 2048, 64, 4, transpose=False, seed=11, expect_kernel=("qvm",))
        run_case("bf16", 16, 1000, 2048, 64, 4, seed=12, expect_kernel=("qmv_rows", "qmv_mma"))


# ---- host-buffer entry point -------------------------------------------------------------------
@pytest.mark.parametrize("pinned", (True, False))
@pytest.mark.parametrize("M", (16, 64))
def test_qmm_host_buffers(pinned, M):
    """b200q_qmm_host with pinned (result written by the kernel straight to host memory when small)
    and pageable (staged copy) host buffers gives the same result as the device call."""
    import ctypes
    from mlx_b200 import _lib
    lib = _lib.load()
    N, K, g = 1024, 512, 64
    wq, s, b = O.quantize(make_w(3, (N, K), "bf16"), g, 4, "bf16")
    x = make_x(4, (M, K), "bf16")
    ref = O.qmm_f32_from(x, wq, s, b, "bf16", transpose=True, group_size=g, bits=4)
    wq_t, s_t, b_t = u32_to_torch(wq), to_torch(s, "bf16"), to_torch(b, "bf16")
    x_host = to_torch(x, "bf16").cpu()
    y_host = torch.zeros(M, N, dtype=torch.bfloat16)
    if pinned:
        x_host, y_host = x_host.pin_memory(), y_host.pin_memory()
    x_dev = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    y_dev = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    need = max(int(lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M, N, K, g, 4, 1)), 256)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    for _ in range(2):
        rc = lib.b200q_qmm_host(P(x_host), P(x_dev), P(wq_t), P(s_t), P(b_t), P(y_dev), P(y_host), _lib.BF16, M, N, K, g, 4, 1,
                                P(ws), ws.numel(), None)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
    ok, rel = qmm_close(O.to_f32(y_host.view(torch.int16).numpy().view(np.uint16), "bf16"), ref)
    assert ok, rel


def test_quantize_then_matmul_on_a_reused_buffer():
    """The decode kernels start under programmatic dependent launch.  By default they request the
    weights only after the previous kernel of the stream has finished, so a quantize (or any other
    producer of wq / scales / biases) directly in front of the matmul, writing into buffers the
    previous matmul has just read, gives the same bits as a fully serialised run."""
    dtype, M, N, K, g, bits = "bf16", 16, 4096, 4096, 64, 4
    x = to_torch(make_x(5, (M, K), dtype), dtype)
    ws = [to_torch(make_w(40 + i, (N, K), dtype), dtype) for i in range(3)]
    wq = torch.empty(N, K * bits // 32, dtype=torch.uint32, device="cuda")
    s = torch.empty(N, K // g, dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(s)
    import ctypes
    from mlx_b200 import _lib
    lib = _lib.load()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = max(int(lib.b200q_qmm_workspace_bytes(_lib.BF16, 1, M, N, K, g, bits, 1)), 256)
    wsp = torch.zeros(need, dtype=torch.uint8, device="cuda")
    outs, refs = [], []
    for rnd in range(6):
        w = ws[rnd % 3]
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        assert lib.b200q_quantize(P(w), _lib.BF16, N, K, g, bits, P(wq), P(s), P(b), st) == 0
        assert lib.b200q_qmm(P(x), P(wq), P(s), P(b), P(y), _lib.BF16, 1, M, N, K, g, bits, 1, 0, P(wsp), wsp.numel(), st) == 0
        outs.append(y)
    torch.cuda.synchronize()
    for rnd in range(6):   # the serialised reference: synchronise between the two calls
        q = mb.quantize(ws[rnd % 3], g, bits)
        torch.cuda.synchronize()
        refs.append(mb.quantized_matmul(x, *q, group_size=g, bits=bits))
        torch.cuda.synchronize()
    for y, r in zip(outs, refs):
        assert torch.equal(y.view(torch.int16), r.view(torch.int16))
