"""Shared helpers for the parity tests: seeded inputs, torch<->numpy carriers, error metric."""
import numpy as np
import torch

import oracle as O

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_torch(a: np.ndarray, dtype: str, device="cuda") -> torch.Tensor:
    """Oracle carrier array -> torch tensor of the real dtype."""
    if dtype == "bf16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def u32_to_torch(a: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32).copy()).view(torch.uint32).to(device)


def from_torch(t: torch.Tensor) -> np.ndarray:
    """torch tensor -> oracle carrier array (bf16 as uint16 bits, uint32 as uint32)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def make_w(seed, shape, dtype, std=0.02):
    rng = np.random.default_rng(seed)
    return O.to_dtype((std * rng.standard_normal(shape)).astype(np.float32), dtype)


def make_x(seed, shape, dtype):
    rng = np.random.default_rng(seed)
    return O.to_dtype(rng.standard_normal(shape).astype(np.float32), dtype)


def qmm_close(y: np.ndarray, y_ref: np.ndarray, rel=1e-2, col_scale=None):
    """|y - y_ref| <= rel*|y_ref| + rel*S element-wise (both float32 arrays), where S is the
    typical output magnitude: rms(y_ref) by default, or `col_scale[n]` (for weights whose rows
    have very different magnitudes: ||w_n||_2 * rms(x), the a-priori scale of output column n).
    Returns (ok, max_err_over_max_ref)."""
    y = y.astype(np.float64)
    y_ref = y_ref.astype(np.float64)
    rms = float(np.sqrt(np.mean(y_ref**2))) if y_ref.size else 0.0
    if col_scale is not None:
        rms = np.asarray(col_scale, dtype=np.float64)
    err = np.abs(y - y_ref)
    ok = bool(np.all(err <= rel * np.abs(y_ref) + rel * rms + 1e-30))
    denom = float(np.max(np.abs(y_ref))) if y_ref.size else 1.0
    return ok, (float(err.max()) / denom if y_ref.size and denom > 0 else 0.0)


def col_scale(wq, s, b, x, dtype, g, bits):
    """||dequant(w)_n||_2 * rms(x) for transpose=True weights [N, K]."""
    wh = O.to_f32(O.dequantize(wq, s, b, g, bits, dtype), dtype).astype(np.float64)
    xf = O.to_f32(x, dtype).astype(np.float64)
    return np.sqrt((wh**2).sum(-1)) * np.sqrt((xf**2).mean())
