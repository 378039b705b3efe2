"""Weight formats in: quantized checkpoints to device buffers without the reference project.

* safetensors files written by the reference (`mx.save_safetensors`, mlx/io/safetensors.cpp):
  `<name>.weight` (uint32, packed), `<name>.scales`, `<name>.biases` triples load as they are:
  the packed layout on disk is the layout the kernels read.
* GGUF files: tensors of type Q4_0 / Q4_1 / Q8_0 are repacked on the device to the affine layout
  (group size 32) by `b200q_gguf_repack`, as the reference's loader does on the host
  (mlx/io/gguf_quants.cpp:11-164: `<name>.weight` -> packed words, plus `<name>.scales` and
  `<name>.biases`); F32 / F16 / BF16 tensors load unchanged.

Only the file parsing runs on the host; there is no CPU repack path.
"""
from __future__ import annotations

import ctypes
import json
import struct
from typing import Dict, Tuple

import numpy as np
import torch

from . import _lib

# ------------------------------------------------------------------------------ safetensors
_ST_DTYPES = {
    "F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16),
    "U32": (np.uint32, torch.uint32), "I32": (np.int32, torch.int32), "U8": (np.uint8, torch.uint8),
    "I64": (np.int64, torch.int64), "U16": (np.uint16, torch.uint16), "I8": (np.int8, torch.int8),
}


def read_safetensors(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    """All tensors of a safetensors file (8-byte little-endian header length, JSON header with
    dtype / shape / data_offsets per tensor, then the raw little-endian data)."""
    with open(path, "rb") as fh:
        (hlen,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(hlen).decode("utf-8"))
        base = 8 + hlen
        out = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] not in _ST_DTYPES:
                raise ValueError(f"[read_safetensors] unsupported dtype {info['dtype']} for {name}")
            npdt, tdt = _ST_DTYPES[info["dtype"]]
            lo, hi = info["data_offsets"]
            fh.seek(base + lo)
            raw = np.frombuffer(fh.read(hi - lo), dtype=npdt).reshape(info["shape"]).copy()
            t = torch.from_numpy(raw.view(np.int32) if npdt is np.uint32 else raw)
            if npdt is np.uint32:
                t = t.view(torch.uint32)
            if tdt is torch.bfloat16:
                t = t.view(torch.bfloat16)
            out[name] = t.to(device)
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Minimal writer (round-trip tests and exporting quantized triples)."""
    rev = {v[1]: k for k, v in _ST_DTYPES.items()}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": rev[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(h)))
        fh.write(h)
        for b in blobs:
            fh.write(b)


def quantized_triples(tensors: Dict[str, torch.Tensor], group_size: int = None, bits: int = None):
    """{prefix: (wq, scales, biases, group_size, bits)} for every `<prefix>.weight` of dtype uint32
    that comes with `.scales` and `.biases`.  The two parameters are tied by
    K = 32 * words / bits = groups * group_size; give one (the reference keeps them in the model's
    config.json) or neither when only one supported pair fits."""
    out = {}
    for name, w in tensors.items():
        if not name.endswith(".weight") or w.dtype != torch.uint32:
            continue
        prefix = name[: -len(".weight")]
        s, b = tensors.get(prefix + ".scales"), tensors.get(prefix + ".biases")
        if s is None or b is None:
            continue
        words, groups = w.shape[-1], s.shape[-1]
        fits = [(g, bt) for g in (32, 64, 128) for bt in (2, 3, 4, 5, 6, 8)
                if words * 32 == groups * g * bt and (group_size in (None, g)) and (bits in (None, bt))]
        if len(fits) != 1:
            raise ValueError(f"[quantized_triples] {prefix}: cannot determine group_size/bits uniquely "
                             f"({words} words, {groups} groups, candidates {fits}); pass group_size or bits")
        out[prefix] = (w, s, b) + fits[0]
    return out


# ------------------------------------------------------------------------------------- GGUF
GGUF_F32, GGUF_F16, GGUF_Q4_0, GGUF_Q4_1, GGUF_Q8_0, GGUF_BF16 = 0, 1, 2, 3, 8, 30
_GGUF_BLOCK = {GGUF_Q4_0: 18, GGUF_Q4_1: 20, GGUF_Q8_0: 34}
_GGUF_SCALAR = {4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d", 0: "<B", 1: "<b", 2: "<H", 3: "<h"}


def _gguf_value(fh, vtype):
    if vtype in _GGUF_SCALAR:
        fmt = _GGUF_SCALAR[vtype]
        return struct.unpack(fmt, fh.read(struct.calcsize(fmt)))[0]
    if vtype == 8:  # string
        (n,) = struct.unpack("<Q", fh.read(8))
        return fh.read(n).decode("utf-8", errors="replace")
    if vtype == 9:  # array
        (et,) = struct.unpack("<I", fh.read(4))
        (n,) = struct.unpack("<Q", fh.read(8))
        return [_gguf_value(fh, et) for _ in range(n)]
    raise ValueError(f"[read_gguf] unknown metadata value type {vtype}")


def read_gguf_raw(path: str):
    """(metadata dict, {name: (gguf_type, shape [outermost first], raw uint8 array)}) of a GGUF v2/v3
    file.  Tensor shapes are stored innermost first in the file and are reversed here."""
    with open(path, "rb") as fh:
        if fh.read(4) != b"GGUF":
            raise ValueError("[read_gguf] not a GGUF file")
        (version,) = struct.unpack("<I", fh.read(4))
        if version < 2:
            raise ValueError(f"[read_gguf] GGUF version {version} is not supported")
        n_tensors, n_kv = struct.unpack("<QQ", fh.read(16))
        meta = {}
        for _ in range(n_kv):
            key = _gguf_value(fh, 8)
            (vt,) = struct.unpack("<I", fh.read(4))
            meta[key] = _gguf_value(fh, vt)
        infos = []
        for _ in range(n_tensors):
            name = _gguf_value(fh, 8)
            (nd,) = struct.unpack("<I", fh.read(4))
            dims = struct.unpack("<" + "Q" * nd, fh.read(8 * nd))
            gtype, offset = struct.unpack("<IQ", fh.read(12))
            infos.append((name, gtype, tuple(reversed(dims)), offset))
        align = int(meta.get("general.alignment", 32))
        data0 = (fh.tell() + align - 1) // align * align
        tensors = {}
        for name, gtype, shape, offset in infos:
            n = int(np.prod(shape)) if shape else 1
            if gtype in _GGUF_BLOCK:
                if shape[-1] % 32:
                    raise ValueError(f"[read_gguf] tensor {name} has incompatible last dim shape: {shape[-1]}")
                nbytes = n // 32 * _GGUF_BLOCK[gtype]
            elif gtype in (GGUF_F16, GGUF_BF16):
                nbytes = 2 * n
            elif gtype == GGUF_F32:
                nbytes = 4 * n
            else:
                raise ValueError(f"[read_gguf] tensor {name}: GGUF type {gtype} is not supported")
            fh.seek(data0 + offset)
            tensors[name] = (gtype, shape, np.frombuffer(fh.read(nbytes), dtype=np.uint8).copy())
    return meta, tensors


def gguf_repack(blocks: torch.Tensor, gguf_type: int, shape) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Raw block bytes (uint8 CUDA tensor) of a Q4_0 / Q4_1 / Q8_0 tensor of logical `shape`
    [.., K] -> (wq uint32 [.., K*bits/32], scales f16 [.., K/32], biases f16 [.., K/32])."""
    if gguf_type not in _GGUF_BLOCK:
        raise ValueError(f"[gguf_repack] GGUF type {gguf_type} is not a supported quantized type")
    if not blocks.is_cuda:
        raise RuntimeError("[gguf_repack] the repack runs on the GPU: pass a CUDA tensor (no CPU fallback)")
    shape = tuple(shape)
    n_blocks = int(np.prod(shape)) // 32
    bits = 8 if gguf_type == GGUF_Q8_0 else 4
    blocks = blocks.contiguous()
    if blocks.numel() != n_blocks * _GGUF_BLOCK[gguf_type]:
        raise ValueError("[gguf_repack] block data does not match the tensor shape")
    dev = blocks.device
    with torch.cuda.device(dev):
        wq = torch.empty(shape[:-1] + (shape[-1] * bits // 32,), dtype=torch.int32, device=dev)
        s = torch.empty(shape[:-1] + (shape[-1] // 32,), dtype=torch.float16, device=dev)
        b = torch.empty_like(s)
        st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        _lib.check(_lib.load().b200q_gguf_repack(vp(blocks), gguf_type, n_blocks, vp(wq), vp(s), vp(b), st))
    return wq.view(torch.uint32), s, b


def load_gguf(path: str, device="cuda") -> Dict[str, torch.Tensor]:
    """Tensors of a GGUF file on `device`; quantized `<name>.weight` tensors come back as the
    triple `<name>.weight` (packed), `<name>.scales`, `<name>.biases` (group size 32), like the
    reference's loader (mlx/io/gguf_quants.cpp:104-164)."""
    _, raw = read_gguf_raw(path)
    out = {}
    for name, (gtype, shape, data) in raw.items():
        if gtype in _GGUF_BLOCK:
            wq, s, b = gguf_repack(torch.from_numpy(data).to(device), gtype, shape)
            prefix = name[: -len(".weight")] if name.endswith(".weight") else name
            for key in (prefix + ".scales", prefix + ".biases"):
                if key in out:
                    raise RuntimeError(f"[load_gguf] Duplicate parameter name {key}")
            out[name], out[prefix + ".scales"], out[prefix + ".biases"] = wq, s, b
        else:
            npdt = {GGUF_F32: np.float32, GGUF_F16: np.float16, GGUF_BF16: np.uint16}[gtype]
            t = torch.from_numpy(data.view(npdt).reshape(shape).copy())
            out[name] = (t.view(torch.bfloat16) if gtype == GGUF_BF16 else t).to(device)
    return out
