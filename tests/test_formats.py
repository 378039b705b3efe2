"""Weight formats: safetensors triples and GGUF blocks.  CPU part: file parsing and the repack
checker against hand-derived blocks and the format definition.  GPU part: the device repack
against the checker, bit for bit, and a matmul through a loaded GGUF tensor."""
import os
import struct
import sys

import numpy as np
import pytest
import torch

import oracle as O
from mlx_b200 import formats


def _blocks(gtype, n, seed=0):
    rng = np.random.default_rng(seed)
    size = formats._GGUF_BLOCK[gtype]
    b = rng.integers(0, 256, size=(n, size), dtype=np.uint8)
    d = (rng.standard_normal(n) * 0.01).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n, 2)
    if gtype == formats.GGUF_Q4_1:
        m = (rng.standard_normal(n) * 0.1).astype(np.float16)
        b[:, 2:4] = m.view(np.uint8).reshape(n, 2)
    return b


def _definition(blocks, gtype):
    """Weights by the GGUF definition, float32: d*(q-8), d*q+m, d*q."""
    n = blocks.shape[0]
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(n, 1)
    if gtype == formats.GGUF_Q8_0:
        return d * blocks[:, 2:].view(np.int8).astype(np.float32)
    q = blocks[:, (2 if gtype == formats.GGUF_Q4_0 else 4):]
    nib = np.concatenate([q & 15, q >> 4], axis=1).astype(np.float32)   # weights 0..15, 16..31
    if gtype == formats.GGUF_Q4_0:
        return d * (nib - 8.0)
    m = blocks[:, 2:4].copy().view(np.float16).astype(np.float32).reshape(n, 1)
    return d * nib + m


@pytest.mark.parametrize("gtype", (formats.GGUF_Q4_0, formats.GGUF_Q4_1, formats.GGUF_Q8_0))
def test_repack_checker_matches_the_format_definition(gtype):
    blocks = _blocks(gtype, 257, seed=gtype)
    wq, s, b = O.gguf_repack(blocks, gtype)
    bits = 8 if gtype == formats.GGUF_Q8_0 else 4
    sf, bf = s.view(np.float16).astype(np.float32)[:, None], b.view(np.float16).astype(np.float32)[:, None]
    if bits == 4:
        q = np.stack([(wq[:, k // 2] >> (4 * (k % 2))) & 15 for k in range(32)], axis=1).astype(np.float32)
    else:
        q = wq.astype(np.float32)
    want = _definition(blocks, gtype)
    # the affine form q*s + b reproduces the definition up to the float16 rounding of the bias
    assert np.allclose(q * sf + bf, want, rtol=0, atol=np.abs(want).max() * 2e-3 + 1e-6)
    if gtype == formats.GGUF_Q4_0:   # -8 d is exact in float16
        assert np.array_equal(q * sf + bf, want)


GGUF_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "gguf_unpack_golden.npz")


def _q4_blocks_from_quants(quants, gtype):
    n = quants.shape[0]
    head = 2 if gtype == formats.GGUF_Q4_0 else 4
    blocks = np.zeros((n, head + 16), dtype=np.uint8)
    blocks[:, 0:2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    blocks[:, head:] = quants
    return blocks


@pytest.mark.parametrize("gtype", (formats.GGUF_Q4_0, formats.GGUF_Q4_1))
def test_repack_checker_nibble_order_matches_reference_golden(gtype):
    """The packed words of the checker equal what the reference's own unpack_32_4
    (mlx/io/gguf_quants.cpp:13-31) produced for the same quant bytes (vectors made by
    tests/golden/make_golden.py from the reference-compiled binary)."""
    gold = np.load(GGUF_GOLDEN)
    wq, _, _ = O.gguf_repack(_q4_blocks_from_quants(gold["quants"], gtype), gtype)
    assert np.array_equal(wq, gold["unpacked"])


@pytest.mark.skipif(not O.have_reference_gguf(), reason="reference-compiled GGUF binary not present")
def test_repack_checker_nibble_order_matches_reference_live():
    quants = np.random.default_rng(11).integers(0, 256, (1000, 16), dtype=np.uint8)
    wq, _, _ = O.gguf_repack(_q4_blocks_from_quants(quants, formats.GGUF_Q4_0), formats.GGUF_Q4_0)
    assert np.array_equal(wq, O.ref_gguf_unpack(quants))


def test_safetensors_round_trip_and_triples(tmp_path):
    rng = np.random.default_rng(1)
    w = (0.02 * rng.standard_normal((64, 256))).astype(np.float32)
    wq, s, b = O.quantize(O.to_dtype(w, "bf16"), 64, 4, "bf16")
    t = {"layers.0.mlp.up_proj.weight": torch.from_numpy(wq.view(np.int32)).view(torch.uint32),
         "layers.0.mlp.up_proj.scales": torch.from_numpy(s).view(torch.bfloat16),
         "layers.0.mlp.up_proj.biases": torch.from_numpy(b).view(torch.bfloat16),
         "norm.weight": torch.ones(256, dtype=torch.float16)}
    path = str(tmp_path / "m.safetensors")
    formats.write_safetensors(path, t)
    back = formats.read_safetensors(path)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k].view(torch.uint8), t[k].view(torch.uint8)), k
    trip = formats.quantized_triples(back, group_size=64)
    assert list(trip) == ["layers.0.mlp.up_proj"] and trip["layers.0.mlp.up_proj"][3:] == (64, 4)
    with pytest.raises(ValueError):
        formats.quantized_triples(back)     # 32 words, 4 groups: (64, 4) and (128, 2)... need a hint


def _write_gguf(path, tensors):
    """Minimal GGUF v3 writer: {name: (type, shape outermost-first, raw bytes)}."""
    def s(x):
        e = x.encode()
        return struct.pack("<Q", len(e)) + e
    head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", len(tensors), 1)
    head += s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", 32)
    off, infos, blobs = 0, b"", []
    for name, (gt, shape, raw) in tensors.items():
        infos += s(name) + struct.pack("<I", len(shape)) + struct.pack("<" + "Q" * len(shape), *reversed(shape))
        infos += struct.pack("<IQ", gt, off)
        pad = (32 - len(raw) % 32) % 32
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    body = head + infos
    body += b"\0" * ((32 - len(body) % 32) % 32)
    with open(path, "wb") as fh:
        fh.write(body + b"".join(blobs))


def test_gguf_parser(tmp_path):
    blocks = _blocks(formats.GGUF_Q4_0, 8 * 4, seed=5)            # [8, 128]
    f = np.arange(12, dtype=np.float32).reshape(3, 4)
    path = str(tmp_path / "m.gguf")
    _write_gguf(path, {"blk.0.ffn_up.weight": (formats.GGUF_Q4_0, (8, 128), blocks.tobytes()),
                       "output_norm.weight": (formats.GGUF_F32, (3, 4), f.tobytes())})
    meta, raw = formats.read_gguf_raw(path)
    assert meta["general.alignment"] == 32
    gt, shape, data = raw["blk.0.ffn_up.weight"]
    assert (gt, shape) == (formats.GGUF_Q4_0, (8, 128)) and np.array_equal(data.reshape(-1, 18), blocks)
    assert np.array_equal(raw["output_norm.weight"][2].view(np.float32).reshape(3, 4), f)
    with pytest.raises(RuntimeError):
        formats.gguf_repack(torch.from_numpy(data), gt, shape)     # CPU tensor: no CPU repack path


@pytest.mark.gpu
@pytest.mark.parametrize("gtype", (formats.GGUF_Q4_0, formats.GGUF_Q4_1, formats.GGUF_Q8_0))
def test_gguf_repack_on_device_is_bit_exact(gtype):
    rows, K = 37, 4096
    blocks = _blocks(gtype, rows * K // 32, seed=10 + gtype)
    wq, s, b = formats.gguf_repack(torch.from_numpy(blocks).cuda(), gtype, (rows, K))
    rq, rs, rb = O.gguf_repack(blocks, gtype)
    bits = 8 if gtype == formats.GGUF_Q8_0 else 4
    assert tuple(wq.shape) == (rows, K * bits // 32) and tuple(s.shape) == (rows, K // 32)
    assert np.array_equal(wq.view(torch.int32).cpu().numpy().view(np.uint8).reshape(rq.shape), rq)
    assert np.array_equal(s.view(torch.int16).cpu().numpy().view(np.uint16).ravel(), rs)
    assert np.array_equal(b.view(torch.int16).cpu().numpy().view(np.uint16).ravel(), rb)


@pytest.mark.gpu
def test_matmul_through_a_loaded_gguf_tensor(tmp_path):
    import mlx_b200 as mb
    N, K = 256, 512
    blocks = _blocks(formats.GGUF_Q4_0, N * K // 32, seed=3)
    path = str(tmp_path / "w.gguf")
    _write_gguf(path, {"ffn.weight": (formats.GGUF_Q4_0, (N, K), blocks.tobytes())})
    t = formats.load_gguf(path)
    assert set(t) == {"ffn.weight", "ffn.scales", "ffn.biases"}
    x = torch.randn(5, K, device="cuda", dtype=torch.float16)
    y = mb.quantized_matmul(x, t["ffn.weight"], t["ffn.scales"], t["ffn.biases"], group_size=32, bits=4)
    want = x.float().cpu().numpy() @ _definition(blocks, formats.GGUF_Q4_0).reshape(N, K).T
    assert np.allclose(y.float().cpu().numpy(), want, rtol=2e-2, atol=2e-2 * np.abs(want).max())
