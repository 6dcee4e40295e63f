"""Seeded synthetic Q4_K weights and activations with the shapes and value distributions of
the benchmark configurations: 4-bit quants uniform in [0,15], 6-bit scales/mins uniform in
[0,63], fp16 d and dmin = |N(0,1)| * 2e-3.  Host (numpy) generators give bit-reproducible
test inputs; the device generator fills large benchmark matrices directly in split tiles."""
from __future__ import annotations

import numpy as np


def pad_n(n: int) -> int:
    return (n + 7) // 8 * 8


def pad_k(k: int) -> int:
    return (k + 255) // 256 * 256


def pack_scale_min(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """[..., 8] 6-bit scales and mins -> [..., 12] packed bytes (the layout decoded by
    get_scale_min_k4, third_party/llama.cpp-q4k/reference.hpp:174-181)."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    p = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    p[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    p[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    p[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return p


def logical_q4k(n: int, k: int, seed: int = 0):
    """Logical matrix: codes uint8 [n, k] in 0..15 and metadata uint8 [n, ceil256(k)/256, 16]
    (fp16 d, fp16 dmin, 12 packed bytes).  Columns >= k do not exist; k need not be a
    multiple of 256."""
    rng = np.random.default_rng(seed)
    tiles_k = pad_k(k) // 256
    codes = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    sc = rng.integers(0, 64, size=(n, tiles_k, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(n, tiles_k, 8), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, tiles_k))) * 2e-3).astype(np.float16)
    dmin = (np.abs(rng.standard_normal((n, tiles_k))) * 2e-3).astype(np.float16)
    meta = np.zeros((n, tiles_k, 16), dtype=np.uint8)
    meta[..., 0:2] = d.view(np.uint8).reshape(n, tiles_k, 2)
    meta[..., 2:4] = dmin.view(np.uint8).reshape(n, tiles_k, 2)
    meta[..., 4:16] = pack_scale_min(sc, mn)
    return codes, meta


def split_tiles(codes: np.ndarray, meta: np.ndarray):
    """Logical -> split-tile bytes (src/format/pack.cpp:175-222): codes
    [padded_n/8][tiles_k][8][128], metadata [padded_n/8][tiles_k][8][16], zero padded."""
    n, k = codes.shape
    pn, pk = pad_n(n), pad_k(k)
    tiles_k = pk // 256
    full = np.zeros((pn, pk), dtype=np.uint8)
    full[:n, :k] = codes
    packed = (full[:, 0::2] | (full[:, 1::2] << 4)).reshape(pn // 8, 8, tiles_k, 128)
    out_codes = np.ascontiguousarray(packed.transpose(0, 2, 1, 3)).reshape(-1)
    m = np.zeros((pn, tiles_k, 16), dtype=np.uint8)
    m[:n] = meta
    out_meta = np.ascontiguousarray(m.reshape(pn // 8, 8, tiles_k, 16).transpose(0, 2, 1, 3)).reshape(-1)
    return out_codes, out_meta


def blocks144(codes: np.ndarray, meta: np.ndarray) -> np.ndarray:
    """Logical (k % 256 == 0) -> 144-byte llama.cpp-native super-blocks [n][k/256][144]:
    element 64c+l in the low nibble of qs[32c+l], element 64c+32+l in its high nibble."""
    n, k = codes.shape
    assert k % 256 == 0
    c = codes.reshape(n, k // 256, 4, 2, 32)
    qs = (c[:, :, :, 0, :] | (c[:, :, :, 1, :] << 4)).reshape(n, k // 256, 128)
    out = np.empty((n, k // 256, 144), dtype=np.uint8)
    out[..., :16] = meta
    out[..., 16:] = qs
    return out


def activations(m: int, k: int, seed: int = 0, scale: float = 1.0, outlier_frac: float = 0.0,
                outlier_gain: float = 20.0) -> np.ndarray:
    """fp32 N(0,1)*scale rows; a fixed seeded set of channels is multiplied by outlier_gain."""
    rng = np.random.default_rng(seed + 1000003)
    x = (rng.standard_normal((m, k)) * scale).astype(np.float32)
    if outlier_frac > 0:
        ch = rng.choice(k, size=max(1, int(round(k * outlier_frac))), replace=False)
        x[:, ch] *= outlier_gain
    return x


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def device_weight(n: int, k: int, seed: int = 0, device="cuda"):
    """Random Q4_K matrix written straight into split tiles on the device (k % 256 == 0,
    n % 8 == 0).  Uniform random bytes are uniform nibbles and uniform 6-bit fields, so the
    distribution equals logical_q4k's; only d/dmin need shaping.  Returns PrefillWeight."""
    import torch
    from .q4k_q8 import PrefillWeight
    assert k % 256 == 0 and n % 8 == 0
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    codes = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device=device, generator=g)
    rows = n * (k // 256)
    meta = torch.randint(0, 256, (rows, 16), dtype=torch.uint8, device=device, generator=g)
    dd = (torch.randn((rows, 2), device=device, generator=g).abs() * 2e-3).to(torch.float16)
    meta[:, 0:4] = dd.view(torch.uint8).reshape(rows, 4)
    return PrefillWeight(codes, meta.reshape(-1), n, k)
