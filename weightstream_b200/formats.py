"""Host-side number formats of the tensor-parallel reduction path (numpy).

Vectorised encoders/decoders for the byte formats the CUDA kernels consume:
FP8 E4M3 (finite-only), FP4 E2M1 packed two per byte, UE8M0 scale bytes and
bf16.  They follow crates/weightstream-core/src/quant.rs of the reference
(f32_to_e4m3 :106-137, f32_to_e2m1 :141-163, f32_to_bf16 :97-101, log2_ceil
:63-73) and its synthetic-weight encoders (crates/weightstream-ref/src/store.rs
:359-419).  They are used to prepare inputs (weights are quantised once, before
sharding) and never sit on the device path.
"""
from __future__ import annotations

import numpy as np

FP4_TABLE = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                      0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def _e4m3_table() -> np.ndarray:
    t = np.empty(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e, m = (b >> 3) & 0xF, b & 7
        if e == 0xF and m == 7:
            t[b] = np.nan
        elif e == 0:
            t[b] = sign * m / 512.0
        else:
            t[b] = sign * 2.0 ** (e - 7) * (1.0 + m / 8.0)
    return t


E4M3_TABLE = _e4m3_table()


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


def e8m0_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    out = np.ldexp(np.float32(1.0), b.astype(np.int32) - 127).astype(np.float32)
    return np.where(b == 0xFF, np.float32(np.nan), out)


def log2_ceil(x: np.ndarray) -> np.ndarray:
    """ceil(log2 x) for positive normal f32, from the exponent field."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    e = ((bits >> 23) & 0xFF).astype(np.int32) - 127
    return e + ((bits & 0x7FFFFF) != 0).astype(np.int32)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rnd = ((bits >> 16) & 1) + 0x7FFF
    return ((bits + rnd) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3(v: np.ndarray) -> np.ndarray:
    """Round to nearest even onto the E4M3 grid, saturating at +-448."""
    v = np.ascontiguousarray(v, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    a = np.abs(v)
    with np.errstate(invalid="ignore", over="ignore"):
        # subnormal region: grid step 1/512
        msub = np.rint(a * np.float32(512.0)).astype(np.int32)
        sub_code = np.where(msub >= 8, 0x08, msub).astype(np.uint8)
        e = ((bits >> 23) & 0xFF).astype(np.int32) - 127
        q = np.ldexp(a, 3 - e).astype(np.float32)
        m8 = np.rint(q).astype(np.int32)
        carry = m8 == 16
        ef = np.where(carry, e + 8, e + 7)
        mant = np.where(carry, 0, m8 - 8)
        norm_code = ((ef << 3) | mant).astype(np.uint8)
    code = np.where(a < np.float32(2.0 ** -6), sub_code, norm_code)
    code = np.where(a >= np.float32(448.0), np.uint8(0x7E), code)
    code = np.where(np.isnan(v), np.uint8(0x7F), code)
    return (sign | code).astype(np.uint8)


def f32_to_e2m1(v: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(v, dtype=np.float32)
    sign = ((v.view(np.uint32) >> 31) << 3).astype(np.uint8)
    a = np.abs(v)
    code = np.full(v.shape, 7, dtype=np.uint8)
    # descending thresholds; the <= / < pattern is ties-to-even on the grid
    code = np.where(a <= 5.0, 6, code)
    code = np.where(a < 3.5, 5, code)
    code = np.where(a <= 2.5, 4, code)
    code = np.where(a < 1.75, 3, code)
    code = np.where(a <= 1.25, 2, code)
    code = np.where(a < 0.75, 1, code)
    code = np.where(a <= 0.25, 0, code)
    return (sign | code.astype(np.uint8)).astype(np.uint8)


def quantize_fp8_blocks(vals: np.ndarray, bn: int = 128, bk: int = 128, scale: str = "f32"):
    """Block-quantise a [rows, cols] fp32 matrix to E4M3 bytes + block scales.

    scale="f32":   one fp32 per (bn x bk) block, scale = amax/448.
    scale="ue8m0": one exponent byte per block, scale = 2^ceil(log2(amax/448)).
    amax is floored at 1e-4 in both.  Returns (w uint8 [rows, cols], scales).
    """
    v = np.ascontiguousarray(vals, dtype=np.float32)
    rows, cols = v.shape
    sr, sc = -(-rows // bn), -(-cols // bk)
    pad = np.zeros((sr * bn, sc * bk), dtype=np.float32)
    pad[:rows, :cols] = np.abs(v)
    amax = pad.reshape(sr, bn, sc, bk).max(axis=(1, 3))
    amax = np.maximum(amax, np.float32(1e-4)).astype(np.float32)
    ratio = (amax / np.float32(448.0)).astype(np.float32)
    if scale == "ue8m0":
        e = log2_ceil(ratio)
        s_val = np.ldexp(np.float32(1.0), e).astype(np.float32)
        s_out = (e + 127).astype(np.uint8)
    elif scale == "f32":
        s_val = ratio
        s_out = ratio
    else:
        raise ValueError(f"unknown scale kind {scale!r}")
    s_full = np.repeat(np.repeat(s_val, bn, axis=0), bk, axis=1)[:rows, :cols]
    q = np.clip((v / s_full).astype(np.float32), -448.0, 448.0)
    return f32_to_e4m3(q), s_out


def quantize_fp4_rows(vals: np.ndarray):
    """MXFP4: E2M1 nibbles (low nibble = even K) + one UE8M0 byte per row per 32 K."""
    v = np.ascontiguousarray(vals, dtype=np.float32)
    rows, cols = v.shape
    assert cols % 32 == 0
    blk = v.reshape(rows, cols // 32, 32)
    amax = np.maximum(np.abs(blk).max(axis=2), np.float32(6.0 * 2.0 ** -126)).astype(np.float32)
    e = log2_ceil((amax / np.float32(6.0)).astype(np.float32))
    s = np.ldexp(np.float32(1.0), e).astype(np.float32)
    q = np.clip((blk / s[:, :, None]).astype(np.float32), -6.0, 6.0)
    codes = f32_to_e2m1(q).reshape(rows, cols)
    packed = (codes[:, 0::2] & 0x0F) | (codes[:, 1::2] << 4)
    return packed.astype(np.uint8), (e + 127).astype(np.uint8)


def dequant_fp8(w: np.ndarray, scales: np.ndarray, bn: int, bk: int) -> np.ndarray:
    rows, cols = w.shape
    s = e8m0_to_f32(scales) if scales.dtype == np.uint8 else scales.astype(np.float32)
    s_full = np.repeat(np.repeat(s, bn, axis=0), bk, axis=1)[:rows, :cols]
    return e4m3_to_f32(w) * s_full


def dequant_fp4(w: np.ndarray, scales: np.ndarray) -> np.ndarray:
    rows, half = w.shape
    out = np.empty((rows, half * 2), dtype=np.float32)
    out[:, 0::2] = FP4_TABLE[w & 0x0F]
    out[:, 1::2] = FP4_TABLE[w >> 4]
    return out * np.repeat(e8m0_to_f32(scales), 32, axis=1)
