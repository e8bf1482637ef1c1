"""Seeded synthetic inputs with the shapes and value distributions of the measured
configurations (no checkpoint exists offline, so nothing here stands in for real
weights):

* attention output projection: x ~ N(0,1) as bf16, W ~ N(0, 0.02) quantised to FP8
  E4M3 with one scale per 128x128 block (scale = amax/448), or per 32x32 block with
  UE8M0 scales (the reference's native layout);
* MoE: router logits ~ N(0,1), softmax, top-k by (value desc, index asc), weights
  renormalised and scaled by 1.5 (crates/weightstream-ref/src/moe.rs:48-69); expert
  weights ~ N(0, 0.02) as MXFP4 (E2M1 + UE8M0 per 32);
* lm_head: as the projection, [vocab, dim].

numpy versions serve the parity tests (same bytes go to the oracle and to the GPU);
the torch versions quantise on the device for tensors too large to build on the host.
"""
from __future__ import annotations

import zlib
from typing import Tuple

import numpy as np

from . import formats as F


def config_seed(name: str, m: int, world: int) -> int:
    return zlib.crc32(f"{name}|m={m}|r={world}".encode()) & 0x7FFFFFFF


def activations_bf16(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    """N(0,1) rounded to bf16; returned as uint16 bit patterns."""
    return F.f32_to_bf16_bits(rng.standard_normal((m, k)).astype(np.float32))


def fp8_weight(rng: np.random.Generator, n: int, k: int, *, scale: str = "f32", bn: int = 128, bk: int = 128,
               std: float = 0.02):
    vals = (rng.standard_normal((n, k)) * std).astype(np.float32)
    return F.quantize_fp8_blocks(vals, bn, bk, scale)


def fp4_experts(rng: np.random.Generator, e: int, n: int, k: int, std: float = 0.02):
    ws, ss = [], []
    for _ in range(e):
        w, s = F.quantize_fp4_rows((rng.standard_normal((n, k)) * std).astype(np.float32))
        ws.append(w)
        ss.append(s)
    return np.stack(ws), np.stack(ss)


def routes(rng: np.random.Generator, m: int, n_experts: int, top_k: int, *, uniform: bool = False,
           route_scale: float = 1.5) -> Tuple[np.ndarray, np.ndarray]:
    """Top-k routing as the reference's gate does it (moe.rs:48-69): softmax scores, order by
    (score desc, index asc), weights = selected / (sum + 1e-20) * route_scale."""
    logits = (rng.uniform(0, 1, (m, n_experts)) if uniform else rng.standard_normal((m, n_experts))).astype(np.float32)
    z = logits - logits.max(axis=1, keepdims=True)
    p = np.exp(z).astype(np.float32)
    p = (p / p.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    order = np.lexsort((np.arange(n_experts)[None, :].repeat(m, 0), -p), axis=1)[:, :top_k]
    w = np.take_along_axis(p, order, axis=1)
    w = (w / (w.sum(axis=1, keepdims=True, dtype=np.float32) + np.float32(1e-20))).astype(np.float32)
    w = (w * np.float32(route_scale)).astype(np.float32)
    return order.astype(np.int32), w


# ----------------------------------------------------------------------------- device-side (torch)
def torch_fp8_weight(n: int, k: int, *, seed: int, device, bn: int = 128, bk: int = 128, std: float = 0.02,
                     rows_per_chunk: int = 8192):
    """W ~ N(0, std) quantised on the device to E4M3 bytes + fp32 (bn x bk) block scales.
    torch's float8_e4m3fn cast rounds to nearest even like the reference encoder; values
    are pre-clamped to +-448, so its NaN-on-overflow rule never triggers."""
    import torch
    assert rows_per_chunk % bn == 0 and k % bk == 0
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.empty((n, k), dtype=torch.uint8, device=device)
    scales = torch.empty((-(-n // bn), k // bk), dtype=torch.float32, device=device)
    for r0 in range(0, n, rows_per_chunk):
        r1 = min(n, r0 + rows_per_chunk)
        v = torch.randn((r1 - r0, k), generator=g, device=device, dtype=torch.float32) * std
        pad = (-(r1 - r0)) % bn
        vp = torch.nn.functional.pad(v.abs(), (0, 0, 0, pad)) if pad else v.abs()
        amax = vp.reshape(-1, bn, k // bk, bk).amax(dim=(1, 3)).clamp_min(1e-4)
        s = amax / 448.0
        scales[r0 // bn:r0 // bn + s.shape[0]] = s
        sf = s.repeat_interleave(bn, 0)[: r1 - r0].repeat_interleave(bk, 1)
        q = (v / sf).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        w[r0:r1] = q.view(torch.uint8)
    return w, scales


def torch_fp4_experts(e: int, n: int, k: int, *, seed: int, device, std: float = 0.02):
    """e experts of MXFP4 [n, k]: packed E2M1 (low nibble = even K) + UE8M0 per row per 32."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w2 = torch.empty((e, n, k // 2), dtype=torch.uint8, device=device)
    s2 = torch.empty((e, n, k // 32), dtype=torch.uint8, device=device)
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=device)
    right = torch.tensor([False, True, False, True, False, True, False], device=device)  # tie goes up?
    for i in range(e):
        v = torch.randn((n, k // 32, 32), generator=g, device=device, dtype=torch.float32) * std
        amax = v.abs().amax(dim=2).clamp_min(6.0 * 2.0 ** -126)
        ratio = amax / 6.0
        bits = ratio.view(torch.int32)
        ex = ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)
        s = torch.ldexp(torch.ones_like(ratio), ex)
        a = (v / s[:, :, None]).clamp(-6.0, 6.0)
        mag = a.abs()
        # thresholds with ties-to-even: <=0.25->0, <0.75->1, <=1.25->2, <1.75->3, <=2.5->4, <3.5->5, <=5->6
        code = torch.zeros_like(mag, dtype=torch.uint8)
        for t, incl_upper in zip(bounds.tolist(), right.tolist()):
            code += (mag >= t).to(torch.uint8) if incl_upper else (mag > t).to(torch.uint8)
        code = code | ((a.view(torch.int32) >> 31) & 1).to(torch.uint8) << 3
        code = code.reshape(n, k)
        w2[i] = (code[:, 0::2] & 0xF) | (code[:, 1::2] << 4)
        s2[i] = (ex + 127).to(torch.uint8)
    return w2, s2
