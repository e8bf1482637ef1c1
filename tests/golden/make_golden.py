"""Generates tests/golden/golden.npz: small seeded inputs for every step of the path together with
the outputs of the CPU oracle (oracle/ws_oracle.c, the restatement of weightstream-ref's arithmetic).

The reference is Rust and cannot be built or imported where this runs, so these vectors are NOT
outputs of the reference itself; what ties the oracle to the reference are the known-answer values
of the reference's own unit tests (tests/test_oracle_kat.py).  The fixture freezes the oracle: a
change of its arithmetic fails tests/test_golden.py on CPU, and the CUDA path is compared with the
same file on the GPU.

    python tests/golden/make_golden.py        # rewrites golden.npz (a few tens of KB)
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from weightstream_b200 import formats as F, synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")


def build() -> dict:
    rng = np.random.default_rng(20240611)
    g = {}
    # activation quantiser (crates/weightstream-ref/src/actquant.rs:21-57), with its edge cases
    x = (rng.standard_normal((3, 256)) * np.exp(rng.uniform(-8, 8, (3, 256)))).astype(np.float32)
    x[0, :32] = 0.0
    x[0, 32:36] = [100.0, -100.0, 3.0, 0.001]
    x[1, :4] = [448.0, -448.0, 464.0, 1e-4]
    q, e = zip(*(O.fp8_act_emit(x[r]) for r in range(3)))
    g["act_x"], g["act_q"], g["act_e"] = x, np.stack(q), np.stack(e)
    # FP8 block-scaled product (actquant.rs:114-138), both scale formats
    for tag, scale, bn, bk in (("f32", "f32", 128, 128), ("ue8m0", "ue8m0", 32, 32)):
        w, sc = synth.fp8_weight(rng, 64, 256, scale=scale, bn=bn, bk=bk)
        xb = synth.activations_bf16(rng, 3, 256)
        g[f"fp8_{tag}_w"], g[f"fp8_{tag}_s"], g[f"fp8_{tag}_x"] = w, sc, xb
        g[f"fp8_{tag}_y"] = O.fp8_gemv(w, sc, F.bf16_bits_to_f32(xb), bn=bn, bk=bk)
    # K-sharded over two ranks and folded in rank order (crates/weightstream-transport/src/ring.rs:399-408)
    w, sc, xb = g["fp8_f32_w"], g["fp8_f32_s"], g["fp8_f32_x"]
    xf = F.bf16_bits_to_f32(xb)
    parts = np.stack([O.fp8_gemv(w[:, a:a + 128], sc, xf[:, a:a + 128], bn=128, bk=128, k0=a) for a in (0, 128)])
    g["fp8_tp2_parts"], g["fp8_tp2_y"] = parts, O.allreduce_fold(parts)
    # MoE down + combine (crates/weightstream-ref/src/moe.rs:75-84, :150)
    w2, s2 = synth.fp4_experts(rng, 4, 32, 256)
    ids, rw = synth.routes(rng, 3, 4, 2)
    hb = F.f32_to_bf16_bits(rng.standard_normal((6, 256)).astype(np.float32))
    g["moe_w2"], g["moe_s2"], g["moe_ids"], g["moe_rw"], g["moe_h"] = w2, s2, ids, rw, hb
    g["moe_y"] = O.moe_down_combine(w2, s2, 0, F.bf16_bits_to_f32(hb), ids, rw)
    # argmax, first maximum wins (crates/weightstream-ref/src/sample.rs:13-23)
    lg = g["fp8_f32_y"].copy()
    lg[1, 5] = lg[1, 40] = lg[1].max() + 1.0
    g["argmax_logits"] = lg
    g["argmax_idx"] = np.array([O.argmax(lg[t]) for t in range(3)], dtype=np.uint32)
    return g


if __name__ == "__main__":
    np.savez_compressed(OUT, **build())
    print(OUT, os.path.getsize(OUT), "bytes")
