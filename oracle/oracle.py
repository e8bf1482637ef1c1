"""ctypes front end of the CPU oracle (``libws_oracle.so``).

TEST INFRASTRUCTURE ONLY: the oracle is the checker for the CUDA library and
must never be reached from the product path.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline / reference arm import this module.

Each wrapper names the reference function it restates; the arithmetic itself is
in ``ws_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libws_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``ws_oracle.c`` with gcc (OpenMP when the runtime is present)."""
    src = os.path.join(_HERE, "ws_oracle.c")
    hdr = os.path.join(_HERE, "ws_oracle.h")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= max(os.path.getmtime(src), os.path.getmtime(hdr))):
        return _LIB_PATH
    base = ["gcc", "-O2", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-std=c11",
            "-shared", "-o", _LIB_PATH, src, "-lm"]
    try:
        subprocess.run(base[:3] + ["-fopenmp"] + base[3:], check=True, capture_output=True)
    except (subprocess.CalledProcessError, FileNotFoundError):
        subprocess.run(base, check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_sz = C.c_size_t
_p = C.c_void_p


def _declare(L: C.CDLL) -> None:
    L.wso_e4m3_to_f32.restype = C.c_float
    L.wso_e4m3_to_f32.argtypes = [C.c_uint8]
    L.wso_e8m0_to_f32.restype = C.c_float
    L.wso_e8m0_to_f32.argtypes = [C.c_uint8]
    L.wso_fp4_to_f32.restype = C.c_float
    L.wso_fp4_to_f32.argtypes = [C.c_uint8]
    L.wso_log2_ceil.restype = C.c_int32
    L.wso_log2_ceil.argtypes = [C.c_float]
    L.wso_pow2i.restype = C.c_float
    L.wso_pow2i.argtypes = [C.c_int32]
    L.wso_ue8m0_round_scale.restype = C.c_float
    L.wso_ue8m0_round_scale.argtypes = [C.c_float, C.c_float]
    L.wso_bf16_to_f32.restype = C.c_float
    L.wso_bf16_to_f32.argtypes = [C.c_uint16]
    L.wso_f32_to_bf16.restype = C.c_uint16
    L.wso_f32_to_bf16.argtypes = [C.c_float]
    L.wso_f32_to_e4m3.restype = C.c_uint8
    L.wso_f32_to_e4m3.argtypes = [C.c_float]
    L.wso_set_e4m3_literal.restype = None
    L.wso_set_e4m3_literal.argtypes = [C.c_int]
    L.wso_get_e4m3_literal.restype = C.c_int
    L.wso_get_e4m3_literal.argtypes = []
    L.wso_f32_to_e2m1.restype = C.c_uint8
    L.wso_f32_to_e2m1.argtypes = [C.c_float]
    L.wso_fp8_snap.restype = None
    L.wso_fp8_snap.argtypes = [_p, _sz, _sz]
    L.wso_fp8_act_emit.restype = None
    L.wso_fp8_act_emit.argtypes = [_p, _sz, _p, _p]
    L.wso_encode_fp8.restype = None
    L.wso_encode_fp8.argtypes = [_p, _sz, _sz, C.c_int, _sz, _sz, _p, _p]
    L.wso_encode_fp4.restype = None
    L.wso_encode_fp4.argtypes = [_p, _sz, _sz, _p, _p]
    L.wso_fp8_gemv.restype = None
    L.wso_fp8_gemv.argtypes = [_p, _sz, _p, C.c_int, _sz, _sz, _sz, _sz, _sz, _sz, _sz,
                               _p, _sz, _sz, _p, _sz, C.c_int]
    L.wso_fp4_gemv.restype = None
    L.wso_fp4_gemv.argtypes = [_p, _p, _sz, _sz, _p, _sz, _sz, _p, _sz, C.c_int]
    L.wso_moe_down_combine.restype = None
    L.wso_moe_down_combine.argtypes = [_p, _p, _sz, _sz, C.c_int32, C.c_int32, _p, _p, _p,
                                       _sz, _sz, _p, C.c_int]
    L.wso_allreduce_fold.restype = None
    L.wso_allreduce_fold.argtypes = [_p, _sz, _sz, _p]
    L.wso_allgather.restype = None
    L.wso_allgather.argtypes = [_p, _sz, _sz, _p]
    L.wso_argmax.restype = C.c_uint32
    L.wso_argmax.argtypes = [_p, _sz]
    L.wso_max_threads.restype = C.c_int
    L.wso_max_threads.argtypes = []


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---- scalar primitives (crates/weightstream-core/src/quant.rs) -------------
def e4m3_to_f32(b: int) -> float:
    return float(lib().wso_e4m3_to_f32(b))


def e8m0_to_f32(b: int) -> float:
    return float(lib().wso_e8m0_to_f32(b))


def fp4_to_f32(nib: int) -> float:
    return float(lib().wso_fp4_to_f32(nib))


def log2_ceil(x: float) -> int:
    return int(lib().wso_log2_ceil(x))


def pow2i(e: int) -> float:
    return float(lib().wso_pow2i(e))


def ue8m0_round_scale(amax: float, fp_max: float) -> float:
    return float(lib().wso_ue8m0_round_scale(amax, fp_max))


def bf16_to_f32(bits: int) -> float:
    return float(lib().wso_bf16_to_f32(bits))


def f32_to_bf16(v: float) -> int:
    return int(lib().wso_f32_to_bf16(v))


def f32_to_e4m3(v: float) -> int:
    return int(lib().wso_f32_to_e4m3(v))


class e4m3_literal:
    """Context manager: inside it the E4M3 encoder returns what
    crates/weightstream-core/src/quant.rs:121 returns as written (the byte of 1.0 for
    |v| in [7.5/512, 8/512)) instead of the byte of 2^-6 that the reference's device
    encoder (crates/weightstream-cuda/kernels/common.cuh:26) and round-to-nearest give."""

    def __enter__(self):
        self.prev = int(lib().wso_get_e4m3_literal())
        lib().wso_set_e4m3_literal(1)
        return self

    def __exit__(self, *exc):
        lib().wso_set_e4m3_literal(self.prev)
        return False


def f32_to_e2m1(v: float) -> int:
    return int(lib().wso_f32_to_e2m1(v))


def max_threads() -> int:
    return int(lib().wso_max_threads())


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """Widen bf16 bit patterns (uint16) to float32 exactly (quant.rs:91)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- activation quantisation (crates/weightstream-ref/src/actquant.rs:21-57)
def fp8_snap(x: np.ndarray, block: int = 32) -> np.ndarray:
    out = _c(x, np.float32).copy()
    lib().wso_fp8_snap(_ptr(out), out.size, block)
    return out


def fp8_act_emit(x: np.ndarray):
    xx = _c(x, np.float32)
    q = np.empty(xx.size, dtype=np.uint8)
    s = np.empty(xx.size // 32, dtype=np.uint8)
    lib().wso_fp8_act_emit(_ptr(xx), xx.size, _ptr(q), _ptr(s))
    return q.reshape(xx.shape), s


# ---- encoders (crates/weightstream-ref/src/store.rs:359-419) ---------------
def encode_fp8(vals: np.ndarray, scale_kind: int, bn: int, bk: int):
    v = _c(vals, np.float32)
    rows, cols = v.shape
    w = np.empty((rows, cols), dtype=np.uint8)
    sshape = (-(-rows // bn), -(-cols // bk))
    s = np.empty(sshape, dtype=np.uint8 if scale_kind == 0 else np.float32)
    lib().wso_encode_fp8(_ptr(v), rows, cols, scale_kind, bn, bk, _ptr(w), _ptr(s))
    return w, s


def encode_fp4(vals: np.ndarray):
    v = _c(vals, np.float32)
    rows, cols = v.shape
    w = np.empty((rows, cols // 2), dtype=np.uint8)
    s = np.empty((rows, -(-cols // 32)), dtype=np.uint8)
    lib().wso_encode_fp4(_ptr(v), rows, cols, _ptr(w), _ptr(s))
    return w, s


# ---- GEMVs (crates/weightstream-ref/src/actquant.rs:114-173) ---------------
def fp8_gemv(w: np.ndarray, scales: np.ndarray, x: np.ndarray, *, bn: int, bk: int,
             row0: int = 0, k0: int = 0, threads: int = 1) -> np.ndarray:
    """y[M, rows] for a weight shard ``w`` (2-D uint8 view, row stride allowed).

    ``scales`` is the FULL tensor's scale matrix (uint8 UE8M0 or float32);
    ``row0``/``k0`` place the shard inside it.  ``x`` is fp32 [M, cols].
    """
    assert w.dtype == np.uint8 and w.ndim == 2 and w.strides[1] == 1
    rows, cols = w.shape
    s = np.ascontiguousarray(scales)
    kind = 0 if s.dtype == np.uint8 else 1
    assert kind == 0 or s.dtype == np.float32
    xx = _c(np.atleast_2d(x), np.float32)
    M = xx.shape[0]
    assert xx.shape[1] == cols
    y = np.empty((M, rows), dtype=np.float32)
    lib().wso_fp8_gemv(_ptr(w), w.strides[0], _ptr(s), kind, bn, bk, s.shape[1], rows, cols,
                       row0, k0, _ptr(xx), cols, M, _ptr(y), rows, threads)
    return y


def fp4_gemv(w: np.ndarray, scales: np.ndarray, x: np.ndarray, threads: int = 1) -> np.ndarray:
    ww = _c(w, np.uint8)
    rows, half = ww.shape
    cols = half * 2
    ss = _c(scales, np.uint8)
    xx = _c(np.atleast_2d(x), np.float32)
    M = xx.shape[0]
    y = np.empty((M, rows), dtype=np.float32)
    lib().wso_fp4_gemv(_ptr(ww), _ptr(ss), rows, cols, _ptr(xx), cols, M, _ptr(y), rows, threads)
    return y


def moe_down_combine(w2: np.ndarray, s2: np.ndarray, e_start: int, h: np.ndarray,
                     route_ids: np.ndarray, route_w: np.ndarray, threads: int = 1) -> np.ndarray:
    """crates/weightstream-ref/src/moe.rs:75-84, :150, :203-207 over a local expert slab.

    w2 [e_len, N, K/2] uint8, s2 [e_len, N, K/32] uint8, h fp32 [M*top_k, K],
    route_ids int32 [M, top_k] (global ids), route_w fp32 [M, top_k].
    """
    ww = _c(w2, np.uint8)
    ss = _c(s2, np.uint8)
    e_len, n, half = ww.shape
    k = half * 2
    ids = _c(route_ids, np.int32)
    rw = _c(route_w, np.float32)
    M, top_k = ids.shape
    hh = _c(h, np.float32).reshape(M * top_k, k)
    y = np.empty((M, n), dtype=np.float32)
    lib().wso_moe_down_combine(_ptr(ww), _ptr(ss), n, k, e_start, e_len, _ptr(hh), _ptr(ids),
                               _ptr(rw), M, top_k, _ptr(y), threads)
    return y


# ---- collectives (crates/weightstream-transport/src/ring.rs:399-408, :426-432)
def allreduce_fold(partials: np.ndarray) -> np.ndarray:
    p = _c(partials, np.float32)
    r = p.shape[0]
    n = p[0].size
    out = np.empty(p.shape[1:], dtype=np.float32)
    lib().wso_allreduce_fold(_ptr(p), r, n, _ptr(out))
    return out


def allgather(contribs: np.ndarray) -> np.ndarray:
    c = _c(contribs, np.float32)
    out = np.empty(c.size, dtype=np.float32)
    lib().wso_allgather(_ptr(c), c.shape[0], c[0].size, _ptr(out))
    return out


# ---- sampling (crates/weightstream-ref/src/sample.rs:13-23) ----------------
def argmax(logits: np.ndarray) -> int:
    l = _c(logits, np.float32)
    return int(lib().wso_argmax(_ptr(l), l.size))
