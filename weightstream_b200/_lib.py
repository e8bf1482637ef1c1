"""ctypes binding of ``libws_tp.so`` (the C ABI in ``include/ws_tp.h``).

There is no fallback: if the CUDA library is missing and cannot be built, or a
call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

WS_MAX_WORLD = 8
WS_IPC_HANDLE_BYTES = 128
WS_OK = 0
WS_ERR_INVALID, WS_ERR_CUDA, WS_ERR_TIMEOUT, WS_ERR_SEQUENCE, WS_ERR_CAPACITY, WS_ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6
WS_SCALE_UE8M0, WS_SCALE_F32 = 0, 1
WS_ACT_BF16, WS_ACT_F32 = 0, 1

STATUS_NAMES = {0: "WS_OK", -1: "WS_ERR_INVALID", -2: "WS_ERR_CUDA", -3: "WS_ERR_TIMEOUT",
                -4: "WS_ERR_SEQUENCE", -5: "WS_ERR_CAPACITY", -6: "WS_ERR_UNSUPPORTED"}

# every symbol include/ws_tp.h declares
EXPORTS = [
    "ws_tp_create", "ws_tp_destroy", "ws_tp_export_handle", "ws_tp_connect_ipc", "ws_tp_connect_local",
    "ws_tp_connect_tcp", "ws_tcp_allgather",
    "ws_tp_check", "ws_tp_last_error", "ws_tp_stats", "ws_tp_num_ctas",
    "ws_fp8_rowpar_gemm_allreduce", "ws_fp8_rowpar_gemm_allreduce_group",
    "ws_moe_down_combine_allreduce", "ws_moe_down_combine_allreduce_group",
    "ws_lm_head_allgather_argmax", "ws_lm_head_allgather_argmax_group",
    "ws_allreduce_f32", "ws_allgather_f32", "ws_allreduce_f32_group", "ws_allgather_f32_group",
    "ws_allreduce_f32_host", "ws_allgather_f32_host", "ws_fp8_rowpar_gemm_allreduce_host",
    "ws_act_quant_fp8", "ws_tp_set_split", "ws_tp_set_kernel", "ws_fp8_gemm_static_scratch", "ws_fp8_gemm_static_scratch_check", "ws_version",
]


class WsError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class TpConfig(C.Structure):
    _fields_ = [("max_m", C.c_int32), ("max_n", C.c_int32), ("max_vocab", C.c_int32),
                ("wait_ms", C.c_int32), ("num_ctas", C.c_int32), ("reserved", C.c_int32 * 3)]


class IpcHandle(C.Structure):
    _fields_ = [("bytes", C.c_uint8 * WS_IPC_HANDLE_BYTES)]


class Fp8GemmArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int64), ("x_dtype", C.c_int32),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("w", C.c_void_p), ("ldw", C.c_int64),
                ("scales", C.c_void_p), ("scale_ld", C.c_int64),
                ("scale_kind", C.c_int32), ("block_n", C.c_int32), ("block_k", C.c_int32),
                ("row0", C.c_int64), ("k0", C.c_int64), ("out", C.c_void_p)]


class MoeDownArgs(C.Structure):
    _fields_ = [("h", C.c_void_p), ("ldh", C.c_int64), ("h_dtype", C.c_int32),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("top_k", C.c_int32),
                ("route_ids", C.c_void_p), ("route_w", C.c_void_p),
                ("w2", C.c_void_p), ("s2", C.c_void_p),
                ("e_start", C.c_int32), ("e_len", C.c_int32), ("out", C.c_void_p)]


class LmHeadArgs(C.Structure):
    _fields_ = [("g", Fp8GemmArgs), ("vocab_row0", C.c_int64), ("vocab", C.c_int32),
                ("reserved", C.c_int32), ("logits", C.c_void_p), ("argmax", C.c_void_p)]


_lib = None


def lib_path() -> str:
    return _build.LIB


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the CUDA library, building it in-tree first when it is absent or stale."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if build_if_missing and (not os.path.exists(path) or _build.is_stale()):
        try:
            _build.build()
        except Exception as exc:  # a prebuilt, newer-than-source library is still usable
            if not os.path.exists(path):
                raise RuntimeError(f"libws_tp.so is missing and could not be built: {exc}") from exc
    if not os.path.exists(path):
        raise RuntimeError("libws_tp.so is missing: run `python -m weightstream_b200.build`")
    L = C.CDLL(path)
    P = C.c_void_p
    st = C.c_int32
    L.ws_version.restype = C.c_char_p
    L.ws_version.argtypes = []
    L.ws_tp_create.restype = st
    L.ws_tp_create.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.POINTER(TpConfig), C.POINTER(P)]
    L.ws_tp_destroy.restype = st
    L.ws_tp_destroy.argtypes = [P]
    L.ws_tp_export_handle.restype = st
    L.ws_tp_export_handle.argtypes = [P, C.POINTER(IpcHandle)]
    L.ws_tp_connect_ipc.restype = st
    L.ws_tp_connect_ipc.argtypes = [P, C.POINTER(IpcHandle), C.c_int32]
    L.ws_tp_connect_tcp.restype = st
    L.ws_tp_connect_tcp.argtypes = [P, C.c_int32, C.c_int32, C.c_char_p, C.c_int32, C.c_int32]
    L.ws_tcp_allgather.restype = st
    L.ws_tcp_allgather.argtypes = [C.c_int32, C.c_int32, C.c_char_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]
    L.ws_tp_connect_local.restype = st
    L.ws_tp_connect_local.argtypes = [C.POINTER(P), C.c_int32]
    L.ws_tp_check.restype = st
    L.ws_tp_check.argtypes = [P, P]
    L.ws_tp_last_error.restype = C.c_char_p
    L.ws_tp_last_error.argtypes = [P]
    L.ws_tp_stats.restype = st
    L.ws_tp_stats.argtypes = [P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.ws_tp_num_ctas.restype = C.c_int32
    L.ws_tp_num_ctas.argtypes = [P]
    L.ws_tp_set_split.restype = st
    L.ws_tp_set_split.argtypes = [P, C.c_int32]
    L.ws_fp8_rowpar_gemm_allreduce.restype = st
    L.ws_fp8_rowpar_gemm_allreduce.argtypes = [P, C.POINTER(Fp8GemmArgs), P]
    L.ws_fp8_rowpar_gemm_allreduce_group.restype = st
    L.ws_fp8_rowpar_gemm_allreduce_group.argtypes = [C.POINTER(P), C.c_int32, C.POINTER(Fp8GemmArgs), C.POINTER(P)]
    L.ws_moe_down_combine_allreduce.restype = st
    L.ws_moe_down_combine_allreduce.argtypes = [P, C.POINTER(MoeDownArgs), P]
    L.ws_moe_down_combine_allreduce_group.restype = st
    L.ws_moe_down_combine_allreduce_group.argtypes = [C.POINTER(P), C.c_int32, C.POINTER(MoeDownArgs), C.POINTER(P)]
    L.ws_lm_head_allgather_argmax.restype = st
    L.ws_lm_head_allgather_argmax.argtypes = [P, C.POINTER(LmHeadArgs), P]
    L.ws_lm_head_allgather_argmax_group.restype = st
    L.ws_lm_head_allgather_argmax_group.argtypes = [C.POINTER(P), C.c_int32, C.POINTER(LmHeadArgs), C.POINTER(P)]
    L.ws_allreduce_f32.restype = st
    L.ws_allreduce_f32.argtypes = [P, P, P, C.c_int64, P]
    L.ws_allgather_f32.restype = st
    L.ws_allgather_f32.argtypes = [P, P, P, C.c_int64, P]
    L.ws_allreduce_f32_group.restype = st
    L.ws_allreduce_f32_group.argtypes = [C.POINTER(P), C.c_int32, C.POINTER(P), C.POINTER(P), C.c_int64, C.POINTER(P)]
    L.ws_allgather_f32_group.restype = st
    L.ws_allgather_f32_group.argtypes = [C.POINTER(P), C.c_int32, C.POINTER(P), C.POINTER(P), C.c_int64, C.POINTER(P)]
    L.ws_allreduce_f32_host.restype = st
    L.ws_allreduce_f32_host.argtypes = [P, P, P, C.c_int64]
    L.ws_allgather_f32_host.restype = st
    L.ws_allgather_f32_host.argtypes = [P, P, P, C.c_int64]
    L.ws_fp8_rowpar_gemm_allreduce_host.restype = st
    L.ws_fp8_rowpar_gemm_allreduce_host.argtypes = [P, C.POINTER(Fp8GemmArgs), P, P]
    L.ws_act_quant_fp8.restype = st
    L.ws_act_quant_fp8.argtypes = [P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, P, P, P]
    L.ws_tp_set_kernel.restype = st
    L.ws_tp_set_kernel.argtypes = [P, C.c_int32]
    L.ws_fp8_gemm_static_scratch.restype = st
    L.ws_fp8_gemm_static_scratch.argtypes = [C.POINTER(Fp8GemmArgs), C.c_int32, P, C.c_char_p, C.c_size_t]
    L.ws_fp8_gemm_static_scratch_check.restype = st
    L.ws_fp8_gemm_static_scratch_check.argtypes = [C.c_int32, P, C.c_char_p, C.c_size_t]
    _lib = L
    return L
