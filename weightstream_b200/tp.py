"""Host-side mirror of the reference's tensor-parallel seam, on top of the C ABI.

The reference (msuiche/weightstream) exposes the path through two Rust
interfaces inside ``crates/weightstream-gpu/src/engine.rs``: the sharding plan
(``Sharding`` :132-145, ``WShard`` :151-156, ``shard_weight`` / ``shard_scale``
:182-280) and ``trait Collectives`` (:287-294: ``allreduce``, ``allgather``,
``stats``).  This module keeps those names, argument meanings and error
behaviour (fail-stop: any failure raises and the step's results are invalid),
and adds the fused operators that replace GEMM launch + collective pairs.

torch is used only for device memory, streams and process-group plumbing.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import (Fp8GemmArgs, IpcHandle, LmHeadArgs, MoeDownArgs, TpConfig, WsError, WS_ACT_BF16,
                   WS_ACT_F32, WS_OK, WS_SCALE_F32, WS_SCALE_UE8M0)


# ----------------------------------------------------------------------------- sharding plan
@dataclass(frozen=True)
class Sharding:
    """engine.rs:132-145.  TP1 by default."""
    world_size: int = 1
    rank: int = 0

    def slice_of(self, length: int) -> Tuple[int, int]:
        """The reference's contiguous equal slice: start = rank*len/world (engine.rs:1477-1480)."""
        if length % self.world_size:
            raise ValueError(f"length {length} does not divide over {self.world_size} ranks")
        per = length // self.world_size
        return self.rank * per, per


@dataclass(frozen=True)
class WShard:
    """engine.rs:151-156: local slice of a sharded row-major matrix."""
    kind: str = "all"          # "all" | "rows" | "cols"
    start: int = 0
    len: int = 0

    @staticmethod
    def All() -> "WShard":
        return WShard("all")

    @staticmethod
    def Rows(start: int, len: int) -> "WShard":
        return WShard("rows", start, len)

    @staticmethod
    def Cols(start: int, len: int) -> "WShard":
        return WShard("cols", start, len)


def shard_weight(view, shape: Sequence[int], shard: WShard, align: int = 32):
    """engine.rs:195-235: slice a row-major byte matrix; starts and lengths must be
    ``align``-aligned (32 in the reference, the scale-tile edge)."""
    rows, cols = shape
    if shard.kind == "all":
        return view
    count = view.numel() if hasattr(view, "numel") else view.size
    if count != rows * cols:
        raise ValueError(f"weight bytes {count} do not tile [{rows}, {cols}]")
    m = view.reshape(rows, cols)
    if shard.kind == "rows":
        if shard.start % align or shard.len % align or shard.start + shard.len > rows:
            raise ValueError(f"row shard [{shard.start}, {shard.start}+{shard.len}) not {align}-aligned in [{rows}]")
        return m[shard.start:shard.start + shard.len]
    if shard.start % align or shard.len % align or shard.start + shard.len > cols:
        raise ValueError(f"col shard [{shard.start}, {shard.start}+{shard.len}) not {align}-aligned in [{cols}]")
    out = m[:, shard.start:shard.start + shard.len]
    return out.contiguous() if hasattr(out, "contiguous") else np.ascontiguousarray(out)


def shard_scale(view, shape: Sequence[int], shard: WShard, block: Tuple[int, int] = (32, 32)):
    """engine.rs:252-280, generalised over the scale block: returns the covering scale
    tiles and the offset (row0, k0) of the shard's first element inside them.

    With the reference's 32x32 tiles and 32-aligned shards the offset is (0, 0); a vocab
    shard that cuts a 128-row tile (129280/8 rows) gets row0 = start % 128."""
    srows, scols = shape
    bn, bk = block
    m = view.reshape(srows, scols)
    if shard.kind == "all":
        return m, 0, 0
    if shard.kind == "rows":
        s0, s1 = shard.start // bn, -(-(shard.start + shard.len) // bn)
        return m[s0:s1], shard.start - s0 * bn, 0
    c0, c1 = shard.start // bk, -(-(shard.start + shard.len) // bk)
    out = m[:, c0:c1]
    out = out.contiguous() if hasattr(out, "contiguous") else np.ascontiguousarray(out)
    return out, 0, shard.start - c0 * bk


# ----------------------------------------------------------------------------- helpers
def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def _act_dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return WS_ACT_BF16
    if t.dtype == torch.float32:
        return WS_ACT_F32
    raise TypeError(f"activations must be bf16 or fp32, got {t.dtype}")


def _scale_kind(t: torch.Tensor) -> int:
    if t.dtype == torch.uint8:
        return WS_SCALE_UE8M0
    if t.dtype == torch.float32:
        return WS_SCALE_F32
    raise TypeError(f"scales must be uint8 (UE8M0) or fp32, got {t.dtype}")


def _np_ptr(a: np.ndarray) -> int:
    """Address of a numpy array's data; three times cheaper than ``a.ctypes.data`` (0.4 against 1.2 us),
    which matters in a call that takes 35 us end to end."""
    try:
        return C.addressof(C.c_char.from_buffer(a))
    except (TypeError, ValueError):  # read-only or empty buffers
        return a.ctypes.data


def _fp8_args(x, w, scales, block, row0, k0, out) -> Fp8GemmArgs:
    if x.dim() != 2 or w.dim() != 2 or scales.dim() != 2:
        raise ValueError("x, w and scales must be 2-D")
    if w.dtype != torch.uint8 and w.dtype != torch.float8_e4m3fn:
        raise TypeError("w must hold E4M3 bytes (uint8 or float8_e4m3fn)")
    if x.stride(1) != 1 or w.stride(1) != 1 or not scales.is_contiguous():
        raise ValueError("x and w need unit inner stride; scales must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"x has k={k} but w has {w.shape[1]} columns")
    a = Fp8GemmArgs()
    a.x, a.ldx, a.x_dtype = x.data_ptr(), (x.stride(0) if m > 1 else k), _act_dtype(x)
    a.m, a.n, a.k = m, n, k
    a.w, a.ldw = w.data_ptr(), w.stride(0)
    a.scales, a.scale_ld, a.scale_kind = scales.data_ptr(), scales.shape[1], _scale_kind(scales)
    a.block_n, a.block_k = block
    a.row0, a.k0 = row0, k0
    a.out = out.data_ptr() if out is not None else None
    return a


class Endpoint:
    """One rank's endpoint (``ws_tp_t``).  Replaces ``tp4::join`` + ``Ring::new``
    (crates/weightstream-gpu/src/tp4.rs:191-312)."""

    def __init__(self, sharding: Sharding = Sharding(), device: Optional[int] = None, *, max_m: int = 64,
                 max_n: int = 7168, max_vocab: int = 0, wait_ms: int = 2000, num_ctas: int = 0):
        self.lib = _lib.load()
        self.sharding = sharding
        self.device = torch.cuda.current_device() if device is None else device
        cfg = TpConfig(max_m=max_m, max_n=max_n, max_vocab=max_vocab, wait_ms=wait_ms, num_ctas=num_ctas)
        h = C.c_void_p()
        st = self.lib.ws_tp_create(sharding.world_size, sharding.rank, self.device, C.byref(cfg), C.byref(h))
        if st != WS_OK:
            raise WsError(st, "ws_tp_create failed")
        self.handle = h
        self._keep: list = []
        self._host_args: dict = {}
        self._host_call = self.lib.ws_fp8_rowpar_gemm_allreduce_host

    # -- life cycle
    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ws_tp_destroy(self.handle)
            self.handle = None
            self._host_args.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ok(self, st: int) -> None:
        if st != WS_OK:
            raise WsError(st, (self.lib.ws_tp_last_error(self.handle) or b"").decode())

    @property
    def world_size(self) -> int:
        return self.sharding.world_size

    @property
    def rank(self) -> int:
        return self.sharding.rank

    def export_handle(self) -> bytes:
        h = IpcHandle()
        self._ok(self.lib.ws_tp_export_handle(self.handle, C.byref(h)))
        return bytes(h.bytes)

    def connect_ipc(self, handles: Sequence[bytes]) -> None:
        arr = (IpcHandle * len(handles))()
        for i, b in enumerate(handles):
            C.memmove(C.byref(arr[i]), b, len(b))
        self._ok(self.lib.ws_tp_connect_ipc(self.handle, arr, len(handles)))

    def connect_process_group(self, group=None) -> None:
        """One process per rank: trade IPC handles over ``torch.distributed``."""
        import torch.distributed as dist
        mine = self.export_handle()
        got: List[Optional[bytes]] = [None] * self.world_size
        dist.all_gather_object(got, mine, group=group)
        self.connect_ipc(got)  # type: ignore[arg-type]
        dist.barrier(group=group)

    def connect_tcp(self, host: str, port: int, timeout_ms: int = 30000) -> None:
        """One process per rank, no host framework: the ranks trade their IPC handles over TCP (rank 0
        listens on host:port), as the reference's control plane does for its ring (ctrl.rs:12-29)."""
        self._ok(self.lib.ws_tp_connect_tcp(self.handle, self.rank, self.world_size, host.encode(), int(port), int(timeout_ms)))

    def set_split(self, on: bool) -> None:
        self._ok(self.lib.ws_tp_set_split(self.handle, int(on)))

    def set_kernel(self, which: int) -> None:
        """0: automatic (default); 1: the mma.sync kernels; 2: the tcgen05 kernels wherever the shape fits;
        3: the CUDA-core kernels (MoE: the decode form)."""
        self._ok(self.lib.ws_tp_set_kernel(self.handle, int(which)))

    def check(self, stream=None) -> None:
        """Synchronise the stream and raise if a kernel recorded an error (fail-stop)."""
        self._ok(self.lib.ws_tp_check(self.handle, _stream_ptr(stream)))

    def stats(self) -> str:
        """Collectives::stats (engine.rs:291-293)."""
        s, l = C.c_uint64(), C.c_uint64()
        self._ok(self.lib.ws_tp_stats(self.handle, C.byref(s), C.byref(l)))
        return f"steps={s.value} launches={l.value}"

    @property
    def launches(self) -> int:
        s, l = C.c_uint64(), C.c_uint64()
        self._ok(self.lib.ws_tp_stats(self.handle, C.byref(s), C.byref(l)))
        return int(l.value)

    @property
    def num_ctas(self) -> int:
        return int(self.lib.ws_tp_num_ctas(self.handle))

    # -- fused operators (device tensors, stream-ordered, no synchronisation)
    def fp8_rowpar_gemm_allreduce(self, x, w, scales, *, block=(128, 128), row0=0, k0=0, out=None, stream=None):
        """emit8 + gemm_q8(wo_b) + Collectives::allreduce (engine.rs:3988-4029)."""
        if out is None:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        a = _fp8_args(x, w, scales, block, row0, k0, out)
        self._ok(self.lib.ws_fp8_rowpar_gemm_allreduce(self.handle, C.byref(a), _stream_ptr(stream)))
        return out

    def moe_down_combine_allreduce(self, h, route_ids, route_w, w2, s2, e_start, *, out=None, stream=None):
        """emit8 + grouped down GEMM + moe_combine_f32 + allreduce (engine.rs:4207-4239, :4513-4522)."""
        a = _moe_args(h, route_ids, route_w, w2, s2, e_start, out)
        if out is None:
            out = torch.empty((route_ids.shape[0], w2.shape[1]), dtype=torch.float32, device=h.device)
            a.out = out.data_ptr()
        self._ok(self.lib.ws_moe_down_combine_allreduce(self.handle, C.byref(a), _stream_ptr(stream)))
        return out

    def lm_head_allgather_argmax(self, x, w, scales, *, vocab_row0, vocab, block=(128, 128), row0=0,
                                 want_logits=True, stream=None):
        """head GEMV + Collectives::allgather + argmax (engine.rs:2647-2667, :2687-2703)."""
        m = x.shape[0]
        logits = torch.empty((m, vocab), dtype=torch.float32, device=x.device) if want_logits else None
        arg = torch.empty((m,), dtype=torch.int32, device=x.device)
        a = LmHeadArgs()
        a.g = _fp8_args(x, w, scales, block, row0, 0, None)
        a.vocab_row0, a.vocab = vocab_row0, vocab
        a.logits = logits.data_ptr() if logits is not None else None
        a.argmax = arg.data_ptr()
        self._ok(self.lib.ws_lm_head_allgather_argmax(self.handle, C.byref(a), _stream_ptr(stream)))
        return logits, arg

    # -- bare collectives on device tensors
    def allreduce_(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        out = torch.empty_like(inp) if out is None else out
        self._ok(self.lib.ws_allreduce_f32(self.handle, inp.data_ptr(), out.data_ptr(), inp.numel(), _stream_ptr(stream)))
        return out

    def allgather_(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if out is None:
            out = torch.empty(inp.numel() * self.world_size, dtype=torch.float32, device=inp.device)
        self._ok(self.lib.ws_allgather_f32(self.handle, inp.data_ptr(), out.data_ptr(), inp.numel(), _stream_ptr(stream)))
        return out

    # -- host-buffer forms
    def fp8_rowpar_gemm_allreduce_host(self, x_host: np.ndarray, w, scales, *, block=(128, 128), row0=0, k0=0,
                                       x_dtype: int = WS_ACT_BF16) -> np.ndarray:
        """Same fused step fed from host memory: activations are copied in and the reduced
        rows copied out inside the call, which returns only when they are valid."""
        m = x_host.shape[0]
        n, k = w.shape
        # the argument struct of a (weight, shape) pair is built once: a decode loop calls this with
        # the same weights every step, and filling a ctypes struct costs as much as the launch
        key = (w.data_ptr(), scales.data_ptr(), m, n, k, w.stride(0), tuple(block), row0, k0, x_dtype)
        hit = self._host_args.get(key)
        if hit is None:
            a = Fp8GemmArgs()
            a.x, a.ldx, a.x_dtype = None, k, x_dtype
            a.m, a.n, a.k = m, n, k
            a.w, a.ldw = w.data_ptr(), w.stride(0)
            a.scales, a.scale_ld, a.scale_kind = scales.data_ptr(), scales.shape[1], _scale_kind(scales)
            a.block_n, a.block_k = block
            a.row0, a.k0 = row0, k0
            if len(self._host_args) >= 4096:
                self._host_args.clear()
            hit = self._host_args[key] = (a, C.byref(a), w, scales)  # the tensors stay alive with their entry
        out = np.empty((m, n), dtype=np.float32)
        xh = x_host if x_host.flags["C_CONTIGUOUS"] else np.ascontiguousarray(x_host)
        st = self._host_call(self.handle, hit[1], _np_ptr(xh), _np_ptr(out))
        if st != WS_OK:
            self._ok(st)
        return out


def _moe_args(h, route_ids, route_w, w2, s2, e_start, out) -> MoeDownArgs:
    if w2.dim() != 3 or s2.dim() != 3:
        raise ValueError("w2 must be [e_len, n, k/2] and s2 [e_len, n, k/32]")
    if not (w2.is_contiguous() and s2.is_contiguous() and route_ids.is_contiguous() and route_w.is_contiguous()):
        raise ValueError("expert slab and routing tensors must be contiguous")
    if route_ids.dtype != torch.int32 or route_w.dtype != torch.float32:
        raise TypeError("route_ids must be int32 and route_w float32")
    e_len, n, half = w2.shape
    m, top_k = route_ids.shape
    a = MoeDownArgs()
    a.h, a.ldh, a.h_dtype = h.data_ptr(), (h.stride(0) if h.shape[0] > 1 else half * 2), _act_dtype(h)
    a.m, a.n, a.k, a.top_k = m, n, half * 2, top_k
    a.route_ids, a.route_w = route_ids.data_ptr(), route_w.data_ptr()
    a.w2, a.s2 = w2.data_ptr(), s2.data_ptr()
    a.e_start, a.e_len = e_start, e_len
    a.out = out.data_ptr() if out is not None else None
    return a


class Collectives:
    """``trait Collectives`` (engine.rs:287-294) over an :class:`Endpoint`: host slice in,
    owned host vector out, bit-identical on every rank; any error raises (fail-stop)."""

    def __init__(self, endpoint: Endpoint):
        self.ep = endpoint
        self.coll_count = 0

    def allreduce(self, input: Sequence[float]) -> np.ndarray:
        inp = np.ascontiguousarray(input, dtype=np.float32)
        if inp.size == 0:
            raise WsError(_lib.WS_ERR_INVALID, "collective input len 0 not in 1..")
        out = np.empty_like(inp)
        self.ep._ok(self.ep.lib.ws_allreduce_f32_host(self.ep.handle, inp.ctypes.data, out.ctypes.data, inp.size))
        self.coll_count += 1
        return out

    def allgather(self, contribution: Sequence[float]) -> np.ndarray:
        inp = np.ascontiguousarray(contribution, dtype=np.float32)
        if inp.size == 0:
            raise WsError(_lib.WS_ERR_INVALID, "collective input len 0 not in 1..")
        out = np.empty(inp.size * self.ep.world_size, dtype=np.float32)
        self.ep._ok(self.ep.lib.ws_allgather_f32_host(self.ep.handle, inp.ctypes.data, out.ctypes.data, inp.size))
        self.coll_count += 1
        return out

    def stats(self) -> str:
        return f"collectives={self.coll_count} {self.ep.stats()}"


class LocalGroup:
    """All ranks of a group driven by one process: several devices with peer access, or
    several virtual ranks on ONE device (one cooperative kernel runs every rank, which is
    how the multi-rank exchange is exercised on a single GPU)."""

    def __init__(self, world: int, devices: Optional[Sequence[int]] = None, **cfg):
        devs = list(devices) if devices is not None else [torch.cuda.current_device()] * world
        if len(devs) != world:
            raise ValueError("one device id per rank")
        self.world = world
        self.eps = [Endpoint(Sharding(world, r), devs[r], **cfg) for r in range(world)]
        self.lib = self.eps[0].lib
        arr = (C.c_void_p * world)(*[e.handle for e in self.eps])
        self._handles = arr
        if world > 1:
            self.eps[0]._ok(self.lib.ws_tp_connect_local(arr, world))

    def close(self) -> None:
        for e in self.eps:
            e.close()

    def _streams(self):
        ptrs = []
        for e in self.eps:
            with torch.cuda.device(e.device):
                ptrs.append(_stream_ptr())
        return (C.c_void_p * self.world)(*ptrs)

    def set_split(self, on: bool) -> None:
        for e in self.eps:
            e.set_split(on)

    def set_kernel(self, which: int) -> None:
        for e in self.eps:
            e.set_kernel(which)

    def check(self) -> None:
        for e in self.eps:
            with torch.cuda.device(e.device):
                e.check()

    def fp8_rowpar_gemm_allreduce(self, xs, ws, scales, *, block=(128, 128), row0s=None, k0s=None):
        outs = [torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device) for x, w in zip(xs, ws)]
        args = (Fp8GemmArgs * self.world)()
        for r in range(self.world):
            args[r] = _fp8_args(xs[r], ws[r], scales[r], block, row0s[r] if row0s else 0, k0s[r] if k0s else 0, outs[r])
        self.eps[0]._ok(self.lib.ws_fp8_rowpar_gemm_allreduce_group(self._handles, self.world, args, self._streams()))
        return outs

    def moe_down_combine_allreduce(self, hs, route_ids, route_ws, w2s, s2s, e_starts):
        outs = [torch.empty((route_ids[r].shape[0], w2s[r].shape[1]), dtype=torch.float32, device=hs[r].device)
                for r in range(self.world)]
        args = (MoeDownArgs * self.world)()
        for r in range(self.world):
            args[r] = _moe_args(hs[r], route_ids[r], route_ws[r], w2s[r], s2s[r], e_starts[r], outs[r])
        self.eps[0]._ok(self.lib.ws_moe_down_combine_allreduce_group(self._handles, self.world, args, self._streams()))
        return outs

    def lm_head_allgather_argmax(self, xs, ws, scales, *, vocab, block=(128, 128), vocab_row0s, row0s=None,
                                 want_logits=True):
        m = xs[0].shape[0]
        logits = [torch.empty((m, vocab), dtype=torch.float32, device=x.device) if want_logits else None for x in xs]
        amax = [torch.empty((m,), dtype=torch.int32, device=x.device) for x in xs]
        args = (LmHeadArgs * self.world)()
        for r in range(self.world):
            a = LmHeadArgs()
            a.g = _fp8_args(xs[r], ws[r], scales[r], block, row0s[r] if row0s else 0, 0, None)
            a.vocab_row0, a.vocab = vocab_row0s[r], vocab
            a.logits = logits[r].data_ptr() if want_logits else None
            a.argmax = amax[r].data_ptr()
            args[r] = a
        self.eps[0]._ok(self.lib.ws_lm_head_allgather_argmax_group(self._handles, self.world, args, self._streams()))
        return logits, amax

    def _coll(self, fn, inputs, out_len):
        outs = [torch.empty(out_len, dtype=torch.float32, device=t.device) for t in inputs]
        ins = (C.c_void_p * self.world)(*[t.data_ptr() for t in inputs])
        ous = (C.c_void_p * self.world)(*[t.data_ptr() for t in outs])
        self.eps[0]._ok(fn(self._handles, self.world, ins, ous, inputs[0].numel(), self._streams()))
        return outs

    def allreduce(self, inputs):
        return self._coll(self.lib.ws_allreduce_f32_group, inputs, inputs[0].numel())

    def allgather(self, inputs):
        return self._coll(self.lib.ws_allgather_f32_group, inputs, inputs[0].numel() * self.world)


def act_quant_fp8(x: torch.Tensor, stream=None):
    """act_quant_fp8_emit (crates/weightstream-cuda/kernels/actquant.cu:47-83): E4M3 bytes and
    one UE8M0 exponent byte per 32 values, bit-exact with the reference's CPU rule."""
    L = _lib.load()
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((m, k // 32), dtype=torch.uint8, device=x.device)
    st = L.ws_act_quant_fp8(x.data_ptr(), x.stride(0), _act_dtype(x), m, k, q.data_ptr(), s.data_ptr(), _stream_ptr(stream))
    if st != WS_OK:
        raise WsError(st, "ws_act_quant_fp8 rejected its arguments")
    return q, s
