"""CPU-rank simulation of the one-shot exchange (test infrastructure, like the oracle).

R threads play R ranks.  Each rank owns slot memory double-banked by step parity and one
flag per (bank, source rank) carrying the step sequence number -- the protocol the CUDA
kernels run over NVLink, restated on host buffers so that rank order, cross-rank bit
identity, run-ahead safety and the fail-stop rules can be tested with no GPU:

* every rank stores its vector into slot [bank][my rank] of EVERY rank, then sets the flag
  (crates/weightstream-transport/src/ring.rs:338-390 does the same in two RDMA hops);
* a rank waits, with a deadline, until all R flags of the bank carry this step's sequence
  number (ring.rs:439-458: a timeout aborts the step, nothing is computed on partial data;
  ring.rs:488-499: a sequence number that is neither this step's nor an earlier one aborts);
* all-reduce adds the slots left to right in rank order (ring.rs:399-408); all-gather
  concatenates them (ring.rs:426-432).

``tagged=True`` restates the all-reduce the fused kernels use: no flag; every value travels
as one 64-bit word {step sequence, fp32 bits} and the receiver polls each word until its tag is
this step's.  Same rank order, same fail-stop rules, same two banks.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

import numpy as np


class ExchangeTimeout(RuntimeError):
    pass


class ExchangeOutOfSequence(RuntimeError):
    pass


class RankMemory:
    def __init__(self, world: int, elems: int):
        self.slots = np.zeros((2, world, elems), dtype=np.float32)
        self.flags = np.zeros((2, world), dtype=np.uint32)
        self.words = np.zeros((2, world, elems), dtype=np.uint64)  # tagged all-reduce words


class SimGroup:
    def __init__(self, world: int, elems: int, wait_s: float = 1.0, tagged: bool = False):
        self.world, self.elems, self.wait_s, self.tagged = world, elems, wait_s, tagged
        self.mem = [RankMemory(world, elems) for _ in range(world)]
        self.step = [0] * world
        # fault injection (host side only): drop[(src, dst)] = True loses src's message to dst
        self.drop = {}
        self.seq_override = {}

    def _exchange(self, rank: int, vec: np.ndarray) -> int:
        n = vec.size
        if n == 0 or n > self.elems:
            raise ValueError(f"collective input len {n} not in 1..={self.elems}")
        self.step[rank] += 1
        seq = self.step[rank]
        bank = seq & 1
        send_seq = self.seq_override.get(rank, seq)
        for p in range(self.world):
            if self.drop.get((rank, p)):
                continue
            self.mem[p].slots[bank, rank, :n] = vec          # data first ...
            self.mem[p].flags[bank, rank] = send_seq          # ... then the flag (release)
        deadline = time.monotonic() + self.wait_s
        mine = self.mem[rank]
        while True:
            f = mine.flags[bank].copy()
            if np.all(f == seq):
                return bank
            bad = [int(v) for v in f if v > seq]
            if bad:
                raise ExchangeOutOfSequence(f"collective out of sequence: got step {bad[0]} at step {seq} (fail-stop)")
            if time.monotonic() >= deadline:
                have = [r for r in range(self.world) if f[r] == seq]
                raise ExchangeTimeout(f"all-reduce wait timeout after {int(self.wait_s * 1e3)} ms "
                                      f"(have {have} of {self.world}); fail-stop, aborting")
            time.sleep(0)

    def _allreduce_tagged(self, rank: int, v: np.ndarray) -> np.ndarray:
        n = v.size
        if n == 0 or n > self.elems:
            raise ValueError(f"collective input len {n} not in 1..={self.elems}")
        self.step[rank] += 1
        seq = self.step[rank]
        bank = seq & 1
        send_seq = self.seq_override.get(rank, seq)
        word = (np.uint64(send_seq) << np.uint64(32)) | v.view(np.uint32).astype(np.uint64)
        for p in range(self.world):
            if not self.drop.get((rank, p)):
                self.mem[p].words[bank, rank, :n] = word  # value and tag in one store
        deadline = time.monotonic() + self.wait_s
        mine = self.mem[rank].words[bank]
        while True:
            w = mine[:, :n].copy()
            tags = (w >> np.uint64(32)).astype(np.uint32)
            if np.all(tags == seq):
                vals = (w & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32)
                acc = vals[0].copy()
                for r in range(1, self.world):
                    acc = (acc + vals[r]).astype(np.float32)
                return acc
            if np.any(tags > seq):
                raise ExchangeOutOfSequence(f"collective out of sequence: got step {int(tags.max())} at step {seq} (fail-stop)")
            if time.monotonic() >= deadline:
                have = [r for r in range(self.world) if np.all(tags[r] == seq)]
                raise ExchangeTimeout(f"all-reduce wait timeout after {int(self.wait_s * 1e3)} ms "
                                      f"(have {have} of {self.world}); fail-stop, aborting")
            time.sleep(0)

    def allreduce(self, rank: int, vec: np.ndarray) -> np.ndarray:
        v = np.ascontiguousarray(vec, dtype=np.float32)
        if self.tagged:
            return self._allreduce_tagged(rank, v)
        bank = self._exchange(rank, v)
        s = self.mem[rank].slots[bank]
        acc = s[0, :v.size].copy()
        for r in range(1, self.world):
            acc = (acc + s[r, :v.size]).astype(np.float32)
        return acc

    def allgather(self, rank: int, vec: np.ndarray) -> np.ndarray:
        v = np.ascontiguousarray(vec, dtype=np.float32)
        bank = self._exchange(rank, v)
        return self.mem[rank].slots[bank][:, :v.size].reshape(-1).copy()


def run_ranks(world: int, fn: Callable[[int], object], skip: Optional[List[int]] = None):
    """Run fn(rank) on one thread per rank; returns results (or the exception raised)."""
    out: List[object] = [None] * world

    def body(r):
        try:
            out[r] = fn(r)
        except Exception as e:  # noqa: BLE001 - handed back to the test
            out[r] = e

    ts = [threading.Thread(target=body, args=(r,)) for r in range(world) if not (skip and r in skip)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out
