"""The TCP rendezvous that trades IPC handles between ranks (csrc/ws_bootstrap.cu): no device involved,
so it runs on CPU with one thread per rank (ctypes releases the GIL while a rank blocks in the call)."""
import ctypes as C
import socket
import threading

import pytest

from weightstream_b200 import _lib

WS_OK, WS_ERR_INVALID, WS_ERR_TIMEOUT = 0, -1, -3


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(world, port, blobs, ranks=None, worlds=None, timeout_ms=5000, delay_rank0=0.0):
    L = _lib.load()
    ranks = list(range(world)) if ranks is None else ranks
    out = [None] * len(ranks)
    status = [None] * len(ranks)

    def work(i):
        import time
        r = ranks[i]
        if r == 0 and delay_rank0:
            time.sleep(delay_rank0)
        w = world if worlds is None else worlds[i]
        src = C.create_string_buffer(blobs[i], len(blobs[i]))
        dst = C.create_string_buffer(w * len(blobs[i]))
        status[i] = L.ws_tcp_allgather(r, w, b"127.0.0.1", port, src, dst, len(blobs[i]), timeout_ms)
        out[i] = dst.raw

    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(ranks))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(30)
    return status, out


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_every_rank_receives_all_handles_in_rank_order(world):
    blobs = [bytes([(r * 17 + i) & 0xFF for i in range(128)]) for r in range(world)]
    status, out = run_ranks(world, free_port(), blobs)
    assert status == [WS_OK] * world
    for r in range(world):
        assert out[r] == b"".join(blobs)


def test_ranks_that_start_before_the_listener_keep_trying():
    world = 3
    blobs = [bytes([r]) * 128 for r in range(world)]
    status, out = run_ranks(world, free_port(), blobs, delay_rank0=0.5)
    assert status == [WS_OK] * world and out[2] == b"".join(blobs)


def test_a_missing_rank_is_a_timeout_on_everyone():
    world = 3
    blobs = [bytes([r]) * 128 for r in range(2)]
    status, _ = run_ranks(world, free_port(), blobs, ranks=[0, 1], timeout_ms=400)
    assert status == [WS_ERR_TIMEOUT, WS_ERR_TIMEOUT]


def test_a_rank_of_another_group_is_refused():
    blobs = [bytes([r]) * 128 for r in range(2)]
    status, _ = run_ranks(2, free_port(), blobs, ranks=[0, 1], worlds=[2, 3], timeout_ms=1500)
    assert status[0] == WS_ERR_INVALID      # rank 0 saw a header for a world of three
    assert status[1] in (WS_ERR_INVALID, WS_ERR_TIMEOUT)


def test_arguments_are_checked():
    L = _lib.load()
    buf = C.create_string_buffer(128)
    assert L.ws_tcp_allgather(2, 2, b"127.0.0.1", 4000, buf, buf, 128, 100) == WS_ERR_INVALID   # rank out of range
    assert L.ws_tcp_allgather(0, 2, b"127.0.0.1", 0, buf, buf, 128, 100) == WS_ERR_INVALID      # no port
    assert L.ws_tcp_allgather(0, 2, b"no such host.invalid", 4000, buf, buf, 128, 100) == WS_ERR_INVALID
