"""The allocation-free FP8 GEMM entry point (ws_fp8_gemm_static_scratch).

Some callers cannot let a library allocate device memory for them: a host runtime that
carves one arena at start-up and treats any later cudaMalloc as a bug, or a plug-in that has
no endpoint object to own scratch.  For them the library carries its scratch inside its own
image.  This test calls that entry point through the C ABI twice in a row (the second call
finds the first call's leftovers in the shared scratch) and checks both results against the
regular entry point, and checks that oversize requests are refused with a message.

It is collected last on purpose, so that a run stopping at the first failure has already
run every other test; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    d = np.linalg.norm(got.astype(np.float64) - want.astype(np.float64))
    return float(d / max(np.linalg.norm(want.astype(np.float64)), 1e-30))


def test_static_scratch_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    from weightstream_b200 import _lib, synth, tp
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = _lib.load()
    # n = 7168 gives every CTA 48 or 49 rows (ragged tiles); the kernel keeps its status word and step counter in the scratch
    n, k = 7168, 2048
    rng = np.random.default_rng(77)
    w, sc = synth.fp8_weight(rng, n, k)
    wd, sd = torch.from_numpy(w).to(dev), torch.from_numpy(sc).to(dev)
    ep = tp.Endpoint(max_m=8, max_n=n)
    stream = tp._stream_ptr()
    err = C.create_string_buffer(256)
    try:
        for call, m in enumerate((3, 8)):
            xb = synth.activations_bf16(rng, m, k)
            xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
            want = ep.fp8_rowpar_gemm_allreduce(xd, wd, sd)
            ep.check()
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
            a = tp._fp8_args(xd, wd, sd, (128, 128), 0, 0, out)
            st = L.ws_fp8_gemm_static_scratch(C.byref(a), 0, stream, err, len(err))
            assert st == _lib.WS_OK, err.value.decode()
            torch.cuda.synchronize()
            got, ref = out.cpu().numpy(), want.cpu().numpy()
            assert np.isfinite(got).all(), f"call {call}: output not fully written"
            assert rel_l2(got, ref) < 5e-5, f"call {call}: rel L2 {rel_l2(got, ref):.3e}"
        # beyond the stated maximum: refused, with a message, before anything is launched
        xb = synth.activations_bf16(rng, 9, k)
        xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
        out = torch.zeros((9, n), dtype=torch.float32, device=dev)
        a = tp._fp8_args(xd, wd, sd, (128, 128), 0, 0, out)
        st = L.ws_fp8_gemm_static_scratch(C.byref(a), 0, stream, err, len(err))
        assert st == _lib.WS_ERR_CAPACITY and b"exceeds" in err.value
    finally:
        ep.close()
