"""The allocation-free FP8 GEMM entry point (ws_fp8_gemm_static_scratch).

Some callers cannot let a library allocate device memory for them: a host runtime that
carves one arena at start-up and treats any later cudaMalloc as a bug, or a plug-in that has
no endpoint object to own scratch.  For them the library carries its scratch inside its own
image.  This test calls that entry point through the C ABI several times in a row (every call
after the first finds the previous call's leftovers in the shared scratch), reads the launch's
status back with ws_fp8_gemm_static_scratch_check, and checks each result three ways: bit for
bit against the regular entry point running the same kernel formulation, within the path's
tolerance against the CPU oracle, and fully written.  Oversize requests must be refused with a
message before anything is launched.

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


def test_static_scratch_matches_regular_entry_point_and_oracle(oracle):
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    from weightstream_b200 import _lib, formats as F, synth, tp
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = _lib.load()
    stream = tp._stream_ptr()
    err = C.create_string_buffer(256)
    rng = np.random.default_rng(77)

    def run_case(ep, w, sc, wd, sd, m, block, row0, k0, call):
        k = wd.shape[1]
        n = wd.shape[0]
        xb = synth.activations_bf16(rng, m, k)
        xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
        want = ep.fp8_rowpar_gemm_allreduce(xd, wd, sd, block=block, row0=row0, k0=k0)
        ep.check()
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
        a = tp._fp8_args(xd, wd, sd, block, row0, k0, out)
        st = L.ws_fp8_gemm_static_scratch(C.byref(a), 0, stream, err, len(err))
        assert st == _lib.WS_OK, err.value.decode()
        st = L.ws_fp8_gemm_static_scratch_check(0, stream, err, len(err))  # synchronises and reads the status word
        assert st == _lib.WS_OK, err.value.decode()
        got, ref = out.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}: output not fully written"
        # same kernel formulation on both sides (the endpoint is told to use it for every row count)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), f"call {call}: differs from the regular entry point"
        cpu = oracle.fp8_gemv(w, sc, F.bf16_bits_to_f32(xb), bn=block[0], bk=block[1], row0=row0, k0=k0,
                              threads=oracle.max_threads())
        e = rel_l2(got, cpu)
        assert e <= 1e-3 and e < 5e-5, f"call {call}: rel L2 vs the oracle {e:.3e}"

    # n = 7168 gives every CTA 48 or 49 rows (ragged tiles); the kernel keeps its status word and step counter in the scratch
    n, k = 7168, 2048
    w, sc = synth.fp8_weight(rng, n, k)
    wd, sd = torch.from_numpy(w).to(dev), torch.from_numpy(sc).to(dev)
    ep = tp.Endpoint(max_m=8, max_n=n)
    ep.set_kernel(1)  # the formulation the allocation-free entry point always uses, so results can be compared bit for bit
    try:
        for call, m in enumerate((3, 8, 1)):
            run_case(ep, w, sc, wd, sd, m, (128, 128), 0, 0, call)
        # the reference's native scale layout (UE8M0 per 32x32) on a shard that starts inside the scale matrix
        nfull, kfull, row0, k0, n2, k2 = 1024, 1024, 256, 384, 512, 512
        wf, scf = synth.fp8_weight(rng, nfull, kfull, scale="ue8m0", bn=32, bk=32)
        wsh = np.ascontiguousarray(wf[row0:row0 + n2, k0:k0 + k2])
        wd2, sd2 = torch.from_numpy(wsh).to(dev), torch.from_numpy(np.ascontiguousarray(scf)).to(dev)
        for call, m in enumerate((2, 5)):
            run_case(ep, wsh, scf, wd2, sd2, m, (32, 32), row0, k0, 10 + call)
        # beyond the stated maximum: refused, with a message, before anything is launched
        xb = synth.activations_bf16(rng, 9, k)
        xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
        out = torch.zeros((9, n), dtype=torch.float32, device=dev)
        a = tp._fp8_args(xd, wd, sd, (128, 128), 0, 0, out)
        st = L.ws_fp8_gemm_static_scratch(C.byref(a), 0, stream, err, len(err))
        assert st == _lib.WS_ERR_CAPACITY and b"exceeds" in err.value
        assert L.ws_fp8_gemm_static_scratch_check(64, stream, err, len(err)) == _lib.WS_ERR_INVALID
    finally:
        ep.close()
