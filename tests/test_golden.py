"""The committed fixture tests/golden/golden.npz (made by tests/golden/make_golden.py from the CPU
oracle) against (1) the oracle as it is now, bit for bit, on CPU, and (2) the CUDA path through the
C ABI on a GPU, within the path's tolerance (1e-3 relative L2 on fp32 outputs, identical bytes for
the quantiser, identical argmax, identical bits on all ranks)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


# ----------------------------------------------------------------------------- CPU: the oracle has not drifted
def test_oracle_reproduces_the_fixture(oracle, gold):
    from weightstream_b200 import formats as F
    for r in range(3):
        q, e = oracle.fp8_act_emit(gold["act_x"][r])
        assert np.array_equal(q, gold["act_q"][r]) and np.array_equal(e, gold["act_e"][r])
    for tag, bn, bk in (("f32", 128, 128), ("ue8m0", 32, 32)):
        y = oracle.fp8_gemv(gold[f"fp8_{tag}_w"], gold[f"fp8_{tag}_s"], F.bf16_bits_to_f32(gold[f"fp8_{tag}_x"]), bn=bn, bk=bk)
        assert np.array_equal(bits(y), bits(gold[f"fp8_{tag}_y"]))
    assert np.array_equal(bits(oracle.allreduce_fold(gold["fp8_tp2_parts"])), bits(gold["fp8_tp2_y"]))
    y = oracle.moe_down_combine(gold["moe_w2"], gold["moe_s2"], 0, F.bf16_bits_to_f32(gold["moe_h"]), gold["moe_ids"], gold["moe_rw"])
    assert np.array_equal(bits(y), bits(gold["moe_y"]))
    assert [oracle.argmax(gold["argmax_logits"][t]) for t in range(3)] == list(gold["argmax_idx"])


def test_fixture_generator_is_deterministic(oracle, gold):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    again = mod.build()
    assert sorted(again) == sorted(gold.files)
    for k in gold.files:
        assert np.array_equal(np.ascontiguousarray(again[k]).view(np.uint8), np.ascontiguousarray(gold[k]).view(np.uint8)), k


# ----------------------------------------------------------------------------- GPU: the CUDA path against the fixture
def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)))


@pytest.mark.gpu
def test_cuda_path_matches_the_fixture(gold):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    from weightstream_b200 import tp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)

    def t(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    def bf16(a):
        return t(a.view(np.int16)).view(torch.bfloat16)

    # quantiser: identical bytes
    q, e = tp.act_quant_fp8(t(gold["act_x"]))
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), gold["act_q"]) and np.array_equal(e.cpu().numpy(), gold["act_e"])
    # FP8 product, one rank, both scale formats
    ep = tp.Endpoint(max_m=8, max_n=64, max_vocab=64)
    try:
        for tag, blk in (("f32", (128, 128)), ("ue8m0", (32, 32))):
            y = ep.fp8_rowpar_gemm_allreduce(bf16(gold[f"fp8_{tag}_x"]), t(gold[f"fp8_{tag}_w"]), t(gold[f"fp8_{tag}_s"]), block=blk)
            ep.check()
            assert rel_l2(y.cpu().numpy(), gold[f"fp8_{tag}_y"]) < 5e-5
        # MoE down + combine
        y = ep.moe_down_combine_allreduce(bf16(gold["moe_h"]), t(gold["moe_ids"]), t(gold["moe_rw"]), t(gold["moe_w2"]), t(gold["moe_s2"]), 0)
        ep.check()
        assert rel_l2(y.cpu().numpy(), gold["moe_y"]) < 5e-5
        # lm_head mode on the same weights: logits and first-maximum argmax
        logits, am = ep.lm_head_allgather_argmax(bf16(gold["fp8_f32_x"]), t(gold["fp8_f32_w"]), t(gold["fp8_f32_s"]), vocab_row0=0, vocab=64)
        ep.check()
        assert rel_l2(logits.cpu().numpy(), gold["fp8_f32_y"]) < 5e-5
        assert [int(a) for a in am.cpu()] == [int(np.argmax(gold["fp8_f32_y"][r])) for r in range(3)]
    finally:
        ep.close()
    # K over two (virtual) ranks, folded in rank order, identical bits on both
    grp = tp.LocalGroup(2, max_m=8, max_n=64)
    try:
        w, sc, xb = gold["fp8_f32_w"], t(gold["fp8_f32_s"]), gold["fp8_f32_x"]
        xs = [bf16(np.ascontiguousarray(xb[:, a:a + 128])) for a in (0, 128)]
        ws = [t(w[:, a:a + 128]) for a in (0, 128)]
        outs = grp.fp8_rowpar_gemm_allreduce(xs, ws, [sc, sc], k0s=[0, 128])
        grp.check()
        a, b = outs[0].cpu().numpy(), outs[1].cpu().numpy()
        assert np.array_equal(bits(a), bits(b))
        assert rel_l2(a, gold["fp8_tp2_y"]) < 5e-5
    finally:
        grp.close()
