"""Worker of tests/test_gpu_multiproc.py: one process per GPU (torchrun), endpoints joined through
CUDA IPC handles traded over torch.distributed; every fused operator checked against the oracle
and for bit-identical results across ranks."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from weightstream_b200 import formats as F, synth, tp  # noqa: E402


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b.astype(np.float64)))


def same_everywhere(t: torch.Tensor, world: int) -> bool:
    got = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(got, t)
    return all(torch.equal(g.view(torch.int32), got[0].view(torch.int32)) for g in got)


def main():
    world, rank, lr = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    sh = tp.Sharding(world, rank)
    vocab = 16 * 101 * world
    ep = tp.Endpoint(sh, lr, max_m=64, max_n=7168, max_vocab=vocab, wait_ms=5000)
    ep.connect_process_group()
    rng = np.random.default_rng(7)  # same tensors on every rank
    # o_proj, K sliced
    n, k = 7168, 2048
    w, sc = synth.fp8_weight(rng, n, k)
    for m in (1, 11, 40):  # 11 and 40 rows run on the tcgen05 kernel (CTA pairs sending tagged words to every rank)
        xb = synth.activations_bf16(rng, m, k)
        xf = F.bf16_bits_to_f32(xb)
        k0, kl = sh.slice_of(k)
        xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)[:, k0:k0 + kl].contiguous()
        wd = torch.from_numpy(np.ascontiguousarray(w[:, k0:k0 + kl])).to(dev)
        out = ep.fp8_rowpar_gemm_allreduce(xd, wd, torch.from_numpy(sc).to(dev), k0=k0)
        ep.check()
        parts = [O.fp8_gemv(w[:, a:a + kl], sc, xf[:, a:a + kl], bn=128, bk=128, k0=a, threads=4)
                 for a in range(0, k, kl)]
        want = O.allreduce_fold(np.stack(parts))
        assert rel(out.cpu().numpy(), want) < 5e-5, f"o_proj m={m}"
        assert same_everywhere(out, world), "o_proj ranks differ"
    # bare collectives, host-buffer trait
    c = tp.Collectives(ep)
    v = (np.arange(5000, dtype=np.float32) * 0.25 + rank).astype(np.float32)
    red = c.allreduce(v)
    exp = v - rank
    acc = exp + 0.0
    for r in range(1, world):
        acc = (acc + (exp + np.float32(r))).astype(np.float32)
    assert np.array_equal(red, acc)
    gat = c.allgather(v[:100])
    assert np.array_equal(gat, np.concatenate([exp[:100] + np.float32(r) for r in range(world)]))
    # MoE, experts by id
    E, top_k, nn, kk = 8 * world, 6, 1024, 512
    w2, s2 = synth.fp4_experts(rng, E, nn, kk)
    ids, rw = synth.routes(rng, 5, E, top_k)
    hb = F.f32_to_bf16_bits(rng.standard_normal((5 * top_k, kk)).astype(np.float32))
    e0, el = sh.slice_of(E)
    y = ep.moe_down_combine_allreduce(torch.from_numpy(hb.view(np.int16)).to(dev).view(torch.bfloat16),
                                      torch.from_numpy(ids).to(dev), torch.from_numpy(rw).to(dev),
                                      torch.from_numpy(w2[e0:e0 + el]).to(dev), torch.from_numpy(s2[e0:e0 + el]).to(dev), e0)
    ep.check()
    hf = F.bf16_bits_to_f32(hb)
    want = O.allreduce_fold(np.stack([O.moe_down_combine(w2[a:a + el], s2[a:a + el], a, hf, ids, rw) for a in range(0, E, el)]))
    assert rel(y.cpu().numpy(), want) < 5e-5, "moe"
    assert same_everywhere(y, world), "moe ranks differ"
    # the same step at the measured expert shape's K (2048) with 40 tokens: several passes per expert
    kk2, mm = 2048, 40
    w2b, s2b = synth.fp4_experts(rng, E, 512, kk2)
    ids2, rw2 = synth.routes(rng, mm, E, top_k)
    hb2 = F.f32_to_bf16_bits(rng.standard_normal((mm * top_k, kk2)).astype(np.float32))
    y2 = ep.moe_down_combine_allreduce(torch.from_numpy(hb2.view(np.int16)).to(dev).view(torch.bfloat16),
                                       torch.from_numpy(ids2).to(dev), torch.from_numpy(rw2).to(dev),
                                       torch.from_numpy(w2b[e0:e0 + el]).to(dev), torch.from_numpy(s2b[e0:e0 + el]).to(dev), e0)
    ep.check()
    hf2 = F.bf16_bits_to_f32(hb2)
    want2 = O.allreduce_fold(np.stack([O.moe_down_combine(w2b[a:a + el], s2b[a:a + el], a, hf2, ids2, rw2) for a in range(0, E, el)]))
    assert rel(y2.cpu().numpy(), want2) < 5e-5, "moe, 40 tokens"
    assert same_everywhere(y2, world), "moe (40 tokens) ranks differ"
    # lm_head, vocab sliced
    wv, sv = synth.fp8_weight(rng, vocab, 512)
    xv = synth.activations_bf16(rng, 2, 512)
    v0, vl = sh.slice_of(vocab)
    svd = torch.from_numpy(sv).to(dev)
    s_r, row0, _ = tp.shard_scale(svd, svd.shape, tp.WShard.Rows(v0, vl), block=(128, 128))
    logits, am = ep.lm_head_allgather_argmax(torch.from_numpy(xv.view(np.int16)).to(dev).view(torch.bfloat16),
                                             torch.from_numpy(wv[v0:v0 + vl]).to(dev), s_r.contiguous(),
                                             vocab_row0=v0, vocab=vocab, row0=row0)
    ep.check()
    lw = O.fp8_gemv(wv, sv, F.bf16_bits_to_f32(xv), bn=128, bk=128, threads=4)
    assert rel(logits.cpu().numpy(), lw) < 5e-5, "lm_head"
    assert [int(a) for a in am.cpu()] == [O.argmax(lw[t]) for t in range(2)]
    assert same_everywhere(logits, world)
    # the decode form: argmax only (one merged candidate per rank crosses the links), 1 row and 40 rows
    for m in (2, 40):
        xm = synth.activations_bf16(rng, m, 512)
        _, am2 = ep.lm_head_allgather_argmax(torch.from_numpy(xm.view(np.int16)).to(dev).view(torch.bfloat16),
                                             torch.from_numpy(wv[v0:v0 + vl]).to(dev), s_r.contiguous(),
                                             vocab_row0=v0, vocab=vocab, row0=row0, want_logits=False)
        ep.check()
        lm = O.fp8_gemv(wv, sv, F.bf16_bits_to_f32(xm), bn=128, bk=128, threads=4)
        assert [int(a) for a in am2.cpu()] == [O.argmax(lm[t]) for t in range(m)], f"argmax-only lm_head m={m}"
        assert same_everywhere(am2, world)
    # a second endpoint brought up over the library's own TCP rendezvous (no torch.distributed involved
    # in the handle exchange): the same o_proj step gives the same bits
    ep2 = tp.Endpoint(sh, lr, max_m=16, max_n=7168, wait_ms=5000)
    ep2.connect_tcp("127.0.0.1", int(os.environ.get("MASTER_PORT", "29500")) + 173, timeout_ms=20000)
    xb = synth.activations_bf16(rng, 1, k)
    k0, kl = sh.slice_of(k)
    xd = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)[:, k0:k0 + kl].contiguous()
    wd = torch.from_numpy(np.ascontiguousarray(w[:, k0:k0 + kl])).to(dev)
    scd = torch.from_numpy(sc).to(dev)
    o1 = ep.fp8_rowpar_gemm_allreduce(xd, wd, scd, k0=k0)
    ep.check()
    o2 = ep2.fp8_rowpar_gemm_allreduce(xd, wd, scd, k0=k0)
    ep2.check()
    assert torch.equal(o1.view(torch.int32), o2.view(torch.int32)), "endpoint connected over TCP differs"
    ep2.close()
    ep.close()
    dist.barrier()
    if rank == 0:
        print("MP_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
