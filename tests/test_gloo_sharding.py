"""World-size-2 (and 4) ranks on CPU over gloo: the host-side sharding plan of the path.

Each rank slices the SAME quantised tensors with the reference's rule (rank*len/world,
crates/weightstream-gpu/src/engine.rs:1477-1480, :1194-1195, :3107-3108), computes its partial with
the oracle, and the ranks trade partials over gloo.  The rank-ordered fold must be identical on
every rank and within summation noise of the unsharded oracle; the gathered lm_head logits
must be the unsharded logits bit for bit (no summation crosses ranks there)."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from weightstream_b200 import formats as F, synth
    from weightstream_b200.tp import Sharding, WShard, shard_scale, shard_weight
    sh = Sharding(world, rank)
    rng = np.random.default_rng(123)              # same seed on every rank: same full tensors
    n, k, m = 256, 1024, 3
    w, sc = synth.fp8_weight(rng, n, k)
    x = F.bf16_bits_to_f32(synth.activations_bf16(rng, m, k))
    # --- o_proj: K slices, fp32 partials, rank-ordered fold
    k0, kl = sh.slice_of(k)
    wl = shard_weight(w, (n, k), WShard.Cols(k0, kl))
    sl, _, kofs = shard_scale(sc, sc.shape, WShard.Cols(k0, kl), block=(128, 128))
    part = O.fp8_gemv(wl, sl, x[:, k0:k0 + kl], bn=128, bk=128, k0=kofs)
    got = [torch.zeros(m, n) for _ in range(world)]
    dist.all_gather(got, torch.from_numpy(part))
    folded = O.allreduce_fold(np.stack([g.numpy() for g in got]))
    full = O.fp8_gemv(w, sc, x, bn=128, bk=128)
    rel = float(np.linalg.norm(folded - full) / np.linalg.norm(full))
    # --- lm_head: vocab slices that cut a 128-row scale block, gathered logits, argmax
    vocab = 16 * 26 * world                        # shard of 416 rows: not a multiple of 128
    wv, sv = synth.fp8_weight(rng, vocab, 256)
    xv = F.bf16_bits_to_f32(synth.activations_bf16(rng, 1, 256))
    v0, vl = sh.slice_of(vocab)
    wvl = shard_weight(wv, (vocab, 256), WShard.Rows(v0, vl), align=16)
    svl, row0, _ = shard_scale(sv, sv.shape, WShard.Rows(v0, vl), block=(128, 128))
    lg = O.fp8_gemv(wvl, np.ascontiguousarray(svl), xv, bn=128, bk=128, row0=row0)
    parts = [torch.zeros(1, vl) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(lg))
    gathered = O.allgather(np.stack([p.numpy()[0] for p in parts]))
    lfull = O.fp8_gemv(wv, sv, xv, bn=128, bk=128)[0]
    # --- MoE: experts by id
    E, top_k = 8 * world, 3
    w2, s2 = synth.fp4_experts(rng, E, 64, 256)
    ids, rw = synth.routes(rng, 2, E, top_k)
    h = F.bf16_bits_to_f32(F.f32_to_bf16_bits(rng.standard_normal((2 * top_k, 256)).astype(np.float32)))
    e0, el = sh.slice_of(E)
    pm = O.moe_down_combine(w2[e0:e0 + el], s2[e0:e0 + el], e0, h, ids, rw)
    pms = [torch.zeros(2, 64) for _ in range(world)]
    dist.all_gather(pms, torch.from_numpy(pm))
    mfold = O.allreduce_fold(np.stack([t.numpy() for t in pms]))
    mfull = O.moe_down_combine(w2, s2, 0, h, ids, rw)
    q.put((rank, folded.tobytes(), rel, bool(np.array_equal(gathered.view(np.uint32), lfull.view(np.uint32))),
           O.argmax(gathered) == O.argmax(lfull), mfold.tobytes(),
           float(np.linalg.norm(mfold - mfull) / np.linalg.norm(mfull))))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_ranks_agree_and_match_unsharded(world, oracle):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world + (os.getpid() % 200)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in res:
        assert r[1] == res[0][1], "o_proj fold differs across ranks"
        assert r[5] == res[0][5], "MoE fold differs across ranks"
        assert r[2] < 1e-5 and r[6] < 1e-5
        assert r[3] and r[4]
