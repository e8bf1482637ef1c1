"""Exchange semantics on CPU ranks (threads): rank-ordered sum, bit identity across ranks,
run-ahead over the two banks, and the fail-stop rules, all without a GPU.  Faults are made
on the host: a rank that never joins, a dropped message, a wrong sequence number."""
import numpy as np
import pytest

from oracle.exchange_sim import ExchangeOutOfSequence, ExchangeTimeout, SimGroup, run_ranks


def gate(rnd, rank, n, world):
    rng = np.random.default_rng(rnd * 100 + rank)
    v = ((rng.integers(0, 1001, n) - 500).astype(np.float32))
    v[3::7] = (np.uint32(0x6E000000) | rng.integers(0, 1 << 23, v[3::7].size).astype(np.uint32)).view(np.float32)
    v[4::7] = -(np.uint32(0x6E000000) | rng.integers(0, 1 << 23, v[4::7].size).astype(np.uint32)).view(np.float32)
    v[5::7] = (rng.integers(0, 1 << 23, v[5::7].size).astype(np.uint32)).view(np.float32)
    carrier = rank == rnd % world
    v[0] = np.finfo(np.float32).max if carrier else 1e-40
    v[1] = -np.finfo(np.float32).max if carrier else 1e-40
    return v


@pytest.mark.parametrize("tagged", [False, True])  # flags + slots, or {step, value} words
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rank_ordered_sum_and_bit_identity(oracle, world, tagged):
    n = 512
    g = SimGroup(world, n, tagged=tagged)
    for rnd in range(5):  # consecutive steps alternate banks
        ins = [gate(rnd, r, n, world) for r in range(world)]
        red = run_ranks(world, lambda r: g.allreduce(r, ins[r]))
        want = oracle.allreduce_fold(np.stack(ins))
        for r in range(world):
            assert np.array_equal(red[r].view(np.uint32), want.view(np.uint32))
        gat = run_ranks(world, lambda r: g.allgather(r, ins[r][:100]))
        for r in range(world):
            assert np.array_equal(gat[r].view(np.uint32), np.concatenate([v[:100] for v in ins]).view(np.uint32))


def test_order_matters_so_the_order_is_fixed(oracle):
    # the property crates/weightstream-transport/src/ring.rs:614-630 states: f32 addition is not
    # associative, so "same bits on every rank" needs one fixed order
    vals = [np.array([x], np.float32) for x in (1e20, 1.0, -1e20, 1.0)]
    g = SimGroup(4, 1)
    a = run_ranks(4, lambda r: g.allreduce(r, vals[r]))
    perm = [0, 2, 1, 3]
    g2 = SimGroup(4, 1)
    b = run_ranks(4, lambda r: g2.allreduce(r, vals[perm[r]]))
    assert a[0].view(np.uint32)[0] != b[0].view(np.uint32)[0]


@pytest.mark.parametrize("tagged", [False, True])
def test_run_ahead_by_one_step_is_safe(tagged):
    """A fast rank may push step s+1 while a slow rank still reads step s: the banks keep them apart."""
    import time
    world, n = 2, 64
    g = SimGroup(world, n, wait_s=2.0, tagged=tagged)
    a0, a1 = np.full(n, 1.0, np.float32), np.full(n, 2.0, np.float32)
    b0, b1 = np.full(n, 10.0, np.float32), np.full(n, 20.0, np.float32)

    def fast(_):
        x = g.allreduce(0, a0)
        y = g.allreduce(0, b0)       # runs ahead into the other bank
        return x, y

    def slow(_):
        x = g.allreduce(1, a1)
        time.sleep(0.2)
        y = g.allreduce(1, b1)
        return x, y

    out = run_ranks(2, lambda r: fast(r) if r == 0 else slow(r))
    for r in range(2):
        assert np.all(out[r][0] == 3.0) and np.all(out[r][1] == 30.0)


def test_tagged_words_many_steps_with_jitter(oracle):
    """Forty consecutive tagged-word steps with ranks sleeping at random: every step's sum is the
    rank-ordered fold of that step's inputs (no word of another step is ever taken for this one)."""
    import time
    world, n, steps = 4, 96, 40
    g = SimGroup(world, n, wait_s=5.0, tagged=True)
    ins = [[gate(s, r, n, world) for r in range(world)] for s in range(steps)]

    def body(r):
        rng = np.random.default_rng(1000 + r)
        got = []
        for s in range(steps):
            if rng.random() < 0.3:
                time.sleep(float(rng.random()) * 0.003)
            got.append(g.allreduce(r, ins[s][r]))
        return got

    out = run_ranks(world, body)
    for s in range(steps):
        want = oracle.allreduce_fold(np.stack(ins[s]))
        for r in range(world):
            assert np.array_equal(out[r][s].view(np.uint32), want.view(np.uint32)), (s, r)


@pytest.mark.parametrize("tagged", [False, True])
def test_missing_rank_times_out_fail_stop(tagged):
    g = SimGroup(4, 16, wait_s=0.05, tagged=tagged)
    out = run_ranks(4, lambda r: g.allreduce(r, np.ones(16, np.float32)), skip=[2])
    for r in (0, 1, 3):
        assert isinstance(out[r], ExchangeTimeout) and "fail-stop" in str(out[r])


@pytest.mark.parametrize("tagged", [False, True])
def test_dropped_message_times_out_only_the_receiver(tagged):
    g = SimGroup(2, 8, wait_s=0.05, tagged=tagged)
    g.drop[(0, 1)] = True
    out = run_ranks(2, lambda r: g.allreduce(r, np.ones(8, np.float32)))
    assert isinstance(out[1], ExchangeTimeout)
    assert not isinstance(out[0], Exception) and np.all(out[0] == 2.0)


@pytest.mark.parametrize("tagged", [False, True])
def test_wrong_sequence_number_aborts(tagged):
    # ring.rs:488-499: a step number from the future is a protocol error, not data
    g = SimGroup(2, 8, wait_s=0.2, tagged=tagged)
    g.seq_override[1] = 7
    out = run_ranks(2, lambda r: g.allreduce(r, np.ones(8, np.float32)))
    assert isinstance(out[0], ExchangeOutOfSequence)


def test_length_limits():
    g = SimGroup(1, 8)
    with pytest.raises(ValueError):
        g.allreduce(0, np.zeros(0, np.float32))
    with pytest.raises(ValueError):
        g.allreduce(0, np.zeros(9, np.float32))
