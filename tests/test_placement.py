"""The host-side planner of usage-driven expert placement (pm_placement_*; the reference's `Adapt`,
src/moe.rs:246-278,1965-2069): decayed scores, the margin against going back and forth, the byte
budget, and what a round does to the ranks' loads. No GPU work."""
import numpy as np
import pytest

import pelica_b200 as pb


def _loads(pl):
    return pl.scores(0)[1]


def test_scores_decay_as_the_reference(tmp_path):
    pl = pb.Placement(2, 8, 2)
    u = np.array([10, 0, 0, 0, 0, 0, 0, 3], np.uint32)
    pl.observe(1, u)
    pl.observe(1, u + np.array([4, 0, 0, 0, 0, 0, 0, 0], np.uint32))  # counters are cumulative
    s, r = pl.scores(1)
    assert s[0] == np.float32(np.float32(10.0) * np.float32(0.944) + np.float32(4.0))
    assert s[7] == np.float32(np.float32(3.0) * np.float32(0.944))
    assert r[0] == s[0] and r[1] == s[7]
    assert not pl.scores(0)[0].any()  # the other layer saw nothing
    # a wrapped counter still gives the increase (u32 arithmetic, src/moe.rs:1978)
    pl2 = pb.Placement(1, 2, 1)
    pl2.observe(0, np.array([0xFFFFFFF0, 0], np.uint32))
    pl2.observe(0, np.array([0x00000010, 0], np.uint32))
    assert pl2.scores(0)[0][0] == np.float32(np.float32(0xFFFFFFF0) * np.float32(0.944) + np.float32(32.0))
    pl.close()
    pl2.close()


def test_a_round_evens_out_the_ranks():
    E, W = 32, 4
    rng = np.random.default_rng(0)
    usage = (1000.0 / np.arange(1, E + 1) ** 1.2).astype(np.uint32)  # Zipf: rank 0 holds the hot experts
    pl = pb.Placement(1, E, W)
    pl.observe(0, usage)
    before = _loads(pl)
    swaps = pl.plan(expert_bytes=1 << 20, budget_bytes=1 << 30)
    after = _loads(pl)
    assert swaps and after.max() < before.max() and after.max() - after.min() < before.max() - before.min()
    assert abs(after.sum() - before.sum()) < 1e-2 * before.sum()
    slots = pl.slots(0)
    assert sorted(slots) == list(range(E))
    # every swap cleared the reference's margin, hot against cold
    s = pl.scores(0)[0]
    for _, hot, cold in swaps:
        assert s[hot] >= s[cold] * 1.25 + 1.5
    # the same scores again: nothing goes back and forth
    assert pl.plan(1 << 20, 1 << 30) == [] or _loads(pl).max() <= after.max()
    again = pl.plan(1 << 20, 1 << 30)
    assert len(again) <= len(swaps)
    pl.close()
    del rng


def test_budget_margin_and_single_rank():
    E, W = 16, 2
    usage = np.zeros(E, np.uint32)
    usage[:8] = 100  # rank 0 serves everything
    pl = pb.Placement(1, E, W)
    pl.observe(0, usage)
    assert pl.plan(expert_bytes=1 << 20, budget_bytes=(1 << 20)) == []          # not even one swap fits
    three = pl.plan(expert_bytes=1 << 20, budget_bytes=6 * (1 << 20))           # 2 * expert_bytes a swap
    assert len(three) == 3
    assert len(pl.plan(1 << 20, 1 << 30, max_swaps=1)) == 1
    pl.close()
    # near-equal use: inside the margin, nothing moves
    flat = pb.Placement(1, E, W)
    u = np.full(E, 40, np.uint32)
    u[0] = 48
    flat.observe(0, u)
    assert flat.plan(1 << 20, 1 << 30) == []
    flat.close()
    one = pb.Placement(1, E, 1)
    one.observe(0, usage)
    assert one.plan(1 << 20, 1 << 30) == []
    one.close()
    with pytest.raises(pb.PelicaError):
        pb.Placement(1, 10, 4)  # experts do not split over the ranks
