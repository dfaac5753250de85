"""Size-independent properties of the CPU oracle: what must hold for any input, whatever the
values are. They guard the checker itself (the parity tests compare the CUDA path with it);
the same properties are asserted on the CUDA path at full widths in test_gpu_fullwidth.py."""
import numpy as np
import pytest

from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal


def _layer(oracle, name, seed=3):
    cfg = SMALL[name]
    W = synth.make_weights(cfg, seed)
    return cfg, oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_plan_is_a_stable_counting_sort(oracle, seed):
    """Every pair lands exactly once; an expert's pairs are contiguous, in ascending
    (token, k) order (src/moe_kernels.rs:1083-1129, src/ds4.rs:1461-1472); experts without
    pairs are not listed."""
    rng = np.random.default_rng(seed)
    T, K, E = 37, 4, 19
    ids = np.stack([rng.choice(E, K, replace=False) for _ in range(T)]).astype(np.uint32)
    p = oracle.plan(ids, E)
    P = T * K
    pos = np.asarray(p["pair_pos"]).reshape(-1)
    assert sorted(pos.tolist()) == list(range(P))
    na = int(p["n_active"])
    cnt = np.asarray(p["count"])[:na]
    off = np.asarray(p["offset"])[:na]
    act = np.asarray(p["active"])[:na]
    assert cnt.sum() == P and np.all(cnt > 0)
    assert np.all(np.diff(act.astype(np.int64)) > 0)
    assert off.tolist() == np.concatenate([[0], np.cumsum(cnt)[:-1]]).tolist()
    flat = ids.reshape(-1)
    for a in range(na):
        mine = np.nonzero(flat == act[a])[0]  # ascending (token, k) = ascending flat index
        assert pos[mine].tolist() == list(range(int(off[a]), int(off[a] + cnt[a])))
        assert np.asarray(p["pair_token"])[off[a]:off[a] + cnt[a]].tolist() == (mine // K).tolist()
    assert set(act.tolist()) == set(np.unique(flat).tolist())


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4"])
def test_route_is_per_token_and_picks_distinct_experts(oracle, name):
    cfg, L = _layer(oracle, name)
    x = synth.make_activations(23, cfg.d, 5)
    ids, w = L.route(x)
    assert ids.shape == (23, cfg.top_k) and w.shape == ids.shape
    for t in range(23):
        assert len(set(ids[t].tolist())) == cfg.top_k
        assert np.all(ids[t] < cfg.n_exp)
    assert np.all(np.isfinite(w))
    # one token at a time gives the same rows: routing is per token
    for t in (0, 7, 22):
        i1, w1 = L.route(x[t:t + 1])
        assert i1[0].tolist() == ids[t].tolist()
        assert bits_equal(w1[0], w[t])


@pytest.mark.parametrize("name", ["c1", "c2"])
def test_softmax_routing_ignores_a_common_logit_shift_in_its_choice(oracle, name):
    """Adding one constant to every logit of a token cannot change which experts a softmax
    router picks (the scores keep their order)."""
    cfg, L = _layer(oracle, name)
    rng = np.random.default_rng(9)
    lg = rng.standard_normal((11, cfg.n_exp)).astype(np.float32)
    ids0, _ = L.route_logits(lg)
    ids1, _ = L.route_logits((lg + np.float32(0.5)).astype(np.float32))
    # (a shift by an exact binary fraction keeps distinct logits distinct at this magnitude)
    assert ids0.tolist() == ids1.tolist()


@pytest.mark.parametrize("n", [256, 1024])
def test_q8x_blocks(oracle, n):
    """Q8x::new (src/ds4_cpu.rs:31-58): |x - d*q| <= d/2 per value, the block's largest value
    maps to +-127, the eight partial sums add up to the block sum, a zero block stays zero."""
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    x[256 - 7:256] = 0.0
    q, d, bs = oracle.q8x(x)
    q, bs = q.astype(np.int32), bs.astype(np.int64)
    nb = n // 256
    assert q.size == n and d.size == nb
    for b in range(nb):
        xb, qb = x[b * 256:(b + 1) * 256].astype(np.float64), q[b * 256:(b + 1) * 256]
        assert np.abs(qb).max() == 127
        assert np.all(np.abs(xb - float(d[b]) * qb) <= 0.5 * float(d[b]) * (1 + 1e-6))
        assert bs.reshape(nb, -1)[b].sum() == qb.sum()
    zq, zd, _ = oracle.q8x(np.zeros(256, np.float32))
    assert not zq.any()


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c6", "c10", "c11", "c12"])
def test_layer_rows_do_not_depend_on_the_batch(oracle, name):
    """A token's output row has the same bits whether it is evaluated alone or in a batch:
    every step of the path is per token, and combine adds in fixed k order
    (src/moe_kernels.rs:1798-1808). This is the layer-level form of the reference's
    multi_matches_single (src/ds4_cpu.rs:476)."""
    cfg, L = _layer(oracle, name, seed=7)
    x = synth.make_activations(6, cfg.d, 8)
    y = L.forward(x)
    for t in (0, 3, 5):
        assert bits_equal(L.forward(x[t:t + 1])[0], y[t])
    # and a permutation of the batch permutes the rows
    perm = np.array([4, 0, 5, 2, 1, 3])
    assert bits_equal(L.forward(np.ascontiguousarray(x[perm])), y[perm])


def test_combine_scales_exactly_with_a_power_of_two(oracle):
    """combine is a fixed-order sum of w * row: doubling every expert output doubles the result
    bit for bit (no rounding changes under a power-of-two scale)."""
    cfg, L = _layer(oracle, "c2", seed=4)
    x = synth.make_activations(5, cfg.d, 6)
    ids, w = L.route(x)
    p = oracle.plan(ids, cfg.n_exp)
    rng = np.random.default_rng(2)
    po_ = rng.standard_normal((ids.size, cfg.d)).astype(np.float32)
    y1 = oracle.combine(L.desc, po_, p["pair_pos"], w)
    y2 = oracle.combine(L.desc, (po_ * np.float32(2.0)).astype(np.float32), p["pair_pos"], w)
    assert bits_equal(y2, (y1 * np.float32(2.0)).astype(np.float32))


@pytest.mark.parametrize("ty", ["Q4_K", "Q6_K", "Q5_K", "Q8_0", "IQ4_NL", "IQ4_XS", "IQ3_S", "MXFP4"])
def test_dequant_is_deterministic_and_finite(oracle, ty):
    """Encoders and decoders of every block format: decoding twice gives the same bits, every
    value is finite, and the encoder's output decodes to within the format's step of its input."""
    tid = getattr(synth, ty)
    rng = np.random.default_rng(11)
    m = (rng.standard_normal((4, 512)) * 0.05).astype(np.float32)
    blocks = synth.encode_matrix(tid, m)
    a = oracle.dequant(tid, blocks, m.size)
    b = oracle.dequant(tid, blocks, m.size)
    assert bits_equal(a, b)
    assert np.all(np.isfinite(a))
    err = np.abs(a.reshape(m.shape) - m).max()
    assert err <= 0.35 * np.abs(m).max()  # 3- to 8-bit codes on a block maximum
