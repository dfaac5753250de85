"""The expert products, the combine and whole layers against the oracle
(through the C ABI): bit-exact where the path is integer + ordered float
(Q8x activations), within the stated tolerance for f32 activations."""
import os

import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal, make_pair, tol_ok

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def check(cfg, got, want):
    if cfg.act_quant == synth.AQ_Q8X_256:
        assert bits_equal(got, want), np.abs(got - want).max()
    else:
        assert tol_ok(got, want), np.abs(got - want).max()


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("T", [1, 7, 8, 9, 64])
def test_layer_forward(ctx, oracle, name, T):
    cfg = SMALL[name]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 21)
    x = synth.make_activations(T, cfg.d, 300 + T)
    check(cfg, gl.forward(x), ol.forward(x))
    gl.close()


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_split_steps(ctx, oracle, name):
    cfg = SMALL[name]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 22)
    T = 19
    x = synth.make_activations(T, cfg.d, 5)
    ids, w = gl.route(x)
    ids_o, w_o = ol.route(x)
    assert np.array_equal(ids, ids_o) and bits_equal(w, w_o)
    po_out = ol.experts(x, ids, w)
    pg_out = gl.experts(x, ids, w)
    check(cfg, pg_out, po_out)
    plan = oracle.plan(ids, cfg.n_exp)
    y_o = oracle.combine(ol.desc, po_out, plan["pair_pos"], w)
    y_g = gl.combine(po_out, ids, w)
    assert bits_equal(y_g, y_o)
    # accumulate into an existing residual
    base = synth.make_activations(T, cfg.d, 6)
    y_o2 = oracle.combine(ol.desc, po_out, plan["pair_pos"], w, y=base.copy())
    y_g2 = gl.combine(po_out, ids, w, y=base.copy())
    assert bits_equal(y_g2, y_o2)
    gl.close()


def test_empty_batch_and_limits(ctx, oracle):
    cfg = SMALL["c2"]
    _, gl, _ = make_pair(oracle, pb, ctx, cfg, 23)
    y = gl.forward(np.zeros((0, cfg.d), np.float32))
    assert y.shape == (0, cfg.d)
    with pytest.raises(pb.PelicaError):
        gl.lib.pm_moe_forward  # noqa: B018
        pb._check(gl.lib.pm_moe_forward(gl.h, None, 1 << 20, None, 0))
    gl.close()
    # a layer without weights refuses to run
    g2 = pb.MoeLayer(ctx, cfg)
    with pytest.raises(pb.PelicaError):
        g2.forward(np.zeros((1, cfg.d), np.float32))
    g2.close()
    with pytest.raises(pb.PelicaError):
        pb.MoeLayer(ctx, cfg.scaled(d=300))


def test_zero_and_extreme_activations(ctx, oracle):
    cfg = SMALL["c2"]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 24)
    x = synth.make_activations(6, cfg.d, 9)
    x[1] = 0.0                      # all-zero token: d = 0 blocks
    x[2, :256] = 0.0                # one zero block
    x[3] *= 1e4
    x[4] *= 1e-6
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()


def test_clamped_swiglu_and_in_combine_fold(ctx, oracle):
    cfg = SMALL["c2"].scaled(act=synth.ACT_SILU_CLAMP, act_limit=0.05, weight_fold=synth.FOLD_IN_COMBINE)
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 25)
    x = synth.make_activations(11, cfg.d, 10) * 3
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()


def test_f32_activations_on_k_quants(ctx, oracle):
    """The generic engine's arithmetic (f32 activations x dequantised weights,
    src/moe_kernels.rs:1170-1229) on Q4_K / Q6_K experts."""
    cfg = SMALL["c2"].scaled(act_quant=synth.AQ_F32, weight_fold=synth.FOLD_IN_COMBINE)
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 26)
    x = synth.make_activations(5, cfg.d, 11)
    assert tol_ok(gl.forward(x), ol.forward(x))
    gl.close()


def test_sigmoid_gated_shared_expert(ctx, oracle):
    cfg = SMALL["c4"].scaled(shared=synth.SHARED_SIGMOID_GATED)
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 27)
    x = synth.make_activations(5, cfg.d, 12)
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()


def test_expert_parallel_shards_sum_to_the_whole(ctx, oracle):
    """Two contexts' worth of local experts: each shard returns the outputs of
    the experts it holds (zeros elsewhere); pair outputs add up to the full layer's."""
    cfg = SMALL["c2"]
    W = synth.make_weights(cfg, 28)
    full = pb.MoeLayer(ctx, cfg).load(W)
    half = cfg.n_exp // 2
    shards = [pb.MoeLayer(ctx, cfg.scaled(first_local_expert=f, n_exp_local=half)).load(W) for f in (0, half)]
    x = synth.make_activations(13, cfg.d, 13)
    ids, w = full.route(x)
    whole = full.experts(x, ids, w)
    parts = [s.experts(x, ids, w) for s in shards]
    assert bits_equal(parts[0] + parts[1], whole)
    assert np.all((parts[0] == 0) | (parts[1] == 0))
    for l in [full, *shards]:
        l.close()


def test_usage_counters(ctx, oracle):
    cfg = SMALL["c2"]
    _, gl, _ = make_pair(oracle, pb, ctx, cfg, 29)
    x = synth.make_activations(40, cfg.d, 14)
    ids, _ = gl.route(x)
    gl.forward(x)
    gl.forward(x)
    want = 2 * np.bincount(ids.ravel(), minlength=cfg.n_exp)
    assert np.array_equal(gl.usage(), want)
    gl.close()


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c6", "c9", "c10", "c11", "c12"])
def test_golden_fixtures(ctx, name):
    """The committed vectors (tests/golden), no oracle involved."""
    from tests.golden.make_golden import case

    g = np.load(os.path.join(GOLDEN, f"layer_{name}.npz"))
    cfg, W, x = case(name)
    gl = pb.MoeLayer(ctx, cfg).load(W)
    ids, w = gl.route(x)
    assert np.array_equal(ids, g["ids"]) and bits_equal(w, g["w"])
    check(cfg, gl.forward(x), g["y"])
    gl.close()


def test_stack_matches_oracle(ctx, oracle):
    cfg = SMALL["c2"]
    n_layers = 3
    ols, gls = [], []
    for l in range(n_layers):
        ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 40 + l)
        ols.append(ol)
        gls.append(gl)
    st = pb.Stack(ctx, gls, eps=1e-6)
    for T in (1, 5):
        x = np.random.default_rng(T).normal(0, 1, (T, cfg.d)).astype(np.float32)
        want = oracle.stack_forward(ols, 1e-6, x)
        got = st.forward(x)
        assert bits_equal(got, want)
    st.close()
    for g in gls:
        g.close()


def test_synthetic_fill_round_trips_through_the_oracle(ctx, oracle):
    """Weights generated on the device, read back as GGUF bytes, give the same
    layer output on the CPU checker."""
    for name in ("c2", "c3", "c4"):
        cfg = SMALL[name]
        gl = pb.MoeLayer(ctx, cfg).fill_synthetic(77, 0.02, 0.02 if cfg.logit_bias else 0.0, cfg.select_bias_sigma)
        W = gl.get_weights()
        ol = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
        x = synth.make_activations(4, cfg.d, 15)
        check(cfg, gl.forward(x), ol.forward(x))
        # the generated weights look like N(0, 0.02)
        deq = oracle.dequant(cfg.type_gate, W["gate"][0], cfg.ff * cfg.d)
        assert 0.015 < deq.std() < 0.025 and abs(deq.mean()) < 2e-3
        gl.close()


@pytest.mark.parametrize("T", [1, 9, 40])
def test_q4k_with_32_block_activations_has_the_oracle_bits(ctx, oracle, T):
    """The labelled second activation mode (Q4_K rows against 32-value int8 blocks with an f16
    scale): integer sums and an ordered float tail, so the bits are the oracle's."""
    cfg = SMALL["c12"]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 31)
    x = synth.make_activations(T, cfg.d, 400 + T)
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()
