"""Router logits, top-k (every gating variant, ties, group-limited selection)
and the dispatch plan: bit-exact against the oracle through the C ABI."""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import bits_equal

pytestmark = pytest.mark.gpu


def layers(oracle, ctx, cfg, seed, **extra):
    rng = np.random.default_rng(seed)
    W = {"router": rng.normal(0, cfg.sigma, (cfg.n_exp, cfg.d)).astype(np.float32)}
    if cfg.logit_bias:
        W["logit_bias"] = synth.bf16_round(rng.normal(0, cfg.sigma, cfg.n_exp).astype(np.float32))
    if cfg.select_bias_sigma:
        W["select_bias"] = rng.normal(0, cfg.select_bias_sigma, cfg.n_exp).astype(np.float32)
    W.update(extra)
    ol = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    gl = pb.MoeLayer(ctx, cfg)
    rc = gl.lib.pm_layer_set_router(gl.h, W["router"].ctypes.data, synth.F32,
                                    W["logit_bias"].ctypes.data if "logit_bias" in W else None,
                                    W["select_bias"].ctypes.data if "select_bias" in W else None)
    assert rc == 0
    return ol, gl


ROUTE_CASES = {
    "c1-softmax": synth.C1_OLMOE,
    "c2-softmax-renorm": synth.C2_QWEN3,
    "c3-selected-bias": synth.C3_GPTOSS,
    "c4-sigmoid-groups": synth.C4_DSV3.scaled(shared=0),
    "sigmoid-bias-scale": synth.C4_DSV3.scaled(n_group=0, topk_group=0, n_exp=160, shared=0),
    "sqrt-softplus": synth.C4_DSV3.scaled(gating=synth.GATE_SQRT_SOFTPLUS, n_group=0, topk_group=0, w_scale=1.5,
                                          shared=0),
    "q4x-16-of-512": synth.C2_QWEN3.scaled(gating=synth.GATE_SOFTMAX_SELECTED, n_exp=512, top_k=16, d=1024),
    "ragged-experts": synth.C2_QWEN3.scaled(n_exp=77, top_k=5, d=256),
    # a token's row beyond the 48 KB a kernel gets without asking: the few-token router stages it whole
    "wide-16384": synth.C2_QWEN3.scaled(n_exp=24, top_k=4, d=16384, ff=256),
}


@pytest.mark.parametrize("name", list(ROUTE_CASES))
def test_route_bit_exact(ctx, oracle, name):
    cfg = ROUTE_CASES[name]
    ol, gl = layers(oracle, ctx, cfg, 7)
    for T in (1, 7, 64, 257):
        x = synth.make_activations(T, cfg.d, 100 + T)
        lg_o = ol.router_logits(x)
        lg_g = gl.router_logits(x)
        assert bits_equal(lg_g, lg_o)
        ids_o, w_o = ol.route_logits(lg_o)
        ids_g, w_g = gl.route(x)
        assert np.array_equal(ids_g, ids_o)
        assert bits_equal(w_g, w_o)
    gl.close()


def test_ties_go_to_the_lower_index(ctx, oracle):
    for gating in (synth.GATE_SOFTMAX_ALL, synth.GATE_SIGMOID, synth.GATE_SOFTMAX_SELECTED):
        cfg = synth.C2_QWEN3.scaled(n_exp=100, top_k=8, d=256, gating=gating)
        ol, gl = layers(oracle, ctx, cfg, 1)
        lg = np.zeros((3, 100), np.float32)
        lg[1, [99, 64, 33, 32, 2]] = 2.0
        lg[2] = np.repeat(np.arange(25, dtype=np.float32), 4)[::-1]  # runs of 4 equal values
        ids_o, w_o = ol.route_logits(lg)
        ids_g, w_g = gl.route_logits(lg)
        assert ids_o[0].tolist() == list(range(8))
        assert ids_o[1].tolist() == [2, 32, 33, 64, 99, 0, 1, 3]
        assert np.array_equal(ids_g, ids_o) and bits_equal(w_g, w_o)
        gl.close()


def test_group_limited_ties_and_masking(ctx, oracle):
    cfg = synth.C4_DSV3.scaled(n_exp=64, n_group=8, topk_group=2, top_k=8, d=256, shared=0, select_bias_sigma=0.0)
    ol, gl = layers(oracle, ctx, cfg, 2)
    lg = np.full((2, 64), -4.0, np.float32)
    lg[0, 40:46] = 3.0       # group 5 clearly best (6 experts)
    lg[0, 8:10] = 2.0        # group 1 second (two high scores)
    lg[0, 56] = 2.5          # group 7 has one higher score but a lower top-2 sum
    # row 1: all equal -> groups 0 and 1, experts 0..7
    ids_o, w_o = ol.route_logits(lg)
    ids_g, w_g = gl.route_logits(lg)
    assert sorted(ids_o[0].tolist()) == [8, 9, 40, 41, 42, 43, 44, 45]
    assert ids_o[1].tolist() == list(range(8))
    assert np.array_equal(ids_g, ids_o) and bits_equal(w_g, w_o)
    gl.close()


@pytest.mark.parametrize("T,K,E", [(0, 8, 128), (1, 8, 128), (9, 4, 32), (300, 8, 128), (4096, 8, 256), (1000, 16, 512)])
def test_plan_bit_exact(ctx, oracle, T, K, E):
    cfg = synth.C2_QWEN3.scaled(n_exp=E, top_k=K, d=256)
    gl = pb.MoeLayer(ctx, cfg)
    rng = np.random.default_rng(T + K)
    # skewed: many experts get nothing, a few get most
    p = 1.0 / np.arange(1, E + 1) ** 1.2
    p /= p.sum()
    ids = np.stack([rng.choice(E, K, replace=False, p=p) for _ in range(T)]).astype(np.uint32) if T else \
        np.zeros((0, K), np.uint32)
    want = oracle.plan(ids, E)
    got = gl.plan(ids)
    assert got["n_active"] == want["n_active"]
    for k in ("active", "offset", "count", "pair_token", "pair_pos"):
        assert np.array_equal(got[k], want[k]), k
    # properties: ascending experts; ascending tokens inside an expert; pair_pos inverts
    na = got["n_active"]
    assert np.all(np.diff(got["active"][:na].astype(np.int64)) > 0)
    for a in range(na):
        seg = got["pair_token"][got["offset"][a]:got["offset"][a] + got["count"][a]].astype(np.int64)
        assert np.all(np.diff(seg) >= 0)
    gl.close()


def test_plan_rejects_bad_ids(ctx):
    cfg = synth.C2_QWEN3.scaled(n_exp=16, top_k=2, d=256)
    gl = pb.MoeLayer(ctx, cfg)
    with pytest.raises(pb.PelicaError):
        gl.plan(np.array([[1, 16]], np.uint32))
    gl.close()


def test_bf16_router_weights(ctx, oracle):
    """A router stored as bf16 (GLM's `router_scores`, src/forward.rs:117): the logits are the
    reference's `dot_bf16` (src/quant.rs:282-304), bit for bit, which in turn equals `dot_f32`
    over the widened values."""
    cfg = synth.C4_DSV3.scaled(n_group=0, topk_group=0, n_exp=64, d=1024, shared=0)
    rng = np.random.default_rng(17)
    r32 = synth.bf16_round(rng.normal(0, cfg.sigma, (cfg.n_exp, cfg.d)).astype(np.float32))
    bits = np.ascontiguousarray((r32.view(np.uint32) >> 16).astype(np.uint16))
    sb = rng.normal(0, cfg.select_bias_sigma, cfg.n_exp).astype(np.float32)
    gl = pb.MoeLayer(ctx, cfg)
    pb._check(gl.lib.pm_layer_set_router(gl.h, bits.ctypes.data, synth.BF16, None, sb.ctypes.data))
    ol = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), {"router": r32, "select_bias": sb})
    for T in (1, 9, 70):
        x = synth.make_activations(T, cfg.d, 500 + T)
        lg = gl.router_logits(x)
        for t in (0, T - 1):
            for e in (0, 13, cfg.n_exp - 1):
                assert np.float32(oracle.dot_bf16(bits[e], x[t])).view(np.uint32) == lg[t, e].view(np.uint32)
        assert bits_equal(lg, ol.router_logits(x))
        ids_o, w_o = ol.route(x)
        ids_g, w_g = gl.route(x)
        assert np.array_equal(ids_g, ids_o) and bits_equal(w_g, w_o)
    gl.close()


def test_width_limit(ctx):
    with pytest.raises(pb.PelicaError) as e:
        pb.MoeLayer(ctx, synth.C2_QWEN3.scaled(n_exp=8, top_k=2, d=65536, ff=256))
    assert e.value.code == -7
