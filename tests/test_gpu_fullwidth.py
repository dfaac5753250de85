"""Parity at the row widths and token counts the benchmarks run, not only at the reduced
shapes: the DeepSeek-V3-shaped layer (hidden 7168, 256 experts in 8 groups of 32, shared
expert), the gpt-oss-shaped layer (hidden = intermediate = 2880: 90 MXFP4 blocks a row, not
a multiple of 256), and 4096 / 8192 tokens in ONE call on the Qwen3-shaped layer (the
reference chunks at 4096 tokens, src/ds4.rs:45; this operator must not need to).

Weights are generated on the GPU and read back for the CPU checker. Where the checker
would need minutes for every token, the whole batch is routed and planned on both sides
(bit-exact) and the layer output is compared on a seeded sample of tokens: a token's output
depends on no other token."""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import bits_equal, device_pair, tol_ok

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(1200)]


@pytest.mark.parametrize("T", [1, 64, 300])
def test_c4_full_width_layer(ctx, oracle, T):
    """d 7168 (28 blocks a gate/up row), ff 2048, routing over all 256 experts with the
    group-limited selection (8 groups, 4 kept, top-8), selection bias, shared expert on every
    token; this context holds experts 96..111 (a 16-expert shard, as one of 16 ranks would)."""
    cfg = synth.C4_DSV3.scaled(first_local_expert=96, n_exp_local=16)
    ol, gl = device_pair(oracle, pb, ctx, cfg, 4100)
    x = synth.make_activations(T, cfg.d, 4200 + T)
    ids, w = gl.route(x)
    ids_o, w_o = ol.route(x)
    assert np.array_equal(ids, ids_o) and bits_equal(w, w_o)
    # every token's picks lie in 4 of the 8 groups
    assert all(len({int(e) // 32 for e in row}) <= 4 for row in ids)
    before = ctx.path_counts()
    got = gl.forward(x)
    after = ctx.path_counts()
    if T >= 32:
        assert after["tensor"] > before["tensor"]
    assert bits_equal(got, ol.forward(x))
    gl.close()


@pytest.mark.parametrize("T", [1, 8, 300])
def test_c3_full_width_layer(ctx, oracle, T):
    """d = ff = 2880, 32 experts, top-4 with softmax over the picks, router bias, expert
    biases, the gpt-oss GLU; f32 activations: tolerance 1e-3 relative + 1e-4 of the RMS."""
    cfg = synth.C3_GPTOSS
    ol, gl = device_pair(oracle, pb, ctx, cfg, 4300)
    x = synth.make_activations(T, cfg.d, 4400 + T)
    ids, w = gl.route(x)
    ids_o, w_o = ol.route(x)
    assert np.array_equal(ids, ids_o) and bits_equal(w, w_o)
    before = ctx.path_counts()
    got = gl.forward(x)
    after = ctx.path_counts()
    if T >= 32:  # 90 blocks a row: 45 K chunks of the bf16 tensor-core kernel
        assert after["tensor"] - before["tensor"] >= 2
    want = ol.forward(x)
    assert tol_ok(got, want), float(np.abs(got - want).max())
    gl.close()


@pytest.mark.parametrize("T", [4096, 8192])
def test_many_tokens_in_one_call(ctx, oracle, T):
    cfg = synth.C2_QWEN3
    ol, gl = device_pair(oracle, pb, ctx, cfg, 4500)
    x = synth.make_activations(T, cfg.d, 4600)
    ids, w = gl.route(x)
    ids_o, w_o = ol.route(x)
    assert np.array_equal(ids, ids_o) and bits_equal(w, w_o)
    plan = gl.plan(ids)
    plan_o = oracle.plan(ids, cfg.n_exp)
    for k in ("n_active", "active", "offset", "count", "pair_token", "pair_pos"):
        assert np.array_equal(plan[k], plan_o[k]), k
    got = gl.forward(x)
    pick = np.sort(np.random.default_rng(T).choice(T, 40, replace=False))
    pick[0], pick[-1] = 0, T - 1
    want = ol.forward(x[pick])
    assert bits_equal(got[pick], want)
    # usage counters of the one call: every pair counted once
    assert int(gl.usage().sum()) == T * cfg.top_k
    gl.close()
