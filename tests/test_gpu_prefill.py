"""The tensor-core (tcgen05 int8) expert products against the general kernels and
the oracle: same bits (the integer sums are exact, the float tail keeps block order)."""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal, make_pair

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


@pytest.mark.parametrize("name", ["c1", "c2", "c4"])
@pytest.mark.parametrize("T", [32, 77, 300])
def test_tensor_core_path_matches_oracle_and_general(ctx, oracle, name, T):
    cfg = SMALL[name]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 31)
    x = synth.make_activations(T, cfg.d, 400 + T)
    ctx.set_tensor_core_min_tokens(32)
    c0 = ctx.path_counts()
    tc = gl.forward(x)
    c1 = ctx.path_counts()
    # which kernels served the call: gate/up and down of the routed experts (and of the shared one)
    assert c1["tensor"] - c0["tensor"] >= 2 and c1["general"] == c0["general"]
    ctx.set_tensor_core_min_tokens(0)
    general = gl.forward(x)
    c2 = ctx.path_counts()
    assert c2["tensor"] == c1["tensor"] and c2["general"] - c1["general"] >= 2
    ctx.set_tensor_core_min_tokens(32)
    assert bits_equal(tc, general)
    assert bits_equal(tc, ol.forward(x))
    gl.close()


def test_tensor_core_path_skewed_routing_and_empty_experts(ctx, oracle):
    """Most tokens on a few experts (several token tiles per expert), many experts unused."""
    cfg = SMALL["c5"]
    W = synth.make_weights(cfg, 32)
    W["logit_bias"] = synth.zipf_router_bias(cfg.n_exp, 3, s=1.2, dead=8, strength=2.0)
    ol = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    gl = pb.MoeLayer(ctx, cfg).load(W)
    x = synth.make_activations(700, cfg.d, 9)
    ids, _ = gl.route(x)
    counts = np.bincount(ids.ravel(), minlength=cfg.n_exp)
    assert counts.max() > 256 and (counts == 0).sum() >= 4
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()


def test_tensor_core_path_full_width_rows(ctx, oracle):
    """Full row widths of the benchmark shapes (d 2048 -> 8 blocks, ff 1024 -> 4 blocks), few experts."""
    cfg = synth.C1_OLMOE.scaled(n_exp=8, top_k=2)
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 33)
    x = synth.make_activations(150, cfg.d, 10)
    assert bits_equal(gl.forward(x), ol.forward(x))
    gl.close()


@pytest.mark.parametrize("T", [32, 77, 300])
def test_mxfp4_tensor_core_path(ctx, oracle, T):
    """MXFP4 weights with f32 activations (the gpt-oss path) on the bf16 tensor-core kernels:
    the activations are split hi + lo into two bf16 operands, so parity is the layer tolerance
    (1e-3 relative + 1e-4 of the RMS), against the oracle and against the general f32 kernels.
    The reduced shape has ff = 160: the down products end in a chunk of a single 32-value block."""
    from tests.helpers import tol_ok

    cfg = SMALL["c3"]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 35)
    x = synth.make_activations(T, cfg.d, 700 + T)
    ctx.set_tensor_core_min_tokens(32)
    c0 = ctx.path_counts()
    tc = gl.forward(x)
    c1 = ctx.path_counts()
    assert c1["tensor"] - c0["tensor"] >= 2 and c1["general"] == c0["general"]
    ctx.set_tensor_core_min_tokens(0)
    general = gl.forward(x)
    ctx.set_tensor_core_min_tokens(32)
    want = ol.forward(x)
    assert tol_ok(general, want)
    assert tol_ok(tc, want), float(np.abs(tc - want).max())
    # the split leaves 2^-17 of each activation behind: far inside the tolerance
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    assert float(np.abs(tc.astype(np.float64) - want).max()) < 2e-4 * rms + 1e-3 * float(np.abs(want).max())
    gl.close()
