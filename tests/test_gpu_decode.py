"""The persistent one-token decode kernel against the general kernels and the
oracle: same bits, at reduced and at full layer shapes."""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal, make_pair

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


def build_stack(ctx, cfg, n_layers, seed):
    layers = [pb.MoeLayer(ctx, cfg).fill_synthetic(seed + l) for l in range(n_layers)]
    return pb.Stack(ctx, layers, eps=1e-6), layers


@pytest.mark.parametrize("name,n_layers", [("c2", 3), ("c1", 2), ("c5", 4)])
def test_decode_kernel_small_shapes(ctx, oracle, name, n_layers):
    cfg = SMALL[name]
    ols, gls = [], []
    for l in range(n_layers):
        ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 60 + l)
        ols.append(ol)
        gls.append(gl)
    st = pb.Stack(ctx, gls)
    assert st.decode_kernel
    for i in range(4):  # consecutive calls reuse the exchange buffers
        x = np.random.default_rng(i).normal(0, 1, (1, cfg.d)).astype(np.float32)
        want = oracle.stack_forward(ols, 1e-6, x)
        got = st.forward(x)
        assert bits_equal(got, want), i
        st.set_mode(True)
        assert bits_equal(st.forward(x), want)
        st.set_mode(False)
    st.status()
    st.close()
    for g in gls:
        g.close()


@pytest.mark.parametrize("n_exp", [24, 128])
def test_decode_kernel_equal_logits_pick_lowest_indices(ctx, oracle, n_exp):
    """Ties: rows of the router repeated (and all-zero rows) make logits equal bit for bit;
    the pick must then go by ascending expert index, as K rounds of (max, lowest index) do.
    128 experts take the ranking's eight-keys-at-a-time path, 24 the general one."""
    cfg = synth.C2_QWEN3.scaled(d=512, ff=256, n_exp=n_exp)
    ols, gls = [], []
    for l in range(3):
        W = synth.make_weights(cfg, 300 + l)
        r = W["router"]
        if l == 0:
            r[:] = 0.0                      # every logit equal: experts 0..K-1
        elif l == 1:
            r[1::2] = r[0::2]               # pairs of equal logits
        else:
            r[n_exp // 2:] = r[: n_exp // 2]  # equal logits a quarter boundary apart
        ols.append(oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W))
        gls.append(pb.MoeLayer(ctx, cfg).load(W))
    st = pb.Stack(ctx, gls)
    assert st.decode_kernel
    for i in range(3):
        x = np.random.default_rng(40 + i).normal(0, 1, (1, cfg.d)).astype(np.float32)
        want = oracle.stack_forward(ols, 1e-6, x)
        assert bits_equal(st.forward(x), want), i
        st.set_mode(True)
        assert bits_equal(st.forward(x), want)
        st.set_mode(False)
    st.status()
    st.close()
    for g in gls:
        g.close()


@pytest.mark.parametrize("key", ["c2", "c1"])
def test_decode_kernel_full_shape(ctx, oracle, key):
    """Full layer shapes (Qwen3-30B-A3B: d 2048, 128 experts, ff 768, Q4_K/Q6_K;
    OLMoE: 64 experts, ff 1024, Q4_K), 3 layers; weights generated on the device and
    read back for the CPU checker."""
    cfg = synth.CONFIGS[key]
    st, layers = build_stack(ctx, cfg, 3, 900)
    if key == "c2":
        assert st.decode_kernel  # C1's slices (ff 1024) do not fit one SM's shared memory: general path
    x = np.random.default_rng(5).normal(0, 1, (1, cfg.d)).astype(np.float32)
    got = st.forward(x)
    st.set_mode(True)
    general = st.forward(x)
    st.set_mode(False)
    assert bits_equal(got, general)
    ols = [oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), l.get_weights()) for l in layers]
    want = oracle.stack_forward(ols, 1e-6, x)
    assert bits_equal(got, want)
    # device-resident call, many times: the result does not drift
    dx = ctx.alloc(cfg.d * 4).upload(x)
    dy = ctx.alloc(cfg.d * 4)
    for _ in range(20):
        st.forward_dev(dx, 1, dy)
    st.status()
    assert bits_equal(dy.download(np.float32, (1, cfg.d)), want)
    # usage counters saw every call
    assert int(layers[0].usage().sum()) == cfg.top_k * 22
    st.close()
    for l in layers:
        l.close()


def test_shapes_outside_the_decode_kernel_use_the_general_path(ctx, oracle):
    cfg = SMALL["c3"]  # f32 activations on MXFP4: not a decode-kernel shape
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 70)
    st = pb.Stack(ctx, [gl])
    assert not st.decode_kernel
    x = np.random.default_rng(1).normal(0, 1, (1, cfg.d)).astype(np.float32)
    got = st.forward(x)
    want = oracle.stack_forward([ol], 1e-6, x)
    from tests.helpers import tol_ok

    assert tol_ok(got, want)
    st.close()
    gl.close()
