"""Failure behaviour on the GPU, without a fault: a bounded device-side wait is made to run
out (a short limit against an event that cannot arrive), the kernel returns, the host
reports the error, and the same context keeps working. Also: expert ids in device buffers
are range-checked on the device, and a layer (re)loaded after its stack was created is seen."""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal, make_pair

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


def test_decode_kernel_wait_runs_out_and_the_stack_falls_back(ctx, oracle):
    cfg = SMALL["c2"]
    ols, gls = [], []
    for l in range(3):
        ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 800 + l)
        ols.append(ol)
        gls.append(gl)
    st = pb.Stack(ctx, gls)
    assert st.decode_kernel
    x = np.random.default_rng(1).normal(0, 1, (1, cfg.d)).astype(np.float32)
    want = oracle.stack_forward(ols, 1e-6, x)
    assert bits_equal(st.forward(x), want)
    ctx.set_wait_limit_ns(200_000)  # 0.2 ms
    st.fault_next_call()
    with pytest.raises(pb.PelicaError) as e:
        st.forward(x)
    assert e.value.code == -6
    with pytest.raises(pb.PelicaError) as e:
        st.status()
    assert e.value.code == -6
    ctx.set_wait_limit_ns(2_000_000_000)
    assert not st.decode_kernel          # the general kernels from now on ...
    assert bits_equal(st.forward(x), want)  # ... with the same bits
    st.close()
    # the GPU and the context are intact: a new stack runs the decode kernel again
    st2 = pb.Stack(ctx, gls)
    assert st2.decode_kernel
    n0 = ctx.path_counts()["decode"]
    assert bits_equal(st2.forward(x), want)
    assert ctx.path_counts()["decode"] == n0 + 1
    st2.status()
    st2.close()
    for g in gls:
        g.close()


def test_tensor_core_wait_runs_out_and_the_next_call_is_clean(ctx, oracle):
    cfg = SMALL["c2"]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 810)
    x = synth.make_activations(96, cfg.d, 811)
    want = ol.forward(x)
    ctx.set_tensor_core_min_tokens(32)
    assert bits_equal(gl.forward(x), want)
    ctx.set_wait_limit_ns(200_000)
    ctx.tc_fault_block(1)  # the products of block 1 are never issued nor signalled
    with pytest.raises(pb.PelicaError) as e:
        gl.forward(x)
    assert e.value.code == -6
    ctx.tc_fault_block(-1)
    ctx.set_wait_limit_ns(2_000_000_000)
    # tensor memory and the barrier were released: the same call now succeeds, same bits
    n0 = ctx.path_counts()["tensor"]
    assert bits_equal(gl.forward(x), want)
    assert ctx.path_counts()["tensor"] > n0
    gl.close()


def test_expert_ids_in_device_buffers_are_range_checked(ctx, oracle):
    cfg = SMALL["c2"]
    ol, gl, _ = make_pair(oracle, pb, ctx, cfg, 820)
    T, K = 9, cfg.top_k
    x = synth.make_activations(T, cfg.d, 821)
    ids, w = gl.route(x)
    pair_out = ol.experts(x, ids, w)
    bad = ids.copy()
    bad[3, 2] = cfg.n_exp + 5
    bad[7, 0] = 0xFFFFFFF0
    # host ids: refused before anything is launched
    with pytest.raises(pb.PelicaError) as e:
        gl.combine(pair_out, bad, w)
    assert e.value.code == -1
    # device ids: the plan kernels leave the pairs out and flag the call
    dbad = ctx.alloc(bad.nbytes).upload(bad)
    E = cfg.n_exp
    r = dict(n_active=np.zeros(1, np.int32), active=np.zeros(E, np.uint32), offset=np.zeros(E, np.uint32),
             count=np.zeros(E, np.uint32), pair_token=np.zeros(T * K, np.uint32), pair_pos=np.zeros(T * K, np.uint32))
    po_ = pb.PlanOut(*[r[k].ctypes.data for k in ("n_active", "active", "offset", "count", "pair_token", "pair_pos")])
    import ctypes

    assert gl.lib.pm_plan(gl.h, dbad.ptr, T, ctypes.byref(po_)) == -1
    assert int(r["count"].sum()) == T * K - 2           # the two bad pairs are in no expert's list
    assert (r["pair_pos"].reshape(T, K)[[3, 7], [2, 0]] == 0xFFFFFFFF).all()
    dx = ctx.alloc(x.nbytes).upload(x)
    dw = ctx.alloc(w.nbytes).upload(w)
    out = np.zeros((T * K, cfg.d), np.float32)
    assert gl.lib.pm_experts(gl.h, dx.ptr, T, dbad.ptr, dw.ptr, out.ctypes.data) == -1
    assert b"outside the layer" in gl.lib.pm_last_error()
    # the context is intact and the error does not stick
    assert bits_equal(gl.forward(x), ol.forward(x))
    ctx.sync()
    for b in (dbad, dx, dw):
        b.free()
    gl.close()


def test_router_set_after_stack_creation_is_seen(ctx, oracle):
    """A selection bias is only allocated when it is first set: a stack created before that
    must not keep routing without it (decode kernel and recorded graphs alike)."""
    cfg = SMALL["c2"].scaled(select_bias_sigma=0.5)
    W = synth.make_weights(cfg, 830)
    Wn = dict(W)
    sb = Wn.pop("select_bias")
    gl = pb.MoeLayer(ctx, cfg).load(Wn)          # no selection bias yet
    st = pb.Stack(ctx, [gl, gl])
    x = np.random.default_rng(2).normal(0, 1, (1, cfg.d)).astype(np.float32)
    ol0 = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), Wn)
    assert bits_equal(st.forward(x), oracle.stack_forward([ol0, ol0], 1e-6, x))
    router = np.ascontiguousarray(W["router"], np.float32)
    pb._check(gl.lib.pm_layer_set_router(gl.h, router.ctypes.data, synth.F32, None, sb.ctypes.data))
    ol1 = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    want = oracle.stack_forward([ol1, ol1], 1e-6, x)
    assert not bits_equal(want, oracle.stack_forward([ol0, ol0], 1e-6, x))  # the bias changes the picks
    assert bits_equal(st.forward(x), want)       # decode kernel
    st.set_mode(True)
    for _ in range(3):                           # general kernels, recorded as a graph on the way
        assert bits_equal(st.forward(x), want)
    st.close()
    gl.close()
