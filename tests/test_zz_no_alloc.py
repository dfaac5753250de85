"""pm_route_noalloc, the routing entry point for hosts that cannot let the library
allocate (all device memory in their own pool, latency-critical loops, fixed
memory budgets): it keeps its scratch in a fixed array inside the library.

Checked through the C ABI against pm_route (same bits), on two calls in a row so
that what the first call left in the shared scratch cannot leak into the second.
Collected last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth

pytestmark = pytest.mark.gpu


def _layer(ctx, cfg, seed):
    rng = np.random.default_rng(seed)
    router = rng.normal(0, cfg.sigma, (cfg.n_exp, cfg.d)).astype(np.float32)
    sel = rng.normal(0, 0.01, cfg.n_exp).astype(np.float32) if cfg.select_bias_sigma else None
    ly = pb.MoeLayer(ctx, cfg)
    pb._check(ly.lib.pm_layer_set_router(ly.h, router.ctypes.data, synth.F32, None,
                                         sel.ctypes.data if sel is not None else None))
    return ly


@pytest.mark.parametrize("cfg", [synth.C2_QWEN3, synth.C4_DSV3.scaled(shared=0)], ids=["softmax", "sigmoid-groups"])
def test_route_noalloc_matches_route_twice(ctx, cfg):
    ly = _layer(ctx, cfg, 3)
    K = cfg.top_k
    # second call: fewer tokens and different data, so stale logits of the first would show
    for T, seed in ((256, 10), (37, 11)):
        x = synth.make_activations(T, cfg.d, seed)
        want_ids, want_w = ly.route(x)
        dx = ctx.alloc(x.nbytes).upload(x)
        dids = ctx.alloc(T * K * 4)
        dw = ctx.alloc(T * K * 4)
        free0 = ctx.device_free_bytes()
        ly.route_noalloc(dx, T, dids, dw)
        ctx.sync()
        free1 = ctx.device_free_bytes()
        # nothing was allocated (or freed) by the call: the device's free memory is unchanged
        assert free0 == free1
        got_ids = dids.download(np.uint32, (T, K))
        got_w = dw.download(np.float32, (T, K))
        assert np.array_equal(got_ids, want_ids)
        assert np.array_equal(got_w.view(np.uint32), want_w.view(np.uint32))
        for b in (dx, dids, dw):
            b.free()
    ly.close()


def test_route_noalloc_refuses_what_it_cannot_do(ctx):
    cfg = synth.C2_QWEN3
    ly = _layer(ctx, cfg, 4)
    T = 257  # one more than the fixed scratch holds
    dx = ctx.alloc(T * cfg.d * 4)
    dids = ctx.alloc(T * cfg.top_k * 4)
    dw = ctx.alloc(T * cfg.top_k * 4)
    with pytest.raises(pb.PelicaError) as e:
        ly.route_noalloc(dx, T, dids, dw)
    assert e.value.code == -7 and "256" in str(e.value)
    # host pointers would need staging memory: refused, not silently allocated
    x = np.zeros((1, cfg.d), np.float32)
    rc = ly.lib.pm_route_noalloc(ly.h, x.ctypes.data, 1, dids.ptr, dw.ptr)
    assert rc == -1
    for b in (dx, dids, dw):
        b.free()
    ly.close()
