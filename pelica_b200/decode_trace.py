"""Prints the timeline of the persistent decode kernel: every CTA stamps the global timer at 16
points of every layer (pm_stack_trace); this tool runs a Qwen3-30B-A3B-shaped stack for a few tokens
with the trace on and reports, per point, the minimum / median / maximum over the CTAs (median over
the layers), in nanoseconds after the first CTA entered the layer.

    python -m pelica_b200.decode_trace [layers]
"""
import sys

import numpy as np

import pelica_b200 as pb
from pelica_b200 import synth

POINTS = ["layer entered", "residual stream here", "router logit published", "all logits here", "scores done",
          "selection known", "first gate/up chunk landed", "warp 0's gate/up rows done", "h arrival counters seen",
          "h quantised", "down units done", "residual stream published", "h arrival flag raised",
          "warp 0 saw its h counters", "warp 0 read its first h block", "down copies issued"]


def main():
    n_layers = int(sys.argv[1]) if len(sys.argv) > 1 else 12
    cfg = synth.CONFIGS["c2"]
    ctx = pb.Context(0)
    layers = [pb.MoeLayer(ctx, cfg).fill_synthetic(100 + i) for i in range(n_layers)]
    stack = pb.Stack(ctx, layers)
    x = np.random.default_rng(0).normal(0, 1, (1, cfg.d)).astype(np.float32)
    dx, dy = ctx.alloc(cfg.d * 4).upload(x), ctx.alloc(cfg.d * 4)
    for _ in range(5):
        stack.forward_dev(dx, 1, dy)
    stack.trace(enable=True)
    for _ in range(3):
        stack.forward_dev(dx, 1, dy)
    stack.status()
    t = stack.trace().astype(np.float64)  # [CTA][layer][point]
    t[t < 1e9] = np.nan
    first = np.nanmin(t[:, :, 0], axis=0)
    rel = t[:, :, :16] - first[None, :, None]
    print(f"layer period {np.median(np.diff(first[2:])):.0f} ns")
    for i, name in enumerate(POINTS):
        a = rel[:, 2:, i]
        print(f"  {name:32s} {np.nanmedian(np.nanmin(a, axis=0)):7.0f} {np.nanmedian(np.nanmedian(a, axis=0)):7.0f} "
              f"{np.nanmedian(np.nanmax(a, axis=0)):7.0f}")
    ctx.timer_start()
    n = 50
    for _ in range(n):
        stack.forward_dev(dx, 1, dy)
    ms = ctx.timer_stop() / n
    print(f"{n_layers} layers: {ms * 1e3:.1f} us a token, {ms * 1e3 / n_layers:.2f} us a layer (the kernel variant that stamps)")


if __name__ == "__main__":
    main()
