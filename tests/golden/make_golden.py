"""Writes the golden fixtures of tests/golden/ from the CPU oracle.

The reference (Rust + WGSL) cannot be built or imported where this repository
is built and its tests store no expected numbers for this path, so these
fixtures freeze the oracle's own outputs on seeded inputs: they pin the oracle
against drift and give the CUDA path fixed vectors to hit.

    python -m tests.golden.make_golden [names ...]     (default: every fixture)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from pelica_b200 import synth  # noqa: E402

SHAPES = {
    "c1": synth.C1_OLMOE.scaled(d=256, ff=256, n_exp=8, top_k=2),
    "c2": synth.C2_QWEN3.scaled(d=256, ff=256, n_exp=12, top_k=4),
    "c3": synth.C3_GPTOSS.scaled(d=96, ff=64, n_exp=6, top_k=2),
    "c4": synth.C4_DSV3.scaled(d=256, ff=256, n_exp=16, top_k=4, n_group=4, topk_group=2, shared_ff=256),
    "c6": synth.C6_Q8_0.scaled(d=160, ff=96, n_exp=8, top_k=2),
    "c9": synth.C9_IQ3S.scaled(d=256, ff=96, n_exp=8, top_k=2),
    "c10": synth.C10_Q5K.scaled(d=256, ff=256, n_exp=8, top_k=2),
    "c11": synth.C11_GLM.scaled(d=256, ff=128, n_exp=8, top_k=2, shared_ff=128),
    "c12": synth.C12_Q4K_Q8_0.scaled(d=256, ff=256, n_exp=8, top_k=2),
}


def case(name):
    cfg = SHAPES[name]
    seed = {"c1": 101, "c2": 102, "c3": 103, "c4": 104, "c6": 106, "c9": 109, "c10": 110, "c11": 111, "c12": 112}[name]
    W = synth.make_weights(cfg, seed)
    x = synth.make_activations(5, cfg.d, seed + 1000)
    return cfg, W, x


def main():
    from oracle import pelica_oracle as po

    for name in (sys.argv[1:] or SHAPES):
        cfg, W, x = case(name)
        L = po.Layer(po.LayerDesc(**cfg.desc_fields()), W)
        ids, w = L.route(x)
        y = L.forward(x)
        np.savez_compressed(os.path.join(HERE, f"layer_{name}.npz"), ids=ids, w=w, y=y)
        print(name, ids[0], y[0, :3])


if __name__ == "__main__":
    main()
