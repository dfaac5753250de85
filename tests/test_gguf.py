"""GGUF container: write -> read round trip, the MoE configuration derived from the metadata
(src/moe.rs:746-765) and, on a GPU, a layer loaded from a file against the same layer loaded
from memory."""
import os

import numpy as np
import pytest

from pelica_b200 import gguf, synth
from tests.helpers import SMALL, bits_equal


def _file(tmp_path, name, n_layers=2, **kw):
    cfg = SMALL[name]
    layers = [synth.make_weights(cfg, 50 + i) for i in range(n_layers)]
    path = os.path.join(tmp_path, f"{name}.gguf")
    gguf.write_moe_layers(path, cfg, layers, **kw)
    return cfg, layers, path


@pytest.mark.parametrize("name", ["c1", "c2", "c4", "c6", "c9", "c10"])
def test_round_trip_and_config(tmp_path, name):
    cfg, layers, path = _file(str(tmp_path), name)
    with gguf.GGUFFile(path) as g:
        assert g.version == 3 and g.arch == "qwen3moe" and g.alignment == 32
        assert all(t.offset % 32 == 0 for t in g.tensors.values())
        got = gguf.moe_config(g, 1)
        for f in ("d", "ff", "n_exp", "top_k", "norm_w", "type_gate", "type_up", "type_down", "act_quant", "shared",
                  "shared_ff"):
            assert getattr(got, f) == getattr(cfg, f), f
        assert got.gating == (synth.GATE_SIGMOID if cfg.gating == synth.GATE_SIGMOID else synth.GATE_SOFTMAX_ALL)
        for i, want in enumerate(layers):
            w = gguf.layer_weights(g, i, cfg)
            for k in ("router", "gate", "up", "down"):
                assert np.array_equal(np.asarray(w[k]).ravel(), np.asarray(want[k]).ravel()), k
            if "select_bias" in want:
                assert bits_equal(w["select_bias"], want["select_bias"])
            if cfg.shared:
                assert np.array_equal(w["shared_down"], want["shared_down"])


@pytest.mark.parametrize("name,between", [("c2", False), ("c2", True), ("c4", True), ("c9", True)])
def test_repacked_layout(tmp_path, name, between):
    """Each expert's three pieces side by side (`*_expm`, src/repack.rs:1-24): the same weights come
    back, other tensors that sat between the expert tensors are found at their new offsets, and undoing
    restores the file byte for byte."""
    cfg, layers, path = _file(str(tmp_path), name, router_between=between)
    before = open(path, "rb").read()
    assert gguf.repack(path) == 2 and gguf.repack(path) == 0
    after = open(path, "rb").read()
    assert len(after) == len(before) and after != before
    with gguf.GGUFFile(path) as g:
        assert gguf.layer_is_repacked(g, 0) and "blk.1.ffn_up_exps.weight" not in g.tensors
        assert gguf.moe_config(g, 1).type_down == cfg.type_down
        # an expert is one contiguous run of the file: gate, up, down
        t = [g.tensor(f"blk.1.{p}_expm.weight") for p in gguf.PIECES]
        lens = [i.nbytes // cfg.n_exp for i in t]
        base = min(i.offset for i in t)
        e = 3
        run = np.frombuffer(after, np.uint8, sum(lens), base + e * sum(lens))
        want = np.concatenate([np.asarray(layers[1][k][e]).ravel() for k in ("gate", "up", "down")])
        assert np.array_equal(run, want)
        for i, want in enumerate(layers):
            w = gguf.layer_weights(g, i, cfg)
            for k in ("router", "gate", "up", "down"):
                assert np.array_equal(np.asarray(w[k]).reshape(-1), np.asarray(want[k]).reshape(-1)), k
            if cfg.shared:
                assert np.array_equal(w["shared_up"], want["shared_up"])
    assert gguf.repack(path, undo=True) == 2
    assert open(path, "rb").read() == before


def test_half_repacked_layer_is_refused(tmp_path):
    cfg, _, path = _file(str(tmp_path), "c1", 1)
    data = bytearray(open(path, "rb").read())
    at = data.index(b"blk.0.ffn_up_exps.weight")
    data[at:at + 24] = b"blk.0.ffn_up_expm.weight"
    open(path, "wb").write(data)
    with gguf.GGUFFile(path) as g:
        with pytest.raises(gguf.GGUFError):
            gguf.layer_weights(g, 0, cfg)


def test_rejects_bad_files(tmp_path):
    p = os.path.join(str(tmp_path), "x.gguf")
    open(p, "wb").write(b"GGML" + b"\0" * 60)
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(p)
    cfg, _, path = _file(str(tmp_path), "c1", 1)
    data = open(path, "rb").read()
    open(p, "wb").write(data[: len(data) - 4096])  # truncated download (src/gguf.rs:385)
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(p)
    with gguf.GGUFFile(path) as g:
        with pytest.raises(gguf.GGUFError):
            g.tensor("blk.9.ffn_gate_exps.weight")


def test_oracle_layer_from_file(tmp_path, oracle):
    cfg, layers, path = _file(str(tmp_path), "c2")
    x = synth.make_activations(5, cfg.d, 77)
    with gguf.GGUFFile(path) as g:
        a = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), gguf.layer_weights(g, 1, cfg)).forward(x)
    b = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), layers[1]).forward(x)
    assert bits_equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("name,repacked", [("c2", False), ("c4", False), ("c2", True), ("c9", True)])
def test_layer_loaded_from_file(tmp_path, ctx, name, repacked):
    import pelica_b200 as pb

    cfg, layers, path = _file(str(tmp_path), name, router_between=repacked)
    if repacked:
        assert gguf.repack(path) == 2
    x = synth.make_activations(9, cfg.d, 78)
    with gguf.GGUFFile(path) as g:
        over = {k: getattr(cfg, k) for k in ("gating", "n_group", "topk_group", "w_scale", "select_bias_sigma")}
        got = gguf.load_moe_layer(ctx, g, 1, **over).forward(x)
    want = pb.MoeLayer(ctx, cfg).load(layers[1]).forward(x)
    assert bits_equal(got, want)
