"""Expert parallelism on GPUs: the exchange of pelica_b200.ep around the C-ABI
compute, against the unsharded layer (same bits)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal, tol_ok

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", ["c2", "c4", "c3"])
def test_single_rank_exchange_matches_forward(ctx, name):
    """World size 1: every pair is 'sent' to this rank; exercises the row-serving
    entry points (pm_experts_rows, pm_shared, pm_combine) on device pointers."""
    import torch

    from pelica_b200.ep import CudaBackend, ExpertParallelLayer

    cfg = SMALL[name]
    W = synth.make_weights(cfg, 90)
    tctx = pb.Context(0, stream=torch.cuda.current_stream().cuda_stream)
    layer = pb.MoeLayer(tctx, cfg).load(W)
    ep = ExpertParallelLayer(CudaBackend(layer), cfg.n_exp)
    x = synth.make_activations(33, cfg.d, 7)
    want = layer.forward(x)
    got = ep.forward(torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    got = got.cpu().numpy()
    if cfg.act_quant == synth.AQ_Q8X_256:
        assert bits_equal(got, want)
    else:
        assert tol_ok(got, want)
    assert ep.forward(torch.zeros((0, cfg.d), device="cuda")).shape == (0, cfg.d)
    layer.close()
    tctx.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("name", ["c2", "c4"])
def test_two_gpus_match_the_unsharded_layer(ctx, tmp_path, name):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "ep_gpu_worker.py"), name,
                                       str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o[-2000:]))
    assert all(rc == 0 for rc, _ in outs), outs
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 91)
    layer = pb.MoeLayer(ctx, cfg).load(W)
    want = layer.forward(synth.make_activations(50, cfg.d, 6))
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(2)])
    assert bits_equal(got, want)
    layer.close()


# ---- the same through the C ABI (pm_ep_*: NCCL inside the library) ----

@pytest.mark.parametrize("name", ["c2", "c4", "c3"])
@pytest.mark.parametrize("T", [0, 5, 70])
def test_c_abi_single_rank(ctx, name, T):
    """World size 1 through pm_moe_forward_ep: the whole pipeline (counts all-gather, wire
    records, the second workspace for served rows, combine) with every pair staying on the rank.
    Q8x layers: the same bits as pm_moe_forward; f32 layers: the layer tolerance (70 tokens take
    the tensor-core kernels on both sides)."""
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 92)
    layer = pb.MoeLayer(ctx, cfg).load(W)
    ep = pb.ExpertParallel(ctx, pb.ep_unique_id(), 0, 1)
    x = synth.make_activations(T, cfg.d, 8) if T else np.zeros((0, cfg.d), np.float32)
    got = ep.forward(layer, x)
    want = layer.forward(x)
    if cfg.act_quant == synth.AQ_Q8X_256:
        assert bits_equal(got, want)
    else:
        assert tol_ok(got, want)
    st = ep.last_stats()
    assert st["rows_sent"] == 0 and st["bytes_sent"] == 0  # nothing leaves a world of one
    # a layer that does not hold the rank's shard is refused
    other = pb.MoeLayer(ctx, cfg.scaled(first_local_expert=0, n_exp_local=cfg.n_exp // 2)).load(W)
    with pytest.raises(pb.PelicaError) as e:
        ep.forward(other, x)
    assert e.value.code == -1
    other.close()
    ep.close()
    layer.close()


@pytest.mark.parametrize("name", ["c2", "c4"])
def test_c_abi_two_gpus_match_the_unsharded_layer(ctx, tmp_path, name):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    T_total = 90  # 45 tokens a rank: the tensor-core kernels serve the received rows
    procs = []
    for r in range(2):
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "ep_c_worker.py"), name, str(tmp_path),
                                       str(r), "2", str(T_total)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o[-2000:]))
    assert all(rc == 0 for rc, _ in outs), outs
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 91)
    layer = pb.MoeLayer(ctx, cfg).load(W)
    want = layer.forward(synth.make_activations(T_total, cfg.d, 6))
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(2)])
    assert bits_equal(got, want)
    st = [np.load(tmp_path / f"stats{r}.npy") for r in range(2)]
    assert int(st[0][0]) == int(st[1][1]) and int(st[1][0]) == int(st[0][1])  # rows sent by one = received by the other
    assert int(st[0][0]) > 0
    # after the placement round (planned swaps plus one forced swap across the ranks): the same bits
    got2 = np.concatenate([np.load(tmp_path / f"y2_{r}.npy") for r in range(2)])
    assert bits_equal(got2, want)
    slots = [np.load(tmp_path / f"slots{r}.npy") for r in range(2)]
    assert np.array_equal(slots[0], slots[1]) and sorted(slots[0]) == list(range(cfg.n_exp))
    assert not np.array_equal(slots[0], np.arange(cfg.n_exp))
    assert np.array_equal(np.load(tmp_path / "swaps0.npy"), np.load(tmp_path / "swaps1.npy"))
    layer.close()



@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_slot_table_and_swaps_on_one_rank(ctx, name):
    """Placement tables (`loc`, src/moe.rs:262-263): weights loaded slot by slot under a random
    permutation, then experts swapped in place - the outputs and the per-expert use counters are those
    of the layer that keeps expert e in slot e."""
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 93)
    E = cfg.n_exp
    ref = pb.MoeLayer(ctx, cfg).load(W)
    x = synth.make_activations(70, cfg.d, 9)
    want = ref.forward(x)
    want_usage = ref.usage()
    perm = np.random.default_rng(4).permutation(E).astype(np.int32)  # slot of expert e
    Wp = dict(W)
    for k in ("gate", "up", "down", "bias_gate", "bias_up", "bias_down"):
        if k in W:
            a = np.empty_like(np.asarray(W[k]))
            a[perm] = np.asarray(W[k])
            Wp[k] = a
    layer = pb.MoeLayer(ctx, cfg).load(Wp)
    ep = pb.ExpertParallel(ctx, pb.ep_unique_id(), 0, 1)
    ep.set_slots(layer, perm)
    check = bits_equal if cfg.act_quant == synth.AQ_Q8X_256 else tol_ok
    assert check(ep.forward(layer, x), want)
    assert np.array_equal(layer.usage(), want_usage)
    x3 = synth.make_activations(3, cfg.d, 10)  # a few tokens: the one-launch routing applies the table itself
    assert check(ep.forward(layer, x3), ref.forward(x3))
    assert np.array_equal(layer.usage(), ref.usage())
    ep.swap_experts(layer, 1, 5)
    ep.swap_experts(layer, 5, 2)
    slots = ep.get_slots(layer)
    assert sorted(slots) == list(range(E)) and slots[5] == perm[2] and slots[2] == perm[1] and slots[1] == perm[5]
    assert check(ep.forward(layer, x), want)
    with pytest.raises(pb.PelicaError) as e:
        ep.set_slots(layer, np.zeros(E, np.int32))  # not a permutation
    assert e.value.code == -1
    ep.set_slots(layer, None)  # expert e in slot e again: the weights are not there, the outputs differ
    assert not bits_equal(ep.forward(layer, x), want)
    ep.close()
    layer.close()
    ref.close()
