"""Expert parallelism, host logic: two gloo ranks on the CPU (oracle compute),
checked against the unsharded layer. No GPU involved; the failure case is made on
the host (a rank that never enters the exchange)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from pelica_b200 import synth
from tests.helpers import SMALL, bits_equal

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_ranks(mode, tmp_path, world=2, timeout=240):
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "ep_worker.py"), mode, str(tmp_path)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o))
    return outs


@pytest.mark.timeout(600)
@pytest.mark.parametrize("mode", ["even", "uneven"])
def test_two_ranks_match_the_unsharded_layer(oracle, tmp_path, mode):
    outs = run_ranks(mode, tmp_path)
    assert all(rc == 0 for rc, _ in outs), outs
    cfg = SMALL["c2"]
    W = synth.make_weights(cfg, 77)
    x = synth.make_activations(22, cfg.d, 5)
    want = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W).forward(x)
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(2)])
    assert bits_equal(got, want)
    stats = [np.load(tmp_path / f"stats{r}.npy") for r in range(2)]
    # every pair sent is served exactly once somewhere
    assert sum(s[0] for s in stats) == sum(s[1] for s in stats) == 22 * cfg.top_k


@pytest.mark.timeout(600)
def test_a_rank_that_never_joins_surfaces_as_an_error(tmp_path):
    outs = run_ranks("peer_fails", tmp_path)
    assert outs[0][0] == 0, outs[0]
    err = (tmp_path / "err0.txt")
    assert err.exists(), outs  # rank 0's exchange ended with an exception instead of hanging
