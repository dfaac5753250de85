"""One rank of the expert-parallel GPU test through the C ABI (pm_ep_*); launched by
tests/test_gpu_ep.py. No framework in this process: the communicator's id travels through a file."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import pelica_b200 as pb  # noqa: E402
from pelica_b200 import synth  # noqa: E402
from tests.helpers import SMALL  # noqa: E402


def main():
    name, out_dir, rank, world, T_total = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5])
    idf = os.path.join(out_dir, "ep_id.bin")
    if rank == 0:
        uid = pb.ep_unique_id()
        with open(idf + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(idf + ".tmp", idf)
    else:
        t0 = time.time()
        while not os.path.exists(idf):
            if time.time() - t0 > 120:
                raise SystemExit("no communicator id after 120 s")
            time.sleep(0.05)
        uid = open(idf, "rb").read()
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 91)
    per = cfg.n_exp // world
    ctx = pb.Context(rank)
    layer = pb.MoeLayer(ctx, cfg.scaled(first_local_expert=rank * per, n_exp_local=per)).load(W)
    ep = pb.ExpertParallel(ctx, uid, rank, world)
    ep.set_timeout_ms(120000)
    x_all = synth.make_activations(T_total, cfg.d, 6)
    lo, hi = T_total * rank // world, T_total * (rank + 1) // world
    for _ in range(2):  # twice: workspaces are reused
        y = ep.forward(layer, x_all[lo:hi])
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y)
    np.save(os.path.join(out_dir, f"stats{rank}.npy"), np.array(list(ep.last_stats().values()), np.uint64))
    # a round of usage-driven placement: every rank plans from the same counters (the use of all the
    # ranks' tokens; the router is replicated), carries out the same swaps, and the outputs do not change
    ids, _ = layer.route(x_all)
    usage = np.bincount(ids.ravel(), minlength=cfg.n_exp).astype(np.uint32)
    pl = pb.Placement(1, cfg.n_exp, world)
    pl.observe(0, usage)
    swaps = pl.plan(cfg.expert_bytes(), 1 << 30)
    for _, a, b in swaps:
        ep.swap_experts(layer, a, b)
    assert np.array_equal(ep.get_slots(layer), pl.slots(0))
    ep.swap_experts(layer, 0, cfg.n_exp - 1)  # and one swap the planner did not ask for, across the ranks
    y2 = ep.forward(layer, x_all[lo:hi])
    np.save(os.path.join(out_dir, f"y2_{rank}.npy"), y2)
    np.save(os.path.join(out_dir, f"swaps{rank}.npy"), np.array(swaps, np.int32).reshape(-1, 3))
    np.save(os.path.join(out_dir, f"slots{rank}.npy"), ep.get_slots(layer))
    pl.close()
    ep.close()
    layer.close()
    ctx.close()


if __name__ == "__main__":
    main()
