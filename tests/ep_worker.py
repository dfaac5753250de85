"""Worker for the CPU expert-parallel tests: one gloo rank. The local compute is
the CPU oracle (test infrastructure), the exchange logic is pelica_b200.ep's."""
import datetime
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from oracle import pelica_oracle as po  # noqa: E402
from pelica_b200 import synth  # noqa: E402
from pelica_b200.ep import ExpertParallelLayer  # noqa: E402
from tests.helpers import SMALL  # noqa: E402


class OracleBackend:
    """The five local operations of the exchange, on the CPU checker."""

    def __init__(self, cfg, W, first, n_local):
        self.cfg = cfg
        local = cfg.scaled(first_local_expert=first, n_exp_local=n_local)
        self.full = po.Layer(po.LayerDesc(**cfg.desc_fields()), W)
        self.rows = po.Layer(po.LayerDesc(**local.scaled(top_k=1).desc_fields()), W)
        self.desc = self.full.desc

    def route(self, x):
        ids, w = self.full.route(x.numpy()) if x.shape[0] else (np.zeros((0, self.cfg.top_k), np.uint32),
                                                                np.zeros((0, self.cfg.top_k), np.float32))
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

    def plan(self, ids):
        p = po.plan(ids.numpy().astype(np.uint32), self.cfg.n_exp)
        return torch.from_numpy(p["pair_token"].astype(np.int32)), torch.from_numpy(p["pair_pos"].astype(np.int32))

    def experts_rows(self, x_rows, eids, w):
        if x_rows.shape[0] == 0:
            return x_rows.clone()
        e = eids.numpy().astype(np.uint32).reshape(-1, 1)
        out = self.rows.experts(x_rows.numpy(), e, w.numpy().reshape(-1, 1))  # in plan order
        pos = po.plan(e, self.cfg.n_exp)["pair_pos"]
        return torch.from_numpy(np.ascontiguousarray(out[pos]))

    def shared(self, x):
        return None

    def combine(self, pair_out, ids, w, shared):
        T = ids.shape[0]
        if T == 0:
            return torch.zeros((0, self.cfg.d))
        p = po.plan(ids.numpy().astype(np.uint32), self.cfg.n_exp)
        return torch.from_numpy(po.combine(self.desc, pair_out.numpy(), p["pair_pos"], w.numpy()))


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "peer_fails" and rank == 1:
        # a rank that never joins the exchange: made on the host, no device involved
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
        sys.exit(0)
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8 if mode == "peer_fails" else 120))
    cfg = SMALL["c2"]
    W = synth.make_weights(cfg, 77)
    per = cfg.n_exp // world
    be = OracleBackend(cfg, W, rank * per, per)
    ep = ExpertParallelLayer(be, cfg.n_exp)
    T_total = 22
    x_all = synth.make_activations(T_total, cfg.d, 5)
    if mode == "uneven":
        bounds = [0, T_total] if world == 1 else [0] + [T_total] * world  # rank 0 owns every token
    else:
        bounds = [T_total * r // world for r in range(world + 1)]
    x = torch.from_numpy(x_all[bounds[rank]:bounds[rank + 1]])
    try:
        y = ep.forward(x)
    except Exception as e:  # the surviving rank of "peer_fails" lands here
        open(os.path.join(out_dir, f"err{rank}.txt"), "w").write(repr(e))
        sys.exit(0 if mode == "peer_fails" else 1)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    np.save(os.path.join(out_dir, f"stats{rank}.npy"), np.array([ep.last_stats["pairs_sent"], ep.last_stats["rows_served"]]))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
