"""One NCCL rank of the GPU expert-parallel test (launched by tests/test_gpu_ep.py)."""
import datetime
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import pelica_b200 as pb  # noqa: E402
from pelica_b200 import synth  # noqa: E402
from pelica_b200.ep import CudaBackend, ExpertParallelLayer  # noqa: E402
from tests.helpers import SMALL  # noqa: E402


def main():
    name, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", local))
    cfg = SMALL[name]
    W = synth.make_weights(cfg, 91)
    per = cfg.n_exp // world
    ctx = pb.Context(local, stream=torch.cuda.current_stream().cuda_stream)
    layer = pb.MoeLayer(ctx, cfg.scaled(first_local_expert=rank * per, n_exp_local=per)).load(W)
    ep = ExpertParallelLayer(CudaBackend(layer), cfg.n_exp)
    T_total = 50
    x_all = synth.make_activations(T_total, cfg.d, 6)
    lo, hi = T_total * rank // world, T_total * (rank + 1) // world
    x = torch.from_numpy(x_all[lo:hi]).cuda()
    for _ in range(2):  # twice: workspaces are reused
        y = ep.forward(x)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.cpu().numpy())
    dist.barrier()
    layer.close()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
