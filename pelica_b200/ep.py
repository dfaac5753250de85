"""Expert parallelism for layers whose experts exceed one GPU.

Expert e lives on rank e // (E / W). Router weights, selection bias and the shared
expert are replicated; tokens are data-parallel: every rank routes its own tokens,
sends each (token, expert) pair's activation row to the rank that owns the expert
(all-to-all-v), runs its local experts over the rows it received, sends the outputs
back (all-to-all-v) and combines them in k order with its shared-expert output.

The closest thing in the reference is the bridge RUN op: activations and per-expert
(token, weight) rows out, outputs back (src/bridge.rs:412-466, host side
src/ds4.rs:1527-1552,1695-1713). Here the transport is `torch.distributed`
(NCCL over NVLink on GPUs, gloo in the CPU tests), the compute is the C-ABI library.

Pairs leave in dispatch-plan order (ascending expert, then ascending token), so the
rows for one destination rank are contiguous and the returned outputs ARE the
plan-ordered pair outputs `pm_combine` takes: no permutation on the way back.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

try:  # plumbing only: device memory views and the process group
    import torch
    import torch.distributed as dist
except ImportError:  # pragma: no cover
    torch = None
    dist = None


class CudaBackend:
    """The local compute of one rank: a MoeLayer holding experts [first, first+n_local)."""

    def __init__(self, layer):
        self.layer = layer
        self.desc = layer.desc
        self.lib = layer.lib
        self._plan_bufs = {}  # (T, K, device) -> the dispatch plan's output tensors, reused across calls

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def route(self, x):
        T, K = x.shape[0], self.desc.top_k
        ids = torch.empty((T, K), dtype=torch.int32, device=x.device)
        w = torch.empty((T, K), dtype=torch.float32, device=x.device)
        if T:
            self._check(self.lib.pm_route(self.layer.h, self._p(x), T, self._p(ids), self._p(w)))
        return ids, w

    def plan(self, ids):
        from . import PlanOut

        T, K = ids.shape
        E = self.desc.n_exp
        dev = ids.device
        out = self._plan_bufs.get((T, K, dev))
        if out is None:
            out = dict(n_active=torch.zeros(1, dtype=torch.int32, device=dev),
                       active=torch.zeros(E, dtype=torch.int32, device=dev),
                       offset=torch.zeros(E, dtype=torch.int32, device=dev),
                       count=torch.zeros(E, dtype=torch.int32, device=dev),
                       pair_token=torch.zeros(max(T * K, 1), dtype=torch.int32, device=dev),
                       pair_pos=torch.zeros(max(T * K, 1), dtype=torch.int32, device=dev))
            self._plan_bufs[(T, K, dev)] = out
        po = PlanOut(*[out[k].data_ptr() for k in ("n_active", "active", "offset", "count", "pair_token", "pair_pos")])
        self._check(self.lib.pm_plan(self.layer.h, self._p(ids), T, C.byref(po)))
        return out["pair_token"][:T * K], out["pair_pos"][:T * K]

    def experts_rows(self, x_rows, eids, w):
        R = x_rows.shape[0]
        out = torch.empty_like(x_rows)
        if R:
            self._check(self.lib.pm_experts_rows(self.layer.h, self._p(x_rows), R, self._p(eids), self._p(w),
                                                 self._p(out)))
        return out

    def shared(self, x):
        if not self.desc.shared or x.shape[0] == 0:
            return None
        out = torch.empty_like(x)
        self._check(self.lib.pm_shared(self.layer.h, self._p(x), x.shape[0], self._p(out)))
        return out

    def combine(self, pair_out, ids, w, shared, into=None):
        T = ids.shape[0]
        y = into if into is not None else torch.empty((T, self.desc.d), dtype=torch.float32, device=ids.device)
        if T:
            self._check(self.lib.pm_combine(self.layer.h, self._p(pair_out), self._p(ids), self._p(w),
                                            self._p(shared) if shared is not None else None, T, self._p(y),
                                            1 if into is not None else 0))
        return y

    def rmsnorm(self, x, eps=1e-6):
        out = torch.empty_like(x)
        if x.shape[0]:
            self._check(self.lib.pm_rmsnorm(self.layer.ctx.h, self._p(x), x.shape[0], x.shape[1], eps, self._p(out)))
        return out

    def _check(self, rc):
        from . import _check

        _check(rc)


class ExpertParallelLayer:
    """One MoE layer sharded by expert over the ranks of a process group."""

    def __init__(self, backend, n_exp: int, group=None, validate: bool = True):
        self.be = backend
        self.validate = validate  # host check of the received expert ids (two small device reads per call)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_exp % self.world:
            raise ValueError(f"{n_exp} experts do not split over {self.world} ranks")
        self.n_exp = n_exp
        self.per_rank = n_exp // self.world
        self.last_stats = {}

    def owner(self, e):
        return e // self.per_rank

    def _a2a(self, send, send_counts, recv_counts):
        """all-to-all-v of rows (dim 0)."""
        out = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        if self.world == 1:
            out.copy_(send)
            return out
        dist.all_to_all_single(out, send.contiguous(), output_split_sizes=list(recv_counts),
                               input_split_sizes=list(send_counts), group=self.group)
        return out

    def forward(self, x, add_into=None):
        """x [T_local, d] f32 (this rank's tokens, already normed) -> y [T_local, d];
        with add_into (a [T_local, d] tensor, the residual) the result is added into it."""
        be, W = self.be, self.world
        T = x.shape[0]
        ids, w = be.route(x)
        K = ids.shape[1]
        P = T * K
        pair_token, pair_pos = be.plan(ids)
        pos = pair_pos.long()
        # per pair, in plan order: its expert and (the bits of) its routing weight, side by side
        # so that they travel in one exchange
        pair_ew = torch.empty((P, 2), dtype=torch.int32, device=x.device)
        pair_ew[pos] = torch.stack((ids.reshape(-1).to(torch.int32), w.reshape(-1).view(torch.int32)), dim=1)
        pair_e = pair_ew[:, 0]
        # plan order is ascending expert, so each destination's pairs are contiguous
        send_counts = torch.bincount(pair_e.long() // self.per_rank, minlength=W).to(torch.int64)
        if W > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts = send_counts.clone()
        sc, rc = send_counts.tolist(), recv_counts.tolist()  # one small host read per layer call
        send_x = x.index_select(0, pair_token.long())
        recv_x = self._a2a(send_x, sc, rc)
        recv_ew = self._a2a(pair_ew, sc, rc)
        recv_e = recv_ew[:, 0].contiguous()
        recv_w = recv_ew[:, 1].contiguous().view(torch.float32)
        lo = self.rank * self.per_rank
        if self.validate and recv_e.numel() and (int(recv_e.min()) < lo or int(recv_e.max()) >= lo + self.per_rank):
            raise RuntimeError(f"rank {self.rank}: received a pair for an expert outside [{lo}, {lo + self.per_rank})")
        out_rows = be.experts_rows(recv_x, recv_e, recv_w)
        pair_out = self._a2a(out_rows, rc, sc)  # back: plan order of the sender
        shared = be.shared(x)
        y = be.combine(pair_out, ids, w, shared, add_into) if add_into is not None else be.combine(pair_out, ids, w, shared)
        self.last_stats = {"pairs_sent": int(P), "rows_served": int(sum(rc)),
                           "bytes_dispatched": int(P) * x.shape[1] * 4}
        return y
