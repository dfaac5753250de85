#!/usr/bin/env python
"""Benchmark of the MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--layers L] [--tokens T] [--no-cpu] [--no-ep]

Default workload (`c2_decode`): the Qwen3-30B-A3B-shaped 48-layer MoE stack, decode at batch 1
(hidden 2048, 128 experts, softmax top-8 renormalised, ff 768, gate/up Q4_K, down Q6_K,
synthetic N(0,0.02) weights generated on the device, residual add + RMS norm between
layers). A step is one token through all layers.

`value`  : tokens/s with the token's activation already in HBM (CUDA events on the
           library's stream).
`e2e`    : tokens/s through the C-ABI call with pinned HOST buffers: host->device copy of
           the activation and device->host read of the result inside the timed region.
`ep`     : (default workload, every N) the sharded path on the same ranks: the
           DeepSeek-V3-shaped expert-parallel layer subset, 4096-token prefill through
           pm_moe_forward_ep (NCCL dispatch and combine inside the library).
At N>1 every rank runs its own replica of the default stack on its own tokens (the path
shards by token with no data-path collective at these shapes); the value is the aggregate.

Other workloads: c2_prefill, c1_decode, c1_prefill, c3_decode, c3_prefill, c5_sweep (one
Zipf-routed layer over 1..8192 tokens), c4_prefill_ep, c4_decode64_ep, c4_decode1_ep
(expert-parallel, run under torchrun for N>1).

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from pelica_b200 import synth  # noqa: E402

SEED = 0xC0FFEE

# Libraries below (the collective library for one) may print to standard output; the one JSON
# line is the only thing this program may write there. Everything else goes to standard error.
_REAL_STDOUT = os.dup(1)
os.dup2(2, 1)


def emit(line: dict):
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return {"hbm_gbs": j["hbm_gbs"], "bf16_tflops": j["bf16_tflops"],
                "bf16_tflops_sustained": j.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


WORKLOADS = {
    # name: (config key, tokens per step, description)
    "c2_decode": ("c2", 1, "Qwen3-30B-A3B-shaped 48-layer MoE stack, decode batch 1"),
    "c2_prefill": ("c2", 512, "Qwen3-30B-A3B-shaped 48-layer MoE stack, 512-token prefill"),
    "c1_decode": ("c1", 1, "OLMoE-1B-7B-shaped single MoE layer, decode batch 1"),
    "c1_prefill": ("c1", 64, "OLMoE-1B-7B-shaped single MoE layer, 64-token prefill"),
    "c3_decode": ("c3", 1, "gpt-oss-20b-shaped 24-layer MoE stack, decode batch 1"),
    "c3_prefill": ("c3", 2048, "gpt-oss-20b-shaped 24-layer MoE stack, 2048-token prefill"),
    "c5_sweep": ("c5", 512, "Qwen3-30B-A3B-shaped single layer, Zipf(1.2) routing, token batch swept 1..8192"),
    # expert-parallel: experts sharded over the ranks, NCCL dispatch/combine inside the library
    "c4_prefill_ep": ("c4", 4096, "DeepSeek-V3-shaped expert-parallel MoE (layer subset), 4096-token prefill"),
    "c4_decode64_ep": ("c4", 64, "DeepSeek-V3-shaped expert-parallel MoE (layer subset), decode batch 64"),
    "c4_decode1_ep": ("c4", 1, "DeepSeek-V3-shaped expert-parallel MoE (layer subset), decode batch 1"),
}
# workloads whose dominant kernels are bound by the tensor pipe (the rest: HBM)
TENSOR_BOUND = {"c3_prefill", "c4_prefill_ep"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs (read-only)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.rows = []
        self.first = 0
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def begin(self):
        """The timed region starts here: earlier samples (warm-up) are dropped."""
        self.first = len(self.rows)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows[self.first:]:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local, dist


def share_bytes(dist, rank, local, payload, n):
    """rank 0's `payload` (n bytes) on every rank (torch.distributed as plumbing)."""
    if dist is None:
        return payload
    import torch

    t = torch.zeros(n, dtype=torch.uint8, device=f"cuda:{local}")
    if rank == 0:
        t.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(t, 0)
    return bytes(t.cpu().numpy().tobytes())


def max_over_ranks(dist, local, values):
    if dist is None:
        return list(values)
    import torch

    t = torch.tensor(list(values), device=f"cuda:{local}", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


# ---------------------------------------------------------------------------
# the sharded path: expert parallelism through pm_moe_forward_ep
# ---------------------------------------------------------------------------
def ep_measure(pb, ctx, dist, world, rank, local, cfg, n_layers, T, steps, warmup):
    """T tokens (split over the ranks) through n_layers expert-parallel layers per step:
    x += moe(rmsnorm(x)) per layer. Returns the record rank 0 reports."""
    import ctypes as C

    per = cfg.n_exp // world
    uid = share_bytes(dist, rank, local, pb.ep_unique_id() if rank == 0 else b"", 128)
    ep = pb.ExpertParallel(ctx, uid, rank, world)
    layers = []
    for l in range(n_layers):
        ly = pb.MoeLayer(ctx, cfg.scaled(first_local_expert=rank * per, n_exp_local=per))
        # the replicated parts (router, biases, shared expert) come out identical on every rank:
        # they are seeded by the layer only; the experts by (layer, first local expert)
        ly.fill_synthetic(SEED + 7919 * l, cfg.sigma, 0.0, cfg.select_bias_sigma)
        layers.append(ly)
    Tl = T * (rank + 1) // world - T * rank // world
    d = cfg.d
    POOL = 4
    rng = np.random.default_rng(SEED + rank)
    host_pool = [rng.normal(0, 1, (max(Tl, 1), d)).astype(np.float32) for _ in range(POOL)]
    pool = [ctx.alloc(max(Tl, 1) * d * 4).upload(h) for h in host_pool]
    xb = ctx.alloc(max(Tl, 1) * d * 4)
    xn = ctx.alloc(max(Tl, 1) * d * 4)
    lib = ctx.lib

    def step(src):
        pb._check(lib.pm_copy(ctx.h, xb.ptr, src, max(Tl, 1) * d * 4))
        for ly in layers:
            if Tl:
                pb._check(lib.pm_rmsnorm(ctx.h, xb.ptr, Tl, d, C.c_float(1e-6), xn.ptr))
            ep.forward_dev(ly, xn, Tl, xb, accumulate=True)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    for i in range(warmup):
        step(pool[i % POOL].ptr)
    barrier()
    launches0 = ctx.launches
    ctx.timer_start()
    for i in range(steps):
        step(pool[(warmup + i) % POOL].ptr)
    ms = ctx.timer_stop() / steps
    barrier()
    launches = (ctx.launches - launches0) / steps
    stats = ep.last_stats()
    # the experts one step touches (for the byte side of the roofline): the use counters around one step,
    # every rank's tokens together
    u0 = [ly.usage().astype(np.int64) for ly in layers]
    ctx.profile(True)
    step(pool[0].ptr)
    phases = {k: v[0] for k, v in ctx.profile_read().items() if v[1]}
    ctx.profile(False)
    hit = np.stack([(ly.usage().astype(np.int64) - u) > 0 for ly, u in zip(layers, u0)]).astype(np.float64)
    if dist is not None:
        import torch

        t = torch.tensor(hit, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        hit = t.cpu().numpy()
    distinct = int(hit.sum())  # (layer, expert) pairs read in a step
    # end to end: host tokens in, host result out, every step
    hxs = []  # the tokens of the device-resident run, in pinned memory: the same routing
    for h in host_pool:
        p = ctx.pinned((max(Tl, 1), d))
        p[:] = h
        hxs.append(p)
    hy = ctx.pinned((max(Tl, 1), d))
    barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        step(hxs[(warmup + i) % POOL].ctypes.data)
        pb._check(lib.pm_copy(ctx.h, hy.ctypes.data, xb.ptr, max(Tl, 1) * d * 4))
    e2e_ms = (time.perf_counter() - t0) / steps * 1e3
    barrier()
    ms, e2e_ms = max_over_ranks(dist, local, [ms, e2e_ms])
    pk = peaks()
    pairs = T * cfg.top_k
    flops = 2 * 3 * d * cfg.ff * (pairs + T * (1 if cfg.shared else 0)) * n_layers
    exch = phases.get("fused", 0.0)
    # bytes a step must read: the experts hit once each, and on every rank the replicated router and
    # shared expert, plus the activations in and out
    shared_bytes = cfg.scaled(ff=cfg.shared_ff, has_expert_bias=0).expert_bytes() if cfg.shared else 0
    step_bytes = distinct * cfg.expert_bytes() + n_layers * world * (shared_bytes + cfg.n_exp * d * 4) + 2 * T * d * 4 * n_layers
    tensor_roof = {"bound": "tensor", "unit": "TFLOP/s", "achieved": flops / (ms * 1e-3) / 1e12 / world,
                   "peak": pk["bf16_tflops_sustained"],
                   "peak_source": pk["source"] + " (bf16 dense sustained; the kernels run int8)",
                   "frac": flops / (ms * 1e-3) / 1e12 / world / pk["bf16_tflops_sustained"], "per": "GPU",
                   "kernel": "k_tc (tcgen05 int8 grouped expert products)"}
    hbm_roof = {"bound": "hbm", "unit": "GB/s", "achieved": step_bytes / (ms * 1e-3) / 1e9 / world, "peak": pk["hbm_gbs"],
                "peak_source": pk["source"], "frac": step_bytes / (ms * 1e-3) / 1e9 / world / pk["hbm_gbs"], "per": "GPU",
                "bytes_per_step": step_bytes, "experts_read_per_step": distinct,
                "kernel": "whole step (expert products dominate)"}
    # few tokens per expert: the step is bound by reading the experts it touches; many: by the products
    few = T * cfg.top_k < 32 * cfg.n_exp
    rec = {
        "workload": f"DeepSeek-V3-shaped expert-parallel MoE, {n_layers} of {cfg.n_layers} layers, {T} tokens per step",
        "tokens_per_s": T / (ms / 1e3), "ms_per_step": ms, "n_gpus": world, "experts_per_gpu": per,
        "tokens_per_step": T, "layers": n_layers,
        "e2e": {"value": T / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": T * d * 4, "d2h_bytes_per_step": T * d * 4},
        "gpu_launches_per_step_rank0": launches,
        "rank0_phases_ms_per_step": phases,
        "rank0_exchange_ms_per_step": exch, "rank0_kernel_ms_per_step": sum(phases.values()) - exch,
        "rank0_wire_bytes_per_layer": {"sent": stats["bytes_sent"], "received": stats["bytes_received"],
                                       "rows_sent": stats["rows_sent"], "rows_received": stats["rows_received"]},
        "roofline": dict(hbm_roof if few else tensor_roof, other_bound=tensor_roof if few else hbm_roof),
        "tokens_per_s_full_model": T / (ms / 1e3) * n_layers / cfg.n_layers,
        "scaling": "strong",
    }
    for b in pool + [xb, xn]:
        b.free()
    ep.close()
    for ly in layers:
        ly.close()
    return rec


def run_ep(args, cfg, n_layers, T, desc):
    """The expert-parallel workloads as the bench's own line."""
    world, rank, local, dist = dist_setup()
    import pelica_b200 as pb

    ctx = pb.Context(local)
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
        clocks.begin()
    rec = ep_measure(pb, ctx, dist, world, rank, local, cfg, n_layers, T, args.steps, args.warmup)
    clk = clocks.stop() if rank == 0 else None
    if rank == 0:
        line = {
            "metric": "moe_tokens_per_s", "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 x u4 -> i32 (tcgen05 kind::i8), f32 scales",
            "data": "synthetic",
            "config": {"workload": desc, "tokens_per_step": T, "layers": n_layers, "of_layers": cfg.n_layers,
                       "hidden": cfg.d, "experts": cfg.n_exp, "experts_per_gpu": rec["experts_per_gpu"],
                       "top_k": cfg.top_k, "ff": cfg.ff, "parallelism": f"ep{world}", "seed": SEED,
                       "l2": f"inputs larger than L2: {rec['experts_per_gpu'] * cfg.expert_bytes() * n_layers / 1e9:.1f} GB "
                             "of experts per GPU"},
            "e2e": rec["e2e"], "gpu_launches": int(rec["gpu_launches_per_step_rank0"] * args.steps), "clocks": clk,
            "roofline": dict(rec["roofline"], traffic=None),
            "ep": {k: rec[k] for k in ("rank0_phases_ms_per_step", "rank0_exchange_ms_per_step", "rank0_kernel_ms_per_step",
                                       "rank0_wire_bytes_per_layer", "tokens_per_s_full_model")},
        }
        emit(line)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# the reference arm and the CPU baseline: the oracle's restatement of the reference's CPU path
# ---------------------------------------------------------------------------
def cpu_sample(cfg, weights_per_layer, xs, threads):
    """The reference's CPU path (restated, AVX-512 VNNI, threaded as the reference threads
    it) on a bounded sample: the given layers x the given tokens, one token at a time
    (decode). Returns seconds per (token, layer)."""
    from oracle import pelica_oracle as po

    layers = [po.Layer(po.LayerDesc(**cfg.desc_fields()), W) for W in weights_per_layer]
    layers[0].forward_fast(xs[:1], threads)  # warm-up
    t0 = time.perf_counter()
    n = 0
    for x in xs:
        h = x[None, :].copy()
        for L in layers:
            xn = po.rmsnorm(h, 1e-6)
            h = h + L.forward_fast(xn, threads)
            n += 1
    return (time.perf_counter() - t0) / n, h


def weight_gbs(cfg, n_layers, tok_s, T):
    """GB/s of expert + router bytes the CPU path streams at `tok_s` (decode: top_k experts a token)."""
    per_layer = min(cfg.n_exp, T * cfg.top_k) * cfg.expert_bytes() + cfg.n_exp * cfg.d * 4
    return per_layer * n_layers * (tok_s / T) / 1e9


def run_reference(args, cfg, n_layers, T, desc):
    """--impl reference: the reference's CPU implementation of the path (the oracle's
    restatement of its fast path; the Rust original cannot be built here) on host cores."""
    # rank 0 alone runs and prints this arm; the other ranks leave without work (no process group:
    # nothing here uses a GPU)
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import pelica_oracle as po

    threads = os.cpu_count() or 1
    sample_layers = min(2, n_layers)
    Ws = [synth.make_weights(cfg, SEED + l) for l in range(sample_layers)]
    layers = [po.Layer(po.LayerDesc(**cfg.desc_fields()), W) for W in Ws]
    rng = np.random.default_rng(SEED)
    tok = max(1, T)

    def step():
        x = rng.normal(0, 1, (tok, cfg.d)).astype(np.float32)
        for L in layers:
            x = x + L.forward_fast(po.rmsnorm(x, 1e-6), threads)
        return x

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    # a step here = sample_layers of n_layers layers: scale to the whole stack
    ms_full = dt * 1e3 * n_layers / sample_layers
    value = tok / (ms_full / 1e3)
    line = {
        "impl": "reference", "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x u4/u6 -> i32, f32 scales", "data": "synthetic",
        "config": {"workload": desc, "tokens_per_step": tok, "layers": n_layers, "hidden": cfg.d, "experts": cfg.n_exp,
                   "top_k": cfg.top_k, "ff": cfg.ff, "parallelism": "host cores", "seed": SEED},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "weight_gb_per_s": weight_gbs(cfg, n_layers, value, tok),
                         "sample": f"{sample_layers} of {n_layers} layers per step (numpy-encoded weights), "
                                   f"time scaled x{n_layers / sample_layers:g}; AVX-512 VNNI={bool(po.lib().po_have_vnni())}"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def algorithmic_bytes_per_step(cfg, n_layers, T, distinct_experts_per_layer):
    """Bytes one step must move: the distinct experts hit (gate+up+down blocks, biases), the
    router, the shared expert, and the activations in and out, per layer."""
    per_layer = distinct_experts_per_layer * cfg.expert_bytes() + cfg.n_exp * cfg.d * 4 + 2 * T * cfg.d * 4
    if cfg.shared:
        sh = cfg.scaled(ff=cfg.shared_ff, has_expert_bias=0)
        per_layer += sh.expert_bytes()
    return per_layer * n_layers


# dram__bytes_read + dram__bytes_write of k_decode_mega in an ncu capture of a 4-layer launch
# (profiles/k_decode_mega_c2_decode.md), per layer
NCU_DRAM_BYTES_PER_LAYER_C2_DECODE = (102226688 + 4401152) // 4


def run_sweep(args, cfg, desc):
    """C5: one Zipf-routed layer, the token batch swept; which kernel family served each size."""
    import pelica_b200 as pb

    ctx = pb.Context(0)
    ly = pb.MoeLayer(ctx, cfg).fill_synthetic(SEED, cfg.sigma, 0.0, 0.0)
    router = np.empty((cfg.n_exp, cfg.d), np.float32)
    pb._check(ly.lib.pm_layer_get_router(ly.h, router.ctypes.data, None, None))
    # (strength 0.6: the pair counts' log-log slope over the 64 most popular experts comes out at -1.2
    # under top-8 selection of N(0, 0.9) logits; 8 experts are pushed to never win)
    bias = synth.zipf_router_bias(cfg.n_exp, 3, s=1.2, dead=8, strength=0.6)
    pb._check(ly.lib.pm_layer_set_router(ly.h, router.ctypes.data, synth.F32, bias.ctypes.data, None))
    st = pb.Stack(ctx, [ly])
    pk = peaks()
    out = []
    for T in (1, 8, 64, 512, 4096, 8192):
        x = synth.make_activations(T, cfg.d, 11 + T)
        ids, _ = ly.route(x)
        distinct = int(len(np.unique(ids)))
        counts = np.bincount(ids.ravel(), minlength=cfg.n_exp)
        dx = ctx.alloc(x.nbytes).upload(x)
        dy = ctx.alloc(x.nbytes)
        reps = max(3, min(200, 2000 // T))
        for _ in range(3):
            ly.forward_dev(dx, T, dy)
        ctx.sync()
        p0 = ctx.path_counts()
        l0 = ctx.launches
        ctx.timer_start()
        for _ in range(reps):
            ctx.flush_l2()  # the same layer every repetition: evict its weights between calls
            ly.forward_dev(dx, T, dy)
        ms_all = ctx.timer_stop()
        ctx.timer_start()
        for _ in range(reps):
            ctx.flush_l2()
        ms_flush = ctx.timer_stop()
        ms = (ms_all - ms_flush) / reps
        p1 = ctx.path_counts()
        byt = algorithmic_bytes_per_step(cfg, 1, T, distinct)
        flops = 2 * 3 * cfg.d * cfg.ff * T * cfg.top_k
        out.append({"tokens": T, "ms": ms, "tokens_per_s": T / (ms / 1e3), "distinct_experts": distinct,
                    "max_tokens_on_one_expert": int(counts.max()), "experts_without_tokens": int((counts == 0).sum()),
                    "kernels": {k: (p1[k] - p0[k]) // reps for k in p1 if p1[k] != p0[k]},
                    "launches": (ctx.launches - l0) // reps,
                    "hbm_frac": byt / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                    "tensor_frac": flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"]})
        dx.free()
        dy.free()
    mid = out[3]
    line = {"metric": "moe_tokens_per_s", "value": mid["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": 3, "ms_per_step": mid["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 x u4 -> i32, f32 scales", "data": "synthetic",
            "config": {"workload": desc, "value_is": "the 512-token point", "layers": 1, "hidden": cfg.d, "experts": cfg.n_exp,
                       "top_k": cfg.top_k, "ff": cfg.ff, "l2": "L2 flushed between repetitions (the flush is timed "
                       "separately and subtracted)", "seed": SEED},
            "sweep": out}
    emit(line)
    st.close()
    ly.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_decode", choices=list(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers")
    ap.add_argument("--tokens", type=int, default=0, help="override the tokens per step of a workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ep", action="store_true", help="skip the expert-parallel record of the default workload")
    args = ap.parse_args()

    key, T, desc = WORKLOADS[args.workload]
    if args.tokens:
        T, desc = args.tokens, f"{desc} [tokens per step overridden: {args.tokens}]"
    cfg = synth.CONFIGS[key]
    n_layers = args.layers or cfg.n_layers
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20  # each CPU step is a bounded sample; keep the arm within minutes
        run_reference(args, cfg, n_layers, T, desc)
        return
    if args.workload.endswith("_ep"):
        if args.steps > 50:
            args.steps = 20
        run_ep(args, cfg, args.layers or 2, T, desc)
        return
    if args.workload == "c5_sweep":
        run_sweep(args, cfg, desc)
        return
    if T > 1 and args.steps > 50:
        args.steps = 20  # prompt-sized steps take milliseconds each
    world, rank, local, dist = dist_setup()
    import pelica_b200 as pb

    ctx = pb.Context(local)
    layers = []
    for l in range(n_layers):
        ly = pb.MoeLayer(ctx, cfg)
        ly.fill_synthetic(SEED + 7919 * l + 104729 * rank, cfg.sigma, cfg.sigma if cfg.logit_bias else 0.0,
                          cfg.select_bias_sigma)
        layers.append(ly)
    stack = pb.Stack(ctx, layers, eps=1e-6)
    d = cfg.d

    # a pool of distinct inputs: consecutive steps route differently
    POOL = 64 if T == 1 else 4
    rng = np.random.default_rng(SEED + rank)
    pool = rng.normal(0, 1, (POOL, T, d)).astype(np.float32)
    dpool = [ctx.alloc(T * d * 4).upload(pool[i]) for i in range(POOL)]
    dout = ctx.alloc(T * d * 4)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    # ---- device-resident throughput ----
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()  # (nvidia-smi needs a moment before its first sample: started ahead of the warm-up)
    for i in range(args.warmup):
        stack.forward_dev(dpool[i % POOL], T, dout)
    barrier()
    launches0 = ctx.launches
    clocks.begin()
    ctx.timer_start()
    for i in range(args.steps):
        stack.forward_dev(dpool[(args.warmup + i) % POOL], T, dout)
    ms = ctx.timer_stop()
    barrier()
    launches = ctx.launches - launches0
    # a short timed region (few steps) holds no 50 ms clock sample: the same steps go on, untimed, until
    # the window from the start of the timed region is about 1.5 s, and the record says so
    extra = 0
    if ms < 1500.0 and args.steps > 0:
        extra = int(min(20000, (1500.0 - ms) / max(ms / args.steps, 1e-3)))
        for i in range(extra):
            stack.forward_dev(dpool[i % POOL], T, dout)
        barrier()
    clk = clocks.stop() if rank == 0 else None
    if clk is not None:
        clk["window"] = "the timed region" if not extra else f"the timed region and {extra} more identical steps after it (untimed)"

    # ---- per-phase timing of the same steps (roofline of the dominant kernel) ----
    ctx.profile(True)
    prof_steps = min(args.steps, 50)
    for i in range(prof_steps):
        stack.forward_dev(dpool[i % POOL], T, dout)
    phases = ctx.profile_read()
    ctx.profile(False)

    # ---- end to end through the C ABI with pinned host buffers ----
    hx = ctx.pinned((T, d))
    hy = ctx.pinned((T, d))
    for i in range(max(3, args.warmup // 4)):
        hx[:] = pool[i % POOL]
        stack.forward(hx, hy)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        np.copyto(hx, pool[(args.warmup + i) % POOL])
        stack.forward(hx, hy)
    e2e_s = time.perf_counter() - t0
    barrier()
    checksum = float(np.abs(hy).sum())

    # distinct experts per layer actually hit (decode: top_k; prefill: measured on layer 0)
    if T == 1:
        distinct = cfg.top_k
    else:
        ids, _ = layers[0].route(synth.make_activations(T, d, 1))
        distinct = len(np.unique(ids))

    ms_step, e2e_ms = max_over_ranks(dist, local, [ms / args.steps, e2e_s / args.steps * 1e3])

    # ---- the sharded path on the same ranks (default workload only) ----
    ep_rec = None
    if args.workload == "c2_decode" and not args.no_ep:
        try:
            c4 = synth.CONFIGS["c4"]
            ep_rec = ep_measure(pb, ctx, dist, world, rank, local, c4, 2, 4096, 5, 3)
        except Exception as e:  # the record is an addition: never lose the line to it
            ep_rec = {"failed": repr(e)}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk = peaks()
    value = world * T / (ms_step / 1e3)
    e2e_value = world * T / (e2e_ms / 1e3)
    bytes_step = algorithmic_bytes_per_step(cfg, n_layers, T, distinct)
    flops_step = 2 * 3 * d * cfg.ff * T * cfg.top_k * n_layers
    # the dominant phase of the step
    dom = max(phases, key=lambda k: phases[k][0])
    dom_ms, dom_spans = phases[dom]
    phases_ms = {k: v[0] / prof_steps for k, v in phases.items() if v[1]}
    if args.workload in TENSOR_BOUND:
        # the expert products (gate/up + down phases) against the sustained bf16 peak
        prod_ms = phases_ms.get("gateup", 0.0) + phases_ms.get("down", 0.0)
        ach = flops_step / (prod_ms * 1e-3) / 1e12 if prod_ms else 0.0
        roof = {"bound": "tensor", "unit": "TFLOP/s", "peak": pk["bf16_tflops_sustained"],
                "peak_source": pk["source"] + " (bf16 dense sustained)", "kernel": "gateup + down (k_tc_mx, tcgen05 bf16)",
                "achieved": ach, "frac": ach / pk["bf16_tflops_sustained"], "flops_per_step": flops_step,
                "ms_of_the_products_per_step": prod_ms, "traffic": None,
                "note": "useful flops (2 x 3 x d x ff x pairs); the kernel runs every product twice (activations "
                        "split hi + lo into two bf16 operands), so its tensor work is twice this"}
    else:
        phase_bytes = {
            "gateup": distinct * (synth.row_bytes(cfg.type_gate, d) + synth.row_bytes(cfg.type_up, d)) * cfg.ff,
            "down": distinct * synth.row_bytes(cfg.type_down, cfg.ff) * d,
            "fused": bytes_step / n_layers if phases.get("fused", (0, 0))[1] == prof_steps * n_layers else bytes_step,
        }
        roof = {"bound": "hbm", "peak": pk["hbm_gbs"], "unit": "GB/s", "peak_source": pk["source"], "kernel": dom,
                "traffic": None}
        if dom == "fused" and key == "c2":
            roof["kernel"] = "k_decode_mega (one launch per token)"
            roof["traffic"] = NCU_DRAM_BYTES_PER_LAYER_C2_DECODE * (n_layers if phases["fused"][1] != prof_steps * n_layers else 1)
            roof["traffic_source"] = "ncu capture of a 4-layer launch, scaled by layers"
        if dom in phase_bytes and dom_spans:
            per_launch_bytes = phase_bytes[dom]
            per_launch_ms = dom_ms / dom_spans
            roof["achieved"] = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9
            roof["bytes_per_launch"] = per_launch_bytes
            roof["ms_per_launch"] = per_launch_ms
        else:
            roof["achieved"] = bytes_step / (ms_step * 1e-3) / 1e9
        roof["frac"] = roof["achieved"] / roof["peak"]
    roof["whole_step"] = {"hbm_gbs": bytes_step / (ms_step * 1e-3) / 1e9,
                          "hbm_frac": bytes_step / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], "bytes_per_step": bytes_step,
                          "tflops": flops_step / (ms_step * 1e-3) / 1e12}
    roof["phases_ms_per_step"] = phases_ms
    if clk and clk.get("sm_mhz"):
        roof["ms_per_step_x_sm_mhz"] = ms_step * clk["sm_mhz"]

    line = {
        "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x u4/u6 -> i32, f32 scales" if cfg.act_quant else "f32 x mxfp4 (bf16 hi+lo on the tensor cores from 32 tokens)",
        "data": "synthetic",
        "config": {"workload": desc, "tokens_per_step": T, "layers": n_layers, "hidden": d, "experts": cfg.n_exp,
                   "top_k": cfg.top_k, "ff": cfg.ff, "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB of "
                   f"weights read per step from a {n_layers * cfg.n_exp * cfg.expert_bytes() / 1e9:.1f} GB set",
                   "parallelism": f"replicas x{world}" if world > 1 else "1 gpu", "seed": SEED},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": T * d * 4,
                "d2h_bytes_per_step": T * d * 4, "checksum": checksum},
        "gpu_launches": int(launches),
        "kernel_families": ctx.path_counts(),
        "clocks": clk,
        "roofline": roof,
    }
    if ep_rec is not None:
        line["ep"] = ep_rec

    # ---- CPU baseline on a bounded sample of the same workload (rank 0, N=1) ----
    if world == 1 and not args.no_cpu:
        try:
            from oracle import pelica_oracle as po

            threads = os.cpu_count() or 1
            sl = min(2, n_layers)
            Ws = [layers[l].get_weights() for l in range(sl)]
            ntok = 8 if T == 1 else 1
            if T == 1:
                xs = pool[:ntok, 0, :]
                sec, h_cpu = cpu_sample(cfg, Ws, xs, threads)
                cpu_tok_s = 1.0 / (sec * n_layers)
                sample = f"{ntok} tokens x {sl} of {n_layers} layers, one token at a time, scaled to {n_layers} layers"
                # the same sample on the GPU, checked against the CPU checker's exact path
                st2 = pb.Stack(ctx, layers[:sl], eps=1e-6)
                got = st2.forward(xs[-1:].copy())
                ols = [po.Layer(po.LayerDesc(**cfg.desc_fields()), W) for W in Ws]
                want = po.stack_forward(ols, 1e-6, xs[-1:].copy())
                line["parity_sample"] = {"bit_exact": bool(np.array_equal(got.view(np.uint32), want.view(np.uint32))),
                                         "max_abs_diff": float(np.abs(got - want).max())}
                st2.close()
            else:
                layers_o = [po.Layer(po.LayerDesc(**cfg.desc_fields()), W) for W in Ws]
                x = pool[0]
                layers_o[0].forward_fast(x[:8], threads)
                t0 = time.perf_counter()
                h = x
                for L in layers_o:
                    h = h + L.forward_fast(po.rmsnorm(h, 1e-6), threads)
                sec = (time.perf_counter() - t0) / sl
                cpu_tok_s = T / (sec * n_layers)
                sample = f"{T} tokens x {sl} of {n_layers} layers, scaled to {n_layers} layers"
            line["cpu_baseline"] = {"value": cpu_tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": sample, "avx512_vnni": bool(po.lib().po_have_vnni()),
                                    "weight_gb_per_s": weight_gbs(cfg, n_layers, cpu_tok_s, T)}
        except Exception as e:  # the baseline is a reported figure; never lose the GPU line to it
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {e!r}"}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
