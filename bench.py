#!/usr/bin/env python
"""Benchmark of the MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2_decode|c2_prefill|c1_decode|c3_decode|c4_layers_decode] [--layers L]

Default workload (N=1): the Qwen3-30B-A3B-shaped 48-layer MoE stack, decode at batch 1
(hidden 2048, 128 experts, softmax top-8 renormalised, ff 768, gate/up Q4_K, down Q6_K,
synthetic N(0,0.02) weights generated on the device, residual add + RMS norm between
layers). A step is one token through all layers.

`value`  : tokens/s with the token's activation already in HBM (CUDA events on the
           library's stream).
`e2e`    : tokens/s through the C-ABI call with pinned HOST buffers: host->device copy of
           the activation and device->host read of the result inside the timed region.
At N>1 every rank runs its own replica of the stack on its own tokens (the path shards by
token with no data-path collective at these shapes); the value is the aggregate.

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
    # expert-parallel: experts sharded over the ranks, NCCL all-to-all dispatch/combine
    "c4_prefill_ep": ("c4", 4096, "DeepSeek-V3-shaped expert-parallel MoE (layer subset), 4096-token prefill"),
    "c4_decode64_ep": ("c4", 64, "DeepSeek-V3-shaped expert-parallel MoE (layer subset), decode batch 64"),
}


def run_ep(args, cfg, n_layers, T, desc):
    """Expert-parallel workloads: tokens split over the ranks, experts sharded, all-to-all
    dispatch and combine per layer; one step = T tokens through n_layers layers."""
    import torch
    import torch.distributed as dist

    import pelica_b200 as pb
    from pelica_b200.ep import CudaBackend, ExpertParallelLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = pb.Context(local, stream=torch.cuda.current_stream().cuda_stream)
    per = cfg.n_exp // world
    layers = []
    for l in range(n_layers):
        ly = pb.MoeLayer(ctx, cfg.scaled(first_local_expert=rank * per, n_exp_local=per))
        # the replicated parts (router, biases, shared expert) come out identical on every rank:
        # they are seeded by the layer only; the experts by (layer, first local expert)
        ly.fill_synthetic(SEED + 7919 * l, cfg.sigma, 0.0, cfg.select_bias_sigma)
        layers.append(ExpertParallelLayer(CudaBackend(ly), cfg.n_exp, validate=False))
    be0 = layers[0].be
    Tl = T // world
    POOL = 4
    g = torch.Generator(device="cuda").manual_seed(SEED + rank)
    pool = [torch.randn((Tl, cfg.d), generator=g, device="cuda", dtype=torch.float32) for _ in range(POOL)]

    def step(i):
        x = pool[i % POOL].clone()
        for L in layers:
            L.forward(be0.rmsnorm(x), add_into=x)
        return x

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    clocks.begin()
    launches0 = ctx.launches
    ctx.timer_start()
    for i in range(args.steps):
        step(args.warmup + i)
    ms = ctx.timer_stop() / args.steps
    barrier()
    clk = clocks.stop() if rank == 0 else None
    launches = ctx.launches - launches0
    ctx.profile(True)
    step(0)
    phases = {k: v[0] for k, v in ctx.profile_read().items() if v[1]}
    ctx.profile(False)
    # e2e: host tokens in, host result out, per step
    hx = torch.empty((Tl, cfg.d), dtype=torch.float32).pin_memory()
    hy = torch.empty((Tl, cfg.d), dtype=torch.float32).pin_memory()
    hx.copy_(pool[0].cpu())
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        x = hx.cuda(non_blocking=True)
        for L in layers:
            L.forward(be0.rmsnorm(x), add_into=x)
        hy.copy_(x, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
    barrier()
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank == 0:
        pk = peaks()
        pairs = T * cfg.top_k
        macs = 3 * cfg.d * cfg.ff * (pairs + T * (1 if cfg.shared else 0)) * n_layers  # expert products per step
        flops = 2 * macs
        line = {
            "metric": "moe_tokens_per_s", "value": T / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 x u4 -> i32 (tcgen05 kind::i8), f32 scales",
            "data": "synthetic",
            "config": {"workload": desc, "tokens_per_step": T, "layers": n_layers, "of_layers": cfg.n_layers,
                       "hidden": cfg.d, "experts": cfg.n_exp, "experts_per_gpu": per, "top_k": cfg.top_k, "ff": cfg.ff,
                       "parallelism": f"ep{world}", "seed": SEED,
                       "l2": f"inputs larger than L2: {per * cfg.expert_bytes() * n_layers / 1e9:.1f} GB of experts per GPU"},
            "e2e": {"value": T / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": Tl * cfg.d * 4 * world, "d2h_bytes_per_step": Tl * cfg.d * 4 * world},
            "gpu_launches": int(launches), "clocks": clk,
            "roofline": {"bound": "tensor", "unit": "TFLOP/s", "achieved": flops / (ms * 1e-3) / 1e12 / world,
                         "peak": pk["bf16_tflops_sustained"], "peak_source": pk["source"] + " (bf16 dense sustained; the kernel runs int8)",
                         "frac": flops / (ms * 1e-3) / 1e12 / world / pk["bf16_tflops_sustained"], "traffic": None,
                         "kernel": "k_tc (tcgen05 int8 grouped expert products)", "per": "GPU",
                         "tokens_per_s_full_model": T / (ms / 1e3) * n_layers / cfg.n_layers,
                         "phases_ms_per_step_rank0": phases},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def algorithmic_bytes_per_step(cfg, n_layers, T, distinct_experts_per_layer):
    """Bytes one step must move: the distinct experts hit (gate+up+down blocks, biases), the
    router, the shared expert, and the activations in and out, per layer."""
    per_layer = distinct_experts_per_layer * cfg.expert_bytes() + cfg.n_exp * cfg.d * 4 + 2 * T * cfg.d * 4
    if cfg.shared:
        sh = cfg.scaled(ff=cfg.shared_ff, has_expert_bias=0)
        per_layer += sh.expert_bytes()
    return per_layer * n_layers


# (102,226,176 + 3,290,880) bytes over the 4 layers of the captured launch
NCU_DRAM_BYTES_PER_LAYER_C2_DECODE = (102217472 + 3546112) // 4


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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


def dist_setup(n_gpus):
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


def cpu_sample(cfg, weights_per_layer, xs, threads):
    """The reference's CPU path (restated, AVX-512 VNNI, threaded as the reference threads
    it) on a bounded sample: the given layers x the given tokens, one token at a time
    (decode). Returns seconds per (token, layer)."""
    from oracle import pelica_oracle as po

    layers = [po.Layer(po.LayerDesc(**cfg.desc_fields()), W) for W in weights_per_layer]
    # warm-up
    layers[0].forward_fast(xs[:1], threads)
    t0 = time.perf_counter()
    n = 0
    for x in xs:
        h = x[None, :].copy()
        for L in layers:
            xn = po.rmsnorm(h, 1e-6)
            h = h + L.forward_fast(xn, threads)
            n += 1
    return (time.perf_counter() - t0) / n, h


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
    sub = cfg
    Ws = [synth.make_weights(sub, SEED + l) for l in range(sample_layers)]
    layers = [po.Layer(po.LayerDesc(**sub.desc_fields()), W) for W in Ws]
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
        "config": {"workload": desc, "tokens_per_step": tok, "layers": n_layers},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{sample_layers} of {n_layers} layers per step (numpy-encoded weights), "
                                   f"time scaled x{n_layers / sample_layers:g}; AVX-512 VNNI={bool(po.lib().po_have_vnni())}"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_decode", choices=list(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers")
    ap.add_argument("--tokens", type=int, default=0, help="override the tokens per step of a workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
        run_ep(args, cfg, args.layers or 2, T, desc)
        return
    world, rank, local, dist = dist_setup(args.gpus)
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
    POOL = 64
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
    clk = clocks.stop() if rank == 0 else None
    launches = ctx.launches - launches0

    # ---- per-phase timing of the same steps (roofline of the dominant kernel) ----
    ctx.profile(True)
    for i in range(min(args.steps, 50)):
        stack.forward_dev(dpool[i % POOL], T, dout)
    phases = ctx.profile_read()
    ctx.profile(False)
    prof_steps = min(args.steps, 50)

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

    # distinct experts per layer actually hit (decode: top_k; prefill: measured from usage)
    if T == 1:
        distinct = cfg.top_k
    else:
        ids, _ = layers[0].route(synth.make_activations(T, d, 1))
        distinct = len(np.unique(ids))

    ms_step = ms / args.steps
    if dist is not None:
        import torch

        t = torch.tensor([ms_step, e2e_s / args.steps * 1e3], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_ms = t.tolist()
    else:
        e2e_ms = e2e_s / args.steps * 1e3
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk = peaks()
    value = world * T / (ms_step / 1e3)
    e2e_value = world * T / (e2e_ms / 1e3)
    bytes_step = algorithmic_bytes_per_step(cfg, n_layers, T, distinct)
    # the dominant phase of the step
    dom = max(phases, key=lambda k: phases[k][0])
    dom_ms, dom_spans = phases[dom]
    phase_bytes = {
        "gateup": distinct * (synth.row_bytes(cfg.type_gate, d) + synth.row_bytes(cfg.type_up, d)) * cfg.ff,
        "down": distinct * synth.row_bytes(cfg.type_down, cfg.ff) * d,
        "fused": bytes_step / n_layers if phases.get("fused", (0, 0))[1] == prof_steps * n_layers else bytes_step,
    }
    roof = {"bound": "hbm", "peak": pk["hbm_gbs"], "unit": "GB/s", "peak_source": pk["source"], "kernel": dom,
            "traffic": None}
    if dom == "fused" and key == "c2":
        # dram__bytes_read + dram__bytes_write of k_decode_mega from the committed ncu summary of the
        # decode kernel (4 layers captured; the bytes grow with the layer count)
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
    roof["whole_step"] = {"achieved": bytes_step / (ms_step * 1e-3) / 1e9,
                          "frac": bytes_step / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"],
                          "bytes_per_step": bytes_step}
    roof["phases_ms_per_step"] = {k: v[0] / prof_steps for k, v in phases.items() if v[1]}

    line = {
        "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x u4/u6 -> i32, f32 scales" if cfg.act_quant else "f32 x mxfp4",
        "data": "synthetic",
        "config": {"workload": desc, "tokens_per_step": T, "layers": n_layers, "hidden": d, "experts": cfg.n_exp,
                   "top_k": cfg.top_k, "ff": cfg.ff, "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB of "
                   f"weights read per step from a {n_layers * cfg.n_exp * cfg.expert_bytes() / 1e9:.1f} GB set",
                   "parallelism": f"replicas x{world}" if world > 1 else "1 gpu", "seed": SEED},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": T * d * 4,
                "d2h_bytes_per_step": T * d * 4, "checksum": checksum},
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": roof,
    }

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
                                    "sample": sample, "avx512_vnni": bool(po.lib().po_have_vnni())}
        except Exception as e:  # the baseline is a reported figure; never lose the GPU line to it
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {e!r}"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
