#!/usr/bin/env python
"""Benchmark of the DiT-MoE sparse MoE block (the hot path of DICE) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--variant gelu_tanh|swiglu] [--layers L]

One *step* is one pass of a batch of tokens through the MoE blocks of all
``L`` layers of the model (28 for DiT-XL/2), each layer with its own weights.
``value`` is tokens per second through one MoE block, summed over all GPUs:
``n_gpus * tokens_per_gpu * L / step_time``.

* N = 1: the single-GPU DiT-XL/2 configuration (batch 32 x 2 CFG, 256 tokens
  per image = 16384 tokens, hidden 1152, 8 experts, top-2).
* N > 1 (under torchrun): the expert-parallel configuration (8 experts sharded
  over the ranks, per-GPU batch 16 x 2 CFG = 8192 tokens, synchronous
  all-to-all dispatch/combine); per-GPU work is fixed ("weak" scaling).

Inputs are synthetic (seeded Gaussian activations, N(0, 0.02) weights).  The
expert shape follows the benchmark configuration's wording by default
(``--variant gelu_tanh``: fc1, GELU-tanh, fc2, renormalised top-2 weights, no
shared expert); ``--variant swiglu`` measures the block exactly as the
reference computes it (SwiGLU experts, un-normalised weights, shared expert).

``--impl reference`` times the CPU restatement of the reference path (the
oracle) on the host cores, on a bounded sample of the same workload.

Beyond the contract's keys the line carries: ``roofline`` (grouped GEMM, from
CUDA events around the FFN launches inside the timed region), ``roofline_hbm``
(router, row gather and combine kernels timed on per-layer inputs, against the
measured copy bandwidth), ``gpu_reference`` (the reference's algorithm in stock
PyTorch CUDA operations on the same GPUs: a comparator, not the product),
``variants`` (N = 1: the reference-true SwiGLU block next to the GELU-tanh
one), ``ep_parity`` and ``load`` (N > 1: the expert-parallel layer 0 against an
unsharded block with the same weights on the rank's own tokens; rows per rank
and per expert), ``phases_us_per_layer`` (N > 1) and ``host_us_per_layer``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HIDDEN = 1152
EXPERTS = 8
MLP_RATIO = 4
TOKENS_PER_IMAGE = 256
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one grouped-GEMM launch of this workload,
# scaled from the ncu capture summarised under profiles/ (None until a capture exists)
GEMM_TRAFFIC_BYTES = 452.8e6  # mean of fc1 (417.4 MB) and fc2 (488.3 MB) of the ncu capture summarised under profiles/


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", default="gelu_tanh", choices=["gelu_tanh", "swiglu"])
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    # beyond the default configurations (manual runs; the JSON line names what was run)
    ap.add_argument("--shape", default="xl", choices=["xl", "g1792", "g1408"],
                    help="xl: DiT-XL/2 (h=1152, 8 experts, 256 tokens/image); g1792 / g1408: DiT-G/2-like "
                         "(16 experts, 1024 tokens/image, 8 x2 images per GPU, 40 layers)")
    ap.add_argument("--ep-mode", default="sync", choices=["sync", "displaced", "interweaved"])
    ap.add_argument("--ep-async-mode", default="all", choices=["all", "shallow", "deep", "interleaved"])
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="synchronous expert parallelism through NCCL all-to-all instead of the NVLink peer-memory exchange")
    ap.add_argument("--auto-gc", action="store_true", help="drop send buffers of completed exchanges (ep_cache_init auto_gc)")
    ap.add_argument("--no-full-model", action="store_true",
                    help="skip the latency of one sampling step of the full DiT-MoE model (attention etc. in PyTorch)")
    ap.add_argument("--phases", action="store_true",
                    help="after the timed runs, time the phases of the block (router, count exchange, dispatch, expert "
                         "FFN, combine ...) with CUDA events on a few more steps and add them to the JSON line")
    ap.add_argument("--skip", action="store_true", help="conditional communication: noskip step 2, 'low' strategy")
    ap.add_argument("--route", default="router",
                    help="router (Gaussian activations through the block's own router: near-uniform load) or "
                         "zipf:S[:T]: one constant input channel and a per-expert router bias log(p_e)/T with "
                         "p_e ~ 1/rank^S over a seeded permutation of the experts, so that the logits are "
                         "N(0,1) + log(p_e)/T and the expert load is skewed")
    ap.add_argument("--sync-steps", type=int, default=0,
                    help="asynchronous modes: the first S of the timed steps are forced-synchronous steps "
                         "(the warm-up steps of diffusion/warmup.py:11-20)")
    ap.add_argument("--no-gpu-reference", action="store_true", help="skip the stock-PyTorch comparator on the GPU")
    ap.add_argument("--no-variants", action="store_true", help="N = 1: skip the SwiGLU block next to the GELU-tanh one")
    return ap.parse_args()


def apply_shape(args):
    global HIDDEN, EXPERTS, TOKENS_PER_IMAGE
    if args.shape != "xl":
        HIDDEN = 1792 if args.shape == "g1792" else 1408
        EXPERTS = 16
        TOKENS_PER_IMAGE = 1024
        if args.layers == 28:
            args.layers = 40


def workload(n_gpus: int, shape: str = "xl"):
    if shape != "xl":
        tokens = 8 * 2 * TOKENS_PER_IMAGE
        return tokens, (f"DiT-G/2-MoE-like MoE blocks (hidden {HIDDEN}, 16 experts), {n_gpus} GPU(s): per-GPU batch 8 x2 CFG x "
                        f"1024 tokens")
    images = 32 if n_gpus == 1 else 16
    tokens = images * 2 * TOKENS_PER_IMAGE
    name = ("DiT-XL/2-MoE MoE blocks, 1 GPU: batch 32 x2 CFG x 256 tokens" if n_gpus == 1 else
            f"DiT-XL/2-MoE MoE blocks, expert parallel over {n_gpus} GPUs: per-GPU batch 16 x2 CFG x 256 tokens, sync all-to-all")
    return tokens, name


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- #
# model construction
# --------------------------------------------------------------------------- #


def _param_seed(seed, layer, name):
    import zlib

    return (seed * 1000003 + layer * 7919 + zlib.crc32(name.encode())) % (2 ** 31 - 1)


def zipf_route(spec):
    """(s, temperature) of ``--route zipf:S[:T]``, or None."""
    if spec == "router":
        return None
    parts = spec.split(":")
    if parts[0] != "zipf" or len(parts) not in (2, 3):
        raise SystemExit(f"--route {spec}: expected router or zipf:S[:T]")
    return float(parts[1]), float(parts[2]) if len(parts) == 3 else 1.0


ZIPF_CHANNEL_VALUE = 4.0  # the constant input channel that carries the router bias


def build_blocks(layers, variant, para_mode, device, seed=0, route=None, only_layer=None):
    """One block per layer.  Every parameter is drawn from its own seed (layer, parameter name), so that a
    rank's trimmed expert-parallel block and an unsharded block hold the same values for the same expert."""
    from dice_b200.moe_block import SparseMoeBlock

    blocks = []
    gen = torch.Generator(device=device)
    for layer in (range(layers) if only_layer is None else [only_layer]):
        with torch.device(device):
            blk = SparseMoeBlock(HIDDEN, MLP_RATIO, EXPERTS, 2, pretraining_tp=1, layer_idx=layer, total_layers=layers,
                                 para_mode=para_mode, expert_act=variant, shared_expert=(variant == "swiglu"))
        blk = blk.to(torch.bfloat16).eval()
        for name, p in blk.named_parameters():
            gen.manual_seed(_param_seed(seed, layer, name))
            p.data.normal_(0.0, 0.02, generator=gen)
        if route is not None:
            # logits = N(0, 1) (unit-norm rows against N(0,1) activations) + log(p_e) / T through channel 0
            s_exp, temp = route
            gen.manual_seed(_param_seed(seed, layer, "zipf"))
            w = torch.randn(EXPERTS, HIDDEN, generator=gen, device=device) / (HIDDEN - 1) ** 0.5
            perm = torch.randperm(EXPERTS, generator=gen, device=device)
            p_e = 1.0 / (perm.float() + 1.0) ** s_exp
            w[:, 0] = torch.log(p_e / p_e.sum()) / temp / ZIPF_CHANNEL_VALUE
            blk.gate.weight.data.copy_(w)
        blk.gate.norm_topk_prob = variant == "gelu_tanh"
        blocks.append(blk)
    return blocks


def full_model_step(blocks, tokens, device, begin_step, barrier, ep, steps=10):
    """Latency of one sampling step (CFG-doubled forward + Euler update) of the full DiT-MoE model built around the
    same MoE blocks; the backbone is a measurement harness in plain PyTorch (bench_dit_model.py)."""
    import torch.distributed as dist

    from bench_dit_model import DiTBackbone

    latent = int(round((TOKENS_PER_IMAGE) ** 0.5)) * 2
    images = tokens // TOKENS_PER_IMAGE // 2
    model = DiTBackbone(blocks, HIDDEN, latent=latent).to(device=device, dtype=torch.bfloat16).eval()
    g = torch.Generator(device=device).manual_seed(5)
    z = torch.randn(images, 4, latent, latent, generator=g, device=device).bfloat16()
    cond = torch.randint(0, 1000, (images,), generator=g, device=device)
    null = torch.full((images,), 1000, device=device)

    def step(i):
        begin_step()
        return model.sampling_step(z, cond, null, t=1.0 - i / 50.0, dt=1.0 / 50.0)

    def measure():
        for i in range(3):
            step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
        if ep:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return round(float(ms.item()), 3)

    model.set_fused_glue(False)
    plain = measure()
    model.set_fused_glue(True)
    fused = measure()
    return {"ms_per_step": fused, "ms_per_step_glue_in_torch": plain, "images_per_gpu": images, "latent": latent,
            "note": "MoE blocks: dice_b200 kernels, with the LayerNorm + modulation in front of the block and the gated "
                    "residual behind it inside them (ms_per_step) or as PyTorch element-wise kernels "
                    "(ms_per_step_glue_in_torch); backbone (attention, adaLN, embeddings): PyTorch bf16 harness"}


def small_batch_serving(blocks, device, images=2, steps=20):
    """One sampling step of the full model at a serving-size batch (2 images x2 CFG), where the step is bounded by
    the host: eager against the same step captured once into a CUDA graph (dice_b200.serving.GraphedStep)."""
    from bench_dit_model import DiTBackbone
    from dice_b200.serving import GraphedStep

    latent = int(round((TOKENS_PER_IMAGE) ** 0.5)) * 2
    model = DiTBackbone(blocks, HIDDEN, latent=latent).to(device=device, dtype=torch.bfloat16).eval()
    g = torch.Generator(device=device).manual_seed(6)
    z = torch.randn(images, 4, latent, latent, generator=g, device=device).bfloat16()
    cond = torch.randint(0, 1000, (images,), generator=g, device=device)
    null = torch.full((images,), 1000, device=device)

    def step(zz):
        return model.sampling_step(zz, cond, null, t=0.5, dt=1.0 / 50.0)

    def timed(fn):
        for _ in range(3):
            fn(z)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn(z)
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) / steps, 3)

    eager = timed(step)
    try:
        graphed = timed(GraphedStep(step, z, modules=[model]))
    except Exception as exc:  # a capture that the installed driver refuses is reported, not fatal
        return {"images": images, "eager_ms_per_step": eager, "graphed_ms_per_step": None, "error": str(exc)[:200]}
    return {"images": images, "tokens": 2 * images * TOKENS_PER_IMAGE, "eager_ms_per_step": eager,
            "graphed_ms_per_step": graphed,
            "note": "full DiT-MoE sampling step (PyTorch backbone + dice_b200 MoE blocks), one CUDA graph per step"}


def phase_times(step_fn, layers, steps=3):
    """GPU time of each named phase of the block (the section names the reference's profiler uses,
    ep_fwd.py:88-172, models.py:305-375), per layer, on this rank: CUDA events around every phase."""
    import collections
    import contextlib

    from dice_b200.expertpara import diep

    events = collections.defaultdict(list)

    class Phases:
        @staticmethod
        @contextlib.contextmanager
        def scope(name, stream=None, cpu=False):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            yield
            e.record()
            events[name].append((s, e))

    diep._profiler()  # make sure the hook variable exists
    saved, diep._prof_cls = diep._prof_cls, Phases
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step_fn()
    t1.record()
    torch.cuda.synchronize()
    diep._prof_cls = saved
    out = {k: round(sum(a.elapsed_time(b) for a, b in v) / steps / layers * 1e3, 1) for k, v in events.items()}
    out["whole_layer"] = round(t0.elapsed_time(t1) / steps / layers * 1e3, 1)
    return out


def ffn_flops(tokens, variant):
    """Algorithmic FLOPs of one grouped-GEMM launch pair: the routed experts (2 rows per token) and, in the
    SwiGLU variant, the shared expert of width 2h that rides in the same launches (every token once)."""
    rows = 2 * tokens
    per_row = (6 if variant == "swiglu" else 4) * HIDDEN * MLP_RATIO * HIDDEN
    shared = tokens * 6 * HIDDEN * 2 * HIDDEN if variant == "swiglu" else 0
    return rows * per_row + shared


def hbm_rooflines(blocks, xs, peak_gbs, reps=10):
    """The HBM-bound kernels of the block, each timed alone with CUDA events over all layers' inputs (one
    distinct 37.7 MB input per layer: the working set between two uses of a buffer exceeds the 126 MB L2),
    against their algorithmic bytes: router N*h*2 + E*h*2 + 24 N + 4 E; row gather and combine N*h*2 + R*h*2 +
    4 R (+ 8 N of gate weights for the combine)."""
    from dice_b200 import ops

    n, h, e = xs[0].shape[0] * xs[0].shape[1], xs[0].shape[2], EXPERTS
    r = 2 * n
    x2 = [x.view(-1, h) for x in xs]
    gw = [b._gate_weight(torch.bfloat16) for b in blocks]
    routed = [ops.router_top2(x, w) for x, w in zip(x2, gw)]
    plans = [ops.permute_plan(idx.view(-1), e) for idx, _, _, _ in routed]
    rows = [torch.empty((r, h), dtype=torch.bfloat16, device=xs[0].device) for _ in range(min(len(xs), 4))]
    outs = [torch.empty((n, h), dtype=torch.bfloat16, device=xs[0].device) for _ in range(min(len(xs), 4))]

    def timed(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (reps * len(xs))

    def run_router():
        for x, w in zip(x2, gw):
            ops.router_top2(x, w)

    def run_plan():
        for idx, _, _, _ in routed:
            ops.permute_plan(idx.view(-1), e)

    def run_gather():
        for i, (x, (pos, _, _)) in enumerate(zip(x2, plans)):
            ops.permute_rows(x, pos, 2, out=rows[i % len(rows)])

    def run_combine():
        for i, ((_, w, _, _), (pos, _, _)) in enumerate(zip(routed, plans)):
            src = rows[i % len(rows)]
            ops.unpermute_combine(src, pos[0::2], src, pos[1::2], w[:, 0], w[:, 1], n, out=outs[i % len(outs)])

    run_gather()
    bytes_of = {"router": n * h * 2 + e * h * 2 + 24 * n + 4 * e, "row_gather": n * h * 2 + r * h * 2 + 4 * r,
                "combine": n * h * 2 + r * h * 2 + 4 * r + 8 * n}
    out = {}
    for name, fn in (("router", run_router), ("row_gather", run_gather), ("combine", run_combine)):
        t = timed(fn)
        gbs = bytes_of[name] / t / 1e9
        out[name] = {"us": round(t * 1e6, 2), "bytes": bytes_of[name], "achieved": round(gbs, 1), "peak": peak_gbs,
                     "unit": "GB/s", "frac": round(gbs / peak_gbs, 4)}
    out["permute_plan"] = {"us": round(timed(run_plan) * 1e6, 2), "note": "3 launches on 4-byte indices: latency-bound"}
    return out


def gpu_reference(blocks, xs, ep, budget_steps=2):
    """The reference's algorithm in stock PyTorch CUDA operations (bench_torch_reference.py) on the same blocks
    and inputs: tokens/s of this rank, a comparator only."""
    import bench_torch_reference as R

    fwd = R.block_forward_ep if ep else R.block_forward
    n_layers = min(len(blocks), 4)
    for blk, x in zip(blocks[:2], xs[:2]):
        fwd(blk, x)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(budget_steps):
        for blk, x in zip(blocks[:n_layers], xs[:n_layers]):
            fwd(blk, x)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (budget_steps * n_layers), n_layers


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #


def run_ours(args):
    import torch.distributed as dist

    from dice_b200 import _lib, ops
    from dice_b200.moe_block import ExpertPack, ParaMode

    lib = _lib.load()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    ep = world > 1
    if ep:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    tokens, wl_name = workload(world, args.shape)
    is_async = ep and args.ep_mode != "sync"
    route = zipf_route(args.route)
    para_mode = ParaMode(ep=ep, ep_async=is_async, ep_async_mode=args.ep_async_mode if is_async else None,
                         ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0)
    blocks = build_blocks(args.layers, args.variant, para_mode, device, route=route)
    step_counter = [10 ** 6]
    if ep:
        from dice_b200.expertpara import diep, ep_fwd, p2p

        diep.ep_cache_init(args.layers, auto_gc=args.auto_gc, noskip_step=2 if args.skip else 1,
                           skip_mode="low" if args.skip else None, async_pipeline=args.ep_mode == "interweaved",
                           selective_async_strategy=args.ep_async_mode if is_async else None)
        ep_fwd.use_latest_expert_weights(True)
        p2p.enable(not args.nccl_exchange)
        wl_name += f", {args.ep_mode} exchange" + (f" ({args.ep_async_mode} layers async)" if is_async else "") + (
            ", conditional communication" if args.skip else "")
    if route is not None:
        wl_name += f", router logits N(0,1) + Zipf(s={route[0]}) bias / T={route[1]}"
    gen = torch.Generator(device=device).manual_seed(1000 + rank)

    def make_input(g=gen, dev=device):
        x = torch.randn(tokens // TOKENS_PER_IMAGE, TOKENS_PER_IMAGE, HIDDEN, generator=g, device=dev).bfloat16()
        if route is not None:
            x[..., 0] = ZIPF_CHANNEL_VALUE
        return x

    # one distinct input per layer: together with >150 MB of expert weights per layer the working set
    # between two uses of any buffer is far larger than the 126 MB L2
    xs = [make_input() for _ in range(args.layers)]
    host_in = [make_input(torch.Generator().manual_seed(7 + i), "cpu").pin_memory() for i in range(2)]
    host_out = [torch.empty_like(host_in[0]).pin_memory() for _ in range(2)]
    dev_in = [torch.empty_like(xs[0]) for _ in range(2)]

    def begin_step(forced=False):
        # what the sampler does around each model call (rectified_flow.py:91-114)
        if not ep:
            return
        step_counter[0] -= 1
        diep.ep_set_step(step_counter[0])
        if forced:
            diep.diep_force_sync()
            diep.ep_cache_clear()

    def forced_step():
        begin_step(forced=True)
        y = None
        for blk, x in zip(blocks, xs):
            y = blk(x)
        diep.diep_cancel_sync()
        return y

    def step_device():
        begin_step()
        y = None
        for blk, x in zip(blocks, xs):
            y = blk(x)
        return y

    # end to end: every step copies its inputs from pinned host memory and its result back, double-buffered on
    # two copy streams so that the copies of neighbouring steps run under the blocks of this one
    main = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0, "checksum": 0.0}

    def step_e2e():
        i = e2e_state["i"]
        b = i & 1
        e2e_state["i"] = i + 1
        begin_step()
        with torch.cuda.stream(copy_in):
            if i >= 2:
                copy_in.wait_event(ev_free[b])   # the blocks of step i-2 have read this buffer
            dev_in[b].copy_(host_in[b], non_blocking=True)
            ev_in[b].record(copy_in)
        main.wait_event(ev_in[b])
        y = None
        for blk in blocks:
            y = blk(dev_in[b])
        ev_free[b].record(main)
        ev_done[b].record(main)
        if i >= 2:
            ev_out[b].synchronize()              # the host has the result of step i-2 before its buffer is reused
            e2e_state["checksum"] += float(host_out[b][0, 0, 0])
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(ev_done[b])
            y.record_stream(copy_out)
            host_out[b].copy_(y, non_blocking=True)
            ev_out[b].record(copy_out)

    def e2e_drain():
        for b in range(2):
            ev_out[b].synchronize()
            e2e_state["checksum"] += float(host_out[b][0, 0, 0])

    def barrier():
        if ep:
            dist.barrier()
        torch.cuda.synchronize()

    sync_steps = args.sync_steps if is_async else 0

    def timed(fn, steps, sampler=None, tail=None, sync_steps=0):
        barrier()
        if sampler is not None:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            if i < sync_steps:
                forced_step()
            else:
                fn()
        if tail is not None:
            tail()
        e1.record()
        barrier()
        clocks = sampler.stop() if sampler is not None else None
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if ep:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), clocks

    ep_parity = load = None
    if ep:
        # Layer 0 of the expert-parallel model against an unsharded block with the same weights on this rank's
        # own tokens (a synchronous step, so the same step's results come back): multi-GPU correctness in the line.
        single = build_blocks(args.layers, args.variant, ParaMode(), device, route=route, only_layer=0)[0]
        if is_async:
            begin_step(forced=True)
        else:
            begin_step()
        y_ep = blocks[0](xs[0])
        for blk, x in zip(blocks[1:], xs[1:]):
            blk(x)
        if is_async:
            diep.diep_cancel_sync()
        y_one = single(xs[0])
        idx_ep, w_ep, hist, _ = ops.router_top2(xs[0].view(-1, HIDDEN), blocks[0]._gate_weight(torch.bfloat16),
                                                renorm=blocks[0].gate.norm_topk_prob)
        idx_one, _, _, _ = ops.router_top2(xs[0].view(-1, HIDDEN), single._gate_weight(torch.bfloat16),
                                           renorm=single.gate.norm_topk_prob)
        rel = ((y_ep.float() - y_one.float()).norm() / y_one.float().norm()).reshape(1)
        stats = torch.stack([rel[0], (idx_ep != idx_one).any().float(), (y_ep != y_one).any().float()])
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        ep_parity = {"routing_equal": bool(stats[1].item() == 0), "max_rel_err": float(stats[0].item()),
                     "bit_identical": bool(stats[2].item() == 0), "layer": 0,
                     "against": "unsharded single-GPU block, same weights, this rank's tokens; max over ranks"}
        hists = [torch.zeros_like(hist) for _ in range(world)]
        dist.all_gather(hists, hist)
        per_expert = torch.stack(hists).sum(0).float()
        per_rank = per_expert.view(EXPERTS // world, world).sum(0)  # expert e lives on rank e mod W
        load = {"rows_per_rank_max_over_mean": round(float(per_rank.max() / per_rank.mean()), 3),
                "rows_per_expert_max_over_mean": round(float(per_expert.max() / per_expert.mean()), 3), "layer": 0}
        del single, y_one
    for _ in range(max(args.warmup, 3)):
        step_device()
    # FFN launch durations, measured on the launching stream inside the timed region
    ExpertPack.timing = []
    # time one FFN call in five (5 does not divide the calls per step, so every layer gets its turn); the clocks of
    # this rank's GPU are sampled by rank 0 only: eight polling nvidia-smi processes slow every rank's launches down
    ExpertPack.timing_every = 5
    launches0 = lib.dice_kernel_launches()
    total_ms, clocks = timed(step_device, args.steps, ClockSampler(local_rank) if rank == 0 else None, sync_steps=sync_steps)
    launches = lib.dice_kernel_launches() - launches0
    ffn_events = ExpertPack.timing
    ExpertPack.timing = None
    torch.cuda.synchronize()
    routed = [s.elapsed_time(e) for tag, s, e in ffn_events if tag.startswith("routed")]
    for blk in blocks:
        blk.check_status()
    exchange = "nccl"
    capacity = None
    if ep:
        if p2p._exchange is not None:
            p2p._exchange.check()
            exchange = "nvlink peer memory (own kernels)"
            capacity = {"rows": p2p._exchange.capacity_rows, "lossless": p2p._exchange.lossless}

    # host cost of enqueueing one layer: two steps right after a synchronisation, while the launch queue is short
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(2):
        step_device()
    host_us = (time.perf_counter() - t0) / (2 * args.layers) * 1e6
    torch.cuda.synchronize()

    for _ in range(2):
        step_e2e()
    e2e_drain()
    e2e_state["i"] = 0
    e2e_ms, _ = timed(step_e2e, args.steps, tail=e2e_drain)

    phases = phase_times(step_device, args.layers) if (args.phases or ep) else None
    dit = None if args.no_full_model else full_model_step(blocks, tokens, device, begin_step, barrier, ep, steps=10)

    ms_per_step = total_ms / args.steps
    value = world * tokens * args.layers / (ms_per_step * 1e-3)
    e2e_value = world * tokens * args.layers / (e2e_ms / args.steps * 1e-3)

    pk, pk_src = peaks()
    peak_tf = pk.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    # one FFN call = 2 grouped-GEMM launches; rows per rank = 2 * tokens under uniform routing
    # (conditional communication sends one row per token on skip steps: the FLOP count below would be wrong)
    gemm_launches = 2 * len(routed)
    gemm_ms = sum(routed) / max(gemm_launches, 1)
    flops_per_launch = ffn_flops(tokens, args.variant) / 2
    achieved = flops_per_launch / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    roofline = {"kernel": "grouped_gemm_pair_kernel (tcgen05 cta_group::2, fc1+fc2 of the routed experts"
                          + (" and the shared expert" if args.variant == "swiglu" else "") + ")", "bound": "tensor",
                "achieved": round(achieved, 1), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(achieved / peak_tf, 4),
                "peak_source": f"bf16_tflops_sustained of {pk_src}", "frac_of_burst": round(
                    achieved / pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]), 4), "avg_launch_ms": round(gemm_ms, 4),
                "launches_timed": gemm_launches, "launches_in_region": 2 * args.layers * args.steps,
                "flops_per_launch": flops_per_launch,
                "traffic": GEMM_TRAFFIC_BYTES if (world == 1 and args.variant == "gelu_tanh" and args.shape == "xl") else None,
                "traffic_source": "ncu capture summarised in profiles/grouped_gemm_dit_xl2_moe_block.md"}

    if args.skip or route is not None:
        roofline.update({"achieved": None, "frac": None, "frac_of_burst": None,
                         "note": "rows per launch vary (conditional communication / skewed routing)"})
    roofline_hbm = hbm_rooflines(blocks, xs, pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    line = {
        "metric": "moe_block_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl_name, "variant": args.variant, "layers_per_step": args.layers, "tokens_per_gpu": tokens,
                   "hidden": HIDDEN, "experts": EXPERTS, "top_k": 2, "ffn": MLP_RATIO * HIDDEN,
                   "parallelism": "ep%d" % world if ep else "single", "exchange": exchange if ep else None,
                   "forced_sync_steps_in_region": sync_steps,
                   "l2": "per-layer inputs and weights (>150 MB per layer) exceed the 126 MB L2; no explicit flush"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                "h2d_bytes_per_step": host_in[0].numel() * 2, "d2h_bytes_per_step": host_out[0].numel() * 2,
                "copies": "double-buffered on two copy streams; the host reads every step's result"},
        "gpu_launches": int(launches),
        "gpu_launches_note": "kernels the library launched inside the timed region on this rank (its own launch counter)",
        "clocks": clocks, "roofline": roofline, "roofline_hbm": roofline_hbm,
        "tokens_per_s_per_gpu": round(value / world, 1), "host_us_per_layer": round(host_us, 1),
    }
    if ep and exchange != "nccl":
        x = p2p._exchange
        follows = p2p.return_follows() and x.rows_done is not None
        line["config"]["receive_layout"] = "regions (no count exchange)" if x.region_rows else "packed (count exchange)"
        line["config"]["return_of_a_sync_exchange"] = (
            f"follows the second GEMM on {p2p.follow_ctas()} CTAs" if follows else "after the FFN, on all SMs")
    if ep_parity is not None:
        line["ep_parity"] = ep_parity
        line["load"] = load
        line["receive_capacity"] = capacity
    if phases is not None:
        line["phases_us_per_layer"] = phases
    if dit is not None:
        line["dit_sampling_step"] = dit
    if world == 1 and dit is not None:
        line["small_batch_serving"] = small_batch_serving(blocks, device)
    if not args.no_gpu_reference:
        t_ref, n_ref = gpu_reference(blocks, xs, ep)
        ref_ms = torch.tensor([t_ref], device=device)
        if ep:
            dist.all_reduce(ref_ms, op=dist.ReduceOp.MAX)
        ref_value = world * tokens / float(ref_ms.item())
        line["gpu_reference"] = {
            "value": round(ref_value, 1), "unit": "tokens/s", "us_per_block": round(float(ref_ms.item()) * 1e6, 1),
            "kind": "port", "speedup": round(value / ref_value, 2),
            "what": "the reference's algorithm in stock PyTorch CUDA ops (ATen, cuBLAS" + (", NCCL all_to_all_single per "
                    "expert slot" if ep else "") + "; per-expert Python loop, host reads for split sizes) on the same GPUs, "
                    f"bf16, same blocks and inputs, {n_ref} layers x 2 passes: bench_torch_reference.py"}
    if world == 1 and not args.no_variants and args.variant == "gelu_tanh" and args.shape == "xl" and route is None:
        sw_blocks = build_blocks(args.layers, "swiglu", para_mode, device)

        def step_swiglu():
            for blk, x in zip(sw_blocks, xs):
                blk(x)

        for _ in range(3):
            step_swiglu()
        sw_steps = max(5, args.steps // 2)
        sw_ms, _ = timed(step_swiglu, sw_steps)
        line["variants"] = {"swiglu": {
            "value": round(tokens * args.layers / (sw_ms / sw_steps * 1e-3), 1), "unit": "tokens/s",
            "ms_per_step": round(sw_ms / sw_steps, 4), "steps": sw_steps,
            "what": "the block as the reference computes it: SwiGLU experts, un-normalised top-2 weights, shared expert"}}
        del sw_blocks
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(blocks, xs, args.variant, budget_s=12.0)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if ep:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# CPU baseline / reference arm (the oracle, timed; never the product path)
# --------------------------------------------------------------------------- #


def _oracle_weights(blk, variant):
    sd = {k: v.detach().float().cpu() for k, v in blk.state_dict().items()}
    if variant == "swiglu":
        ex = [tuple(sd[f"experts.{i}.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj")) for i in range(EXPERTS)]
        sh = tuple(sd[f"shared_experts.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj"))
    else:
        ex = [tuple(sd[f"experts.{i}.{p}.weight"] for p in ("fc1", "fc2")) for i in range(EXPERTS)]
        sh = None
    return sd["gate.weight"], ex, sh


def _oracle_block(x, weights, variant):
    from oracle import moe_oracle as O

    wg, ex, sh = weights
    return O.moe_block_forward(x, wg, ex, sh, act=variant, renorm=(variant == "gelu_tanh"))["out"]


def cpu_baseline(blocks, xs, variant, budget_s):
    """The oracle (fp32, all host threads) on whole blocks of the same workload until ~budget_s elapsed."""
    threads = torch.get_num_threads()
    weights = _oracle_weights(blocks[0], variant)
    x = xs[0].float().cpu()
    with torch.no_grad():
        _oracle_block(x[:2], weights, variant)  # warm-up on a slice
        t0 = time.perf_counter()
        n = 0
        while True:
            _oracle_block(x, weights, variant)
            n += 1
            if time.perf_counter() - t0 > budget_s or n >= 8:
                break
        dt = time.perf_counter() - t0
    tokens = x.shape[0] * x.shape[1]
    return {"value": round(tokens * n / dt, 1), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{n} full MoE block(s) of layer 0 ({tokens} tokens, fp32, torch CPU, {threads} threads, "
                      f"os.cpu_count()={os.cpu_count()})"}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference path, on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    tokens, wl_name = workload(world, args.shape)
    # torchrun exports OMP_NUM_THREADS=1; the reference arm may use every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    f = MLP_RATIO * HIDDEN
    rn = lambda *s: torch.randn(*s, generator=g) * 0.02
    wg = rn(EXPERTS, HIDDEN)
    if args.variant == "swiglu":
        ex = [(rn(f, HIDDEN), rn(f, HIDDEN), rn(HIDDEN, f)) for _ in range(EXPERTS)]
        sh = (rn(2 * HIDDEN, HIDDEN), rn(2 * HIDDEN, HIDDEN), rn(HIDDEN, 2 * HIDDEN))
    else:
        ex = [(rn(f, HIDDEN), rn(HIDDEN, f)) for _ in range(EXPERTS)]
        sh = None
    x = torch.randn(tokens // TOKENS_PER_IMAGE, TOKENS_PER_IMAGE, HIDDEN, generator=g)
    # bounded sample: one step = ONE block (not all layers) over the full token batch
    with torch.no_grad():
        for _ in range(min(args.warmup, 2)):
            _oracle_block(x, (wg, ex, sh), args.variant)
        steps = min(args.steps, 10)
        t0 = time.perf_counter()
        for _ in range(steps):
            _oracle_block(x, (wg, ex, sh), args.variant)
        dt = time.perf_counter() - t0
    value = tokens * steps / dt
    sample = (f"{steps} timed block passes of {tokens} tokens (1 layer per step instead of {args.layers}); fp32 torch CPU, "
              f"{threads} threads, os.cpu_count()={os.cpu_count()}")
    line = {
        "impl": "reference", "metric": "moe_block_tokens_per_s", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": round(dt / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "variant": args.variant, "layers_per_step": 1, "tokens_per_gpu": tokens,
                   "hidden": HIDDEN, "experts": EXPERTS, "top_k": 2, "ffn": f},
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    apply_shape(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py measures the CUDA path and needs a GPU (there is no CPU fallback); "
                             "use --impl reference for the CPU baseline")
        run_ours(args)


if __name__ == "__main__":
    main()
