"""Generate the fixtures in this directory from the unmodified reference.

Run on a machine that has the reference checkout (CPU only, gloo ranks):

    python tests/golden/make_golden.py [--reference-root /path/to/DICE]

It writes

* ``block_small.npz``   one small SparseMoeBlock forward (fp32): inputs,
  state dict, routing, expert histogram and output, produced by the
  reference's ``models.SparseMoeBlock`` (models.py:276-382);
* ``block_c0.npz``      the 2x256x1152, 8-expert fp32 block with N(0, 0.02)
  weights from seed 0: routing, histogram and a row subsample of the output
  (weights are regenerated from the seed by the test, not stored);
* ``ep_<mode>.npz``     outputs of the reference's expert-parallel path
  (expertpara/ep_fwd.py, expertpara/diep.py) on 4 gloo ranks, 4 layers and 8
  sampling steps for the synchronous, displaced, interweaved, selective and
  conditional-communication modes, together with the inputs and state dicts
  needed to replay them.

Nothing here is imported by the package; the fixtures are consumed by the
tests only.
"""
import argparse
import os
import socket
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

# --------------------------------------------------------------------------- #
# shared definitions (the tests import these to replay the fixtures)
# --------------------------------------------------------------------------- #

EP_WORLD = 4
EP_LAYERS = 4
EP_STEPS = 8
EP_TOKENS = 16  # per rank, after flattening [B, T]
EP_HIDDEN = 8
EP_EXPERTS = 8
EP_MLP_RATIO = 4

# name -> (ParaMode kwargs, ep_cache_init kwargs, use_latest_expert_weights)
EP_MODES = {
    "sync": (dict(ep=True), None, None),
    "displaced_all": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="all"),
        False,
    ),
    "displaced_all_latest": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="all"),
        True,
    ),
    "displaced_warm2_stride3": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=2, strided_sync=3, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="all", auto_gc=True),
        False,
    ),
    "interweaved_all": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="all"),
        False,
    ),
    "interweaved_all_gc_warm1": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=1, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="all", auto_gc=True),
        True,
    ),
    "interweaved_shallow": (
        dict(ep=True, ep_async=True, ep_async_mode="shallow", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="shallow"),
        False,
    ),
    "interweaved_deep": (
        dict(ep=True, ep_async=True, ep_async_mode="deep", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="deep"),
        False,
    ),
    "interweaved_interleaved": (
        dict(ep=True, ep_async=True, ep_async_mode="interleaved", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="interleaved"),
        False,
    ),
    "displaced_skip_low": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="all", noskip_step=2, skip_mode="low"),
        False,
    ),
    "displaced_skip_high": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="all", noskip_step=2, skip_mode="high"),
        False,
    ),
    "interweaved_skip_low": (
        dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=True, selective_async_strategy="all", noskip_step=2, skip_mode="low"),
        False,
    ),
    "displaced_deep_skip_low_latest": (
        dict(ep=True, ep_async=True, ep_async_mode="deep", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0),
        dict(async_pipeline=False, selective_async_strategy="deep", noskip_step=2, skip_mode="low"),
        True,
    ),
    "sync_skip3_low": (
        dict(ep=True),
        dict(async_pipeline=False, selective_async_strategy=None, noskip_step=3, skip_mode="low"),
        False,
    ),
}


def ep_layer_state_dict(layer: int):
    """Deterministic small state dict for layer ``layer`` (same on all ranks)."""
    g = torch.Generator().manual_seed(100 + layer)
    h, f, e = EP_HIDDEN, EP_MLP_RATIO * EP_HIDDEN, EP_EXPERTS
    sd = {"gate.weight": torch.randn(e, h, generator=g) * 0.5}
    for i in range(e):
        sd[f"experts.{i}.gate_proj.weight"] = torch.randn(f, h, generator=g) * 0.3
        sd[f"experts.{i}.up_proj.weight"] = torch.randn(f, h, generator=g) * 0.3
        sd[f"experts.{i}.down_proj.weight"] = torch.randn(h, f, generator=g) * 0.3
    sd["shared_experts.gate_proj.weight"] = torch.randn(2 * h, h, generator=g) * 0.3
    sd["shared_experts.up_proj.weight"] = torch.randn(2 * h, h, generator=g) * 0.3
    sd["shared_experts.down_proj.weight"] = torch.randn(h, 2 * h, generator=g) * 0.3
    return sd


def ep_input(rank: int, step_pos: int, layer: int) -> torch.Tensor:
    """Input of ``layer`` at the ``step_pos``-th executed step on ``rank``."""
    g = torch.Generator().manual_seed(7919 * (rank + 1) + 101 * step_pos + layer)
    return torch.randn(1, EP_TOKENS, EP_HIDDEN, generator=g)


def c0_weights(seed: int = 0, hidden: int = 1152, experts: int = 8, ratio: int = 4):
    """N(0, 0.02) weights of the 2x256x1152 configuration, drawn in a fixed
    order from one generator: router, then per expert gate/up/down, then the
    shared expert gate/up/down."""
    g = torch.Generator().manual_seed(seed)
    f = ratio * hidden
    sd = {"gate.weight": torch.randn(experts, hidden, generator=g) * 0.02}
    for i in range(experts):
        sd[f"experts.{i}.gate_proj.weight"] = torch.randn(f, hidden, generator=g) * 0.02
        sd[f"experts.{i}.up_proj.weight"] = torch.randn(f, hidden, generator=g) * 0.02
        sd[f"experts.{i}.down_proj.weight"] = torch.randn(hidden, f, generator=g) * 0.02
    sd["shared_experts.gate_proj.weight"] = torch.randn(2 * hidden, hidden, generator=g) * 0.02
    sd["shared_experts.up_proj.weight"] = torch.randn(2 * hidden, hidden, generator=g) * 0.02
    sd["shared_experts.down_proj.weight"] = torch.randn(hidden, 2 * hidden, generator=g) * 0.02
    return sd


def c0_input(seed: int = 1, hidden: int = 1152) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(2, 256, hidden, generator=g)


C0_ROW_STRIDE = 16  # rows of the output kept in block_c0.npz


# --------------------------------------------------------------------------- #
# generation (needs the reference)
# --------------------------------------------------------------------------- #


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gen_block_small(ref, out_dir):
    torch.manual_seed(1234)
    h, e = 32, 8
    pm = ref.models.ParaMode()
    blk = ref.models.SparseMoeBlock(h, 4, e, 2, pretraining_tp=1, layer_idx=0, total_layers=1, para_mode=pm).eval()
    x = torch.randn(3, 37, h)  # 111 tokens: ragged against every tile size
    with torch.no_grad():
        idx, w, _ = blk.gate(x)
        y = blk(x)
    arrays = {f"sd.{k}": v.detach().numpy() for k, v in blk.state_dict().items()}
    arrays.update(
        x=x.numpy(),
        topk_idx=idx.numpy(),
        topk_weight=w.numpy(),
        hist=torch.bincount(idx.view(-1), minlength=e).numpy(),
        out=y.numpy(),
    )
    np.savez_compressed(os.path.join(out_dir, "block_small.npz"), **arrays)


def _gen_block_c0(ref, out_dir):
    pm = ref.models.ParaMode()
    blk = ref.models.SparseMoeBlock(1152, 4, 8, 2, pretraining_tp=1, layer_idx=0, total_layers=1, para_mode=pm).eval()
    blk.load_state_dict(c0_weights())
    x = c0_input()
    with torch.no_grad():
        idx, w, _ = blk.gate(x)
        y = blk(x)
    np.savez_compressed(
        os.path.join(out_dir, "block_c0.npz"),
        topk_idx=idx.numpy(),
        topk_weight=w.numpy(),
        hist=torch.bincount(idx.view(-1), minlength=8).numpy(),
        out_rows=y.view(-1, 1152)[::C0_ROW_STRIDE].numpy(),
    )


def _ep_worker(rank, world, port, mode_name, ref_root, ret):
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    from oracle.reference_shim import load_reference
    from oracle.moe_oracle import forced_sync_schedule

    ref = load_reference(ref_root)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank)
    pm_kwargs, cache_kwargs, use_latest = EP_MODES[mode_name]
    pm = ref.models.ParaMode(num_sampling_steps=EP_STEPS, **pm_kwargs)
    blocks = []
    for layer in range(EP_LAYERS):
        blk = ref.models.SparseMoeBlock(
            EP_HIDDEN, EP_MLP_RATIO, EP_EXPERTS, 2, pretraining_tp=1, layer_idx=layer, total_layers=EP_LAYERS, para_mode=pm
        ).eval()
        # trim_state_dict recognises expert keys by the substring ".experts." (etrim.py:52)
        full = {"moe." + k: v for k, v in ep_layer_state_dict(layer).items()}
        kept = ref.etrim.trim_state_dict(full, EP_EXPERTS)
        blk.load_state_dict({k[len("moe.") :]: v for k, v in kept.items()})
        blocks.append(blk)
    if cache_kwargs is not None:
        ref.diep.ep_cache_init(EP_LAYERS, **cache_kwargs)
    else:
        ref.diep.ep_cache_init(EP_LAYERS)
    ref.ep_fwd._use_latest_expert_weights = use_latest
    is_async = bool(pm_kwargs.get("ep_async"))
    schedule = forced_sync_schedule(
        EP_STEPS, pm_kwargs.get("ep_async_warm_up") or 0, pm_kwargs.get("strided_sync") or 0, pm_kwargs.get("ep_async_cool_down") or 0
    )
    outs = np.zeros((EP_STEPS, EP_LAYERS, EP_TOKENS, EP_HIDDEN), dtype=np.float32)
    with torch.no_grad():
        for pos, i in enumerate(range(EP_STEPS, 0, -1)):
            ref.diep.ep_set_step(i)
            forced = is_async and schedule[pos]
            if forced:
                ref.diep.diep_force_sync()
                ref.diep.ep_cache_clear()
            for layer, blk in enumerate(blocks):
                outs[pos, layer] = blk(ep_input(rank, pos, layer))[0].numpy()
            if forced:
                ref.diep.diep_cancel_sync()
    ret[rank] = outs
    dist.barrier()
    dist.destroy_process_group()


def _gen_ep(mode_name, ref_root, out_dir):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, EP_WORLD, port, mode_name, ref_root, ret)) for r in range(EP_WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join()
        assert p.exitcode == 0, f"rank failed in mode {mode_name}"
    outs = np.stack([ret[r] for r in range(EP_WORLD)])  # [W, steps, layers, N, h]
    np.savez_compressed(os.path.join(out_dir, f"ep_{mode_name}.npz"), out=outs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=None, help="DICE checkout (default: $DICE_REFERENCE_ROOT or ../reference)")
    ap.add_argument("--only", default=None, help="comma-separated subset: block_small,block_c0,ep")
    args = ap.parse_args()
    from oracle.reference_shim import load_reference

    from oracle.reference_shim import DEFAULT_REFERENCE_ROOT

    args.reference_root = args.reference_root or DEFAULT_REFERENCE_ROOT
    ref = load_reference(args.reference_root)
    only = set(args.only.split(",")) if args.only else {"block_small", "block_c0", "ep"}
    if "block_small" in only:
        _gen_block_small(ref, HERE)
    if "block_c0" in only:
        _gen_block_c0(ref, HERE)
    if "ep" in only:
        for name in EP_MODES:
            _gen_ep(name, args.reference_root, HERE)
            print("generated", name, flush=True)


if __name__ == "__main__":
    main()
