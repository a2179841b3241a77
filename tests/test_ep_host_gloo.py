"""The expert-parallel host logic among CPU gloo ranks, replayed against the
outputs of the unmodified reference (tests/golden/ep_*.npz: 4 ranks, 4 layers,
8 sampling steps, every exchange mode).  Device kernels are replaced by the
oracle here; their own parity is covered by the GPU tests."""
import os
import socket
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as G  # noqa: E402  (shared definitions of the fixtures)


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, modes, ret):
    import torch.distributed as dist
    import torch.nn as nn

    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    from oracle import moe_oracle as O
    from oracle_ops import OracleOps

    from dice_b200.expertpara import diep, ep_fwd
    from dice_b200.expertpara.etrim import trim_module_list, trim_state_dict
    from dice_b200.moe_block import MoeMLP, ParaMode, layer_is_async

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank)
    ep_fwd.set_device_ops(OracleOps())
    results = {}
    for mode_name in modes:
        pm_kwargs, cache_kwargs, use_latest = G.EP_MODES[mode_name]
        pm = ParaMode(num_sampling_steps=G.EP_STEPS, **pm_kwargs)
        layers = []
        for layer in range(G.EP_LAYERS):
            sd = {"moe." + k: v for k, v in G.ep_layer_state_dict(layer).items()}
            sd = {k[4:]: v for k, v in trim_state_dict(sd, G.EP_EXPERTS).items()}
            experts = trim_module_list(
                nn.ModuleList([MoeMLP(G.EP_HIDDEN, G.EP_MLP_RATIO * G.EP_HIDDEN, 1) for _ in range(G.EP_EXPERTS)]),
                G.EP_EXPERTS)
            experts.load_state_dict({k[len("experts."):]: v for k, v in sd.items() if k.startswith("experts.")})
            shared = [sd[f"shared_experts.{n}.weight"] for n in ("gate_proj", "up_proj", "down_proj")]
            layers.append((sd["gate.weight"], experts, shared))
        diep.ep_cache_init(G.EP_LAYERS, **(cache_kwargs or {}))
        ep_fwd._use_latest_expert_weights = use_latest
        is_async = bool(pm_kwargs.get("ep_async"))
        schedule = O.forced_sync_schedule(G.EP_STEPS, pm_kwargs.get("ep_async_warm_up") or 0,
                                          pm_kwargs.get("strided_sync") or 0, pm_kwargs.get("ep_async_cool_down") or 0)
        outs = np.zeros((G.EP_STEPS, G.EP_LAYERS, G.EP_TOKENS, G.EP_HIDDEN), dtype=np.float32)
        with torch.no_grad():
            for pos, i in enumerate(range(G.EP_STEPS, 0, -1)):
                diep.ep_set_step(i)
                forced = is_async and schedule[pos]
                if forced:
                    diep.diep_force_sync()
                    diep.ep_cache_clear()
                for layer, (w_gate, experts, shared) in enumerate(layers):
                    x = G.ep_input(rank, pos, layer)[0]
                    idx, w, _ = O.gate_top2(x, w_gate)
                    partial = diep.ep_skip_enabled()
                    y = ep_fwd.moe_infer_ep(
                        inp=x, experts=experts, flat_expert_indices=idx.view(-1), flat_expert_weights=w.view(-1, 1),
                        num_experts_per_tok=2, async_op=layer_is_async(pm, layer, G.EP_LAYERS),
                        skip_mask=diep.ep_skip_mask(idx.numel()) if partial else None,
                        skip_now=diep.ep_skip_now(layer) if partial else None, cache_key=layer)
                    outs[pos, layer] = (y + O.expert_swiglu(x, *shared)).numpy()
                if forced:
                    diep.diep_cancel_sync()
        results[mode_name] = outs
    ret[rank] = results
    dist.barrier()
    dist.destroy_process_group()


def _run(world, modes):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, modes, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0, "a gloo rank failed"
    return [ret[r] for r in range(world)]


def test_all_exchange_modes_match_reference_outputs():
    modes = list(G.EP_MODES)
    per_rank = _run(G.EP_WORLD, modes)
    for name in modes:
        want = np.load(os.path.join(HERE, "golden", f"ep_{name}.npz"))["out"]
        got = np.stack([per_rank[r][name] for r in range(G.EP_WORLD)])
        err = np.abs(got - want).max(axis=(0, 3, 4))  # [steps, layers]
        assert err.max() < 1e-5, f"mode {name}: max |diff| per (step, layer) =\n{err}"
