"""Worker of tests/test_ep_gpu_multi.py: one NCCL rank per GPU (run under torchrun).

Checks the expert-parallel block against the single-device block on the same
seeded inputs: synchronous exchange (same step), displaced (two steps stale),
interweaved over two layers (one step stale), and displaced with conditional
communication (runs, finite, right shapes)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from dice_b200.expertpara import diep, ep_fwd
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    h, e, layers, steps, n_tok = 256, 8, 2, 6, 1000 + 37 * rank  # ragged: ranks hold different token counts

    def make(pm, layer):
        torch.manual_seed(100 + layer)
        full = SparseMoeBlock(h, 4, e, 2, 1, layer, layers, ParaMode(), shared_expert=False)
        sd = {k: v.clone() for k, v in full.state_dict().items()}
        if pm.ep:
            blk = SparseMoeBlock(h, 4, e, 2, 1, layer, layers, pm, shared_expert=False)
            mine = {k: v for k, v in sd.items() if ".experts." not in "." + k or int(k.split(".")[1]) % world == rank}
            blk.load_state_dict(mine)
        else:
            blk = full
        return blk.to(device=dev, dtype=torch.bfloat16).eval()

    g = torch.Generator(device=dev).manual_seed(7 + rank)
    xs = [[torch.randn(1, n_tok, h, generator=g, device=dev).bfloat16() for _ in range(layers)] for _ in range(steps)]
    ref_blocks = [make(ParaMode(), l) for l in range(layers)]
    want = [[ref_blocks[l](xs[t][l]).float() for l in range(layers)] for t in range(steps)]

    def close(a, b, what):
        err = ((a.float() - b).norm() / b.norm()).item()
        assert err < 2e-2, f"rank {rank} {what}: rel err {err}"

    def run(pm, cache_kwargs, check, collect=None):
        blocks = [make(pm, l) for l in range(layers)]
        diep.ep_cache_init(layers, **cache_kwargs)
        ep_fwd.use_latest_expert_weights(False)
        for t in range(steps):
            diep.ep_set_step(steps - t)
            forced = pm.ep_async and t == 0
            if forced:
                diep.diep_force_sync()
                diep.ep_cache_clear()
            for l in range(layers):
                y = blocks[l](xs[t][l])
                assert y.shape == xs[t][l].shape and bool(torch.isfinite(y.float()).all())
                check(t, l, y)
                if collect is not None:
                    collect.append(y.clone())
            if forced:
                diep.diep_cancel_sync()
        for b in blocks:
            b.check_status()

    from dice_b200.expertpara import p2p

    nccl_sync, nccl_skip = [], []
    run(ParaMode(ep=True), {}, lambda t, l, y: close(y, want[t][l], f"sync t={t} l={l}"), nccl_sync)
    run(ParaMode(ep=True), dict(noskip_step=2, skip_mode="low"), lambda t, l, y: None, nccl_skip)
    # the same two runs over NVLink peer memory (no NCCL, no host sync): same kernels, same order -> same bits
    p2p.enable(True)
    peer_sync, peer_skip = [], []
    run(ParaMode(ep=True), {}, lambda t, l, y: close(y, want[t][l], f"peer sync t={t} l={l}"), peer_sync)
    run(ParaMode(ep=True), dict(noskip_step=2, skip_mode="low"), lambda t, l, y: None, peer_skip)
    assert p2p.enabled() and p2p._exchange is not None, "peer-memory exchange was not used"
    # once more with the return fused into the second expert GEMM
    p2p.set_fused_return(True)
    fused_sync = []
    run(ParaMode(ep=True), {}, lambda t, l, y: close(y, want[t][l], f"fused return t={t} l={l}"), fused_sync)
    p2p.set_fused_return(False)
    p2p._exchange.check()
    for a_, b_ in zip(nccl_sync + nccl_skip + nccl_sync, peer_sync + peer_skip + fused_sync):
        assert torch.equal(a_, b_), f"rank {rank}: peer-memory exchange differs from the NCCL exchange"
    p2p.enable(False)
    a = dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0)
    sel = dict(a, ep_async_mode="interleaved")
    async_runs = [
        (a, dict(async_pipeline=False, selective_async_strategy="all"),
         lambda t, l, y: close(y, want[max(0, t - 2)][l], f"displaced t={t} l={l}")),
        (a, dict(async_pipeline=True, selective_async_strategy="all", auto_gc=True),
         lambda t, l, y: close(y, want[max(0, t - 1) if t != 1 else 0][l], f"interweaved t={t} l={l}")),
        (a, dict(async_pipeline=False, selective_async_strategy="all", noskip_step=2, skip_mode="low"), lambda t, l, y: None),
        (a, dict(async_pipeline=True, selective_async_strategy="all", noskip_step=2, skip_mode="low"), lambda t, l, y: None),
        (sel, dict(async_pipeline=False, selective_async_strategy="interleaved"), lambda t, l, y: None),
    ]
    nccl_async = []
    for kw, cache_kw, check in async_runs:
        run(ParaMode(**kw), cache_kw, check, nccl_async)
    # the asynchronous protocols over peer memory (pushes on a side stream) must give the very same bits
    p2p.enable(True)
    peer_async = []
    for kw, cache_kw, check in async_runs:
        run(ParaMode(**kw), cache_kw, check, peer_async)
    p2p._exchange.check()
    assert len(nccl_async) == len(peer_async) == len(async_runs) * steps * layers
    for i, (a_, b_) in enumerate(zip(nccl_async, peer_async)):
        assert torch.equal(a_, b_), f"rank {rank}: asynchronous peer-memory exchange differs from NCCL at output {i}"
    p2p.enable(False)
    mem = diep.ep_cached_tensors_size()
    assert mem > 0 and diep.ep_get_max_mem() >= 0
    dist.barrier()
    if rank == 0:
        print("EP_GPU_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
