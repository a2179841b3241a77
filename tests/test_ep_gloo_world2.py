"""Expert-parallel host logic on small gloo worlds (2 and 4 CPU ranks), in the
manner of the reference's tests/test_ep.py and tests/test_etrim.py: arbitrary
row-wise expert modules, random routing, synchronous output equals the
single-process result, displaced output equals the result of two iterations
earlier; round-robin trimming; a failing rank is detected on the host."""
import os
import socket
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _single_process(experts, k, x, flat_idx, flat_w):
    """What one process computes with all experts (models.py:361-382)."""
    out = torch.zeros_like(x)
    order = flat_idx.argsort(stable=True)
    ends = torch.bincount(flat_idx, minlength=len(experts)).cumsum(0).tolist()
    start = 0
    for e, end in enumerate(ends):
        if end > start:
            rows = order[start:end] // k
            out.index_add_(0, rows, experts[e](x[rows]) * flat_w[order[start:end]])
        start = end
    return out


def _spawn(target, world, *args):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port) + args) for r in range(world)]
    for p in procs:
        p.start()
    codes = []
    for p in procs:
        p.join(300)
        codes.append(p.exitcode)
    return codes


def _setup(rank, world, port):
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    from oracle_ops import OracleOps

    from dice_b200.expertpara import ep_fwd

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank)
    ep_fwd.set_device_ops(OracleOps())
    return dist


def _infer_worker(rank, world, port, seed, async_op, pipeline):
    import torch.nn as nn

    dist = _setup(rank, world, port)
    from dice_b200.expertpara import diep
    from dice_b200.expertpara.ep_fwd import moe_infer_ep

    n_tokens, hidden, n_experts, k, n_iter = 128, 36, 8, 2, 5
    torch.manual_seed(seed)
    experts = []
    for _ in range(n_experts):
        lin = nn.Linear(hidden, hidden)
        nn.init.uniform_(lin.weight, 0.0, 1.0)
        experts.append(lin)
    torch.manual_seed(seed + rank)
    diep.ep_cache_init(1, async_pipeline=pipeline, selective_async_strategy="all" if pipeline else None)
    history = []
    with torch.no_grad():
        for it in range(n_iter):
            if it == 0:
                diep.diep_force_sync()
            elif it == 1:
                diep.diep_cancel_sync()
            x = torch.randn(n_tokens, hidden)
            flat_idx = torch.randint(0, n_experts, (n_tokens * k,))
            if it == 2:
                flat_idx[flat_idx == 3] = 4  # an expert that receives nothing
            flat_w = torch.rand(n_tokens * k, 1)
            got = moe_infer_ep(inp=x, experts=experts, flat_expert_indices=flat_idx, flat_expert_weights=flat_w,
                               num_experts_per_tok=k, async_op=async_op, cache_key=0)
            history.append(_single_process(experts, k, x, flat_idx, flat_w))
            if not async_op:
                want = history[-1]
            else:
                # displaced: two steps stale.  With a single layer the interweaved protocol's
                # "previous asynchronous layer" is the layer itself, so it degenerates to the same.
                want = history[max(0, it - 2)]
            assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), f"rank {rank} iter {it}"
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("seed,async_op,pipeline", [(42, False, False), (42, True, False), (43, True, False), (43, True, True)])
def test_infer_matches_single_process(world, seed, async_op, pipeline):
    assert _spawn(_infer_worker, world, seed, async_op, pipeline) == [0] * world


def _skew_worker(rank, world, port):
    """Zipf-like routing: three quarters of all rows go to the experts of one rank, which then receives about
    three times the mean.  The reference has no capacity (ep_fwd.py:247-293): nothing may be dropped."""
    import torch.nn as nn

    dist = _setup(rank, world, port)
    from dice_b200.expertpara.ep_fwd import moe_infer_ep

    n_tokens, hidden, n_experts, k = 96, 20, 8, 2
    torch.manual_seed(7)
    experts = []
    for _ in range(n_experts):
        lin = nn.Linear(hidden, hidden)
        nn.init.uniform_(lin.weight, 0.0, 1.0)
        experts.append(lin)
    torch.manual_seed(70 + rank)
    hot_rank = 1
    with torch.no_grad():
        for it in range(3):
            x = torch.randn(n_tokens, hidden)
            flat_idx = torch.randint(0, n_experts, (n_tokens * k,))
            hot = torch.rand(n_tokens * k) < 0.75
            flat_idx[hot] = hot_rank + world * torch.randint(0, n_experts // world, (int(hot.sum()),))
            flat_w = torch.rand(n_tokens * k, 1)
            got = moe_infer_ep(inp=x, experts=experts, flat_expert_indices=flat_idx, flat_expert_weights=flat_w,
                               num_experts_per_tok=k, async_op=False, cache_key=0)
            want = _single_process(experts, k, x, flat_idx, flat_w)
            assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), f"rank {rank} iter {it}"
    dist.barrier()
    dist.destroy_process_group()


def test_skewed_routing_drops_nothing():
    assert _spawn(_skew_worker, 4) == [0] * 4


def _trim_worker(rank, world, port, n_experts):
    import torch.nn as nn

    dist = _setup(rank, world, port)
    from dice_b200.expertpara.etrim import DummyExpert, _needed_expert_indices, trim_module_list, trim_state_dict

    mine = _needed_expert_indices(n_experts)
    assert mine == list(range(rank, n_experts, world))
    trimmed = trim_module_list(nn.ModuleList([nn.Linear(4, 4) for _ in range(n_experts)]), n_experts)
    assert len(trimmed) == n_experts
    for i, m in enumerate(trimmed):
        assert isinstance(m, DummyExpert) == (i not in mine)
    with pytest.raises(RuntimeError, match="DummyExpert"):
        trimmed[(rank + 1) % world](torch.zeros(1, 4))
    sd = {f"blocks.0.moe.experts.{i}.weight": torch.rand(4, 4) for i in range(n_experts)}
    sd["blocks.0.moe.gate.weight"] = torch.rand(n_experts, 4)
    kept = trim_state_dict(sd, n_experts)
    assert "blocks.0.moe.gate.weight" in kept
    assert sorted(int(k.split(".")[4]) for k in kept if ".experts." in k) == mine
    dist.destroy_process_group()


@pytest.mark.parametrize("n_experts,world", [(8, 4), (4, 2), (16, 4)])
def test_round_robin_trimming(n_experts, world):
    assert _spawn(_trim_worker, world, n_experts) == [0] * world


def _fault_worker(rank, world, port):
    """Rank 1 raises before the collective; rank 0 must see an error from the
    process group (short timeout) instead of hanging."""
    import datetime

    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    from oracle_ops import OracleOps

    from dice_b200.expertpara import ep_fwd

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank,
                            timeout=datetime.timedelta(seconds=5))
    ep_fwd.set_device_ops(OracleOps())
    import torch.nn as nn

    experts = [nn.Linear(8, 8) for _ in range(4)]
    x = torch.randn(16, 8)
    idx = torch.randint(0, 4, (32,))
    w = torch.rand(32, 1)
    if rank == 1:
        os._exit(7)  # leaves between steps, nothing in flight
    try:
        ep_fwd.moe_infer_ep(inp=x, experts=experts, flat_expert_indices=idx, flat_expert_weights=w,
                            num_experts_per_tok=2, async_op=False, cache_key=0)
    except Exception:
        os._exit(3)  # detected
    os._exit(0)


def test_lost_rank_is_an_error_not_a_hang():
    codes = _spawn(_fault_worker, 2)
    assert codes == [3, 7]


def test_out_of_range_expert_index_is_caught_on_the_host():
    """An expert id beyond the expert list never reaches a collective."""
    def worker(rank, world, port):
        import torch.nn as nn

        dist = _setup(rank, world, port)
        from dice_b200.expertpara.ep_fwd import moe_infer_ep

        experts = [nn.Linear(8, 8) for _ in range(4)]
        idx = torch.randint(0, 4, (32,))
        idx[5] = 9
        try:
            moe_infer_ep(inp=torch.randn(16, 8), experts=experts, flat_expert_indices=idx,
                         flat_expert_weights=torch.rand(32, 1), num_experts_per_tok=2, async_op=False, cache_key=0)
        except (AssertionError, IndexError, RuntimeError):
            dist.destroy_process_group()
            return
        raise SystemExit(1)

    # world of one rank: the check must fire without any peer
    import torch.multiprocessing as mp

    ctx = mp.get_context("fork")
    p = ctx.Process(target=worker, args=(0, 1, _free_port()))
    p.start()
    p.join(120)
    assert p.exitcode == 0
