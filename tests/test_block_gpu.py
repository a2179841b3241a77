"""The SparseMoeBlock module on the GPU against the reference fixtures and the
oracle: routing exactly, activations within 1e-5 (fp32) / 2e-2 relative (bf16)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as G  # noqa: E402


def _block(h, e, sd, device, dtype=torch.float32, **kw):
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    blk = SparseMoeBlock(h, 4, e, 2, pretraining_tp=1, layer_idx=0, total_layers=1, para_mode=ParaMode(), **kw)
    blk.load_state_dict(sd)
    return blk.to(device=device, dtype=dtype).eval()


def _small():
    g = np.load(os.path.join(HERE, "golden", "block_small.npz"))
    sd = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd.")}
    return g, sd


def test_block_small_fp32_matches_reference(cuda_device):
    g, sd = _small()
    blk = _block(32, 8, sd, cuda_device)
    x = torch.from_numpy(g["x"]).to(cuda_device)
    idx, w, _ = blk.gate(x)
    assert np.array_equal(idx.cpu().numpy(), g["topk_idx"])
    np.testing.assert_allclose(w.cpu().numpy(), g["topk_weight"], rtol=1e-5, atol=1e-7)
    y = blk(x)
    blk.check_status()
    assert y.shape == x.shape and y.dtype == torch.float32
    np.testing.assert_allclose(y.cpu().numpy(), g["out"], rtol=1e-5, atol=1e-5)


def test_block_small_bf16_within_tolerance(cuda_device):
    g, sd = _small()
    blk = _block(32, 8, sd, cuda_device, torch.bfloat16)
    x = torch.from_numpy(g["x"]).to(cuda_device).bfloat16()
    y = blk(x)
    blk.check_status()
    # oracle on the bf16-rounded weights and inputs, fp32 arithmetic, routing from the kernel's logits
    sdb = {k: v.bfloat16().float() for k, v in sd.items()}
    ex = [tuple(sdb[f"experts.{i}.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj")) for i in range(8)]
    sh = tuple(sdb[f"shared_experts.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj"))
    r = O.moe_block_forward(x.cpu(), sd["gate.weight"].bfloat16(), [[t.bfloat16() for t in e] for e in ex], None)
    idx, _, _ = blk.gate(x)
    mism = (idx.cpu() != r["topk_idx"]).any(-1).float().mean().item()
    assert mism < 0.03
    xf = x.cpu().float().view(-1, 32)
    from dice_b200 import ops

    idx_k, w_k, _, _ = ops.router_top2(x.view(-1, 32), blk.gate.weight.detach())
    want = O.moe_infer(xf, idx_k.cpu().view(-1), w_k.cpu().view(-1), ex, "swiglu") + O.run_expert(xf, sh, "swiglu")
    err = ((y.cpu().float().view(-1, 32) - want).norm() / want.norm()).item()
    assert err < 2e-2, err


def test_block_c0_fp32_matches_reference(cuda_device):
    """2 x 256 x 1152, 8 experts, fp32, N(0, 0.02) weights from seed 0."""
    g = np.load(os.path.join(HERE, "golden", "block_c0.npz"))
    blk = _block(1152, 8, G.c0_weights(), cuda_device)
    x = G.c0_input().to(cuda_device)
    idx, w, _ = blk.gate(x)
    assert np.array_equal(idx.cpu().numpy(), g["topk_idx"])
    np.testing.assert_allclose(w.cpu().numpy(), g["topk_weight"], rtol=1e-5, atol=1e-7)
    y = blk(x)
    blk.check_status()
    got = y.view(-1, 1152)[:: G.C0_ROW_STRIDE].cpu().numpy()
    np.testing.assert_allclose(got, g["out_rows"], rtol=1e-4, atol=1e-5)
    # the same block in bf16: 2e-2 relative to the fp32 reference output
    yb = blk.to(torch.bfloat16)(x.bfloat16()).float().view(-1, 1152)[:: G.C0_ROW_STRIDE].cpu().numpy()
    rel = np.linalg.norm(yb - g["out_rows"]) / np.linalg.norm(g["out_rows"])
    assert rel < 2e-2, rel


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_variant_against_oracle(cuda_device, dtype):
    """fc1 / GELU-tanh / fc2 experts, renormalised top-2 weights, no shared expert."""
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    torch.manual_seed(3)
    h, e = 128, 8
    blk = SparseMoeBlock(h, 4, e, 2, 1, 0, 1, ParaMode(), expert_act="gelu_tanh", shared_expert=False)
    blk.gate.norm_topk_prob = True
    blk = blk.to(device=cuda_device, dtype=dtype).eval()
    x = torch.randn(2, 301, h, device=cuda_device, dtype=dtype)
    y = blk(x)
    blk.check_status()
    sd = {k: v.detach().float().cpu() for k, v in blk.state_dict().items()}
    ex = [(sd[f"experts.{i}.fc1.weight"], sd[f"experts.{i}.fc2.weight"]) for i in range(e)]
    idx, w, _ = blk.gate(x)
    np.testing.assert_allclose(w.sum(-1).cpu().numpy(), 1.0, rtol=1e-5)
    want = O.moe_infer(x.float().cpu().view(-1, h), idx.cpu().view(-1), w.cpu().view(-1), ex, "gelu_tanh")
    err = ((y.float().cpu().view(-1, h) - want).norm() / want.norm()).item()
    assert err < (1e-5 if dtype == torch.float32 else 2e-2), err
    if dtype == torch.float32:
        r = O.moe_block_forward(x.cpu(), sd["gate.weight"], ex, None, act="gelu_tanh", renorm=True)
        assert torch.equal(idx.cpu(), r["topk_idx"])


def test_gelu_block_with_the_combine_in_the_gemm_epilogue(cuda_device, monkeypatch):
    """The opt-in path (DICE_FFN_COMBINE=1) where the second GEMM adds the gate-weighted rows to the token rows
    itself: same routing, output within 2e-2 of the oracle and within bf16 rounding of the default path."""
    from dice_b200 import moe_block
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    torch.manual_seed(5)
    h, e = 128, 8
    blk = SparseMoeBlock(h, 4, e, 2, 1, 0, 1, ParaMode(), expert_act="gelu_tanh", shared_expert=False)
    blk.gate.norm_topk_prob = True
    blk = blk.to(device=cuda_device, dtype=torch.bfloat16).eval()
    x = torch.randn(2, 301, h, device=cuda_device, dtype=torch.bfloat16)
    default = blk(x)
    monkeypatch.setattr(moe_block, "epilogue_combine", True)
    y = blk(x)
    blk.check_status()
    assert not torch.equal(y, default)  # the other path did run
    sd = {k: v.detach().float().cpu() for k, v in blk.state_dict().items()}
    ex = [(sd[f"experts.{i}.fc1.weight"], sd[f"experts.{i}.fc2.weight"]) for i in range(e)]
    idx, w, _ = blk.gate(x)
    want = O.moe_infer(x.float().cpu().view(-1, h), idx.cpu().view(-1), w.cpu().view(-1), ex, "gelu_tanh")
    assert ((y.float().cpu().view(-1, h) - want).norm() / want.norm()).item() < 2e-2
    assert ((y.float() - default.float()).norm() / default.float().norm()).item() < 1e-2


def test_empty_and_single_token_batches(cuda_device):
    g, sd = _small()
    blk = _block(32, 8, sd, cuda_device)
    y = blk(torch.from_numpy(g["x"][:1, :1]).to(cuda_device))
    np.testing.assert_allclose(y.cpu().numpy(), g["out"][:1, :1], rtol=1e-5, atol=1e-5)
    y0 = blk(torch.zeros(0, 4, 32, device=cuda_device))
    assert y0.shape == (0, 4, 32)


def test_ep_world_of_one_on_gpu(cuda_device):
    """The expert-parallel code path on one GPU (NCCL world of one rank, once over NCCL and once over the
    peer-memory exchange): the synchronous exchange equals the single-device block at every step; the displaced
    exchange returns the result of two steps earlier and the interweaved one (two layers) that of one step
    earlier, at EVERY step (diep.py:196-310; the reference's tests/test_ep.py:113-121 pins the displaced case).
    The blocks have no shared expert, so the whole output is stale and is compared bit for bit."""
    import socket

    import torch.distributed as dist

    from dice_b200.expertpara import diep, ep_fwd, p2p
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", world_size=1, rank=0)
    h, e, layers, steps = 64, 8, 2, 6
    try:
        def make(pm, layer):
            torch.manual_seed(50 + layer)
            blk = SparseMoeBlock(h, 4, e, 2, 1, layer, layers, pm, shared_expert=False)
            return blk.to(device=cuda_device, dtype=torch.bfloat16).eval()

        g = torch.Generator(device="cuda").manual_seed(11)
        xs = [[torch.randn(2, 77 + 5 * l, h, device=cuda_device, generator=g).bfloat16() for l in range(layers)]
              for _ in range(steps)]
        ref = [make(ParaMode(), l) for l in range(layers)]
        want = [[ref[l](xs[t][l]) for l in range(layers)] for t in range(steps)]
        for l in range(layers):  # inputs differ enough between steps for a wrong staleness to show
            assert not torch.allclose(want[0][l].float(), want[1][l].float(), atol=1e-2)
        a = dict(ep=True, ep_async=True, ep_async_mode="all", ep_async_warm_up=0, strided_sync=0, ep_async_cool_down=0)
        cases = [
            ("sync", ParaMode(ep=True), {}, lambda t: t),
            ("displaced", ParaMode(**a), dict(async_pipeline=False, selective_async_strategy="all"), lambda t: max(0, t - 2)),
            ("interweaved", ParaMode(**a), dict(async_pipeline=True, selective_async_strategy="all"), lambda t: max(0, t - 1)),
        ]
        for use_peer_memory in (False, True):
            p2p.enable(use_peer_memory)
            for name, pm, cache_kw, source_step in cases:
                blocks = [make(pm, l) for l in range(layers)]
                diep.ep_cache_init(layers, **cache_kw)
                ep_fwd.use_latest_expert_weights(False)
                for t in range(steps):
                    diep.ep_set_step(steps - t)
                    forced = pm.ep_async and t == 0
                    if forced:
                        diep.diep_force_sync()
                        diep.ep_cache_clear()
                    for l in range(layers):
                        y = blocks[l](xs[t][l])
                        src = source_step(t)
                        assert y.shape == xs[t][l].shape
                        assert torch.equal(y, want[src][l]), f"{name} peer={use_peer_memory} step {t} layer {l}"
                    if forced:
                        diep.diep_cancel_sync()
                for b in blocks:
                    b.check_status()
                assert diep.ep_cached_tensors_size() >= 0
            if use_peer_memory:
                assert p2p._exchange is not None and p2p._exchange.lossless
                p2p._exchange.check()
    finally:
        p2p.enable(False)
        p2p.reset()
        dist.destroy_process_group()
        ep_fwd._use_latest_expert_weights = None


@pytest.mark.parametrize("variant", ["swiglu", "gelu_tanh"])
def test_full_size_block_is_row_independent(cuda_device, variant):
    """Size-independent property at the benchmark's size (16384 tokens, hidden
    1152, 8 experts, bf16): a token's output does not depend on which other
    tokens share the batch, so the block applied to half of the batch gives
    the same bits as the matching half of the full-batch output, although the
    permutation, the segment sizes and the tile list all differ."""
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    torch.manual_seed(0)
    with torch.device(cuda_device):
        blk = SparseMoeBlock(1152, 4, 8, 2, 1, 0, 1, ParaMode(), expert_act=variant,
                             shared_expert=(variant == "swiglu"))
    blk = blk.to(torch.bfloat16).eval()
    for p in blk.parameters():
        p.data.normal_(0.0, 0.02)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(64, 256, 1152, generator=g, device=cuda_device).bfloat16()
    y = blk(x)
    y_half = blk(x[:32].contiguous())
    y_odd = blk(x[1::2].contiguous())
    blk.check_status()
    assert bool(torch.isfinite(y.float()).all())
    assert torch.equal(y[:32], y_half)
    assert torch.equal(y[1::2], y_odd)
    # and the routing histogram adds up
    from dice_b200 import ops

    _, _, hist, _ = ops.router_top2(x.view(-1, 1152), blk.gate.weight.detach())
    assert int(hist.sum()) == 2 * 64 * 256


def test_dependent_launch_changes_nothing(cuda_device):
    """The kernels are launched with programmatic dependent launch (a kernel may become resident while its
    predecessor still runs and waits before touching memory).  A chain of six full-width blocks, repeated three
    times, must give bit-identical outputs with the launch attribute on and off."""
    import subprocess

    root = os.path.dirname(HERE)
    digests = []
    for flag in ("1", "0"):
        env = dict(os.environ, DICE_PDL=flag, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, os.path.join(HERE, "pdl_worker.py")], env=env, capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("DIGEST ")]
        assert lines, r.stdout[-2000:]
        digests.append(lines[-1])
    assert digests[0] == digests[1]
