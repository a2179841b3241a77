"""The CPU oracle against the fixtures generated from the unmodified reference
(tests/golden), and against the reference itself when its checkout is present."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from oracle.reference_shim import load_reference, reference_available

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as G  # noqa: E402


def _experts_from_sd(sd, n):
    ex = [tuple(sd[f"experts.{i}.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj")) for i in range(n)]
    sh = tuple(sd[f"shared_experts.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj"))
    return ex, sh


def test_block_small_matches_reference_fixture():
    g = np.load(os.path.join(HERE, "golden", "block_small.npz"))
    sd = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd.")}
    ex, sh = _experts_from_sd(sd, 8)
    r = O.moe_block_forward(torch.from_numpy(g["x"]), sd["gate.weight"], ex, sh)
    assert np.array_equal(r["topk_idx"].numpy(), g["topk_idx"])
    np.testing.assert_allclose(r["topk_weight"].numpy(), g["topk_weight"], rtol=1e-6, atol=1e-8)
    assert np.array_equal(r["hist"].numpy(), g["hist"])
    np.testing.assert_allclose(r["out"].numpy(), g["out"], rtol=1e-5, atol=1e-6)


def test_block_c0_matches_reference_fixture():
    """2 x 256 tokens, hidden 1152, 8 experts, fp32, N(0, 0.02) weights from seed 0."""
    g = np.load(os.path.join(HERE, "golden", "block_c0.npz"))
    sd = G.c0_weights()
    ex, sh = _experts_from_sd(sd, 8)
    r = O.moe_block_forward(G.c0_input(), sd["gate.weight"], ex, sh)
    assert np.array_equal(r["topk_idx"].numpy(), g["topk_idx"])
    assert np.array_equal(r["hist"].numpy(), g["hist"])
    np.testing.assert_allclose(r["topk_weight"].numpy(), g["topk_weight"], rtol=1e-6, atol=1e-8)
    np.testing.assert_allclose(r["out"].reshape(-1, 1152)[:: G.C0_ROW_STRIDE].numpy(), g["out_rows"], rtol=1e-4, atol=2e-6)


def test_permutation_helpers_round_trip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 16, generator=g)
    flat = torch.randint(0, 8, (74,), generator=g)
    rows, order = O.permute_rows(x, flat, 2)
    assert torch.equal(O.unpermute_rows(rows, order).view(37, 2, 16)[:, 0], x)
    srt = flat[order]
    assert bool((srt[1:] >= srt[:-1]).all())
    # stable: rows of one expert keep their original order
    for e in range(8):
        sel = order[srt == e]
        assert bool((sel[1:] > sel[:-1]).all())


def test_top2_tie_rule():
    s = torch.tensor([[0.1, 0.3, 0.3, 0.3], [0.25, 0.25, 0.25, 0.25], [0.0, 0.5, 0.2, 0.5]])
    _, idx = O.top2_from_scores(s)
    assert idx.tolist() == [[1, 2], [0, 1], [1, 3]]


def test_forced_sync_schedule_matches_warmup_rules():
    # first step always; warm-up steps; strided; cool-down ignored without warm-up/stride (warmup.py:13-14)
    assert O.forced_sync_schedule(8, 0, 0, 0) == [True] + [False] * 7
    assert O.forced_sync_schedule(8, 2, 0, 0) == [True, True, True] + [False] * 5
    assert O.forced_sync_schedule(8, 0, 3, 0) == [True, False, True, False, False, True, False, False]
    assert O.forced_sync_schedule(8, 0, 0, 3) == [True] + [False] * 7
    assert O.forced_sync_schedule(8, 1, 0, 2) == [True, True, False, False, False, False, True, True]


@pytest.mark.skipif(not reference_available(), reason="reference checkout not present")
def test_oracle_against_reference_modules():
    ref = load_reference()
    torch.manual_seed(7)
    pm = ref.models.ParaMode()
    blk = ref.models.SparseMoeBlock(48, 4, 8, 2, pretraining_tp=1, layer_idx=0, total_layers=1, para_mode=pm).eval()
    x = torch.randn(2, 50, 48)
    with torch.no_grad():
        idx, w, _ = blk.gate(x)
        y = blk(x)
    ex, sh = _experts_from_sd(blk.state_dict(), 8)
    r = O.moe_block_forward(x, blk.gate.weight.detach(), ex, sh)
    assert torch.equal(r["topk_idx"], idx)
    torch.testing.assert_close(r["topk_weight"], w, rtol=1e-6, atol=1e-8)
    torch.testing.assert_close(r["out"], y, rtol=1e-5, atol=1e-6)
    # warm-up schedule and layer keys
    import importlib

    warmup = None
    try:
        warmup = importlib.import_module("diffusion.warmup")
    except Exception:
        pass
    if warmup is not None:
        for wu, st, cd in [(0, 0, 0), (2, 0, 0), (0, 3, 0), (1, 0, 2), (5, 4, 3)]:
            p = ref.models.ParaMode(ep=True, ep_async=True, ep_async_warm_up=wu, strided_sync=st, ep_async_cool_down=cd)
            want = [bool(warmup.ep_forced_sync(i, 12, p)) for i in range(12, 0, -1)]
            assert O.forced_sync_schedule(12, wu, st, cd) == want
    ref.diep.ep_cache_init(6, selective_async_strategy="all")
    for strat in ("all", "shallow", "deep", "interleaved"):
        ref.diep._selective_async_strategy = strat
        for key in range(6):
            assert O.past_layer_key(key, 6, strat) == ref.diep._past_layer_key(key)
