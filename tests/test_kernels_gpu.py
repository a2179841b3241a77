"""Parity of each CUDA kernel (called through the C ABI) with the CPU oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _ops():
    from dice_b200 import ops

    return ops


# --------------------------------------------------------------------------- #
# router
# --------------------------------------------------------------------------- #


@pytest.mark.parametrize("n,h,e", [(1, 64, 8), (2, 1152, 8), (127, 1152, 8), (512, 1152, 8), (129, 1792, 16), (333, 256, 5), (64, 128, 32), (40, 128, 64)])
@pytest.mark.parametrize("renorm", [False, True])
def test_router_fp32_bit_exact_routing(cuda_device, n, h, e, renorm):
    ops = _ops()
    g = torch.Generator().manual_seed(n * 7 + h + e)
    x = torch.randn(n, h, generator=g)
    wg = torch.randn(e, h, generator=g) * 0.02
    idx_o, w_o, _ = O.gate_top2(x, wg, renorm)
    idx, w, hist, logits = ops.router_top2(x.to(cuda_device), wg.to(cuda_device), renorm, want_logits=True)
    assert torch.equal(idx.cpu(), idx_o)
    torch.testing.assert_close(w.cpu(), w_o, rtol=1e-5, atol=1e-7)
    assert torch.equal(hist.cpu().long(), O.expert_histogram(idx_o.reshape(-1), e))
    torch.testing.assert_close(logits.cpu(), x @ wg.t(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("n,h,e", [(512, 1152, 8), (2048, 1792, 16), (4096, 1408, 16)])
def test_router_bf16_against_oracle(cuda_device, n, h, e):
    """bf16: logits may differ from the oracle's by one bf16 ulp (plus the
    fp32 summation-order error, which dominates for logits near zero); every
    routing mismatch must be such a near-tie."""
    ops = _ops()
    g = torch.Generator().manual_seed(n + h + e)
    x = torch.randn(n, h, generator=g).bfloat16()
    wg = (torch.randn(e, h, generator=g) * 0.05).bfloat16()
    idx_o, w_o, logits_o = O.gate_top2(x, wg)
    idx, w, hist, logits = ops.router_top2(x.to(cuda_device), wg.to(cuda_device), False, want_logits=True)
    idx, w, logits = idx.cpu(), w.cpu(), logits.cpu()
    # logits within one bf16 ulp of the oracle's
    lf, lo = logits.float(), logits_o.float()
    ulp = torch.maximum(lo.abs(), torch.tensor(2.0 ** -126)).log2().floor().exp2() * 2.0 ** -7
    assert ((lf - lo).abs() <= ulp + 2e-5).all()
    # the kernel's selection is exactly the oracle's selection on the kernel's own logits
    w_sel, idx_sel = O.top2_from_scores(logits.float().softmax(-1))
    assert torch.equal(idx, idx_sel)
    torch.testing.assert_close(w, w_sel, rtol=2e-6, atol=1e-8)
    mism = (idx != idx_o).any(-1)
    # mismatching tokens: the logits of the disputed experts differ by <= 1 ulp in the oracle
    for t in mism.nonzero().flatten().tolist():
        a = set(idx[t].tolist()) ^ set(idx_o[t].tolist())
        vals = lo[t, sorted(a)]
        assert (vals.max() - vals.min()).abs() <= 2 * ulp[t].max() + 4e-5 or set(idx[t].tolist()) == set(idx_o[t].tolist())
    assert mism.float().mean() < 0.02
    assert int(hist.sum()) == 2 * n


def test_selection_tie_rule_matches_cuda_topk(cuda_device):
    """Crafted ties: the selection must reproduce torch.topk(k=2, sorted=False)
    of the CUDA backend on the softmax scores (models.py:186-191)."""
    ops = _ops()
    rows = [
        [0.1, 0.3, 0.3, 0.3, 0.0, 0.0, 0.0, 0.0],
        [0.25, 0.25, 0.25, 0.25, 0.0, 0.0, 0.0, 0.0],
        [1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0],
        [0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 2.0, 2.0],
        [3.0, 0.0, 0.0, 3.0, 0.0, 1.0, 0.0, 0.0],
        [0.0, 1.0, 0.5, 0.5, 0.5, 0.0, 0.0, 0.0],
        [-1.0, -1.0, -2.0, -3.0, -1.0, -4.0, -5.0, -6.0],
    ]
    g = torch.Generator().manual_seed(5)
    rnd = (torch.randn(4096, 8, generator=g) * 2).bfloat16().float()  # many exact ties after bf16 rounding
    logits = torch.cat([torch.tensor(rows), rnd]).to(cuda_device)
    idx, w, hist = ops.top2_from_logits(logits)
    scores = logits.softmax(-1)
    tw, ti = torch.topk(scores, k=2, dim=-1, sorted=False)
    assert torch.equal(idx, ti)
    torch.testing.assert_close(w, tw, rtol=2e-6, atol=1e-8)
    w_o, idx_o = O.top2_from_scores(logits.cpu().softmax(-1))
    assert torch.equal(idx.cpu(), idx_o)


# --------------------------------------------------------------------------- #
# permutation
# --------------------------------------------------------------------------- #


@pytest.mark.parametrize("n,e,k", [(1, 8, 2), (2, 8, 2), (127, 8, 2), (128, 8, 2), (129, 8, 2), (5000, 16, 2), (777, 8, 1), (300, 64, 2)])
def test_permute_plan_is_stable_argsort(cuda_device, n, e, k):
    ops = _ops()
    g = torch.Generator().manual_seed(n + e)
    flat = torch.randint(0, e, (n * k,), generator=g)
    if n >= 127:
        flat[flat == 3] = 2  # an empty expert
    pos, seg, order = ops.permute_plan(flat.to(cuda_device), e, want_order=True)
    order_o = O.stable_expert_order(flat)
    assert torch.equal(order.cpu().long(), order_o)
    inv = torch.empty_like(order_o)
    inv[order_o] = torch.arange(n * k)
    assert torch.equal(pos.cpu().long(), inv)
    hist = O.expert_histogram(flat, e)
    assert torch.equal(seg.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), hist.cumsum(0)]))


def test_permute_plan_all_rows_one_expert_and_empty(cuda_device):
    ops = _ops()
    flat = torch.full((1000,), 5, dtype=torch.int64)
    pos, seg, order = ops.permute_plan(flat.to(cuda_device), 8, want_order=True)
    assert torch.equal(pos.cpu().long(), torch.arange(1000))
    assert seg.cpu().tolist() == [0] * 6 + [1000] * 3
    pos, seg, _ = ops.permute_plan(torch.empty(0, dtype=torch.int64, device=cuda_device), 8)
    assert seg.cpu().tolist() == [0] * 9 and pos.numel() == 0


@pytest.mark.parametrize("n,h,e", [(1, 64, 8), (127, 64, 8), (128, 128, 8), (129, 64, 8), (1000, 256, 16), (16384, 1152, 8), (4096, 1792, 16)])
def test_router_files_a_histogram_per_128_tokens(cuda_device, n, h, e):
    """The bf16 router's per-chunk table equals a bincount of every 128 tokens' selections; routing is unchanged."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(n + h)
    x = torch.randn(n, h, generator=g, device=cuda_device).bfloat16()
    wg = (torch.randn(e, h, generator=g, device=cuda_device) * 0.05).bfloat16()
    idx, w, hist, _ = ops.router_top2(x, wg)
    idx2, w2, chunks, _ = ops.router_top2(x, wg, want_chunks=True)
    assert torch.equal(idx, idx2) and torch.equal(w, w2)
    assert chunks.shape == ((n + 127) // 128, e)
    ic = idx.cpu()
    want = torch.stack([O.expert_histogram(ic[c * 128:(c + 1) * 128].reshape(-1), e) for c in range((n + 127) // 128)])
    assert torch.equal(chunks.cpu().long(), want)
    assert torch.equal(chunks.sum(0), hist)


@pytest.mark.parametrize("n,e,world,k", [(1, 8, 1, 2), (127, 8, 1, 2), (129, 8, 2, 2), (1000, 8, 8, 2), (5000, 16, 8, 2),
                                         (16384, 8, 1, 2), (3000, 16, 4, 2), (300, 64, 1, 2), (777, 8, 4, 1)])
def test_chunked_plan_equals_three_pass_plan(cuda_device, n, e, world, k):
    """dice_permute_plan_chunked (one launch, from per-256-row histograms, keys = (owner rank, local slot) of the
    round-robin placement, optional fused row gather) gives exactly the plan and the rows of
    dice_permute_plan on those keys + dice_permute_rows, which are checked against the oracle's stable argsort."""
    ops = _ops()
    h = 64
    g = torch.Generator().manual_seed(n + e + world)
    flat = torch.randint(0, e, (n * k,), generator=g)
    if n >= 127:
        flat[flat == 3] = 2  # an empty expert
    x = torch.randn(n, h, generator=g).bfloat16().to(cuda_device)
    chunks = torch.stack([O.expert_histogram(flat[c * 256:(c + 1) * 256], e) for c in range((n * k + 255) // 256)])
    chunks = chunks.to(torch.int32).to(cuda_device)
    el = e // world
    keys = (flat % world) * el + flat // world
    pos_w, seg_w, order_w = ops.permute_plan(keys.to(cuda_device), e, want_order=True)
    rows_w = ops.permute_rows(x, pos_w, k)
    order_o = O.stable_expert_order(keys)
    assert torch.equal(order_w.cpu().long(), order_o)
    pos, seg, order, rows = ops.permute_plan_chunked(flat.to(cuda_device), chunks, e, world, x, k, want_order=True)
    assert torch.equal(pos, pos_w) and torch.equal(seg, seg_w) and torch.equal(order, order_w)
    assert torch.equal(rows, rows_w)
    pos2, seg2, _, none = ops.permute_plan_chunked(flat.to(cuda_device), chunks, e, world)
    assert none is None and torch.equal(pos2, pos_w) and torch.equal(seg2, seg_w)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,h,e", [(1, 64, 8), (129, 1152, 8), (512, 1792, 16)])
def test_permute_rows_and_unpermute_combine(cuda_device, dtype, n, h, e):
    ops = _ops()
    g = torch.Generator().manual_seed(n + h)
    x = torch.randn(n, h, generator=g).to(dtype)
    flat = torch.randint(0, e, (n * 2,), generator=g)
    w = torch.rand(n, 2, generator=g)
    shared = torch.randn(n, h, generator=g).to(dtype)
    pos, seg, _ = ops.permute_plan(flat.to(cuda_device), e)
    rows = ops.permute_rows(x.to(cuda_device), pos, 2)
    rows_o, order_o = O.permute_rows(x, flat, 2)
    assert torch.equal(rows.cpu(), rows_o)  # pure data movement: bit exact
    # combine: weighted pair sum of the (here: identity-processed) rows + addend
    wd = w.to(cuda_device)
    out = ops.unpermute_combine(rows, pos[0::2], rows, pos[1::2], wd[:, 0], wd[:, 1], n, addend=shared.to(cuda_device))
    flat_rows = O.unpermute_rows(rows_o, order_o)
    want = (flat_rows.float().view(n, 2, h) * w.view(n, 2, 1)).sum(1) + shared.float()
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.cpu().float(), want, **tol)
    # single-source form with identity index and unit weight = plain un-permute of slot 0
    slot0 = ops.unpermute_combine(rows, pos[0::2], None, None, None, None, n)
    assert torch.equal(slot0.cpu(), x)


def test_permute_round_trip_full_size(cuda_device):
    """Size-independent property at the benchmark's size: permute then
    un-permute with weights (1, 0) returns the input."""
    ops = _ops()
    n, h, e = 16384, 1152, 8
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(n, h, generator=g, device=cuda_device).bfloat16()
    flat = torch.randint(0, e, (2 * n,), generator=g, device=cuda_device)
    pos, seg, order = ops.permute_plan(flat, e, want_order=True)
    assert int(seg[-1]) == 2 * n
    srt = flat[order.long()]
    assert bool((srt[1:] >= srt[:-1]).all())  # sortedness
    rows = ops.permute_rows(x, pos, 2)
    ones = torch.ones(n, 2, device=cuda_device)
    zeros = torch.zeros(n, 2, device=cuda_device)
    back = ops.unpermute_combine(rows, pos[0::2], rows, pos[1::2], ones[:, 0], zeros[:, 1], n)
    assert torch.equal(back, x)


# --------------------------------------------------------------------------- #
# grouped GEMM / FFN
# --------------------------------------------------------------------------- #


def _segments(counts, device):
    return torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=device)


@pytest.mark.parametrize(
    "counts,k,n",
    [
        ([128], 64, 256),        # one tile, one k-block
        ([128], 16, 32),         # a single MMA
        ([128], 128, 256),       # two k-blocks
        ([128], 1152, 256),      # full reduction depth, ring wrap-around
        ([256], 320, 512),       # 2x2 tiles
        ([100], 64, 64),         # ragged rows, narrow n
        ([1, 0, 129, 37], 1152, 1152),  # ragged segments, empty segment, n = 4.5 tiles
        ([300, 300, 300, 300, 300, 300, 300, 300], 1152, 4608),
        ([511, 513], 4608, 1152),
    ],
)
def test_grouped_gemm_store(cuda_device, counts, k, n):
    ops = _ops()
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    r, s = sum(counts), len(counts)
    a = torch.randn(r, k, generator=g).bfloat16()
    w = (torch.randn(s, n, k, generator=g) / math.sqrt(k)).bfloat16()
    seg = _segments(counts, cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.full((r + 3, n), 7.0, dtype=torch.bfloat16, device=cuda_device)  # canary rows
    ops.grouped_gemm(a.to(cuda_device), w.to(cuda_device), seg, ops.EPI_STORE, n, status, out=out)
    torch.cuda.synchronize()
    ops.check_status(status)
    want = torch.cat([a[seg[i] : seg[i + 1]].float() @ w[i].float().t() for i in range(s)])
    torch.testing.assert_close(out[:r].cpu().float(), want, rtol=2e-2, atol=2e-2)
    assert bool((out[r:] == 7.0).all())


@pytest.mark.parametrize("act", ["swiglu", "gelu_tanh"])
@pytest.mark.parametrize("counts,h,f", [([111], 32, 128), ([5, 0, 200, 51], 128, 512), ([130, 126, 257, 0, 3, 64, 64, 380], 1152, 4608)])
def test_grouped_ffn_bf16(cuda_device, act, counts, h, f):
    ops = _ops()
    g = torch.Generator().manual_seed(sum(counts) + h + f)
    r, s = sum(counts), len(counts)
    x = torch.randn(r, h, generator=g).bfloat16()
    mk = lambda *shape: (torch.randn(*shape, generator=g) / math.sqrt(shape[-1])).bfloat16()
    if act == "swiglu":
        experts = [(mk(f, h), mk(f, h), mk(h, f)) for _ in range(s)]
        w1 = torch.stack([ops.pack_w13(e[0].to(cuda_device), e[1].to(cuda_device)) for e in experts])
        w2 = torch.stack([e[2] for e in experts]).to(cuda_device)
    else:
        experts = [(mk(f, h), mk(h, f)) for _ in range(s)]
        w1 = torch.stack([e[0] for e in experts]).to(cuda_device)
        w2 = torch.stack([e[1] for e in experts]).to(cuda_device)
    seg = _segments(counts, cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = ops.grouped_ffn(x.to(cuda_device), w1, w2, seg, act, f, status)
    torch.cuda.synchronize()
    ops.check_status(status)
    want = torch.cat(
        [O.run_expert(x[seg[i] : seg[i + 1]].float(), [t.float() for t in experts[i]], act) for i in range(s)]
    )
    err = (out.cpu().float() - want).norm() / want.norm()
    assert err < 2e-2, f"relative error {err}"
    torch.testing.assert_close(out.cpu().float(), want, rtol=5e-2, atol=5e-2 * want.abs().max().item())


@pytest.mark.parametrize("act", ["swiglu", "gelu_tanh"])
def test_grouped_ffn_fp32(cuda_device, act):
    ops = _ops()
    counts, h, f = [70, 0, 3, 64, 129], 96, 200
    g = torch.Generator().manual_seed(11)
    r, s = sum(counts), len(counts)
    x = torch.randn(r, h, generator=g)
    mk = lambda *shape: torch.randn(*shape, generator=g) / math.sqrt(shape[-1])
    if act == "swiglu":
        experts = [(mk(f, h), mk(f, h), mk(h, f)) for _ in range(s)]
        w1 = torch.stack([ops.pack_w13(e[0].to(cuda_device), e[1].to(cuda_device)) for e in experts])
        w2 = torch.stack([e[2] for e in experts]).to(cuda_device)
    else:
        experts = [(mk(f, h), mk(h, f)) for _ in range(s)]
        w1 = torch.stack([e[0] for e in experts]).to(cuda_device)
        w2 = torch.stack([e[1] for e in experts]).to(cuda_device)
    seg = _segments(counts, cuda_device)
    out = ops.grouped_ffn(x.to(cuda_device), w1, w2, seg, act, f)
    want = torch.cat([O.run_expert(x[seg[i] : seg[i + 1]], experts[i], act) for i in range(s)])
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5)


def test_grouped_gemm_rejects_bad_segments(cuda_device):
    """Non-monotone segment offsets: the kernel records a status code and does
    no work (bounded, no fault)."""
    ops = _ops()
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(2, 32, 64, dtype=torch.bfloat16, device=cuda_device)
    seg = torch.tensor([0, 200, 100], dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    ops.grouped_gemm(a, w, seg, ops.EPI_STORE, 32, status)
    with pytest.raises(RuntimeError, match="segment offsets"):
        ops.check_status(status)


def test_linearity_full_size_ffn_gemm(cuda_device):
    """Size-independent property at the benchmark's shape: the store-epilogue
    GEMM is linear in its input: f(a) + f(b) == f(a + b) up to bf16 rounding,
    and row r of the output depends only on row r and its expert's weights."""
    ops = _ops()
    r, k, n, s = 32768, 1152, 1152, 8
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randn(r, k, generator=g, device=cuda_device).bfloat16()
    w = (torch.randn(s, n, k, generator=g, device=cuda_device) / math.sqrt(k)).bfloat16()
    counts = torch.tensor([4000, 4200, 3900, 4100, 4096, 4096, 4288, 4088])
    seg = _segments(counts.tolist(), cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = ops.grouped_gemm(a, w, seg, ops.EPI_STORE, n, status)
    torch.cuda.synchronize()
    ops.check_status(status)
    # spot-check 64 random rows against fp32 math
    rows = torch.randint(0, r, (64,), generator=torch.Generator().manual_seed(1))
    ends = counts.cumsum(0)
    for row in rows.tolist():
        e = int((ends > row).nonzero()[0])
        want = a[row].float() @ w[e].float().t()
        torch.testing.assert_close(out[row].float(), want, rtol=2e-2, atol=2e-2)
    out2 = ops.grouped_gemm((a * 2).contiguous(), w, seg, ops.EPI_STORE, n, status)
    torch.testing.assert_close(out2.float(), out.float() * 2, rtol=1e-2, atol=1e-2)


def test_exchange_wait_runs_out_and_reports(cuda_device):
    """Failure detection without a fault: a flag that nothing raises makes the
    bounded wait expire; the kernel returns, the status word names the reason
    and the context stays usable."""
    import time

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    flags = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    t0 = time.time()
    rc = lib.dice_ep_wait_flags(flags.data_ptr(), 2, 1, 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 10.0
    with pytest.raises(RuntimeError, match="dispatched rows"):
        ops.check_status(status)
    # a raised flag passes at once, and the device still works
    flags.fill_(5)
    rc = lib.dice_ep_wait_flags(flags.data_ptr(), 2, 5, 1, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert int((flags + 1).sum()) == 48


def test_exchange_wait_limit_is_configurable(cuda_device):
    """dice_ep_set_wait_limit_ms: the bounded waits of the exchange kernels follow the limit set for the device
    (ranks that may stall for seconds between two exchanges need more than the default 2 s)."""
    import time

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    assert lib.dice_ep_set_wait_limit_ms(50) != 0 and lib.dice_ep_set_wait_limit_ms(4 * 3600 * 1000) != 0  # out of range
    flags = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    try:
        assert lib.dice_ep_set_wait_limit_ms(300) == 0
        torch.cuda.synchronize()
        t0 = time.time()
        assert lib.dice_ep_wait_flags(flags.data_ptr(), 2, 1, 1, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        assert 0.25 < time.time() - t0 < 1.5
        with pytest.raises(RuntimeError, match="expert outputs"):
            ops.check_status(status)
    finally:
        assert lib.dice_ep_set_wait_limit_ms(2000) == 0


def test_exchange_world_of_one(cuda_device):
    """The four exchange kernels on one GPU (world of one rank: every 'peer' is
    the rank itself): dispatch + return reproduce the plain permutation."""
    import ctypes

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    n, h, e = 777, 256, 8
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, h, generator=g).bfloat16().to(cuda_device)
    flat = torch.randint(0, e, (2 * n,), generator=g).to(cuda_device)
    pos, seg, _ = ops.permute_plan(flat, e)
    cap = 2 * n + 5
    ctrl = torch.zeros(e + 3 * 64, dtype=torch.int32, device=cuda_device)
    recv = torch.full((cap, h), 3.0, dtype=torch.bfloat16, device=cuda_device)
    back = torch.zeros((2 * n, h), dtype=torch.bfloat16, device=cuda_device)
    meta = torch.zeros(lib.dice_ep_meta_ints(1, e), dtype=torch.int32, device=cuda_device)
    done = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    tab = lambda p: (ctypes.c_void_p * 1)(p)
    f = lambda i: ctrl.data_ptr() + (e + 64 * i) * 4
    for seq in (1, 2):  # twice: the done counters and flags must be reusable
        assert lib.dice_ep_exchange_counts(seg.data_ptr(), tab(ctrl.data_ptr()), tab(f(0)), meta.data_ptr(), 0, 1, e, cap,
                                           seq, status.data_ptr(), st) == 0
        assert lib.dice_ep_dispatch_rows(x.data_ptr(), pos.data_ptr(), seg.data_ptr(), meta.data_ptr(), tab(recv.data_ptr()),
                                         tab(f(1)), done.data_ptr(), n, 2, h, 0, 0, 1, e, cap, seq, 7 * (seq - 1), 0, None, status.data_ptr(), st) == 0
        assert lib.dice_ep_wait_flags(f(1), 1, seq, 0, status.data_ptr(), st) == 0
        assert lib.dice_ep_return_rows(recv.data_ptr(), meta.data_ptr(), tab(back.data_ptr()), tab(f(2)), done[1:].data_ptr(),
                                       h, 0, 0, 1, 2 * n, cap, seq, 5 * (seq - 1), status.data_ptr(), st) == 0
        assert lib.dice_ep_wait_flags(f(2), 1, seq, 1, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        ops.check_status(status)
        want = ops.permute_rows(x, pos, 2)
        assert torch.equal(recv[: 2 * n], want) and torch.equal(back, want)
        assert bool((recv[2 * n:] == 3.0).all())
        m = meta.cpu().tolist()
        assert m[0] == 2 * n and m[1] == 0                                # rows received, state
        assert m[2] == 0 and m[3] == 0 and m[4:6] == [0, 2 * n] and m[6] == 2 * n   # send_base, back_base, src_off, src_cnt
        assert m[7:7 + e + 1] == seg.cpu().tolist()
    # a receive buffer that is too small is reported, not overrun
    assert lib.dice_ep_exchange_counts(seg.data_ptr(), tab(ctrl.data_ptr()), tab(f(0)), meta.data_ptr(), 0, 1, e, 100, 3,
                                       status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="more rows"):
        ops.check_status(status)



@pytest.mark.parametrize("n,h,k,dtype", [(777, 256, 2, torch.bfloat16), (1000, 1152, 2, torch.bfloat16),
                                         (333, 1152, 2, torch.float32), (129, 1792, 1, torch.bfloat16),
                                         (5, 64, 2, torch.bfloat16), (4097, 1152, 2, torch.bfloat16)])
def test_exchange_bulk_copy_pushes_equal_simt_pushes(cuda_device, n, h, k, dtype):
    """Dispatch and return exist in three forms: SIMT kernels (max_ctas < 0), kernels that move the rows with
    cp.async.bulk through shared memory on every SM (max_ctas == 0), and the same on a few four-warp CTAs
    launched as clusters of two (max_ctas > 0, the form that runs next to the expert FFN).  World of one rank, a tenth of the rows left out
    (expert -1, as conditional communication does): both forms must write the same bytes and touch nothing else."""
    import ctypes

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    e = 8
    g = torch.Generator().manual_seed(n + h)
    x = torch.randn(n, h, generator=g).to(dtype).to(cuda_device)
    flat = torch.randint(0, e, (k * n,), generator=g)
    flat[torch.rand(k * n, generator=g) < 0.1] = -1
    flat = flat.to(cuda_device)
    pos, seg, _ = ops.permute_plan(flat, e)
    rows = int(seg[-1].item())
    cap = rows + 3
    code = 0 if dtype == torch.bfloat16 else 1
    st = torch.cuda.current_stream().cuda_stream
    tab = lambda p: (ctypes.c_void_p * 1)(p)
    outs = []
    for max_ctas in (0, -1, 6):
        ctrl = torch.zeros(e + 3 * 64, dtype=torch.int32, device=cuda_device)
        recv = torch.full((cap, h), 3.0, dtype=dtype, device=cuda_device)
        back = torch.full((cap, h), 5.0, dtype=dtype, device=cuda_device)
        meta = torch.zeros(lib.dice_ep_meta_ints(1, e), dtype=torch.int32, device=cuda_device)
        done = torch.zeros(2, dtype=torch.int32, device=cuda_device)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        f = lambda i: ctrl.data_ptr() + (e + 64 * i) * 4
        for seq in (1, 2):
            assert lib.dice_ep_exchange_counts(seg.data_ptr(), tab(ctrl.data_ptr()), tab(f(0)), meta.data_ptr(), 0, 1, e,
                                               cap, seq, status.data_ptr(), st) == 0
            assert lib.dice_ep_dispatch_rows(x.data_ptr(), pos.data_ptr(), seg.data_ptr(), meta.data_ptr(),
                                             tab(recv.data_ptr()), tab(f(1)), done.data_ptr(), n, k, h, code, 0, 1, e, cap,
                                             seq, max_ctas, 0, None, status.data_ptr(), st) == 0
            assert lib.dice_ep_wait_flags(f(1), 1, seq, 0, status.data_ptr(), st) == 0
            assert lib.dice_ep_return_rows(recv.data_ptr(), meta.data_ptr(), tab(back.data_ptr()), tab(f(2)),
                                           done[1:].data_ptr(), h, code, 0, 1, cap, cap, seq, max_ctas, status.data_ptr(),
                                           st) == 0
            assert lib.dice_ep_wait_flags(f(2), 1, seq, 1, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        ops.check_status(status)
        outs.append((recv.clone(), back.clone()))
    (recv_bulk, back_bulk), (recv_simt, back_simt), (recv_few, back_few) = outs
    assert torch.equal(recv_bulk, recv_simt) and torch.equal(back_bulk, back_simt)
    assert torch.equal(recv_bulk, recv_few) and torch.equal(back_bulk, back_few)
    assert bool((recv_bulk[rows:] == 3.0).all()) and bool((back_bulk[rows:] == 5.0).all())
    # and the rows are the permutation of x: row r of the receive order is the token whose slot has pos == r
    p = pos.cpu().view(n, k)
    t_of = torch.full((rows,), -1, dtype=torch.long)
    for s in range(k):
        m = p[:, s] >= 0
        t_of[p[m, s].long()] = torch.nonzero(m).flatten()
    assert bool((t_of >= 0).all())
    assert torch.equal(recv_bulk[:rows].cpu(), x.cpu()[t_of])



@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("max_ctas", [0, -1, 4])
def test_exchange_of_emulated_ranks_on_one_gpu(cuda_device, world, max_ctas):
    """The whole exchange for `world` ranks whose buffers all live on this GPU.  The count matrices and count
    flags are filled in beforehand and every push is launched before the first wait, so no kernel ever waits
    for a later one.  With the identity as expert FFN, every rank must get back exactly its own key-sorted
    rows, and every receive buffer must hold its sources' rows in (source, slot) order.  max_ctas 0: bulk-copy
    pushes, -1: SIMT pushes, 4: bulk-copy pushes on at most four CTAs."""
    import ctypes

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    e, h, k = 8, 256, 2
    el = e // world
    n = [300 + 37 * r for r in range(world)]  # tokens per rank (ragged)
    g = torch.Generator().manual_seed(world)
    xs, poss, segs, sorted_rows = [], [], [], []
    for r in range(world):
        x = torch.randn(n[r], h, generator=g).bfloat16().to(cuda_device)
        expert = torch.randint(0, e, (k * n[r],), generator=g)
        key = (expert % world) * el + expert // world  # (owner rank, local slot) of a round-robin expert
        pos, seg, _ = ops.permute_plan(key.to(cuda_device), e)
        xs.append(x); poss.append(pos); segs.append(seg); sorted_rows.append(ops.permute_rows(x, pos, k))
    seg_host = [s.cpu().tolist() for s in segs]
    recv_rows = [sum(seg_host[s][(d + 1) * el] - seg_host[s][d * el] for s in range(world)) for d in range(world)]
    cap = max(recv_rows) + 7
    flag_base = world * e
    ctrl = [torch.zeros(flag_base + 3 * 64, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    recv = [torch.full((cap, h), 3.0, dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    back_cap = k * max(n) + 2  # every rank offers the same return capacity
    back = [torch.full((back_cap, h), 5.0, dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    meta = [torch.zeros(lib.dice_ep_meta_ints(world, el), dtype=torch.int32, device=cuda_device) for _ in range(world)]
    done = [torch.zeros(2, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    table = lambda ptrs: (ctypes.c_void_p * world)(*ptrs)
    flags = lambda which: table([c.data_ptr() + (flag_base + 64 * which) * 4 for c in ctrl])
    my_flags = lambda r, which: ctrl[r].data_ptr() + (flag_base + 64 * which) * 4
    seq = 1
    counts = torch.tensor([[seg_host[r][i + 1] - seg_host[r][i] for i in range(e)] for r in range(world)], dtype=torch.int32)
    for d in range(world):  # what every rank's count kernel will publish, and the flags that say so
        ctrl[d][:flag_base] = counts.flatten().to(cuda_device)
        ctrl[d][flag_base:flag_base + world] = seq
    for r in range(world):
        assert lib.dice_ep_exchange_counts(segs[r].data_ptr(), table([c.data_ptr() for c in ctrl]), flags(0),
                                           meta[r].data_ptr(), r, world, e, cap, seq, status.data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), meta[r].data_ptr(),
                                         table([t.data_ptr() for t in recv]), flags(1), done[r].data_ptr(), n[r], k, h, 0,
                                         r, world, e, cap, seq, max_ctas, 0, None, status.data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(my_flags(r, 1), world, seq, 0, status.data_ptr(), st) == 0
    for r in range(world):  # identity FFN: the received rows go straight back
        assert lib.dice_ep_return_rows(recv[r].data_ptr(), meta[r].data_ptr(), table([t.data_ptr() for t in back]), flags(2),
                                       done[r][1:].data_ptr(), h, 0, r, world, back_cap, cap, seq, max_ctas,
                                       status.data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(my_flags(r, 2), world, seq, 1, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    ops.check_status(status)
    for r in range(world):
        assert torch.equal(back[r][: k * n[r]], sorted_rows[r]), f"rank {r} did not get its rows back"
        assert bool((back[r][k * n[r]:] == 5.0).all())
    for d in range(world):
        want = torch.cat([sorted_rows[s][seg_host[s][d * el]: seg_host[s][(d + 1) * el]] for s in range(world)])
        assert torch.equal(recv[d][: recv_rows[d]], want), f"receive buffer of rank {d}"
        assert bool((recv[d][recv_rows[d]:] == 3.0).all())


class _EmulatedRanks:
    """Buffers of `world` ranks on one GPU for the exchange kernels, as PeerExchange lays them out per slot."""

    def __init__(self, world, e, h, cap, back_cap, device, lib):
        import ctypes

        self.world, self.e, self.el, self.h, self.cap, self.back_cap = world, e, e // world, h, cap, back_cap
        self.flag_base = world * e
        self.ctrl = [torch.zeros(self.flag_base + 3 * 64, dtype=torch.int32, device=device) for _ in range(world)]
        self.recv = [torch.full((cap + 4, h), 3.0, dtype=torch.bfloat16, device=device) for _ in range(world)]  # 4 guard rows
        self.back = [torch.full((back_cap + 4, h), 5.0, dtype=torch.bfloat16, device=device) for _ in range(world)]
        self.meta = [torch.zeros(lib.dice_ep_meta_ints(world, self.el), dtype=torch.int32, device=device) for _ in range(world)]
        self.done = [torch.zeros(2, dtype=torch.int32, device=device) for _ in range(world)]
        self.status = [torch.zeros(1, dtype=torch.int32, device=device) for _ in range(world)]
        self._ct = ctypes

    def table(self, ptrs):
        return (self._ct.c_void_p * self.world)(*ptrs)

    def flags(self, which):
        return self.table([c.data_ptr() + (self.flag_base + 64 * which) * 4 for c in self.ctrl])

    def my_flags(self, r, which):
        return self.ctrl[r].data_ptr() + (self.flag_base + 64 * which) * 4

    def publish_counts(self, seg_host, seq, ranks=None):
        """What the count kernels of `ranks` would publish on every peer, and the flags that say so."""
        e = self.e
        for r in (range(self.world) if ranks is None else ranks):
            row = torch.tensor([seg_host[r][i + 1] - seg_host[r][i] for i in range(e)], dtype=torch.int32)
            for d in range(self.world):
                self.ctrl[d][r * e:(r + 1) * e] = row.to(self.ctrl[d].device)
                self.ctrl[d][self.flag_base + r] = seq


def _emulated_inputs(world, e, h, n, k, device, seed, hot_owner=None):
    ops = _ops()
    el = e // world
    g = torch.Generator().manual_seed(seed)
    xs, poss, segs = [], [], []
    for r in range(world):
        x = torch.randn(n[r], h, generator=g).bfloat16().to(device)
        expert = torch.randint(0, e, (k * n[r],), generator=g)
        if hot_owner is not None:  # three quarters of the rows go to one rank's experts
            hot = torch.rand(k * n[r], generator=g) < 0.75
            expert[hot] = hot_owner + world * torch.randint(0, el, (int(hot.sum()),), generator=g)
        key = (expert % world) * el + expert // world
        pos, seg, _ = ops.permute_plan(key.to(device), e)
        xs.append(x); poss.append(pos); segs.append(seg)
    return xs, poss, segs


@pytest.mark.parametrize("max_ctas", [0, -1, 4])
def test_exchange_overflow_is_found_by_every_rank_and_touches_nothing(cuda_device, max_ctas):
    """A routing that sends one rank more rows than its receive buffer holds (the reference has no capacity,
    ep_fwd.py:247-293, so this can only be reported, not reproduced): every rank records the overflow in the
    count exchange, the pushes and the return then move nothing, the guard rows behind every buffer stay
    untouched, and no flag is left unraised."""
    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    world, e, h, k = 4, 8, 256, 2
    n = [400, 380, 420, 390]
    xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=21, hot_owner=2)
    seg_host = [s.cpu().tolist() for s in segs]
    el = e // world
    recv_rows = [sum(seg_host[s][(d + 1) * el] - seg_host[s][d * el] for s in range(world)) for d in range(world)]
    cap = 2 * max(n)  # what two average senders fill: too small for the hot rank
    assert recv_rows[2] > cap > max(recv_rows[:2] + recv_rows[3:])
    R = _EmulatedRanks(world, e, h, cap, k * max(n), cuda_device, lib)
    st = torch.cuda.current_stream().cuda_stream
    seq = 1
    R.publish_counts(seg_host, seq)
    for r in range(world):
        assert lib.dice_ep_exchange_counts(segs[r].data_ptr(), R.table([c.data_ptr() for c in R.ctrl]), R.flags(0),
                                           R.meta[r].data_ptr(), r, world, e, cap, seq, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), R.meta[r].data_ptr(),
                                         R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r], k,
                                         h, 0, r, world, e, cap, seq, max_ctas, 0, None, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(R.my_flags(r, 1), world, seq, 0, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_return_rows(R.recv[r].data_ptr(), R.meta[r].data_ptr(), R.table([t.data_ptr() for t in R.back]),
                                       R.flags(2), R.done[r][1:].data_ptr(), h, 0, r, world, R.back_cap, cap, seq, max_ctas,
                                       R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(R.my_flags(r, 2), world, seq, 1, R.status[r].data_ptr(), st) == 0
    torch.cuda.synchronize()
    for r in range(world):
        m = R.meta[r].cpu().tolist()
        assert m[0] == 0 and m[1] == 1, f"rank {r}: meta head {m[:2]}"                  # no rows, state = overflow
        assert all(v == 0 for v in m[2 + 4 * world + 1:2 + 4 * world + 1 + e + 1]), "segments must be empty"
        with pytest.raises(RuntimeError, match="more rows"):
            ops.check_status(R.status[r])
        assert bool((R.recv[r] == 3.0).all()) and bool((R.back[r] == 5.0).all()), f"rank {r}: a buffer was written"
        assert int(R.done[r].sum()) == 0


@pytest.mark.parametrize("max_ctas", [0, 4])
def test_exchange_of_skewed_routing_with_lossless_capacity(cuda_device, max_ctas):
    """Three quarters of all rows go to one rank's experts (it receives about three times the mean).  With the
    receive capacity at world x the largest sender, which no routing can exceed, every row arrives and comes back."""
    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    world, e, h, k = 4, 8, 128, 2
    n = [300, 280, 320, 290]
    xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=31, hot_owner=1)
    seg_host = [s.cpu().tolist() for s in segs]
    el = e // world
    recv_rows = [sum(seg_host[s][(d + 1) * el] - seg_host[s][d * el] for s in range(world)) for d in range(world)]
    assert recv_rows[1] > 2.5 * (sum(recv_rows) / world)
    cap = world * k * max(n)
    R = _EmulatedRanks(world, e, h, cap, k * max(n), cuda_device, lib)
    st = torch.cuda.current_stream().cuda_stream
    seq = 1
    R.publish_counts(seg_host, seq)
    for r in range(world):
        assert lib.dice_ep_exchange_counts(segs[r].data_ptr(), R.table([c.data_ptr() for c in R.ctrl]), R.flags(0),
                                           R.meta[r].data_ptr(), r, world, e, cap, seq, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), R.meta[r].data_ptr(),
                                         R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r], k,
                                         h, 0, r, world, e, cap, seq, max_ctas, 0, None, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(R.my_flags(r, 1), world, seq, 0, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_return_rows(R.recv[r].data_ptr(), R.meta[r].data_ptr(), R.table([t.data_ptr() for t in R.back]),
                                       R.flags(2), R.done[r][1:].data_ptr(), h, 0, r, world, R.back_cap, cap, seq, max_ctas,
                                       R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(R.my_flags(r, 2), world, seq, 1, R.status[r].data_ptr(), st) == 0
    torch.cuda.synchronize()
    for r in range(world):
        ops.check_status(R.status[r])
        assert R.meta[r].cpu().tolist()[:2] == [recv_rows[r], 0]
        want = ops.permute_rows(xs[r], poss[r], k)
        assert torch.equal(R.back[r][: k * n[r]], want), f"rank {r} did not get its rows back"
        assert bool((R.back[r][k * n[r]:] == 5.0).all()) and bool((R.recv[r][recv_rows[r]:] == 3.0).all())


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("max_ctas", [0, -1, 4])
def test_exchange_in_the_region_layout(cuda_device, world, max_ctas):
    """The exchange without a count rendezvous: every source owns a fixed region of each receive buffer, the
    dispatch publishes the source's counts with its rows, and dice_ep_wait_dispatch derives the receiver's segment
    table (with a slab-less segment for the unused rest of every region).  Skewed routing (three quarters of the
    rows to one rank) on `world` ranks whose buffers share this GPU; identity FFN: every rank gets its own rows
    back, every region holds its source's rows in slot order, nothing else is touched.  Twice on the same buffers."""
    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    e, h, k = 8, 128, 2
    el = e // world
    n = [150 + 13 * r for r in range(world)]
    region = k * max(n)
    cap = world * region
    R = _EmulatedRanks(world, e, h, cap, region, cuda_device, lib)
    st = torch.cuda.current_stream().cuda_stream
    matrices = R.table([c.data_ptr() for c in R.ctrl])
    for seq in (1, 2):
        xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=40 + seq, hot_owner=world - 1)
        seg_host = [s.cpu().tolist() for s in segs]
        for r in range(world):
            assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), None,
                                             R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r],
                                             k, h, 0, r, world, e, cap, seq, max_ctas, region, matrices,
                                             R.status[r].data_ptr(), st) == 0
        for r in range(world):
            assert lib.dice_ep_wait_dispatch(R.my_flags(r, 1), R.ctrl[r].data_ptr(), R.meta[r].data_ptr(), r, world, e, region,
                                             seq, R.status[r].data_ptr(), st) == 0
        for r in range(world):  # identity FFN: the received rows go straight back
            assert lib.dice_ep_return_rows(R.recv[r].data_ptr(), R.meta[r].data_ptr(), R.table([t.data_ptr() for t in R.back]),
                                           R.flags(2), R.done[r][1:].data_ptr(), h, 0, r, world, R.back_cap, cap, seq, max_ctas,
                                           R.status[r].data_ptr(), st) == 0
        for r in range(world):
            assert lib.dice_ep_wait_flags(R.my_flags(r, 2), world, seq, 1, R.status[r].data_ptr(), st) == 0
        torch.cuda.synchronize()
        sorted_rows = [ops.permute_rows(xs[r], poss[r], k) for r in range(world)]
        for r in range(world):
            ops.check_status(R.status[r])
            assert torch.equal(R.back[r][: k * n[r]], sorted_rows[r]), f"rank {r} did not get its rows back"
            assert bool((R.back[r][k * n[r]:] == 5.0).all())
        for d in range(world):
            m = R.meta[d].cpu().tolist()
            seg_off = m[2 + 4 * world + 1: 2 + 4 * world + 1 + world * (el + 1) + 1]
            got_total = 0
            for s in range(world):
                lo, hi = seg_host[s][d * el], seg_host[s][(d + 1) * el]
                want = sorted_rows[s][lo:hi]
                assert torch.equal(R.recv[d][s * region: s * region + hi - lo], want), f"region of source {s} at rank {d}"
                # segments of source s: its slots, then the rest of the region
                slots = [seg_host[s][d * el + i] - lo + s * region for i in range(el + 1)]
                assert seg_off[s * (el + 1): s * (el + 1) + el + 1] == slots
                assert m[2 + 2 * world + s] == s * region and m[2 + 3 * world + 1 + s] == hi - lo   # src_off, src_cnt
                got_total += hi - lo
            assert seg_off[-1] == cap and m[0] == got_total and m[1] == 0
            assert bool((R.recv[d][cap:] == 3.0).all())


def test_grouped_gemm_skips_segments_without_a_slab(cuda_device):
    """Segments whose weight slab is -1 (the unused rest of a source's region in the region layout) produce no
    tiles: their output rows stay untouched."""
    ops = _ops()
    g = torch.Generator().manual_seed(77)
    counts, slabs = [100, 300, 0, 140, 260, 50], [0, -1, 1, -1, 1, -1]
    r, k, n = sum(counts), 64, 96
    a = torch.randn(r, k, generator=g).bfloat16()
    w = (torch.randn(2, n, k, generator=g) / 8).bfloat16()
    seg = _segments(counts, cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.full((r, n), 7.0, dtype=torch.bfloat16, device=cuda_device)
    ops.grouped_gemm(a.to(cuda_device), w.to(cuda_device), seg, ops.EPI_STORE, n, status,
                     seg_slab=torch.tensor(slabs, dtype=torch.int32, device=cuda_device), out=out)
    torch.cuda.synchronize()
    ops.check_status(status)
    offs = seg.cpu().tolist()
    for s, slab in enumerate(slabs):
        got = out[offs[s]:offs[s + 1]].cpu().float()
        if slab < 0:
            assert bool((got == 7.0).all())
        elif counts[s]:
            torch.testing.assert_close(got, a[offs[s]:offs[s + 1]].float() @ w[slab].float().t(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("max_ctas", [0, -1])
def test_exchange_failure_reaches_the_peers(cuda_device, max_ctas):
    """Failure detection without a fault: rank 1 of two never publishes its counts, so rank 0's count exchange
    runs out of time (bounded wait).  Rank 0's dispatch then marks its push as failed before it raises the
    flags, and the rank that waits for those rows records "a peer rank reported ..." instead of consuming
    incomplete rows with a clean status."""
    import time

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    world, e, h, k = 2, 8, 128, 2
    n = [200, 200]
    xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=22)
    seg_host = [s.cpu().tolist() for s in segs]
    R = _EmulatedRanks(world, e, h, 4 * max(n), k * max(n), cuda_device, lib)
    st = torch.cuda.current_stream().cuda_stream
    seq = 1
    t0 = time.time()
    assert lib.dice_ep_exchange_counts(segs[0].data_ptr(), R.table([c.data_ptr() for c in R.ctrl]), R.flags(0),
                                       R.meta[0].data_ptr(), 0, world, e, R.cap, seq, R.status[0].data_ptr(), st) == 0
    assert lib.dice_ep_dispatch_rows(xs[0].data_ptr(), poss[0].data_ptr(), segs[0].data_ptr(), R.meta[0].data_ptr(),
                                     R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[0].data_ptr(), n[0], k, h, 0,
                                     0, world, e, R.cap, seq, max_ctas, 0, None, R.status[0].data_ptr(), st) == 0
    # rank 1's own push is played by hand: its dispatch flag on rank 1 is up, so that only rank 0's mark matters
    R.ctrl[1][R.flag_base + 64 + 1] = seq
    assert lib.dice_ep_wait_flags(R.my_flags(1, 1), world, seq, 0, R.status[1].data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 15.0
    assert R.meta[0].cpu().tolist()[:2] == [0, 2]  # no rows, state = the peers' counts never arrived
    with pytest.raises(RuntimeError, match="row counts"):
        ops.check_status(R.status[0])
    with pytest.raises(RuntimeError, match="peer rank reported"):
        ops.check_status(R.status[1])
    assert bool((R.recv[0] == 3.0).all()) and bool((R.recv[1] == 3.0).all())
    # the next exchange on the same buffers is clean again (marks carry the sequence number of the failure)
    seq = 2
    R.publish_counts(seg_host, seq)
    for r in range(world):
        assert lib.dice_ep_exchange_counts(segs[r].data_ptr(), R.table([c.data_ptr() for c in R.ctrl]), R.flags(0),
                                           R.meta[r].data_ptr(), r, world, e, R.cap, seq, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), R.meta[r].data_ptr(),
                                         R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r], k,
                                         h, 0, r, world, e, R.cap, seq, max_ctas, 0, None, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_flags(R.my_flags(r, 1), world, seq, 0, R.status[r].data_ptr(), st) == 0
    torch.cuda.synchronize()
    for r in range(world):
        ops.check_status(R.status[r])


def test_status_is_polled_without_a_synchronisation(cuda_device):
    """ops.poll_status: a status a kernel left on the device surfaces as an exception one or two polls later,
    with no host synchronisation in between (the word travels through a pinned mirror)."""
    ops = _ops()
    word = ops.device_status(cuda_device)
    torch.cuda.synchronize()
    word.zero_()
    ops.poll_status(cuda_device)
    torch.cuda.synchronize()
    ops.poll_status(cuda_device)  # clean
    # non-monotone segments make the grouped GEMM record a status on the shared word
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(2, 32, 64, dtype=torch.bfloat16, device=cuda_device)
    seg = torch.tensor([0, 200, 100], dtype=torch.int32, device=cuda_device)
    ops.grouped_gemm(a, w, seg, ops.EPI_STORE, 32, word)
    raised = False
    for _ in range(3):
        try:
            ops.poll_status(cuda_device)
        except RuntimeError as exc:
            assert "segment offsets" in str(exc)
            raised = True
            break
        torch.cuda.synchronize()  # only so that the test does not depend on timing; the poll itself never waits
    assert raised
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    ops.poll_status(cuda_device)
    torch.cuda.synchronize()
    ops.poll_status(cuda_device)


def test_ffn_with_fused_return_world_of_one(cuda_device):
    """dice_grouped_ffn_return on one GPU: the rows the second GEMM sends "home"
    land where the separate return kernel would put them and equal the plain
    FFN's output bit for bit; the flag is raised by the last CTA."""
    import ctypes

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    n, h, f, e = 500, 128, 512, 4
    g = torch.Generator().manual_seed(12)
    x = torch.randn(n, h, generator=g).bfloat16().to(cuda_device)
    flat = torch.randint(0, e, (2 * n,), generator=g).to(cuda_device)
    mk = lambda *shape: (torch.randn(*shape, generator=g) / math.sqrt(shape[-1])).bfloat16().to(cuda_device)
    w1 = torch.stack([ops.pack_w13(mk(f, h), mk(f, h)) for _ in range(e)])
    w2 = torch.stack([mk(h, f) for _ in range(e)])
    pos, seg, _ = ops.permute_plan(flat, e)
    rows = ops.permute_rows(x, pos, 2)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    want = ops.grouped_ffn(rows, w1, w2, seg, "swiglu", f, status)
    ctrl = torch.zeros(e + 3 * 64, dtype=torch.int32, device=cuda_device)
    back = torch.zeros((2 * n + 3, h), dtype=torch.bfloat16, device=cuda_device)
    meta = torch.zeros(lib.dice_ep_meta_ints(1, e), dtype=torch.int32, device=cuda_device)
    done = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    inter = torch.empty((2 * n, f), dtype=torch.bfloat16, device=cuda_device)
    slab = torch.arange(e, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    tab = lambda p: (ctypes.c_void_p * 1)(p)
    f_cnt, f_back = ctrl.data_ptr() + e * 4, ctrl.data_ptr() + (e + 128) * 4
    for seq in (1, 2):
        back.zero_()
        assert lib.dice_ep_exchange_counts(seg.data_ptr(), tab(ctrl.data_ptr()), tab(f_cnt), meta.data_ptr(), 0, 1, e,
                                           2 * n, seq, status.data_ptr(), st) == 0
        seg_dev = meta[7:7 + e + 1]
        assert lib.dice_grouped_ffn_return(rows.data_ptr(), 2 * n, h, f, 0, w1.data_ptr(), w2.data_ptr(), e,
                                           seg_dev.data_ptr(), slab.data_ptr(), e, inter.data_ptr(), meta.data_ptr(),
                                           tab(back.data_ptr()), tab(f_back), done[1:].data_ptr(), 0, 1, 2 * n, seq, 0,
                                           status.data_ptr(), st) == 0
        assert lib.dice_ep_wait_flags(f_back, 1, seq, 1, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        ops.check_status(status)
        assert torch.equal(back[: 2 * n], want)
        assert bool((back[2 * n:] == 0).all()) and int(done.sum()) == 0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("layout", ["regions", "packed"])
def test_return_push_that_follows_the_second_gemm(cuda_device, layout, world):
    """The return of a synchronous exchange launched on a second stream BEFORE the expert FFN: it sends a chunk of
    rows once the second GEMM has counted the 256-row blocks it lies in as complete.  `world` ranks whose buffers
    share this GPU, skewed routing, real expert weights; every rank must get back exactly what an FFN followed by an
    ordinary return delivers, the block counters must be zero again afterwards, twice on the same buffers."""
    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    e, h, ffn, k = 8, 256, 512, 2
    el = e // world
    n = [900 + 57 * r for r in range(world)]
    region = k * max(n) if layout == "regions" else 0
    cap = world * k * max(n)
    R = _EmulatedRanks(world, e, h, cap, k * max(n), cuda_device, lib)
    n_seg = world * (el + 1) if region else world * el
    seg_slab = torch.tensor([i for _ in range(world) for i in (list(range(el)) + ([-1] if region else []))],
                            dtype=torch.int32, device=cuda_device)
    g = torch.Generator().manual_seed(77)
    w1 = (torch.randn(el, ffn, h, generator=g) / 16).bfloat16().to(cuda_device)
    w2 = (torch.randn(el, h, ffn, generator=g) / 16).bfloat16().to(cuda_device)
    rows_done = torch.zeros(cap // 256 + n_seg + 1, dtype=torch.int32, device=cuda_device)
    status = ops.device_status(cuda_device)
    main, side = torch.cuda.current_stream(), torch.cuda.Stream()
    between = torch.cuda.Event()
    between.record()  # torch creates the CUDA event at the first record
    st = main.cuda_stream
    matrices = R.table([c.data_ptr() for c in R.ctrl])
    seg_base = 2 + 4 * world + 1
    for seq in (1, 2):
        xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=50 + seq, hot_owner=1)
        seg_host = [s.cpu().tolist() for s in segs]
        if not region:  # (the packed layout's capacity here is the lossless one too, so the skew fits)
            R.publish_counts(seg_host, seq)
            for r in range(world):
                assert lib.dice_ep_exchange_counts(segs[r].data_ptr(), matrices, R.flags(0), R.meta[r].data_ptr(), r, world,
                                                   e, cap, seq, R.status[r].data_ptr(), st) == 0
        for r in range(world):
            assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(),
                                             None if region else R.meta[r].data_ptr(),
                                             R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r],
                                             k, h, 0, r, world, e, cap, seq, 0, region, matrices if region else None,
                                             R.status[r].data_ptr(), st) == 0
        for r in range(world):
            if region:
                assert lib.dice_ep_wait_dispatch(R.my_flags(r, 1), R.ctrl[r].data_ptr(), R.meta[r].data_ptr(), r, world, e,
                                                 region, seq, R.status[r].data_ptr(), st) == 0
            else:
                assert lib.dice_ep_wait_flags(R.my_flags(r, 1), world, seq, 0, R.status[r].data_ptr(), st) == 0
        # what an FFN followed by an ordinary return delivers
        outs = []
        for r in range(world):
            seg_dev = R.meta[r][seg_base: seg_base + n_seg + 1]
            outs.append(ops.grouped_ffn(R.recv[r][:cap], w1, w2, seg_dev, "gelu_tanh", ffn, status=status, seg_slab=seg_slab))
        for r in range(world):
            assert lib.dice_ep_return_rows(outs[r].data_ptr(), R.meta[r].data_ptr(), R.table([t.data_ptr() for t in R.back]),
                                           R.flags(2), R.done[r][1:].data_ptr(), h, 0, r, world, R.back_cap, cap, seq, 0,
                                           R.status[r].data_ptr(), st) == 0
        torch.cuda.synchronize()
        want = [b[: k * n[r]].clone() for r, b in enumerate(R.back)]
        for r in range(world):
            R.back[r].fill_(5.0)
            R.ctrl[r][R.flag_base + 128: R.flag_base + 128 + world] = 0  # the return flags, for the second delivery
        torch.cuda.synchronize()
        for r in range(world):
            out = torch.zeros(cap, h, dtype=torch.bfloat16, device=cuda_device)
            seg_dev = R.meta[r][seg_base: seg_base + n_seg + 1]
            def push():
                assert lib.dice_ep_return_rows_following(
                    out.data_ptr(), R.meta[r].data_ptr(), R.table([t.data_ptr() for t in R.back]), R.flags(2),
                    R.done[r][1:].data_ptr(), h, r, world, R.back_cap, cap, seq, 4, rows_done.data_ptr(), rows_done.numel(),
                    seg_slab.data_ptr(), n_seg, R.status[r].data_ptr(), side.cuda_stream) == 0

            if seq == 1:
                # the push is launched FIRST, so that it really has to wait for the GEMM (whose kernel is already
                # loaded: the FFN above ran it)
                side.wait_stream(main)
                push()
                got = ops.grouped_ffn(R.recv[r][:cap], w1, w2, seg_dev, "gelu_tanh", ffn, status=status, seg_slab=seg_slab,
                                      out=out, reserve_sms=4, rows_done=rows_done)
            else:
                # the product's order: FFN first (its first GEMM on all SMs), the push's stream waits for the event
                # between the two GEMMs
                got = ops.grouped_ffn(R.recv[r][:cap], w1, w2, seg_dev, "gelu_tanh", ffn, status=status, seg_slab=seg_slab,
                                      out=out, reserve_sms=4, rows_done=rows_done, first_gemm_done=between)
                side.wait_event(between)
                push()
            main.wait_stream(side)  # the next rank's FFN counts into the same counters
            assert got.data_ptr() == out.data_ptr()
        for r in range(world):
            assert lib.dice_ep_wait_flags(R.my_flags(r, 2), world, seq, 1, R.status[r].data_ptr(), st) == 0
        torch.cuda.synchronize()
        ops.check_status(status)
        assert int(rows_done.abs().sum()) == 0, "the push must leave the block counters at zero"
        for r in range(world):
            ops.check_status(R.status[r])
            assert torch.equal(R.back[r][: k * n[r]], want[r]), f"rank {r}: rows differ from FFN + ordinary return"
            assert bool((R.back[r][k * n[r]:] == 5.0).all())


def test_following_push_gives_up_when_no_block_completes(cuda_device):
    """Failure detection without a fault: the return push that follows a GEMM is launched, but nothing ever counts
    a block of the output as complete.  Every ring's bounded wait runs out, the push records the expired wait,
    moves no row, marks its flags as failed, and the rank that waits for the rows records "a peer rank reported"."""
    import time

    from dice_b200 import _lib

    ops = _ops()
    lib = _lib.load()
    world, e, h, k = 2, 8, 256, 2
    el = e // world
    n = [600, 640]
    region = k * max(n)
    cap = world * region
    R = _EmulatedRanks(world, e, h, cap, region, cuda_device, lib)
    n_seg = world * (el + 1)
    seg_slab = torch.tensor([i for _ in range(world) for i in (list(range(el)) + [-1])], dtype=torch.int32,
                            device=cuda_device)
    rows_done = torch.zeros(cap // 256 + n_seg + 1, dtype=torch.int32, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    matrices = R.table([c.data_ptr() for c in R.ctrl])
    xs, poss, segs = _emulated_inputs(world, e, h, n, k, cuda_device, seed=61)
    seq = 1
    for r in range(world):
        assert lib.dice_ep_dispatch_rows(xs[r].data_ptr(), poss[r].data_ptr(), segs[r].data_ptr(), None,
                                         R.table([t.data_ptr() for t in R.recv]), R.flags(1), R.done[r].data_ptr(), n[r], k,
                                         h, 0, r, world, e, cap, seq, 0, region, matrices, R.status[r].data_ptr(), st) == 0
    for r in range(world):
        assert lib.dice_ep_wait_dispatch(R.my_flags(r, 1), R.ctrl[r].data_ptr(), R.meta[r].data_ptr(), r, world, e, region,
                                         seq, R.status[r].data_ptr(), st) == 0
    torch.cuda.synchronize()
    for r in range(world):
        ops.check_status(R.status[r])
    out = torch.zeros(cap, h, dtype=torch.bfloat16, device=cuda_device)
    t0 = time.time()
    assert lib.dice_ep_return_rows_following(out.data_ptr(), R.meta[0].data_ptr(), R.table([t.data_ptr() for t in R.back]),
                                             R.flags(2), R.done[0][1:].data_ptr(), h, 0, world, R.back_cap, cap, seq, 4,
                                             rows_done.data_ptr(), rows_done.numel(), seg_slab.data_ptr(), n_seg,
                                             R.status[0].data_ptr(), st) == 0
    # rank 1's own return to itself is played by hand, so that only rank 0's mark matters to its wait
    R.ctrl[1][R.flag_base + 128 + 1] = seq
    assert lib.dice_ep_wait_flags(R.my_flags(1, 2), world, seq, 1, R.status[1].data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 15.0
    with pytest.raises(RuntimeError, match="expert outputs that a return push follows"):
        ops.check_status(R.status[0])
    with pytest.raises(RuntimeError, match="peer rank reported"):
        ops.check_status(R.status[1])
    assert bool((R.back[0] == 5.0).all()) and bool((R.back[1] == 5.0).all()), "no row may have moved"
    assert int(rows_done.abs().sum()) == 0
