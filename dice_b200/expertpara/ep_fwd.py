"""Expert-parallel MoE forward: drop-in for the reference's
``expertpara/ep_fwd.py`` (``moe_infer_ep`` :19-197 and helpers :199-354).

Experts are sharded round-robin over the ranks (``etrim.py:23-24``); tokens
stay on the rank that owns them, their (token, slot) rows travel to the expert
owners through an uneven all-to-all (dispatch), run the expert FFN there, and
travel back (combine).  What differs from the reference is *how*, not *what*:

* the histogram, the stable expert sort, the row gather, the expert FFN and
  the un-permute + gate-weighted pair sum are CUDA kernels reached through the
  C ABI (``dice_b200.ops``); the zero-fill + ``index_copy_`` + ``mul_`` +
  ``sum`` tail of the reference (:172-195) is one kernel;
* rows are sorted by ``(owner rank, local slot)`` instead of by expert id, so
  ONE ``all_to_all_single`` per direction and layer moves what the reference
  moves with ``E/W`` calls (:277-291, :326-340); the receive buffer is then
  source-major and the grouped FFN walks its ``(source, slot)`` segments;
* per layer there is one device-to-host read (the gathered ``[W, E]`` count
  matrix, which NCCL needs as host-side split sizes) instead of the
  reference's per-slot ``.tolist()`` calls and tensor-valued slice bounds.

The block output is identical to the reference's for every mode; the row
order *inside* the exchanged buffers is an internal matter.
"""
from __future__ import annotations

import contextlib
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _lib, ops as _dops
from ..ops import _dtype_code, _stream, no_grad
from . import diep, p2p
from .diep import ep_skip_get, ep_skip_put, global_combine_async, global_dispatch_async  # noqa: F401

_use_latest_expert_weights = None
_shared_job = None  # the shared-expert job of the moe_infer_ep call in progress (see proc_experts)


def use_latest_expert_weights(val):
    """ep_fwd.py:12-15: scale the (possibly stale) expert outputs by the
    current step's gate weights (True) or by the cached ones (False)."""
    assert val in [True, False], "val must be a boolean"
    global _use_latest_expert_weights
    _use_latest_expert_weights = val


# --------------------------------------------------------------------------- #
# device operations (CUDA kernels); replaceable only so that the host logic can
# be exercised by CPU gloo ranks in the test-suite
# --------------------------------------------------------------------------- #


class CudaOps:
    """The product's device operations: every method launches dice_b200 CUDA
    kernels and refuses CPU tensors."""

    def plan(self, keys: torch.Tensor, n_keys: int):
        pos, seg, _ = _dops.permute_plan(keys, n_keys)
        return pos, seg

    def plan_chunked(self, flat_idx: torch.Tensor, chunk_hist: torch.Tensor, n_experts: int, world: int):
        """Plan by (owner rank, local slot) in one launch, from the router's per-chunk histograms."""
        pos, seg, _, _ = _dops.permute_plan_chunked(flat_idx, chunk_hist, n_experts, world)
        return pos, seg

    def permute_rows(self, x: torch.Tensor, pos: torch.Tensor, k: int) -> torch.Tensor:
        return _dops.permute_rows(x, pos, k)

    def unpermute_combine(self, src0, idx0, src1, idx1, w0, w1, n_tokens, addend=None, **glue):
        return _dops.unpermute_combine(src0, idx0, src1, idx1, w0, w1, n_tokens, addend=addend, **glue)

    def run_packed_experts(self, rows, pack, seg_counts: Sequence[int], seg_slab: Sequence[int], seg_offsets_dev=None):
        if seg_offsets_dev is not None:
            # segment offsets were derived on the device from the gathered counts: no host-to-device copy,
            # and therefore no stream synchronisation, between the dispatch and the expert FFN
            return pack.run_offsets(rows, seg_offsets_dev, pack.slab_table(seg_slab, rows.device))
        return pack.run_segments(rows, seg_counts, seg_slab)


_ops = CudaOps()


def set_device_ops(ops_obj) -> None:
    """Replace the device operations (used by the CPU tests of the host logic)."""
    global _ops
    _ops = ops_obj


def device_ops():
    return _ops


def _scope(name: str):
    """The reference wraps each phase in ``CudaProfiler.scope`` (ep_fwd.py:88,
    108, 127, 149, 153, 172); keep the same section names when its profiler is
    importable, else time nothing."""
    prof = diep._profiler()
    return prof.scope(name) if prof is not None else contextlib.nullcontext()


# --------------------------------------------------------------------------- #
# counts
# --------------------------------------------------------------------------- #


@no_grad
def exchange_token_counts(token_counts_local: torch.Tensor) -> torch.Tensor:
    """ep_fwd.py:214-245: all-gather the per-expert row counts (expert-id
    order, length E) and return the ``[world_size, E/W]`` counts of rows each
    rank sends to THIS rank's local experts."""
    world_size, rank = dist.get_world_size(), dist.get_rank()
    assert token_counts_local.size(0) % world_size == 0, "Number of experts must be divisible by world size"
    gathered = [torch.zeros_like(token_counts_local) for _ in range(world_size)]
    dist.all_gather(gathered, token_counts_local)
    return torch.stack(gathered, dim=0)[:, rank::world_size]


def _exchange_counts_by_owner(counts_key: torch.Tensor, world_size: int, rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather the local counts, which are laid out ``[owner rank][slot]``,
    and bring the ``[W, E]`` matrix to the host once.  Returns CPU int64
    tensors ``send[W, El]`` (rows this rank sends to rank d's slot i) and
    ``recv[W, El]`` (rows rank s sends to this rank's slot i)."""
    n_local = counts_key.numel() // world_size
    if world_size == 1:
        gathered = counts_key.contiguous()
    else:
        gathered = torch.empty((world_size * counts_key.numel(),), dtype=counts_key.dtype, device=counts_key.device)
        dist.all_gather_into_tensor(gathered, counts_key.contiguous())
    seg_dev = None
    if gathered.is_cuda:
        # offsets of the [source][slot] segments of the receive buffer, kept on the device for the grouped FFN
        mine = gathered.view(world_size, world_size, n_local)[:, rank, :].reshape(-1)
        seg_dev = torch.zeros(mine.numel() + 1, dtype=torch.int32, device=gathered.device)
        torch.cumsum(mine, 0, out=seg_dev[1:])
    host = gathered.to("cpu", torch.int64).view(world_size, world_size, n_local)
    send, recv = host[rank].contiguous(), host[:, rank, :].contiguous()
    recv._dice_seg_offsets = seg_dev
    return send, recv


# --------------------------------------------------------------------------- #
# all-to-all
# --------------------------------------------------------------------------- #


def _all_to_all_rows(send: torch.Tensor, in_counts: torch.Tensor, out_counts: torch.Tensor, async_op: bool):
    """One uneven all-to-all of rows.  ``in_counts``/``out_counts`` are CPU
    ``[W, El]`` tensors; the split towards/from a rank is the row sum."""
    in_splits = in_counts.sum(dim=1).tolist()
    out_splits = out_counts.sum(dim=1).tolist()
    assert send.size(0) == sum(in_splits)
    buf = send.new_empty((sum(out_splits), send.size(1)))
    with _scope("global_dispatch.call_dist"):
        handle = dist.all_to_all_single(buf, send, out_splits, in_splits, async_op=True)
    with _scope("moe.wait"):
        if not async_op:
            handle.wait()
    return buf, [handle]


@no_grad
def global_dispatch(grouped_dup_inp, token_counts_local, token_counts_global, async_op=False):
    """Send owner-sorted rows to the expert owners (ep_fwd.py:247-293).

    ``token_counts_local`` / ``token_counts_global`` are the CPU ``[W, E/W]``
    send / receive counts.  Returns ``(recv_buf, handles)``; the receive
    buffer is ordered ``[source rank][local slot]``.

    With the peer-memory exchange the first argument is a
    :class:`p2p.PendingRows`: the row gather and the dispatch are one kernel
    that writes every row into its owner's receive buffer over NVLink, on the
    current stream, or on the exchange's side stream when ``async_op``."""
    if isinstance(grouped_dup_inp, p2p.PendingRows):
        return _peer_push(grouped_dup_inp.info, async_op, dispatch=grouped_dup_inp)
    return _all_to_all_rows(grouped_dup_inp, token_counts_local, token_counts_global, async_op)


@no_grad
def global_combine(grouped_dup_outp, token_counts_local, token_counts_global, async_op=False):
    """Return expert outputs to the token owners; the mirror image of
    :func:`global_dispatch` (ep_fwd.py:295-342).  With the peer-memory exchange
    ``token_counts_global`` is the :class:`p2p.SegInfo` of the dispatch being
    answered and the rows are written into the token owners' buffers."""
    if isinstance(token_counts_global, p2p.SegInfo):
        if isinstance(grouped_dup_outp, p2p.ReturnedRows):  # the FFN kernel already returned the rows
            info = token_counts_global
            handle = p2p.PeerHandle(info, 1, grouped_dup_outp.event, ordered=grouped_dup_outp.beside_ffn)
            if not async_op:
                handle.wait()
            return info.xchg.back[info.slot][: info.rows_sent], [handle]
        return _peer_push(token_counts_global, async_op, rows_back=grouped_dup_outp)
    return _all_to_all_rows(grouped_dup_outp, token_counts_global, token_counts_local, async_op)


def _peer_push(info, async_op, dispatch=None, rows_back=None):
    """Launch one push of the peer-memory exchange (csrc/p2p_exchange.cu) and
    return ``(buffer the peers fill for this rank, [handle])``."""
    x = info.xchg
    lib, tab, slot = x.lib, info.tab, info.slot
    # 0: the push owns the GPU (one copy-unit warp per SM); an asynchronous push runs next to the expert FFN on
    # the few SMs that the FFN leaves free (p2p.reserve_sms)
    side_ctas = (p2p.side_push_ctas() or -1) if async_op else 0
    p2p.note_push(async_op)
    if async_op and dispatch is not None and dispatch.on_side:
        stream = x.comm_raw  # the count exchange in front already moved this exchange to the side stream
    elif async_op:
        stream = x.fork_to_comm()  # the push runs on the side stream, after what the current stream has produced
        # the caching allocator must not hand these to someone else before the side stream has read them
        for t in ((dispatch.inp, dispatch.pos, dispatch.seg_offsets) if dispatch is not None else (rows_back,)):
            t.record_stream(x._comm)
    else:
        stream = _stream()
    if dispatch is not None:
        inp = dispatch.inp
        _lib.check(lib.dice_ep_dispatch_rows(
            inp.data_ptr(), dispatch.pos.data_ptr(), dispatch.seg_offsets.data_ptr(), x._meta_ptrs[slot], tab["recv"],
            tab["f_disp"], x._done_ptrs[2 * slot], inp.shape[0], dispatch.k_eff, inp.shape[1], _dtype_code(inp), x.rank,
            x.world, x.n_experts, x.min_peer_cap, info.seq, side_ctas, x.region_rows, tab["matrix"], x.status_ptr, stream),
            "dice_ep_dispatch_rows")
        out, which = x._recv_views[slot], 0
    else:
        _lib.check(lib.dice_ep_return_rows(
            rows_back.data_ptr(), x._meta_ptrs[slot], tab["back"], tab["f_back"], x._done_ptrs[2 * slot + 1], x.hidden,
            _dtype_code(rows_back), x.rank, x.world, x.min_peer_rows, x.capacity_rows, info.seq, side_ctas, x.status_ptr,
            stream),
            "dice_ep_return_rows")
        if async_op:
            x.note_output_read_on_side(rows_back)
        out, which = x.back[slot][: info.rows_sent], 1
    # a consumer on another stream must also see what THIS rank's side stream wrote (the meta block of the count
    # exchange, the rows this rank pushed into its own buffers)
    event = x.record_side_event(slot, which) if async_op else None
    handle = p2p.PeerHandle(info, which, event)
    with _scope("moe.wait"):
        if not async_op:
            handle.wait()
    return out, [handle]


# --------------------------------------------------------------------------- #
# experts
# --------------------------------------------------------------------------- #


@no_grad
def proc_experts(inp, experts, token_counts_global, num_local_experts):
    """Run this rank's experts over the received rows (ep_fwd.py:199-211).

    The buffer is ``[source][slot]``-ordered; segment ``(s, i)`` holds
    ``token_counts_global[s, i]`` rows for local slot ``i`` (global expert
    ``rank + i * world_size``).  Expert lists built by ``SparseMoeBlock`` carry
    packed weights and run as one grouped-FFN launch pair; any other list of
    row-wise modules is called segment by segment, as the reference does."""
    if isinstance(token_counts_global, p2p.SegInfo):
        pack = getattr(experts, "_dice_pack", None)
        if pack is not None:
            if inp.dtype == torch.bfloat16 and p2p.fused_return():
                pack.run_offsets_return(inp, token_counts_global)
                return p2p.ReturnedRows(token_counts_global)
            job = _shared_job
            xchg = token_counts_global.xchg
            inter, out = xchg.ffn_buffers(pack.ffn_width(inp.dtype)) if inp.shape[0] == xchg.capacity_rows else (None, None)
            if (out is not None and inp.dtype == torch.bfloat16 and p2p.return_follows() and p2p.reserve_sms() == 0
                    and xchg.rows_done is not None):
                # synchronous exchange: the return push starts beside the FFN and follows its second GEMM
                shared = (job.x, job.pack) if job is not None else None
                returned = []
                res = pack.run_offsets(inp, token_counts_global.seg_dev, xchg.seg_slab_dev,
                                       reserve_sms=p2p.follow_ctas(), shared=shared, inter=inter, out=out,
                                       rows_done=xchg.rows_done, first_gemm_done=xchg._fork,
                                       then=lambda: returned.append(xchg.follow_ffn(token_counts_global, out)))
                if job is not None:
                    job.out = res[1]
                return returned[0]
            if job is not None and inp.dtype == torch.bfloat16:
                outp, job.out = pack.run_offsets(inp, token_counts_global.seg_dev, xchg.seg_slab_dev,
                                                 reserve_sms=p2p.reserve_sms(), shared=(job.x, job.pack), inter=inter, out=out)
                return outp
            return pack.run_offsets(inp, token_counts_global.seg_dev, xchg.seg_slab_dev, reserve_sms=p2p.reserve_sms(),
                                    inter=inter, out=out)
        world_size, rank = token_counts_global.xchg.world, token_counts_global.xchg.rank
        seg_slab = token_counts_global.xchg.seg_slab
        offs = token_counts_global.seg_dev.tolist()  # arbitrary expert modules need the bounds on the host
        outp = torch.empty_like(inp)
        for j, slot in enumerate(seg_slab):
            if slot >= 0 and offs[j + 1] > offs[j]:
                outp[offs[j]:offs[j + 1]] = experts[rank + slot * world_size](inp[offs[j]:offs[j + 1]])
        return outp
    world_size, rank = dist.get_world_size(), dist.get_rank()
    counts = token_counts_global.tolist()  # CPU tensor: no device sync
    seg_counts = [counts[s][i] for s in range(world_size) for i in range(num_local_experts)]
    seg_slab = [i for _ in range(world_size) for i in range(num_local_experts)]
    assert sum(seg_counts) == inp.size(0)
    pack = getattr(experts, "_dice_pack", None)
    if pack is not None:
        seg_dev = getattr(token_counts_global, "_dice_seg_offsets", None)
        if seg_dev is not None:
            return _ops.run_packed_experts(inp, pack, seg_counts, seg_slab, seg_dev)
        return _ops.run_packed_experts(inp, pack, seg_counts, seg_slab)
    outp = torch.empty_like(inp)
    start = 0
    for cnt, slot in zip(seg_counts, seg_slab):
        if cnt:
            outp[start:start + cnt] = experts[rank + slot * world_size](inp[start:start + cnt])
        start += cnt
    return outp


# --------------------------------------------------------------------------- #
# the forward
# --------------------------------------------------------------------------- #


def _slot_views(skip_mask: torch.Tensor, n_tokens: int, device) -> Tuple[Optional[int], torch.Tensor]:
    """From the reference's boolean row mask (one True per token pair,
    diep.py:72-90) derive the skipped slot: a constant for the 'high'/'low'
    patterns, else a per-token int64 tensor on ``device``."""
    m = skip_mask.view(n_tokens, 2)
    assert bool((m.sum(dim=1) == 1).all()), "skip mask must mark exactly one slot per token"
    if bool(m[:, 1].all()):
        return 1, None
    if bool(m[:, 0].all()):
        return 0, None
    return None, m[:, 1].to(device=device, dtype=torch.int64)


_slot_cache = {}


def _skipped_slot(skip_mask: torch.Tensor, n_tokens: int, device):
    key = (id(skip_mask), n_tokens, str(device))
    hit = _slot_cache.get(key)
    if hit is None or hit[0] is not skip_mask:
        const, per_tok = _slot_views(skip_mask.cpu() if skip_mask.is_cuda else skip_mask, n_tokens, device)
        if len(_slot_cache) > 64:
            _slot_cache.clear()
        hit = (skip_mask, const, per_tok)
        _slot_cache[key] = hit
    return hit[1], hit[2]


def _pick(pairs: torch.Tensor, const_slot: Optional[int], per_tok: Optional[torch.Tensor], other: bool) -> torch.Tensor:
    """Column ``slot`` (or the other one) of an ``[N, 2]`` tensor as a 1-D view/tensor."""
    if const_slot is not None:
        s = 1 - const_slot if other else const_slot
        return pairs[:, s]
    sel = (1 - per_tok) if other else per_tok
    return pairs.gather(1, sel.view(-1, 1)).view(-1)


@no_grad
def moe_infer_ep(inp: torch.Tensor, experts: nn.ModuleList, flat_expert_indices, flat_expert_weights,
                 num_experts_per_tok, async_op, skip_mask=None, skip_now=None, cache_key=None, _addend=None,
                 _chunks=None, _glue=None, _shared=None):
    """Expert-parallel replacement of ``SparseMoeBlock.moe_infer``
    (ep_fwd.py:19-197; same arguments and result).

    ``inp`` ``[N, h]``; ``experts`` the block's full expert list (only entries
    ``rank + i*W`` are real); ``flat_expert_indices`` ``[N*k]`` int64;
    ``flat_expert_weights`` ``[N*k, 1]``; ``async_op`` selects the displaced /
    interweaved protocol of :mod:`diep`; ``skip_mask`` / ``skip_now`` drive
    conditional communication; ``cache_key`` is the layer index.  ``_addend``
    (not in the reference) is added to the result inside the combine kernel;
    ``_chunks`` (not in the reference) is the router's per-128-token histogram
    table, from which the plan is a single launch; ``_glue`` (not in the
    reference) is ``(residual [N, h], gate [B, h], tokens per sample)``: the
    DiT block's gated residual, applied by the same combine kernel;
    ``_shared`` (not in the reference) is the block's shared-expert job, which
    rides in this call's grouped-FFN launches and whose output is added in the
    combine kernel."""
    live = p2p._exchange if p2p.enabled() else None  # knows this rank's place without asking c10d per layer
    world_size, rank = (live.world, live.rank) if live is not None else (dist.get_world_size(), dist.get_rank())
    num_total_experts = len(experts)
    num_local_experts = num_total_experts // world_size
    assert num_total_experts % world_size == 0, "Number of experts must be divisible by world size"
    n_tokens, hidden = inp.shape
    k_full = num_experts_per_tok

    partial_skip = skip_mask is not None
    const_slot = per_tok = None
    if partial_skip:
        assert k_full == 2, "only support num_experts_per_tok == 2"
        const_slot, per_tok = _skipped_slot(skip_mask, n_tokens, inp.device)

    # conditional communication: on a skip step only the retained slot of each token travels (:57-66)
    if skip_now:
        assert partial_skip, "skip is not enabled"
        k_eff = k_full // 2
        flat_idx = _pick(flat_expert_indices.view(n_tokens, 2), const_slot, per_tok, other=True).contiguous()
        assert flat_idx.size(0) == n_tokens * k_eff
    else:
        k_eff = k_full
        flat_idx = flat_expert_indices

    # sort key = (owner rank, local slot): rows for one destination are contiguous
    if _chunks is not None and k_eff == k_full and hasattr(_ops, "plan_chunked"):
        pos, seg_offsets = _ops.plan_chunked(flat_idx, _chunks, num_total_experts, world_size)
    else:
        keys = (flat_idx % world_size) * num_local_experts + torch.div(flat_idx, world_size, rounding_mode="floor")
        pos, seg_offsets = _ops.plan(keys, num_total_experts)

    xchg = None
    if inp.is_cuda and p2p.enabled():
        # exchange over NVLink peer memory: counts, dispatch and combine are own kernels, no NCCL, no host sync
        cached_layers = diep._diep_cache_dispatch.capacity if diep._diep_cache_dispatch is not None else 0
        xchg = p2p.get_exchange(num_total_experts, hidden, inp.dtype, n_tokens * k_full, max(1, cached_layers))
    if xchg is not None:
        inp = inp.contiguous()
        slot, seq, tab = xchg.begin(cache_key or 0)
        # An exchange that nobody waits for in this layer (displaced / interweaved) keeps even its count exchange,
        # a rendezvous of all ranks, off the main stream: it runs on the side stream in front of the dispatch.
        # Whoever consumes the exchange later waits for the side stream's event and for the sources' flags.
        side = async_op and not diep._forced_sync
        if xchg.region_rows:
            # every source owns a fixed region of each receive buffer: no count exchange; the dispatch carries this
            # rank's counts and the consumer derives its segment table from them (PeerHandle.wait)
            side = False
        else:
            with _scope("exchange_token_counts"):
                if side:
                    for t in (seg_offsets, pos, inp):
                        t.record_stream(xchg._comm)
                _lib.check(xchg.lib.dice_ep_exchange_counts(
                    seg_offsets.data_ptr(), tab["matrix"], tab["f_cnt"], xchg._meta_ptrs[slot], xchg.rank, xchg.world,
                    xchg.n_experts, xchg.min_peer_cap, seq, xchg.status_ptr, xchg.fork_to_comm() if side else _stream()),
                    "dice_ep_exchange_counts")
        counts_local = None
        counts_global = p2p.SegInfo(xchg, slot, seq, tab, n_tokens * k_eff)
        grouped_dup_inp = p2p.PendingRows(inp, pos, seg_offsets, k_eff, counts_global, on_side=side)
    else:
        with _scope("exchange_token_counts"):
            counts_local, counts_global = _exchange_counts_by_owner(seg_offsets[1:] - seg_offsets[:-1], world_size, rank)
        assert int(counts_local.sum()) == n_tokens * k_eff, "expert index out of range"
        with _scope("local_dispatch"):
            grouped_dup_inp = _ops.permute_rows(inp, pos, k_eff)

    latest_flat_expert_weights = flat_expert_weights
    with _scope("global_dispatch"):
        if not async_op:
            mlp_inp, _ = global_dispatch(grouped_dup_inp, counts_local, counts_global)
            experts_to_calc = experts
        else:
            (mlp_inp, counts_local, counts_global, pos, flat_expert_weights, experts_to_calc) = global_dispatch_async(
                grouped_dup_inp=grouped_dup_inp, token_counts_local=counts_local, token_counts_global=counts_global,
                grouped_idx_dup=pos, flat_expert_weights=flat_expert_weights, experts=experts, cache_key=cache_key)

    global _shared_job
    _shared_job = _shared
    with _scope("moe.mlp"):
        mlp_outp = proc_experts(mlp_inp, experts_to_calc, counts_global, num_local_experts)
    _shared_job = None
    if _shared is not None:  # added by the combine kernel; computed on its own if no launch could carry it
        _addend = _shared.out if _shared.out is not None else _shared.run_alone()

    with _scope("global_combine"):
        if not async_op:
            grouped_dup_outp, _ = global_combine(mlp_outp, counts_local, counts_global)
        else:
            grouped_dup_outp, pos, flat_expert_weights = global_combine_async(
                grouped_dup_outp=mlp_outp, token_counts_local=counts_local, token_counts_global=counts_global,
                grouped_idx_dup=pos, flat_expert_weights=flat_expert_weights, cache_key=cache_key)

    return _finish(grouped_dup_outp, pos, latest_flat_expert_weights, flat_expert_weights, n_tokens, hidden, k_full,
                   partial_skip, const_slot, per_tok, cache_key, _addend, inp, _glue)


def _finish(grouped_dup_outp, pos, latest_flat_expert_weights, flat_expert_weights, n_tokens, hidden, k_full,
            partial_skip, const_slot, per_tok, cache_key, _addend, inp, _glue=None):
    """Un-permute, merge with the skip cache, scale by the gate weights and sum
    each token's pair (ep_fwd.py:172-195) in one kernel."""
    glue = {} if _glue is None else dict(resid=_glue[0], gate=_glue[1], tokens_per_sample=_glue[2])
    weights = latest_flat_expert_weights if _use_latest_expert_weights else flat_expert_weights
    w_pairs = weights.reshape(n_tokens, k_full)
    if w_pairs.dtype != torch.float32:
        w_pairs = w_pairs.float()
    got_rows = grouped_dup_outp.size(0)
    with _scope("local_combine"):
        if partial_skip and got_rows != n_tokens * k_full:
            # the exchange that just completed carried one slot per token: the other comes from the skip cache
            assert got_rows == n_tokens * k_full // 2
            dropped = ep_skip_get(cache_key)
            assert dropped is not None and dropped.shape == (n_tokens, hidden)
            w_kept = _pick(w_pairs, const_slot, per_tok, other=True)
            w_drop = _pick(w_pairs, const_slot, per_tok, other=False)
            if per_tok is not None:
                w_kept, w_drop = w_kept.contiguous(), w_drop.contiguous()
            expert_out = _ops.unpermute_combine(grouped_dup_outp, pos, dropped, None, w_kept, w_drop, n_tokens,
                                                addend=_addend, **glue)
        else:
            assert got_rows == n_tokens * k_full
            pos_pairs = pos.view(n_tokens, k_full)
            if partial_skip:
                # keep the to-be-skipped slot's rows for the next skip step
                ep_skip_put(cache_key, _ops.unpermute_combine(
                    grouped_dup_outp, _pick(pos_pairs, const_slot, per_tok, other=False), None, None, None, None,
                    n_tokens))
            if k_full == 2:
                expert_out = _ops.unpermute_combine(grouped_dup_outp, pos_pairs[:, 0], grouped_dup_outp,
                                                    pos_pairs[:, 1], w_pairs[:, 0], w_pairs[:, 1], n_tokens,
                                                    addend=_addend, **glue)
            else:
                assert k_full == 1, "num_experts_per_tok must be 1 or 2"
                expert_out = _ops.unpermute_combine(grouped_dup_outp, pos_pairs[:, 0], None, None, w_pairs[:, 0],
                                                    None, n_tokens, addend=_addend, **glue)
    assert expert_out.shape == inp.shape, f"{expert_out.shape} != {inp.shape}"
    return expert_out
