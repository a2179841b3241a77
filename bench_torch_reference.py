"""Measurement harness only (not part of the package, not the oracle): the
reference's MoE-block algorithm written with stock PyTorch CUDA operations, so
that ``bench.py`` can put "what the reference's Python would cost on this very
GPU" (ATen kernels, cuBLAS, NCCL; per-expert Python loops and the host
round trips they need) next to the numbers of the dice_b200 kernels.

It follows the reference's call structure, not its text:

* single device: ``MoEGate.forward`` (``models.py:179-217``: linear, softmax,
  ``topk``) and ``SparseMoeBlock.moe_infer`` (``models.py:361-382``: ``argsort``,
  ``bincount`` brought to the host, one expert call per non-empty expert,
  ``mul_`` by the gate weights, ``scatter_reduce_`` into the output);
* expert parallel: ``moe_infer_ep`` (``expertpara/ep_fwd.py:19-197``):
  ``all_gather`` of the expert histogram, ``index_select`` into expert order,
  one ``all_to_all_single`` per local expert slot and direction with split
  sizes read on the host, the local experts in a Python loop, zero-fill +
  ``index_copy_``, ``mul_`` and the pair sum.

The experts are the block's own modules (``MoeMLP`` / ``GeluMLP`` forward in
plain torch), so both arms hold identical weights.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


@torch.no_grad()
def gate(block, x2d):
    scores = F.linear(x2d, block.gate.weight, None).softmax(dim=-1)
    w, idx = torch.topk(scores, k=2, dim=-1, sorted=False)
    if block.gate.norm_topk_prob:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return idx, w


@torch.no_grad()
def block_forward(block, x):
    """One block on one device, the way models.py:302-382 runs it."""
    shape = x.shape
    x2d = x.view(-1, shape[-1])
    idx, w = gate(block, x2d)
    flat_idx, flat_w = idx.view(-1), w.view(-1, 1)
    out = torch.zeros_like(x2d)
    order = flat_idx.argsort()
    ends = flat_idx.bincount().cpu().numpy().cumsum(0)  # the host read of models.py:366
    token_of = order // 2
    start = 0
    for e, end in enumerate(ends):
        if start == end:
            continue
        rows = token_of[start:end]
        y = block.experts[e](x2d[rows])
        y.mul_(flat_w[order[start:end]].to(y.dtype))
        out.scatter_reduce_(0, rows.view(-1, 1).repeat(1, shape[-1]), y, reduce="sum")
        start = end
    if block.n_shared_experts is not None:
        out = out + block.shared_experts(x2d)
    return out.view(shape)


@torch.no_grad()
def block_forward_ep(block, x):
    """One block with experts sharded round-robin over the NCCL ranks, the way ep_fwd.py:19-197 runs it
    (synchronous exchange)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    shape = x.shape
    h = shape[-1]
    x2d = x.view(-1, h)
    idx, w = gate(block, x2d)
    flat_idx, flat_w = idx.view(-1), w.view(-1, 1)
    n_experts = len(block.experts)
    n_local = n_experts // world
    counts_local = torch.bincount(flat_idx, minlength=n_experts)
    gathered = [torch.zeros_like(counts_local) for _ in range(world)]
    dist.all_gather(gathered, counts_local)
    counts_global = torch.stack(gathered, dim=0)[:, rank::world]  # [source, local slot]
    order = flat_idx.argsort()
    send = x2d.index_select(0, order // 2)
    per_slot = counts_local.view(n_local, world)  # expert e = slot * world + owner: one slot's rows are contiguous
    offs = torch.cat([counts_local.new_zeros(1), counts_local.cumsum(0)]).tolist()  # host read, as in ep_fwd.py:262-263
    received = []
    for slot in range(n_local):  # ep_fwd.py:277-291: one all-to-all per local expert slot
        in_splits = per_slot[slot].tolist()
        out_splits = counts_global[:, slot].tolist()
        buf = send.new_empty((sum(out_splits), h))
        dist.all_to_all_single(buf, send[offs[slot * world]:offs[(slot + 1) * world]], out_splits, in_splits)
        received.append((buf, out_splits, in_splits))
    outs = [block.experts[rank + slot * world](buf) if buf.shape[0] else buf
            for slot, (buf, _, _) in enumerate(received)]  # ep_fwd.py:199-211
    back = torch.empty_like(send)
    for slot, (_, out_splits, in_splits) in enumerate(received):  # ep_fwd.py:326-340
        dist.all_to_all_single(back[offs[slot * world]:offs[(slot + 1) * world]], outs[slot].to(send.dtype), in_splits,
                               out_splits)
    final = torch.zeros_like(back)
    final.index_copy_(0, order, back)
    final.mul_(flat_w.to(final.dtype))
    out = final.view(-1, 2, h).sum(dim=1)
    if block.n_shared_experts is not None:
        out = out + block.shared_experts(x2d)
    return out.view(shape)
