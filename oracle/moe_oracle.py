"""CPU restatement of the reference's DiT-MoE block (test infrastructure only).

Every function cites the reference lines it follows (paths are relative to the
reference project's root).  The restatement is checked against the reference's
own modules by ``tests/test_oracle_golden.py`` whenever the reference
checkout is present, and against the fixtures under ``tests/golden`` (generated
from the reference by ``tests/golden/make_golden.py``) everywhere else.

Two variants have no counterpart in the reference and are therefore restated
from its structure only ("parity unpinned" for these two switches):

* ``act="gelu_tanh"``: a two-matrix expert ``fc2(gelu_tanh(fc1(x)))`` run
  through the same dispatch/combine structure as ``models.py:361-382``;
* ``renorm=True``: the reference's dead branch ``models.py:194-196``.

The only deliberate deviation from the reference's text is tie handling in the
top-2 selection.  ``torch.topk(..., sorted=False)`` (``models.py:191``) leaves
slot order and tie choice to the backend; this oracle fixes "larger score
first, lower expert index first among equal scores", which is what the CUDA
backend of ``torch.topk`` produces for k=2 (checked on the GPU by the parity
tests with crafted ties) and what the CPU backend produces on tie-free input.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

# ----------------------------------------------------------------------------
# Router
# ----------------------------------------------------------------------------


def router_logits(x2d: torch.Tensor, w_gate: torch.Tensor) -> torch.Tensor:
    """``logits = F.linear(hidden_states, self.weight, None)`` (models.py:184).

    The product is accumulated in fp32 and rounded to the activation dtype, as
    the library GEMM behind ``F.linear`` does for 16-bit inputs.
    """
    return (x2d.float() @ w_gate.float().t()).to(x2d.dtype)


def top2_from_scores(scores: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-2 of each row: larger score first; among equal scores the lower
    index first (models.py:191, with the tie rule fixed as described in the
    module docstring)."""
    n, e = scores.shape
    idx0 = scores.argmax(dim=-1)  # first maximal value
    masked = scores.clone()
    masked[torch.arange(n), idx0] = -math.inf
    idx1 = masked.argmax(dim=-1)
    idx = torch.stack([idx0, idx1], dim=-1)
    return scores.gather(-1, idx), idx


def gate_top2(
    x2d: torch.Tensor, w_gate: torch.Tensor, renorm: bool = False
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """MoEGate.forward in eval mode (models.py:179-217).

    Returns ``(topk_idx int64 [N,2], topk_weight fp32 [N,2], logits)``.
    Softmax is evaluated in fp32 on the (activation-dtype) logits: that is what
    ``logits.softmax(dim=-1)`` (models.py:186) does under the autocast region
    the reference samples in, and it is the identity for fp32 inputs.
    """
    logits = router_logits(x2d, w_gate)
    scores = logits.float().softmax(dim=-1)
    w, idx = top2_from_scores(scores)
    if renorm:  # models.py:194-196
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return idx, w, logits


# ----------------------------------------------------------------------------
# Experts
# ----------------------------------------------------------------------------


def expert_swiglu(x, gate_w, up_w, down_w):
    """MoeMLP.forward, ``pretraining_tp == 1`` branch (models.py:271)."""
    return F.linear(F.silu(F.linear(x, gate_w)) * F.linear(x, up_w), down_w)


def expert_gelu_tanh(x, fc1_w, fc2_w):
    """Two-matrix expert ``fc2(gelu_tanh(fc1(x)))``; no reference counterpart."""
    return F.linear(F.gelu(F.linear(x, fc1_w), approximate="tanh"), fc2_w)


def run_expert(x: torch.Tensor, weights: Sequence[torch.Tensor], act: str) -> torch.Tensor:
    if act == "swiglu":
        return expert_swiglu(x, *weights)
    if act == "gelu_tanh":
        return expert_gelu_tanh(x, *weights)
    raise ValueError(f"unknown activation {act!r}")


# ----------------------------------------------------------------------------
# Single-device dispatch / combine
# ----------------------------------------------------------------------------


def stable_expert_order(flat_idx: torch.Tensor) -> torch.Tensor:
    """``flat_expert_indices.argsort()`` (models.py:365, ep_fwd.py:100) with the
    order inside an expert fixed to the stable one (row-major: token, then
    slot).  The reference's unstable order only permutes rows inside an expert
    segment, which does not change the block output."""
    return flat_idx.argsort(stable=True)


def expert_histogram(flat_idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """``bincount`` zero-extended to all experts (ep_fwd.py:70-76)."""
    return torch.bincount(flat_idx, minlength=num_experts)


def moe_infer(
    x: torch.Tensor,
    flat_idx: torch.Tensor,
    flat_w: torch.Tensor,
    experts: Sequence[Sequence[torch.Tensor]],
    act: str = "swiglu",
    k: int = 2,
) -> torch.Tensor:
    """SparseMoeBlock.moe_infer (models.py:361-382): sort rows by expert, run
    each non-empty expert on its rows, scale by the gate weight, sum the k
    rows of each token."""
    out = torch.zeros_like(x)
    order = stable_expert_order(flat_idx)
    ends = expert_histogram(flat_idx, len(experts)).cumsum(0).tolist()
    token_of = order // k
    start = 0
    for e, end in enumerate(ends):
        if end > start:
            rows = token_of[start:end]
            y = run_expert(x[rows], experts[e], act)
            y = y * flat_w[order[start:end]].view(-1, 1).to(y.dtype)
            out.index_add_(0, rows, y.to(out.dtype))
        start = end
    return out


def moe_block_forward(
    x: torch.Tensor,
    w_gate: torch.Tensor,
    experts: Sequence[Sequence[torch.Tensor]],
    shared: Optional[Sequence[torch.Tensor]] = None,
    act: str = "swiglu",
    renorm: bool = False,
) -> Dict[str, torch.Tensor]:
    """SparseMoeBlock.forward, eval mode, no expert parallelism
    (models.py:302-358).  Returns the output and the routing it used."""
    shape = x.shape
    x2d = x.reshape(-1, shape[-1])
    idx, w, logits = gate_top2(x2d, w_gate, renorm)
    flat_idx = idx.reshape(-1)
    y = moe_infer(x2d, flat_idx, w.reshape(-1), experts, act)
    if shared is not None:  # models.py:355-357
        y = y + run_expert(x2d, shared, act)
    return {
        "out": y.reshape(shape),
        "topk_idx": idx,
        "topk_weight": w,
        "logits": logits,
        "hist": expert_histogram(flat_idx, len(experts)),
        "order": stable_expert_order(flat_idx),
    }


def modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """models.py:75-76."""
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


def dit_block_moe_half(x, shift_mlp, scale_mlp, gate_mlp, moe_fn, eps: float = 1e-6) -> torch.Tensor:
    """The MoE half of DiTBlock.forward (models.py:518-519) around any block
    function: ``x + gate_mlp.unsqueeze(1) * moe(modulate(norm2(x), shift_mlp,
    scale_mlp))`` with ``norm2 = LayerNorm(hidden, elementwise_affine=False,
    eps=1e-6)`` (models.py:494)."""
    normed = F.layer_norm(x, x.shape[-1:], None, None, eps)
    return x + gate_mlp.unsqueeze(1) * moe_fn(modulate(normed, shift_mlp, scale_mlp))


# ----------------------------------------------------------------------------
# Expert-parallel building blocks (per-rank restatement; the collectives are
# the caller's)
# ----------------------------------------------------------------------------


def permute_rows(x: torch.Tensor, flat_idx: torch.Tensor, k: int):
    """Local dispatch (ep_fwd.py:100-111, 344-347): returns the expert-sorted,
    duplicated rows and the sorted-position -> flat-row map."""
    order = stable_expert_order(flat_idx)
    return x.index_select(0, order // k), order


def unpermute_rows(rows: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    """Local combine (ep_fwd.py:349-354): row ``order[p]`` <- ``rows[p]``."""
    out = torch.zeros_like(rows)
    out.index_copy_(0, order, rows)
    return out


def weighted_pair_sum(rows_flat: torch.Tensor, flat_w: torch.Tensor, k: int) -> torch.Tensor:
    """``final.mul_(w)`` then ``view(N,k,h).sum(1)`` (ep_fwd.py:190-195)."""
    n = rows_flat.shape[0] // k
    return (rows_flat.float() * flat_w.view(-1, 1).float()).view(n, k, -1).sum(1).to(rows_flat.dtype)


def owner_rank(expert: int, world_size: int) -> int:
    """Round-robin expert placement (etrim.py:23-24)."""
    return expert % world_size


def local_expert_ids(rank: int, world_size: int, num_experts: int) -> List[int]:
    """Experts held by ``rank`` (etrim.py:23-24; ep_fwd.py:207)."""
    return list(range(rank, num_experts, world_size))


def proc_experts(
    rows: torch.Tensor,
    counts_global: torch.Tensor,
    experts: Sequence[Optional[Sequence[torch.Tensor]]],
    rank: int,
    world_size: int,
    act: str,
) -> torch.Tensor:
    """ep_fwd.py:199-211: local-expert slot ``i`` (global expert
    ``rank + i*world_size``) runs over ``counts_global.sum(0)[i]`` rows."""
    out = torch.empty_like(rows)
    per_slot = counts_global.sum(dim=0).tolist()
    start = 0
    for i, m in enumerate(per_slot):
        e = rank + i * world_size
        if m:
            out[start : start + m] = run_expert(rows[start : start + m], experts[e], act)
        start += m
    assert start == rows.shape[0]
    return out


def forced_sync_schedule(sample_steps: int, warm_up: int, strided_sync: int, cool_down: int) -> List[bool]:
    """``ep_forced_sync`` for i = sample_steps..1 (diffusion/warmup.py:6-26)."""
    out = []
    for i in range(sample_steps, 0, -1):
        if i == sample_steps:
            out.append(True)
            continue
        if warm_up < 1 and strided_sync < 1:
            out.append(False)
            continue
        rev = sample_steps - i
        need = False
        if 0 < rev <= warm_up:
            need = True
        elif strided_sync > 0 and i % strided_sync == 0:
            need = True
        elif i <= cool_down:
            need = True
        out.append(need)
    return out


def past_layer_key(key: int, total_layers: int, strategy: str) -> int:
    """diep.py:184-194."""
    if strategy == "all":
        return (key - 1) % total_layers
    if strategy == "shallow":
        return (key - 1) % (total_layers // 2)
    if strategy == "deep":
        return (key - 1) % (total_layers // 2) + total_layers // 2
    if strategy == "interleaved":
        return (key - 2) % total_layers
    raise ValueError(f"Unknown selective async strategy: {strategy}")


def layer_is_async(layer_idx: int, total_layers: int, mode: str) -> bool:
    """models.py:328-340."""
    if mode == "shallow":
        return layer_idx < total_layers // 2
    if mode == "deep":
        return layer_idx >= total_layers // 2
    if mode == "all":
        return True
    if mode == "interleaved":
        return layer_idx % 2 == 0
    raise ValueError(f"Invalid ep_async_mode: {mode}")
