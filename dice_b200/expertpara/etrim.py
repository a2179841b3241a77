"""Round-robin expert ownership under expert parallelism.

Rank ``r`` of ``W`` holds experts ``r, r+W, r+2W, ...``; every other entry of a
block's expert list is replaced by a placeholder that raises when called, and
the matching weights are dropped from a state dict before loading.  Mirrors
the reference's ``expertpara/etrim.py`` (:13-67).
"""
from __future__ import annotations

from typing import Dict, List

import torch.distributed as dist
import torch.nn as nn


class DummyExpert(nn.Module):
    """Placeholder for an expert owned by another rank (etrim.py:13-19)."""

    def forward(self, x):
        raise RuntimeError("DummyExpert should not be called")


_etrim_enable = True


def _needed_expert_indices(total_experts: int) -> List[int]:
    return list(range(dist.get_rank(), total_experts, dist.get_world_size()))


def trim_module_list(module_list: nn.ModuleList, total_experts: int) -> nn.ModuleList:
    """etrim.py:26-38."""
    assert _etrim_enable, "Expert trimming is disabled"
    mine = set(_needed_expert_indices(total_experts))
    return nn.ModuleList([m if i in mine else DummyExpert() for i, m in enumerate(module_list)])


def trim_state_dict(state_dict: Dict, total_experts: int) -> Dict:
    """Drop the parameters of experts held elsewhere; keys look like
    ``blocks.11.moe.experts.7.gate_proj.weight`` (etrim.py:40-67)."""
    assert _etrim_enable, "Expert trimming is disabled"
    mine = set(_needed_expert_indices(total_experts))
    kept, removed, out = 0, 0, {}
    for key, value in state_dict.items():
        if ".experts." in key:
            parts = key.split(".")
            expert = int(parts[parts.index("experts") + 1])
            if expert not in mine:
                removed += 1
                continue
            kept += 1
        out[key] = value
    assert removed == kept * (dist.get_world_size() - 1), \
        "Removed experts should be equal to kept experts times (world_size - 1)"
    return out
