"""CPU stand-in for the device operations, backed by the oracle.

Lets the expert-parallel HOST logic (count exchange, all-to-all layout, the
displaced / interweaved cache protocols, conditional communication) run among
CPU gloo ranks.  Test infrastructure only: the package never imports this.
"""
import torch

from oracle import moe_oracle as O


class OracleOps:
    def plan(self, keys, n_keys):
        order = O.stable_expert_order(keys)
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel())
        hist = O.expert_histogram(keys, n_keys)
        seg = torch.cat([torch.zeros(1, dtype=torch.int64), hist.cumsum(0)])
        return pos.to(torch.int32), seg.to(torch.int32)

    def permute_rows(self, x, pos, k):
        out = torch.empty((x.shape[0] * k, x.shape[1]), dtype=x.dtype)
        out[pos.long()] = x.repeat_interleave(k, dim=0)
        return out

    def unpermute_combine(self, src0, idx0, src1, idx1, w0, w1, n_tokens, addend=None):
        def term(src, idx, w):
            rows = src[idx.long()] if idx is not None else src[:n_tokens]
            rows = rows.float()
            return rows * w.view(-1, 1).float() if w is not None else rows

        acc = term(src0, idx0, w0)
        if src1 is not None:
            acc = acc + term(src1, idx1, w1)
        if addend is not None:
            acc = acc + addend.float()
        return acc.to(src0.dtype)

    def run_packed_experts(self, rows, pack, seg_counts, seg_slab):
        raise AssertionError("packed experts are a CUDA-only path")
