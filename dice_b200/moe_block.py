"""The DiT-MoE sparse MoE block on B200 kernels: drop-in for the reference's
``models.py:159-382`` (``MoEGate``, ``MoeMLP``, ``SparseMoeBlock``) and the
``ParaMode`` flag bundle (``models.py:34-71``).

Constructor arguments, attribute names and state-dict keys are the
reference's, so checkpoints load unchanged and ``models.py`` / ``sample_ddp.py``
can use this class in place of their own.  In eval mode on a CUDA device the
forward runs the hand-written kernels (fused router, permute, grouped expert
FFN on the tensor cores, un-permute + weighted combine); there is no CPU or
PyTorch fallback for that path.  Training (``self.training``) is outside the
accelerated path and is expressed with ordinary differentiable torch
operations, as the reference does (``models.py:313-320``).
"""
from __future__ import annotations

import contextlib
import math
import os
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .expertpara.etrim import DummyExpert, trim_module_list


class ParaMode:
    """Parallelism flags handed from the launcher to every block
    (models.py:34-71)."""

    def __init__(self, ep=False, ep_async=False, sp=False, sp_async=False, num_sampling_steps=None,
                 ep_async_warm_up=None, strided_sync=None, ep_async_cool_down=None, sp_async_warm_up=None,
                 ep_async_mode=None):
        if ep_async:
            assert ep
        if sp_async:
            assert sp
        self.ep, self.ep_async, self.sp, self.sp_async = ep, ep_async, sp, sp_async
        self.dp = not ep and not sp
        self.num_sampling_steps = num_sampling_steps
        self.ep_async_warm_up = ep_async_warm_up
        self.strided_sync = strided_sync
        self.sp_async_warm_up = sp_async_warm_up
        self.ep_async_cool_down = ep_async_cool_down
        self.ep_async_mode = ep_async_mode

    def verbose(self):
        if self.dp:
            return "DP"
        name = []
        if self.ep:
            name.append("DiEP" if self.ep_async else "EP")
        if self.sp:
            name.append("DF" if self.sp_async else "SP")
        return "+".join(name)


def _scope(name: str):
    from .expertpara import diep

    prof = diep._profiler()
    return prof.scope(name) if prof is not None else contextlib.nullcontext()


def _compute_dtype(x: torch.Tensor) -> torch.dtype:
    """bf16 for 16-bit inputs and inside an autocast region (where the
    reference's linears run in 16 bits); fp32 inputs outside autocast take the
    fp32 kernels."""
    if x.dtype == torch.float32 and not torch.is_autocast_enabled():
        return torch.float32
    return torch.bfloat16


def layer_is_async(para_mode, layer_idx, total_layers) -> bool:
    """Which layers use the asynchronous exchange under each selective-sync
    mode (models.py:328-340)."""
    if not para_mode.ep_async:
        return False
    mode = para_mode.ep_async_mode
    if mode == "shallow":
        return layer_idx < total_layers // 2
    if mode == "deep":
        return layer_idx >= total_layers // 2
    if mode == "all":
        return True
    if mode == "interleaved":
        return layer_idx % 2 == 0
    raise ValueError(f"Invalid ep_async_mode: {mode}")


class MoEGate(nn.Module):
    """Router parameters and (for training / standalone use) the reference's
    gate arithmetic (models.py:159-217).  ``SparseMoeBlock`` does not call
    ``forward`` in eval mode on CUDA; it feeds ``weight`` to the fused router
    kernel."""

    def __init__(self, embed_dim, num_experts=16, num_experts_per_tok=2, aux_loss_alpha=0.01):
        super().__init__()
        self.top_k = num_experts_per_tok
        self.n_routed_experts = num_experts
        self.scoring_func = "softmax"
        self.alpha = aux_loss_alpha
        self.seq_aux = False
        self.norm_topk_prob = False
        self.gating_dim = embed_dim
        self.weight = nn.Parameter(torch.empty((self.n_routed_experts, self.gating_dim)))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, hidden_states):
        bsz, seq_len, h = hidden_states.shape
        x2d = hidden_states.reshape(-1, h)
        if x2d.is_cuda and not self.training and self.top_k == 2:
            cd = _compute_dtype(x2d)
            idx, w, _, _ = ops.router_top2(x2d.to(cd), self.weight.to(cd), renorm=self.norm_topk_prob)
            return idx, w, None
        scores = F.linear(x2d, self.weight, None).softmax(dim=-1)
        topk_weight, topk_idx = torch.topk(scores, k=self.top_k, dim=-1, sorted=False)
        if self.top_k > 1 and self.norm_topk_prob:
            topk_weight = topk_weight / (topk_weight.sum(dim=-1, keepdim=True) + 1e-20)
        aux_loss = None
        if self.training and self.alpha > 0.0:  # models.py:199-214 (token-level auxiliary loss)
            mask_ce = F.one_hot(topk_idx.view(-1), num_classes=self.n_routed_experts)
            ce = mask_ce.float().mean(0)
            aux_loss = (scores.mean(0) * ce * self.n_routed_experts).sum() * self.alpha
        return topk_idx, topk_weight, aux_loss


class AddAuxiliaryLoss(torch.autograd.Function):
    """Attach the auxiliary loss's gradient to the block output (models.py:220-237)."""

    @staticmethod
    def forward(ctx, x, loss):
        assert loss.numel() == 1
        ctx.dtype = loss.dtype
        ctx.required_aux_loss = loss.requires_grad
        return x

    @staticmethod
    def backward(ctx, grad_output):
        grad_loss = torch.ones(1, dtype=ctx.dtype, device=grad_output.device) if ctx.required_aux_loss else None
        return grad_output, grad_loss


class MoeMLP(nn.Module):
    """One SwiGLU expert: ``down_proj(silu(gate_proj(x)) * up_proj(x))``, no
    biases (models.py:240-273).  The module's own ``forward`` is plain torch
    (used for training and by callers that run a single expert); the block runs
    all experts together through the grouped FFN kernel."""

    def __init__(self, hidden_size, intermediate_size, pretraining_tp=2):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self.act_fn = nn.SiLU()
        self.pretraining_tp = pretraining_tp

    def forward(self, x):
        # the column/row slicing of models.py:253-269 is the same sum in another order
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class GeluMLP(nn.Module):
    """Two-matrix expert ``fc2(gelu_tanh(fc1(x)))`` without biases: the expert
    shape of the synthetic benchmark configurations; it has no counterpart in
    the reference."""

    def __init__(self, hidden_size, intermediate_size):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.fc1 = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.fc2 = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))


class ExpertPack:
    """Kernel-side view of a list of experts: stacked first-layer weights
    (gate/up interleaved for SwiGLU) and second-layer weights of the experts
    this rank holds, in local-slot order, rebuilt when a parameter changes."""

    # when set to a list, every FFN call appends (tag, start_event, end_event) recorded on the
    # launching stream (used by the benchmark to time the grouped-GEMM launches in place)
    timing = None
    timing_every = 1   # record only every n-th call (keeps the host cost of the instrumentation negligible)
    _timing_calls = 0

    @classmethod
    def _want_timing(cls) -> bool:
        if cls.timing is None:
            return False
        cls._timing_calls += 1
        return cls._timing_calls % cls.timing_every == 0

    def __init__(self, experts: Sequence[nn.Module], tag: str = "routed"):
        self._experts = experts
        self._built = {}
        self._calls = 0
        self.status = None
        self.tag = tag
        self._slab_tables = {}

    def _local(self) -> List[nn.Module]:
        return [e for e in self._experts if not isinstance(e, DummyExpert)]

    @staticmethod
    def _params(e: nn.Module):
        if isinstance(e, MoeMLP):
            return "swiglu", (e.gate_proj.weight, e.up_proj.weight, e.down_proj.weight)
        if isinstance(e, GeluMLP):
            return "gelu_tanh", (e.fc1.weight, e.fc2.weight)
        raise TypeError(f"cannot pack expert of type {type(e).__name__}")

    def invalidate(self) -> None:
        """Forget the packed weights (the block calls this when its parameters are replaced or reloaded)."""
        self._built.clear()

    def _signature(self, local):
        return tuple((p.data_ptr(), p._version) for e in local for p in self._params(e)[1])

    def get(self, dtype: torch.dtype):
        hit = self._built.get(dtype)
        if hit is not None:
            # per call only the first parameter is looked at; module-level changes (``.to()``, ``.half()``,
            # ``load_state_dict``) invalidate the pack through the block's hooks, and every 256th call
            # compares all parameters
            self._calls += 1
            p0 = hit[2]
            if p0.data_ptr() == hit[3] and p0._version == hit[4] and (self._calls & 255 or hit[0] == self._signature(self._local())):
                return hit[1]
        local = self._local()
        sig = self._signature(local)
        act = self._params(local[0])[0]
        dev = self._params(local[0])[1][0].device
        if dev.type != "cuda":
            raise RuntimeError("dice_b200 expert weights must live on a CUDA device (no CPU fallback)")
        with torch.no_grad():
            if act == "swiglu":
                ffn = local[0].intermediate_size
                w1 = torch.stack([ops.pack_w13(e.gate_proj.weight.to(dtype), e.up_proj.weight.to(dtype)) for e in local])
                w2 = torch.stack([e.down_proj.weight.to(dtype) for e in local]).contiguous()
            else:
                ffn = local[0].intermediate_size
                w1 = torch.stack([e.fc1.weight.to(dtype) for e in local]).contiguous()
                w2 = torch.stack([e.fc2.weight.to(dtype) for e in local]).contiguous()
            if self.status is None:
                self.status = ops.device_status(dev)
        built = (act, ffn, w1, w2)
        p0 = self._params(local[0])[1][0]
        self._built[dtype] = (sig, built, p0, p0.data_ptr(), p0._version)
        return built

    def ffn_width(self, dtype: torch.dtype) -> int:
        return self.get(dtype)[1]

    def run_offsets(self, rows: torch.Tensor, seg_offsets: torch.Tensor, seg_slab: Optional[torch.Tensor] = None,
                    reserve_sms: int = 0, shared=None, inter=None, out=None, rows_done=None, first_gemm_done=None,
                    then=None):
        """The grouped FFN over ``rows``.  ``shared = (tokens, pack of the shared expert)`` lets the shared expert
        ride in the same launches (bf16); the result is then ``(rows_out, shared_out)``.  ``inter`` / ``out`` are
        caller-owned buffers for the intermediate and the result (allocated per call when None).  ``then()`` is
        called right after the launches (before anything else is recorded on the stream): the place for work on
        another stream that should start beside them."""
        act, ffn, w1, w2 = self.get(rows.dtype)
        extra = None
        if shared is not None:
            sx, spack = shared
            s_act, s_ffn, sw1, sw2 = spack.get(rows.dtype)
            assert s_act == act
            extra = (sx, sw1, sw2, s_ffn)
        if not ExpertPack._want_timing():
            res = ops.grouped_ffn(rows, w1, w2, seg_offsets, act, ffn, status=self.status, seg_slab=seg_slab,
                                  reserve_sms=reserve_sms, shared=extra, inter=inter, out=out, rows_done=rows_done,
                                  first_gemm_done=first_gemm_done)
            if then is not None:
                then()
            return res
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        res = ops.grouped_ffn(rows, w1, w2, seg_offsets, act, ffn, status=self.status, seg_slab=seg_slab,
                              reserve_sms=reserve_sms, shared=extra, inter=inter, out=out, rows_done=rows_done,
                              first_gemm_done=first_gemm_done)
        if then is not None:
            then()
        end.record()
        ExpertPack.timing.append((self.tag if shared is None else self.tag + "+shared", start, end))
        return res

    def run_offsets_combine(self, rows: torch.Tensor, seg_offsets: torch.Tensor, order: torch.Tensor, flat_weights):
        """The grouped FFN with the gate-weighted combine in the second GEMM's epilogue: returns token rows."""
        act, ffn, w1, w2 = self.get(rows.dtype)
        timing = ExpertPack.timing if ExpertPack._want_timing() else None
        if timing is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        out = ops.grouped_ffn_combine(rows, w1, w2, seg_offsets, act, ffn, order, flat_weights, self.status)
        if timing is not None:
            end.record()
            timing.append((self.tag + "+combine", start, end))
        return out

    def run_offsets_return(self, rows: torch.Tensor, info):
        """FFN over the receive buffer of a peer-memory exchange with the
        return fused into the second GEMM (bf16 only): the outputs land in the
        token owners' buffers, nothing is stored locally."""
        from . import _lib

        act, ffn, w1, w2 = self.get(rows.dtype)
        x = info.xchg
        n_rows, h = rows.shape
        inter = torch.empty((n_rows, ffn), dtype=rows.dtype, device=rows.device)
        timing = ExpertPack.timing if ExpertPack._want_timing() else None
        if timing is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        _lib.check(x.lib.dice_grouped_ffn_return(
            rows.data_ptr(), n_rows, h, ffn, ops.ACT_CODES[act], w1.data_ptr(), w2.data_ptr(), w1.shape[0],
            info.seg_dev.data_ptr(), x.seg_slab_dev.data_ptr(), x.n_seg, inter.data_ptr(), x._meta_ptrs[info.slot],
            info.tab["back"], info.tab["f_back"], x._done_ptrs[2 * info.slot + 1], x.rank, x.world, x.min_peer_rows,
            info.seq, 0, self.status.data_ptr(), ops._stream()), "dice_grouped_ffn_return")
        if timing is not None:
            end.record()
            timing.append((self.tag, start, end))

    def slab_table(self, seg_slab: Sequence[int], device) -> torch.Tensor:
        """Device copy of a segment -> weight-slab table (cached: it only depends on world size and slots)."""
        key = (tuple(seg_slab), str(device))
        hit = self._slab_tables.get(key)
        if hit is None:
            hit = torch.tensor(list(seg_slab), dtype=torch.int32, device=device)
            self._slab_tables[key] = hit
        return hit

    def run_segments(self, rows: torch.Tensor, seg_counts: Sequence[int], seg_slab: Sequence[int]):
        """Segments given as host-side counts (the expert-parallel receive layout)."""
        offs = [0]
        for c in seg_counts:
            offs.append(offs[-1] + c)
        seg = torch.tensor(offs, dtype=torch.int32, device=rows.device)
        return self.run_offsets(rows, seg, self.slab_table(seg_slab, rows.device))

    def check(self):
        if self.status is not None:
            ops.check_status(self.status, "grouped expert FFN")


# DICE_FFN_COMBINE=1: blocks without a third addend let the second GEMM's epilogue do the gate-weighted combine
# (dice_grouped_ffn_combine).  Off by default: the 16-byte bf16 reductions cost the GEMM more (about 40 us per layer
# at 16384 tokens, hidden 1152) than the separate combine kernel they replace (about 22 us), and the rounding
# differs from the combine kernel's fp32 sum, so the single-device and expert-parallel paths would stop agreeing
# bit for bit.
epilogue_combine = os.environ.get("DICE_FFN_COMBINE", "0") == "1"
_fold_cached = None


def _fold_shared() -> bool:
    global _fold_cached
    if _fold_cached is None:
        _fold_cached = ops.shared_expert_can_ride()
    return _fold_cached


class SharedJob:
    """The shared expert's work of one block call, waiting for a grouped-FFN launch to ride in: the tokens, the
    shared expert's pack and what is needed to run it on its own if no suitable launch comes by."""

    def __init__(self, x, pack, seg_all, reserve_sms):
        self.x, self.pack, self.seg_all, self.reserve_sms = x, pack, seg_all, reserve_sms
        self.out = None

    def run_alone(self):
        with _scope("moe.mlp_shared"):
            self.out = self.pack.run_offsets(self.x, self.seg_all, reserve_sms=self.reserve_sms)
        return self.out


class SparseMoeBlock(nn.Module):
    """Routed experts + always-on shared expert (models.py:276-382).

    Same constructor as the reference.  Two keyword-only extensions select the
    synthetic benchmark variant: ``expert_act="gelu_tanh"`` builds two-matrix
    GELU-tanh experts, ``shared_expert=False`` drops the shared expert;
    ``self.gate.norm_topk_prob = True`` renormalises the top-2 weights
    (the reference's switch, models.py:170)."""

    def __init__(self, embed_dim, mlp_ratio=4, num_experts=16, num_experts_per_tok=2, pretraining_tp=2,
                 layer_idx=None, total_layers=None, para_mode: ParaMode = None, *, expert_act="swiglu",
                 shared_expert=True):
        super().__init__()
        assert para_mode is not None
        assert expert_act in ("swiglu", "gelu_tanh")
        self.num_experts_per_tok = num_experts_per_tok
        self.expert_act = expert_act
        inter = mlp_ratio * embed_dim

        def make(size):
            return MoeMLP(embed_dim, size, pretraining_tp) if expert_act == "swiglu" else GeluMLP(embed_dim, size)

        self.experts = nn.ModuleList([make(inter) for _ in range(num_experts)])
        if para_mode.ep:
            self.experts = trim_module_list(self.experts, num_experts)  # models.py:288-290
        self.gate = MoEGate(embed_dim=embed_dim, num_experts=num_experts, num_experts_per_tok=num_experts_per_tok)
        self.n_shared_experts = 2 if shared_expert else None
        if self.n_shared_experts is not None:
            self.shared_experts = make(embed_dim * self.n_shared_experts)
        self.layer_idx = layer_idx
        self.total_layers = total_layers
        self.para_mode = para_mode
        self.num_experts = num_experts
        self.experts._dice_pack = ExpertPack(self.experts)
        self._shared_pack = ExpertPack([self.shared_experts], tag="shared") if self.n_shared_experts is not None else None
        self._gate_cast = {}
        self._seg_cache = {}
        self._status = None
        self.register_load_state_dict_post_hook(lambda module, incompatible: module._invalidate_packs())

    def _invalidate_packs(self):
        self.experts._dice_pack.invalidate()
        if self._shared_pack is not None:
            self._shared_pack.invalidate()
        self._gate_cast.clear()

    def _apply(self, fn, *args, **kwargs):
        # .to() / .half() / .cuda() replace the parameters' storage: the packed copies must be rebuilt
        out = super()._apply(fn, *args, **kwargs)
        if hasattr(self, "_gate_cast"):
            self._invalidate_packs()
        return out

    # -- helpers ----------------------------------------------------------------
    def _gate_weight(self, dtype):
        w = self.gate.weight
        sig = (w.data_ptr(), w._version)
        hit = self._gate_cast.get(dtype)
        if hit is None or hit[0] != sig:
            hit = (sig, w.detach().to(dtype).contiguous())
            self._gate_cast[dtype] = hit
        return hit[1]

    def _async_layer(self) -> bool:
        return layer_is_async(self.para_mode, self.layer_idx, self.total_layers)

    def _segment_all(self, n_tokens: int, device) -> torch.Tensor:
        key = (n_tokens, str(device))
        seg = self._seg_cache.get(key)
        if seg is None:
            if len(self._seg_cache) > 16:
                self._seg_cache.clear()
            seg = torch.tensor([0, n_tokens], dtype=torch.int32, device=device)
            self._seg_cache[key] = seg
        return seg

    def _router_status(self, device):
        if self._status is None or self._status.device != device:
            self._status = ops.device_status(device)
        return self._status

    def check_status(self):
        """Raise if a kernel of this block reported an expired wait (synchronises)."""
        if self._status is not None:
            ops.check_status(self._status, "router")
        self.experts._dice_pack.check()
        if self._shared_pack is not None:
            self._shared_pack.check()

    # -- forward ------------------------------------------------------------------
    def forward(self, hidden_states):
        if self.training:
            return self._forward_train(hidden_states)
        if not hidden_states.is_cuda:
            raise RuntimeError("dice_b200.SparseMoeBlock runs on CUDA tensors only (no CPU fallback)")
        return self._forward_infer(hidden_states)

    @torch.no_grad()
    def forward_with_glue(self, x, shift, scale, gate, eps: float = 1e-6):
        """The MoE half of ``DiTBlock.forward`` (models.py:518-519),

            x + gate.unsqueeze(1) * self(modulate(LayerNorm(x), shift, scale)),

        with the LayerNorm (no affine parameters, models.py:494) and the
        modulation (models.py:75-76) in one kernel in front of the router and
        the gated residual inside the combine kernel: two full passes over
        ``[N, h]`` instead of six or seven.  ``x`` is ``[B, T, h]``; ``shift``,
        ``scale`` and ``gate`` are ``[B, h]`` (views are fine).  Training, CPU
        tensors and 16-bit floats other than bf16 take the plain formulation."""
        fusable = (not self.training and x.is_cuda and x.dim() == 3 and x.dtype in (torch.bfloat16, torch.float32))
        if not fusable:
            normed = F.layer_norm(x, x.shape[-1:], None, None, eps)
            return x + gate.unsqueeze(1) * self(normed * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1))
        cd = _compute_dtype(x)
        x = x.contiguous()
        x_in = ops.ln_modulate(x, shift.to(x.dtype), scale.to(x.dtype), eps, out_dtype=cd)
        if x.dtype != cd:  # fp32 residual stream around a 16-bit block: the residual stays in torch
            return x + gate.unsqueeze(1) * self._forward_infer(x_in).to(x.dtype)
        glue = (x.view(-1, x.shape[-1]), gate.to(cd).contiguous(), x.shape[1])
        return self._forward_infer(x_in, _glue=glue)

    @torch.no_grad()
    def _forward_infer(self, hidden_states, _glue=None):
        orig_shape, orig_dtype = hidden_states.shape, hidden_states.dtype
        h = orig_shape[-1]
        cd = _compute_dtype(hidden_states)
        x = hidden_states.reshape(-1, h)
        x = x.contiguous() if x.dtype == cd else x.to(cd)
        n_tokens = x.shape[0]
        assert self.num_experts_per_tok == 2, "the fused router selects exactly two experts per token"
        if not self.layer_idx:  # once per model forward (first layer, or a block used on its own)
            ops.poll_status(x.device)
        reserve = 0
        if self.para_mode.ep:
            from .expertpara import p2p

            reserve = p2p.reserve_sms()
        # bf16: the router also files one histogram per 128 tokens, from which the permutation plan is one launch
        chunked = cd == torch.bfloat16 and (2 * n_tokens + 255) // 256 * self.num_experts <= ops.PLAN_CHUNKED_MAX_INTS
        with _scope("moe.gate"):
            topk_idx, topk_weight, hist, _ = ops.router_top2(x, self._gate_weight(cd), renorm=self.gate.norm_topk_prob,
                                                             status=self._router_status(x.device), want_chunks=chunked)
        chunks = hist if chunked else None
        # The always-on shared expert (models.py:355-357).  In bf16 it rides in the routed experts' two launches as
        # one more problem of their tile list; otherwise it is a launch pair of its own, added inside the combine.
        shared_out = shared_job = None
        if self._shared_pack is not None:
            if cd == torch.bfloat16 and _fold_shared():
                shared_job = SharedJob(x, self._shared_pack, self._segment_all(n_tokens, x.device), reserve)
            else:
                with _scope("moe.mlp_shared"):
                    shared_out = self._shared_pack.run_offsets(x, self._segment_all(n_tokens, x.device), reserve_sms=reserve)
        if not self.para_mode.ep:
            y = self.moe_infer(x, topk_idx.view(-1), topk_weight.view(-1, 1), _addend=shared_out, _chunks=chunks,
                               _glue=_glue, _shared=shared_job)
        else:
            from .expertpara import diep as _diep, ep_fwd as _ep_fwd

            ep_skip_mask, ep_skip_now = _diep.ep_skip_mask, _diep.ep_skip_now
            partial_skip = _diep.ep_skip_enabled()
            y = _ep_fwd.moe_infer_ep(
                inp=x, experts=self.experts, flat_expert_indices=topk_idx.view(-1),
                flat_expert_weights=topk_weight.view(-1, 1), num_experts_per_tok=self.num_experts_per_tok,
                skip_mask=ep_skip_mask(topk_idx.numel()) if partial_skip else None,
                skip_now=ep_skip_now(self.layer_idx) if partial_skip else None,
                async_op=self._async_layer(), cache_key=self.layer_idx, _addend=shared_out, _chunks=chunks, _glue=_glue,
                _shared=shared_job)
        y = y.view(*orig_shape)
        return y if y.dtype == orig_dtype else y.to(orig_dtype)

    @ops.no_grad
    def moe_infer(self, x, flat_expert_indices, flat_expert_weights, _addend=None, _chunks=None, _glue=None,
                  _shared=None):
        """Single-device dispatch -> experts -> weighted combine
        (models.py:361-382), without a host sync: plan + row gather (one
        launch when the router filed per-chunk histograms, else four), two
        grouped GEMMs, combine."""
        assert not self.para_mode.ep
        n_tokens = x.shape[0]
        k = self.num_experts_per_tok
        if (epilogue_combine and _chunks is not None and _addend is None and _shared is None and _glue is None and k == 2
                and n_tokens > 0 and _fold_shared()):
            # nothing but the two expert rows goes into a token's output: the second GEMM can add them itself
            # (models.py:377-381 inside its epilogue), three launches and a memset for the whole dispatch -> combine
            pos, seg, order, rows = ops.permute_plan_chunked(flat_expert_indices, _chunks, self.num_experts, 1, x, k,
                                                             want_order=True)
            w_flat = flat_expert_weights.reshape(-1)
            w_flat = w_flat if w_flat.dtype == torch.float32 else w_flat.float()
            with _scope("moe.mlp"):
                return self.experts._dice_pack.run_offsets_combine(rows, seg, order, w_flat.contiguous())
        if _chunks is not None:
            pos, seg, _, rows = ops.permute_plan_chunked(flat_expert_indices, _chunks, self.num_experts, 1, x, k)
        else:
            pos, seg, _ = ops.permute_plan(flat_expert_indices, self.num_experts)
            rows = ops.permute_rows(x, pos, k)
        with _scope("moe.mlp"):
            if _shared is not None:
                y_rows, _addend = self.experts._dice_pack.run_offsets(rows, seg, shared=(_shared.x, _shared.pack))
            else:
                y_rows = self.experts._dice_pack.run_offsets(rows, seg)
        w = flat_expert_weights.view(n_tokens, k)
        w = w if w.dtype == torch.float32 else w.float()
        pp = pos.view(n_tokens, k)
        resid, gate, tps = _glue if _glue is not None else (None, None, 1)
        return ops.unpermute_combine(y_rows, pp[:, 0], y_rows, pp[:, 1], w[:, 0], w[:, 1], n_tokens, addend=_addend,
                                     resid=resid, gate=gate, tokens_per_sample=tps)

    def _forward_train(self, hidden_states):
        """models.py:313-320 with differentiable torch operations."""
        identity, orig_shape = hidden_states, hidden_states.shape
        topk_idx, topk_weight, aux_loss = self.gate(hidden_states)
        x = hidden_states.view(-1, orig_shape[-1]).repeat_interleave(self.num_experts_per_tok, dim=0)
        flat = topk_idx.view(-1)
        y = torch.empty_like(x)
        for i, expert in enumerate(self.experts):
            sel = flat == i
            if bool(sel.any()):
                y[sel] = expert(x[sel]).to(y.dtype)
        y = (y.view(*topk_weight.shape, -1) * topk_weight.unsqueeze(-1)).sum(dim=1).view(*orig_shape)
        if aux_loss is not None:
            y = AddAuxiliaryLoss.apply(y, aux_loss)
        if self.n_shared_experts is not None:
            y = y + self.shared_experts(identity)
        return y
