"""Device operations of the MoE block: thin wrappers that hand torch CUDA
tensors (device memory + stream only) to the C-ABI kernels.

Every function requires CUDA tensors and the built native library; there is no
CPU or PyTorch fallback.  Names follow the reference's vocabulary: *rows* are
the (token, slot) rows of ``ep_fwd.py:100-111``, *segments* the per-expert runs
of expert-sorted rows.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

DICE_BF16, DICE_F32 = 0, 1
ACT_SWIGLU, ACT_GELU_TANH = 0, 1
EPI_STORE, EPI_GELU_TANH, EPI_SWIGLU = 0, 1, 2
ACT_CODES = {"swiglu": ACT_SWIGLU, "gelu_tanh": ACT_GELU_TANH}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DICE_BF16
    if t.dtype == torch.float32:
        return DICE_F32
    raise TypeError(f"dice_b200 kernels take bfloat16 or float32 tensors, got {t.dtype}")


def _require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "dice_b200 operations run on CUDA tensors only (no CPU fallback); got a tensor on " + str(t.device)
            )


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Raw handle of torch's current stream on the current device."""
    if _raw_stream is not None:  # much cheaper than building a Stream object
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_stream_objects = {}


def current_stream_object() -> "torch.cuda.Stream":
    """torch's current stream as a Stream object, looked up by its raw handle
    (``torch.cuda.current_stream()`` itself costs several microseconds per call,
    which adds up on the per-layer path of the asynchronous exchange)."""
    if _raw_stream is None:
        return torch.cuda.current_stream()
    dev = torch.cuda.current_device()
    key = (dev, _raw_stream(dev))
    obj = _stream_objects.get(key)
    if obj is None:
        if len(_stream_objects) > 64:
            _stream_objects.clear()
        obj = _stream_objects[key] = torch.cuda.current_stream()
    return obj


def no_grad(fn):
    """``@torch.no_grad()`` that costs nothing when gradients are already off
    (the block's forward enters the no-grad region once; the functions below
    it keep the reference's decorators without paying for them again)."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if torch.is_grad_enabled():
            with torch.no_grad():
                return fn(*args, **kwargs)
        return fn(*args, **kwargs)

    return wrapper


def check_status(status: torch.Tensor, what: str = "dice_b200 kernel") -> None:
    """Read a device status word (synchronises) and raise if a kernel's bounded
    wait expired."""
    code = int(status.item())
    if code != 0:
        msg = _lib.load().dice_status_message(code).decode()
        status.zero_()
        raise RuntimeError(f"{what}: device status {code}: {msg}")


class _StatusWord:
    """The status word every kernel of this process reports to on one device,
    with a pinned host mirror that is refreshed by asynchronous copies."""

    def __init__(self, device: torch.device):
        self.dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False


_status_words = {}


def _status_word(device) -> _StatusWord:
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(device)
    if word is None:
        word = _status_words[device] = _StatusWord(device)
    return word


def device_status(device) -> torch.Tensor:
    """The int32 status word shared by the kernels this package launches on
    ``device`` (the first failure wins; see ``dice_status_message``)."""
    return _status_word(device).dev


def poll_status(device=None) -> None:
    """Look at the device status word WITHOUT synchronising: raise if the copy
    enqueued by an earlier call has landed and shows a failure (an expired
    wait, an exchange buffer that was too small, a peer that gave up), then
    enqueue the next copy on the current stream.  Called once per model
    forward and per sampling step by the block and by ``ep_set_step`` /
    ``ep_cache_clear``, so a failure surfaces within a step or two instead of
    turning into silently wrong images."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if torch.cuda.is_current_stream_capturing():
        return
    word = _status_word(device)
    if word.pending:
        if not word.event.query():
            return
        word.pending = False
        code = int(word.host[0])
        if code != 0:
            word.dev.zero_()
            word.host.zero_()
            raise RuntimeError(f"dice_b200 kernels reported device status {code}: "
                               + _lib.load().dice_status_message(code).decode())
    with torch.cuda.device(device):
        word.host.copy_(word.dev, non_blocking=True)
        word.event.record()
    word.pending = True


# --------------------------------------------------------------------------- #
# router
# --------------------------------------------------------------------------- #


def router_top2(
    x2d: torch.Tensor, w_gate: torch.Tensor, renorm: bool = False, want_logits: bool = False,
    status: Optional[torch.Tensor] = None, want_chunks: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Fused gate: returns ``(topk_idx int64 [N,2], topk_weight fp32 [N,2],
    hist int32 [E], logits or None)``; replaces ``MoEGate.forward``
    (models.py:179-217) and the ``bincount`` of ep_fwd.py:70.

    With ``want_chunks`` (bf16 only) the third result is instead the
    per-128-token histogram table ``int32 [ceil(N/128), E]`` that
    :func:`permute_plan_chunked` consumes."""
    _require_cuda(x2d, w_gate)
    assert x2d.dim() == 2 and w_gate.dim() == 2 and x2d.shape[1] == w_gate.shape[1]
    assert x2d.dtype == w_gate.dtype, "router weight must have the activation dtype"
    x2d = x2d.contiguous()
    w_gate = w_gate.contiguous()
    n, h = x2d.shape
    e = w_gate.shape[0]
    idx = torch.empty((n, 2), dtype=torch.int64, device=x2d.device)
    w = torch.empty((n, 2), dtype=torch.float32, device=x2d.device)
    hist = chunks = None
    if want_chunks:
        chunks = torch.empty(((n + 127) // 128, e), dtype=torch.int32, device=x2d.device)
    else:
        hist = torch.empty((e,), dtype=torch.int32, device=x2d.device)
    logits = torch.empty((n, e), dtype=x2d.dtype, device=x2d.device) if want_logits else None
    lib = _lib.load()
    _lib.check(
        lib.dice_router_top2(
            _ptr(x2d), _ptr(w_gate), n, h, e, _dtype_code(x2d), int(renorm), _ptr(idx), _ptr(w), _ptr(hist),
            _ptr(chunks), _ptr(logits), _ptr(status), _stream(),
        ),
        "dice_router_top2",
    )
    return idx, w, (chunks if want_chunks else hist), logits


def top2_from_logits(logits: torch.Tensor, renorm: bool = False):
    """Selection stage only (softmax + top-2 of models.py:186-196)."""
    _require_cuda(logits)
    logits = logits.contiguous()
    n, e = logits.shape
    idx = torch.empty((n, 2), dtype=torch.int64, device=logits.device)
    w = torch.empty((n, 2), dtype=torch.float32, device=logits.device)
    hist = torch.empty((e,), dtype=torch.int32, device=logits.device)
    lib = _lib.load()
    _lib.check(
        lib.dice_top2_from_logits(_ptr(logits), n, e, _dtype_code(logits), int(renorm), _ptr(idx), _ptr(w), _ptr(hist), _stream()),
        "dice_top2_from_logits",
    )
    return idx, w, hist


# --------------------------------------------------------------------------- #
# permutation
# --------------------------------------------------------------------------- #


def permute_plan(flat_idx: torch.Tensor, n_experts: int, want_order: bool = False):
    """Stable counting sort of rows by expert.  Returns ``(pos int32 [R],
    seg_offsets int32 [E+1], order int32 [R] or None)`` where ``pos[r]`` is the
    sorted position of row ``r`` (the inverse of the reference's
    ``flat_expert_indices.argsort()``, ep_fwd.py:100) and ``order`` is that
    argsort itself."""
    _require_cuda(flat_idx)
    assert flat_idx.dtype == torch.int64 and flat_idx.dim() == 1
    flat_idx = flat_idx.contiguous()
    r = flat_idx.shape[0]
    lib = _lib.load()
    nbytes = lib.dice_permute_scratch_bytes(r, n_experts)
    scratch = torch.empty((max(nbytes, 4) // 4,), dtype=torch.int32, device=flat_idx.device)
    pos = torch.empty((r,), dtype=torch.int32, device=flat_idx.device)
    order = torch.empty((r,), dtype=torch.int32, device=flat_idx.device) if want_order else None
    seg = torch.empty((n_experts + 1,), dtype=torch.int32, device=flat_idx.device)
    _lib.check(
        lib.dice_permute_plan(_ptr(flat_idx), r, n_experts, _ptr(scratch), scratch.numel() * 4, _ptr(pos), _ptr(order),
                              _ptr(seg), _stream()),
        "dice_permute_plan",
    )
    return pos, seg, order


def permute_plan_chunked(flat_idx: torch.Tensor, chunk_hist: torch.Tensor, n_experts: int, world: int = 1,
                         x2d: Optional[torch.Tensor] = None, k: int = 2, want_order: bool = False):
    """The plan in one launch from the router's per-128-token histograms
    (``router_top2(..., want_chunks=True)``), ordered by expert id (``world``
    1) or by ``(owner rank, local slot)`` of the round-robin placement
    (``world`` > 1, etrim.py:23-24).  With ``x2d`` the row gather of
    :func:`permute_rows` is part of the same kernel.  Returns ``(pos, seg_offsets,
    order or None, rows or None)``."""
    _require_cuda(flat_idx, chunk_hist, x2d)
    assert flat_idx.dtype == torch.int64 and flat_idx.dim() == 1 and flat_idx.is_contiguous()
    assert chunk_hist.dtype == torch.int32 and chunk_hist.is_contiguous()
    r = flat_idx.shape[0]
    assert chunk_hist.numel() == (r + 255) // 256 * n_experts
    dev = flat_idx.device
    pos = torch.empty((r,), dtype=torch.int32, device=dev)
    order = torch.empty((r,), dtype=torch.int32, device=dev) if want_order else None
    seg = torch.empty((n_experts + 1,), dtype=torch.int32, device=dev)
    rows, h, code = None, 0, 0
    if x2d is not None:
        assert x2d.is_contiguous() and x2d.shape[0] * k == r
        h, code = x2d.shape[1], _dtype_code(x2d)
        rows = torch.empty((r, h), dtype=x2d.dtype, device=dev)
    _lib.check(
        _lib.load().dice_permute_plan_chunked(_ptr(flat_idx), _ptr(chunk_hist), r, n_experts, world, _ptr(pos), _ptr(order),
                                              _ptr(seg), _ptr(x2d), k, h, code, _ptr(rows), _stream()),
        "dice_permute_plan_chunked",
    )
    return pos, seg, order, rows


# the chunked plan adds the whole per-chunk table up in every CTA: beyond this size use the three-pass plan
PLAN_CHUNKED_MAX_INTS = 16384


def permute_rows(x2d: torch.Tensor, pos: torch.Tensor, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[pos[t*k+s]] = x[t]`` — the row gather of ep_fwd.py:107-111."""
    _require_cuda(x2d, pos, out)
    x2d = x2d.contiguous()
    n, h = x2d.shape
    assert pos.dtype == torch.int32 and pos.numel() == n * k
    if out is None:
        out = torch.empty((n * k, h), dtype=x2d.dtype, device=x2d.device)
    assert out.is_contiguous() and out.shape[1] == h and out.shape[0] >= n * k and out.dtype == x2d.dtype
    _lib.check(
        _lib.load().dice_permute_rows(_ptr(x2d), _ptr(pos), n, k, h, _dtype_code(x2d), _ptr(out), _stream()),
        "dice_permute_rows",
    )
    return out


def unpermute_combine(
    src0: torch.Tensor,
    idx0: Optional[torch.Tensor],
    src1: Optional[torch.Tensor],
    idx1: Optional[torch.Tensor],
    w0: Optional[torch.Tensor],
    w1: Optional[torch.Tensor],
    n_tokens: int,
    addend: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    resid: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
    tokens_per_sample: int = 1,
) -> torch.Tensor:
    """``y[t] = w0[t]*src0[idx0[t]] + w1[t]*src1[idx1[t]] + addend[t]`` and
    ``out[t] = resid[t] + gate[t // tokens_per_sample] * y[t]`` (residual and
    gate optional: the DiT block's ``x + gate_mlp * moe(...)``, models.py:519).

    ``idx*`` and ``w*`` may be strided 1-D views (e.g. ``pos[0::2]``); the two
    weight views must share one stride.  Replaces ep_fwd.py:172-195."""
    _require_cuda(src0, idx0, src1, idx1, w0, w1, addend, out, resid, gate)
    h = src0.shape[1]
    assert src0.is_contiguous() and (src1 is None or (src1.is_contiguous() and src1.dtype == src0.dtype))
    for i in (idx0, idx1):
        assert i is None or (i.dtype == torch.int32 and i.dim() == 1 and i.shape[0] == n_tokens)
    w_stride = 1
    for w in (w0, w1):
        if w is not None:
            assert w.dtype == torch.float32 and w.dim() == 1 and w.shape[0] == n_tokens
            w_stride = w.stride(0) if n_tokens > 1 else 1
    if w0 is not None and w1 is not None and n_tokens > 1:
        assert w0.stride(0) == w1.stride(0)
    if addend is not None:
        assert addend.is_contiguous() and addend.shape == (n_tokens, h) and addend.dtype == src0.dtype
    if resid is not None:
        assert resid.is_contiguous() and resid.shape == (n_tokens, h) and resid.dtype == src0.dtype
    if gate is not None:
        assert gate.is_contiguous() and gate.dim() == 2 and gate.shape[1] == h and gate.dtype == src0.dtype
        assert gate.shape[0] * tokens_per_sample >= n_tokens
    if out is None:
        out = torch.empty((n_tokens, h), dtype=src0.dtype, device=src0.device)
    assert out.is_contiguous() and out.shape == (n_tokens, h) and out.dtype == src0.dtype
    s0 = idx0.stride(0) if (idx0 is not None and n_tokens > 1) else 1
    s1 = idx1.stride(0) if (idx1 is not None and n_tokens > 1) else 1
    _lib.check(
        _lib.load().dice_unpermute_combine(
            _ptr(src0), _ptr(idx0), s0, _ptr(src1), _ptr(idx1), s1, _ptr(w0), _ptr(w1), w_stride, _ptr(addend),
            _ptr(resid), _ptr(gate), tokens_per_sample, n_tokens, h, _dtype_code(src0), _ptr(out), _stream(),
        ),
        "dice_unpermute_combine",
    )
    return out


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``LayerNorm(x) * (1 + scale[:, None]) + shift[:, None]`` in one pass
    (``modulate(self.norm2(x), shift_mlp, scale_mlp)``, models.py:75-76, :494,
    :519).  ``x`` is ``[B, T, h]``, ``shift`` / ``scale`` are ``[B, h]`` of
    the same dtype (bf16 or fp32); statistics in fp32."""
    _require_cuda(x, shift, scale)
    assert x.dim() == 3 and shift.shape == (x.shape[0], x.shape[2]) and scale.shape == shift.shape
    assert shift.dtype == x.dtype and scale.dtype == x.dtype
    x, shift, scale = x.contiguous(), shift.contiguous(), scale.contiguous()
    b, t, h = x.shape
    out_dtype = out_dtype or x.dtype
    out = torch.empty((b, t, h), dtype=out_dtype, device=x.device)
    code_out = DICE_BF16 if out_dtype == torch.bfloat16 else DICE_F32
    assert out_dtype in (torch.bfloat16, torch.float32)
    _lib.check(
        _lib.load().dice_ln_modulate(_ptr(x), _ptr(shift), _ptr(scale), b * t, h, t, float(eps), _dtype_code(x), code_out,
                                     _ptr(out), _stream()),
        "dice_ln_modulate",
    )
    return out


# --------------------------------------------------------------------------- #
# expert weights and the grouped FFN
# --------------------------------------------------------------------------- #


def w13_rows(ffn: int) -> int:
    return int(_lib.load().dice_w13_rows(ffn))


def pack_w13(gate_proj: torch.Tensor, up_proj: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Interleave ``gate_proj``/``up_proj`` ([F, h] each, models.py:246-247)
    in 128-row blocks for the SwiGLU epilogue."""
    _require_cuda(gate_proj, up_proj, out)
    gate_proj, up_proj = gate_proj.contiguous(), up_proj.contiguous()
    f, h = gate_proj.shape
    assert up_proj.shape == (f, h) and up_proj.dtype == gate_proj.dtype
    rows = w13_rows(f)
    if out is None:
        out = torch.empty((rows, h), dtype=gate_proj.dtype, device=gate_proj.device)
    assert out.shape == (rows, h) and out.is_contiguous()
    _lib.check(
        _lib.load().dice_pack_w13(_ptr(gate_proj), _ptr(up_proj), h, f, _dtype_code(gate_proj), _ptr(out), _stream()),
        "dice_pack_w13",
    )
    return out


def grouped_gemm(
    a: torch.Tensor,
    w: torch.Tensor,
    seg_offsets: torch.Tensor,
    epilogue: int,
    n_out: int,
    status: torch.Tensor,
    seg_slab: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    reserve_sms: int = 0,
) -> torch.Tensor:
    """One grouped GEMM stage on the tensor cores (bf16):
    ``out[r] = epilogue(a[r] @ w[slab(seg(r))].T)``."""
    _require_cuda(a, w, seg_offsets, status, seg_slab, out)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    assert w.dim() == 3 and a.dim() == 2 and w.shape[2] == a.shape[1]
    assert seg_offsets.dtype == torch.int32 and status.dtype == torch.int32
    n_rows, k_dim = a.shape
    n_slabs, w_rows, _ = w.shape
    n_seg = seg_offsets.numel() - 1
    if out is None:
        out = torch.empty((n_rows, n_out), dtype=torch.bfloat16, device=a.device)
    assert out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= n_rows
    _lib.check(
        _lib.load().dice_grouped_gemm(
            _ptr(a), n_rows, k_dim, _ptr(w), n_slabs, w_rows, _ptr(seg_offsets), _ptr(seg_slab), n_seg, epilogue,
            _ptr(out), out.stride(0), n_out, reserve_sms, _ptr(status), _stream(),
        ),
        "dice_grouped_gemm",
    )
    return out


def _event_handle(event: Optional[torch.cuda.Event]):
    """The cudaEvent_t behind a torch event (torch creates it at the first record)."""
    if event is None:
        return None
    handle = event.cuda_event
    handle = getattr(handle, "value", handle)
    if not handle:
        raise RuntimeError("the event has never been recorded: torch has not created its CUDA event yet")
    return handle


def grouped_ffn(
    rows: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    seg_offsets: torch.Tensor,
    act: str,
    ffn: int,
    status: Optional[torch.Tensor] = None,
    seg_slab: Optional[torch.Tensor] = None,
    inter: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    reserve_sms: int = 0,
    shared=None,
    rows_done: Optional[torch.Tensor] = None,
    first_gemm_done: Optional[torch.cuda.Event] = None,
):
    """Expert FFN over expert-sorted rows (ep_fwd.py:199-211; models.py:368-376).

    ``w1``: packed gate/up ``[S, w13_rows(F), h]`` (swiglu) or fc1 ``[S, F, h]``
    (gelu_tanh); ``w2``: ``[S, h, F]``.  bf16 runs on the tensor cores, fp32 on
    the CUDA cores.  ``reserve_sms`` SMs are left to kernels of other streams
    (the side-stream pushes of the asynchronous exchange).

    ``shared = (tokens [N, h], w1 [1, ..., h], w2 [1, h, Fs], Fs)`` (bf16 only)
    runs the block's shared expert over all tokens inside the same two
    launches; the result is then ``(rows_out, shared_out)``.

    ``rows_done`` (bf16 only): zeroed int32 counters, one per 256-row block of
    the output, that the second GEMM raises as blocks complete (a return push
    on another stream follows them); ``first_gemm_done``: an event recorded
    between the two GEMMs (that push's stream waits for it)."""
    _require_cuda(rows, w1, w2, seg_offsets, status, seg_slab, inter, out, rows_done)
    assert rows.is_contiguous() and w1.is_contiguous() and w2.is_contiguous()
    assert seg_offsets.dtype == torch.int32
    n_rows, h = rows.shape
    n_slabs = w1.shape[0]
    n_seg = seg_offsets.numel() - 1
    assert w2.shape == (n_slabs, h, ffn) and w1.shape[2] == h
    if inter is None:
        inter = torch.empty((max(n_rows, 1), ffn), dtype=rows.dtype, device=rows.device)
    if out is None:
        out = torch.empty((n_rows, h), dtype=rows.dtype, device=rows.device)
    assert inter.is_contiguous() and out.is_contiguous() and inter.shape[1] == ffn and inter.shape[0] >= n_rows
    lib = _lib.load()
    if rows.dtype == torch.bfloat16:
        assert status is not None and status.dtype == torch.int32
        sx = sw1 = sw2 = s_inter = s_out = None
        n_shared = s_ffn = 0
        if shared is not None:
            sx, sw1, sw2, s_ffn = shared
            _require_cuda(sx, sw1, sw2)
            assert sx.is_contiguous() and sx.dtype == rows.dtype and sx.shape[1] == h
            assert sw1.is_contiguous() and sw2.is_contiguous() and sw2.shape == (1, h, s_ffn) and sw1.shape[0] == 1
            n_shared = sx.shape[0]
            s_inter = torch.empty((max(n_shared, 1), s_ffn), dtype=rows.dtype, device=rows.device)
            s_out = torch.empty((n_shared, h), dtype=rows.dtype, device=rows.device)
        _lib.check(
            lib.dice_grouped_ffn(
                _ptr(rows), n_rows, h, ffn, ACT_CODES[act], _ptr(w1), _ptr(w2), n_slabs, _ptr(seg_offsets),
                _ptr(seg_slab), n_seg, _ptr(inter), _ptr(out), _ptr(sx), n_shared, s_ffn, _ptr(sw1), _ptr(sw2),
                _ptr(s_inter), _ptr(s_out), reserve_sms, _ptr(rows_done),
                _event_handle(first_gemm_done), _ptr(status), _stream(),
            ),
            "dice_grouped_ffn",
        )
        return (out, s_out) if shared is not None else out
    assert shared is None, "the shared expert rides along in the bf16 kernel only"
    assert rows_done is None, "block counters are the bf16 kernel's"
    if rows.dtype == torch.float32:
        _lib.check(
            lib.dice_grouped_ffn_f32(
                _ptr(rows), n_rows, h, ffn, ACT_CODES[act], _ptr(w1), _ptr(w2), n_slabs, _ptr(seg_offsets),
                _ptr(seg_slab), n_seg, _ptr(inter), _ptr(out), _stream(),
            ),
            "dice_grouped_ffn_f32",
        )
    else:
        raise TypeError(f"unsupported dtype {rows.dtype}")
    return out


def grouped_ffn_combine(rows: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, seg_offsets: torch.Tensor, act: str,
                        ffn: int, order: torch.Tensor, flat_weights: torch.Tensor, status: torch.Tensor,
                        reserve_sms: int = 0) -> torch.Tensor:
    """Expert FFN over expert-sorted rows with the gate-weighted combine
    (models.py:377-381) inside the second GEMM's epilogue: returns ``[N, h]``
    token rows, ``out[t] = sum_s w[t, s] * ffn(row(t, s))``.  bf16, two rows
    per token; ``order`` is the plan's sorted-position -> flat-row map,
    ``flat_weights`` the fp32 top-2 weights viewed flat."""
    _require_cuda(rows, w1, w2, seg_offsets, order, flat_weights, status)
    assert rows.dtype == torch.bfloat16 and rows.is_contiguous() and w1.is_contiguous() and w2.is_contiguous()
    n_rows, h = rows.shape
    assert n_rows % 2 == 0 and order.dtype == torch.int32 and order.numel() == n_rows
    assert flat_weights.dtype == torch.float32 and flat_weights.is_contiguous() and flat_weights.numel() == n_rows
    n_slabs = w1.shape[0]
    inter = torch.empty((max(n_rows, 1), ffn), dtype=rows.dtype, device=rows.device)
    out = torch.empty((n_rows // 2, h), dtype=rows.dtype, device=rows.device)
    _lib.check(
        _lib.load().dice_grouped_ffn_combine(
            _ptr(rows), n_rows, h, ffn, ACT_CODES[act], _ptr(w1), _ptr(w2), n_slabs, _ptr(seg_offsets), None,
            seg_offsets.numel() - 1, _ptr(inter), _ptr(order), _ptr(flat_weights), 2, _ptr(out), reserve_sms, _ptr(status),
            _stream(),
        ),
        "dice_grouped_ffn_combine",
    )
    return out


def shared_expert_can_ride() -> bool:
    """Whether the grouped-FFN launches can carry the shared expert as an extra
    problem (the CTA-pair kernel can; ``DICE_GEMM_PAIR=0`` selects the
    one-CTA-per-tile kernel, which cannot)."""
    import os

    return os.environ.get("DICE_GEMM_PAIR", "1") != "0"
