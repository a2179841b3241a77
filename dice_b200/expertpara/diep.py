"""Staleness-tolerant (asynchronous) expert parallelism: drop-in for the
reference's ``expertpara/diep.py``.

Module-level state, as in the reference, because the sampler drives it through
free functions (``diffusion/rectified_flow.py:91-114``, ``sample_ddp.py:182-191``):

* a *dispatch* cache and a *combine* cache with one slot per layer
  (:class:`~.ep_cache.All2AllCache`), holding in-flight all-to-all exchanges
  with everything needed to consume them later;
* a *skip* cache (:class:`~.ep_cache.EPSkipCache`) for conditional
  communication.

Protocols (diep.py:196-310), per layer ``l`` and step ``t``:

* forced-sync step: both exchanges run synchronously and their results are
  stored under ``l`` with no handles (the caches were cleared just before);
* displaced (``async_pipeline=False``): consume the dispatch stored under ``l``
  (launched at ``t-1``), launch this step's dispatch; consume the combine stored
  under ``l`` (launched at ``t-1`` with results of ``t-2``'s tokens), launch the
  new combine: outputs are two steps stale;
* interweaved (``async_pipeline=True``): consume the dispatch the *previous
  asynchronous layer* launched earlier in the same step, run THAT layer's
  experts, and file the combine launched now under that layer's key; outputs
  are one step stale.

All cached tensors stay resident in device memory (``auto_gc`` only drops send
buffers of completed exchanges, as in the reference).
"""
from __future__ import annotations

import torch

from ..ops import no_grad as _no_grad
from .ep_cache import All2AllCache, EPSkipCache

_CACHE_DISPATCH_VAL_LEN = 8  # (handles, recv, counts_local, counts_global, pos, weights, experts, send)
_CACHE_COMBINE_VAL_LEN = 5   # (handles, recv, pos, weights, send)

_diep_cache_dispatch = None
_diep_cache_combine = None
_diep_cache_skip = None

_step = 0
_noskip_interval = 1
_enable_skip = False
_skip_mode = None
_async_pipeline = False
_selective_async_strategy = None
_forced_sync = False
_rand_mask = None
_mask_cache = {}
max_mem = -1


def _profiler():
    """The reference's ``CudaProfiler`` when its package is importable and a
    CUDA device is present (its scopes record CUDA events), else None."""
    global _prof_cls
    try:
        return _prof_cls
    except NameError:
        pass
    _prof_cls = None
    try:
        if torch.cuda.is_available():
            from cudaprof.prof import CudaProfiler  # provided by the reference checkout when run inside it

            _prof_cls = CudaProfiler
    except Exception:
        _prof_cls = None
    return _prof_cls


# ---- memory accounting (diep.py:38-55, 312-313) ------------------------------


def ep_all2all_cached_tensors_size():
    return _diep_cache_dispatch.tensors_size() + _diep_cache_combine.tensors_size()


def ep_skip_cached_tensors_size():
    return _diep_cache_skip.tensors_size()


def ep_cached_tensors_size():
    """Bytes held by the three caches."""
    return ep_all2all_cached_tensors_size() + ep_skip_cached_tensors_size()


def ep_get_max_mem():
    return max_mem


# ---- step / skip policy (diep.py:57-98) ----------------------------------------


def _poll_device_status():
    """A failure that a kernel recorded on the device (an expired wait, an
    exchange buffer that was too small, a peer that gave up) becomes a Python
    exception here, without a synchronisation: see ``ops.poll_status``."""
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        from .. import ops

        ops.poll_status()


def ep_set_step(step):
    global _step
    _step = step
    _poll_device_status()


def ep_skip_enabled():
    return _enable_skip


def ep_skip_now(idx):
    """Skip this step's second slot?  Only when conditional communication is on,
    the skip cache holds layer ``idx`` and the step is not a multiple of the
    no-skip interval (diep.py:61-68)."""
    if not _enable_skip or not _diep_cache_skip.contains(idx):
        return False
    return _step % _noskip_interval != 0


def ep_skip_mask(len):
    """Boolean row mask, True = row left out on skip steps: slot 0 of each
    token for 'high', slot 1 for 'low', one random slot per token (drawn once)
    for 'rand' (diep.py:72-90).  Masks are built once per length."""
    global _rand_mask
    if _skip_mode == "rand":
        if _rand_mask is None:
            n = len // 2
            pick = torch.randint(0, 2, (n,))
            mask = torch.zeros((n, 2), dtype=torch.bool)
            mask[torch.arange(n), pick] = True
            _rand_mask = mask.view(-1)
        return _rand_mask
    if _skip_mode not in ("high", "low"):
        raise ValueError(f"Unknown skip mode: {_skip_mode}")
    key = (_skip_mode, len)
    mask = _mask_cache.get(key)
    if mask is None:
        mask = torch.zeros(len, dtype=torch.bool)
        mask[(0 if _skip_mode == "high" else 1)::2] = True
        _mask_cache[key] = mask
    return mask


def ep_wait():
    _diep_cache_dispatch.wait()
    _diep_cache_combine.wait()


# ---- forced synchronisation (diep.py:100-109) ------------------------------------


def diep_force_sync():
    global _forced_sync
    assert not _forced_sync
    _forced_sync = True


def diep_cancel_sync():
    global _forced_sync
    assert _forced_sync
    _forced_sync = False


# ---- set-up (diep.py:112-163) ------------------------------------------------------


def ep_cache_init(cache_capacity, auto_gc=False, noskip_step=1, skip_mode=None, async_pipeline=False,
                  selective_async_strategy=None):
    assert selective_async_strategy in [None, "shallow", "deep", "interleaved", "all"]
    global _selective_async_strategy, _async_pipeline, _noskip_interval, _enable_skip, _skip_mode
    global _diep_cache_dispatch, _diep_cache_combine, _diep_cache_skip, _forced_sync, _rand_mask, max_mem
    _selective_async_strategy = selective_async_strategy
    _async_pipeline = async_pipeline
    _noskip_interval = noskip_step  # every noskip_step-th step communicates both slots
    _enable_skip = noskip_step != 1
    if _enable_skip:
        assert skip_mode is not None
    _skip_mode = skip_mode
    _forced_sync = False
    _rand_mask = None
    max_mem = -1
    _diep_cache_dispatch = All2AllCache(capacity=cache_capacity, gc_send_buf=auto_gc, val_len=_CACHE_DISPATCH_VAL_LEN,
                                        gc_recv_buf=auto_gc and _async_pipeline)
    # the combine cache is consumed a step later in interweaved mode: its receive buffers are never collected
    _diep_cache_combine = All2AllCache(capacity=cache_capacity, gc_send_buf=auto_gc, val_len=_CACHE_COMBINE_VAL_LEN,
                                       gc_recv_buf=False)
    _diep_cache_skip = EPSkipCache(capacity=cache_capacity if _enable_skip else 0)


def ep_cache_clear():
    _poll_device_status()
    _diep_cache_dispatch.clear()
    _diep_cache_combine.clear()
    _diep_cache_skip.clear()


def ep_skip_get(key):
    """Rows cached for the skipped slot of layer ``key``; clears the entry."""
    return _diep_cache_skip.get(key)


def ep_skip_put(key, tensor):
    assert isinstance(tensor, torch.Tensor)
    _diep_cache_skip.put(key, tensor)


# ---- the two protocols (diep.py:178-310) ------------------------------------------


_ep_fwd_module = None


def _ep_fwd():
    """``expertpara.ep_fwd`` (imported late: that module imports this one); looked up through
    ``sys.modules`` semantics once, then cached, but re-read when someone replaced the module attribute."""
    global _ep_fwd_module
    if _ep_fwd_module is None:
        from . import ep_fwd

        _ep_fwd_module = ep_fwd
    return _ep_fwd_module


def _wait(handles):
    if handles is not None:
        for handle in handles:
            handle.wait()


def _past_layer_key(key):
    """The asynchronous layer that ran just before layer ``key`` (wrapping to
    the last one of the previous step), for each selective strategy
    (diep.py:184-194)."""
    total_layers = _diep_cache_dispatch.capacity
    if _selective_async_strategy == "all":
        return (key - 1) % total_layers
    if _selective_async_strategy == "shallow":
        return (key - 1) % (total_layers // 2)
    if _selective_async_strategy == "deep":
        return (key - 1) % (total_layers // 2) + total_layers // 2
    if _selective_async_strategy == "interleaved":
        return (key - 2) % total_layers
    raise ValueError(f"Unknown selective async strategy: {_selective_async_strategy}")


@_no_grad
def global_dispatch_async(grouped_dup_inp, token_counts_local, token_counts_global, grouped_idx_dup,
                          flat_expert_weights, experts, cache_key):
    """Launch this call's dispatch and hand back an earlier one to compute on
    (diep.py:196-259).  Returns ``(recv_rows, counts_local, counts_global,
    pos, weights, experts)`` of the exchange being consumed."""
    global_dispatch = _ep_fwd().global_dispatch
    assert cache_key is not None
    if _forced_sync:
        buf, _ = global_dispatch(grouped_dup_inp, token_counts_local, token_counts_global, async_op=False)
        assert not _diep_cache_dispatch.contains(cache_key)
        _diep_cache_dispatch.put(cache_key, (None, buf, token_counts_local, token_counts_global, grouped_idx_dup,
                                             flat_expert_weights, experts, None))
        return buf, token_counts_local, token_counts_global, grouped_idx_dup, flat_expert_weights, experts

    if _async_pipeline:
        key_to_get = _past_layer_key(cache_key)
        assert _diep_cache_dispatch.contains(key_to_get)
    else:
        key_to_get = cache_key
    (prev_handles, prev_buf, prev_counts_local, prev_counts_global, prev_pos, prev_weights, prev_experts,
     _prev_send) = _diep_cache_dispatch.get(key_to_get)
    _wait(prev_handles)
    _diep_cache_dispatch.manual_gc_recv_buf()
    buf, handles = global_dispatch(grouped_dup_inp, token_counts_local, token_counts_global, async_op=True)
    # the send side stays alive until the exchange completes: the gathered rows, or (peer-memory exchange,
    # where the gather is part of the dispatch kernel) the layer input itself
    send_buf = getattr(grouped_dup_inp, "keepalive", grouped_dup_inp)
    _diep_cache_dispatch.put(cache_key, (handles, buf, token_counts_local, token_counts_global, grouped_idx_dup,
                                         flat_expert_weights, experts, send_buf))
    global max_mem
    max_mem = max(max_mem, ep_cached_tensors_size())
    return prev_buf, prev_counts_local, prev_counts_global, prev_pos, prev_weights, prev_experts


@_no_grad
def global_combine_async(grouped_dup_outp, token_counts_local, token_counts_global, grouped_idx_dup,
                         flat_expert_weights, cache_key):
    """Launch the combine of the rows just computed and hand back the combine
    stored for this layer (diep.py:261-310).  Returns ``(rows, pos, weights)``
    of the exchange being consumed."""
    global_combine = _ep_fwd().global_combine
    assert cache_key is not None
    if _forced_sync:
        buf, _ = global_combine(grouped_dup_outp, token_counts_local, token_counts_global, async_op=False)
        assert not _diep_cache_combine.contains(cache_key)
        _diep_cache_combine.put(cache_key, (None, buf, grouped_idx_dup, flat_expert_weights, None))
        return buf, grouped_idx_dup, flat_expert_weights

    if _async_pipeline:
        key_to_put = _past_layer_key(cache_key)
        assert _diep_cache_combine.contains(cache_key)
    else:
        key_to_put = cache_key
    prev_handles, prev_buf, prev_pos, prev_weights, _prev_send = _diep_cache_combine.get(cache_key)
    _wait(prev_handles)
    buf, handles = global_combine(grouped_dup_outp, token_counts_local, token_counts_global, async_op=True)
    _diep_cache_combine.put(key_to_put, (handles, buf, grouped_idx_dup, flat_expert_weights,
                                         getattr(grouped_dup_outp, "keepalive", grouped_dup_outp)))
    return prev_buf, prev_pos, prev_weights
