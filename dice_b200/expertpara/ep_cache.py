"""Per-layer caches of in-flight all-to-all exchanges and of skipped-slot rows.

Same observable behaviour as the reference's ``expertpara/ep_cache.py``
(``All2AllCache`` :66-186, ``EPSkipCache`` :188-235): one slot per layer, a
value is a fixed-length tuple whose first item is the list of collective work
handles (or None), whose second item is the receive buffer and whose last item
is the send buffer kept alive until the collective completes.  All tensors stay
resident in device memory; nothing is offloaded.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence, Tuple

import torch

HANDLES_IDX = 0
RECV_BUF_IDX = 1
SEND_BUF_IDX = -1


def is_completed(handles: Optional[Sequence[Any]]) -> bool:
    """True when there is nothing left to wait for (ep_cache.py:59-62)."""
    return handles is None or all(h.is_completed() for h in handles)


def _tensor_bytes(item: Any) -> int:
    return item.element_size() * item.numel() if isinstance(item, torch.Tensor) else 0


class All2AllCache:
    """``capacity`` slots of ``val_len``-tuples (ep_cache.py:66-186)."""

    def __init__(self, capacity: int, val_len: int, gc_send_buf: bool, cl_name: Optional[str] = None,
                 gc_recv_buf: bool = False):
        self.capacity = capacity
        self.val_len = val_len
        self.gc_send_buf = gc_send_buf
        self.gc_recv_buf = gc_recv_buf
        self.cl_name = cl_name
        self.cache: List[Optional[Tuple]] = [None] * capacity
        self._bytes: List[int] = [0] * capacity  # tensor bytes per slot, kept current by put / release / clear

    # -- completion ---------------------------------------------------------
    def wait(self) -> None:
        """Wait for every handle still stored (ep_cache.py:84-90)."""
        for entry in self.cache:
            if entry is not None and entry[HANDLES_IDX] is not None:
                for handle in entry[HANDLES_IDX]:
                    handle.wait()

    def clear(self) -> None:
        self.cache = [None] * self.capacity
        self._bytes = [0] * self.capacity

    # -- access ---------------------------------------------------------------
    def put(self, key: int, value: Tuple) -> None:
        """Store ``value`` under ``key``; with ``gc_send_buf`` the send buffers
        of completed exchanges are dropped first (ep_cache.py:96-111)."""
        assert isinstance(key, int) and len(value) == self.val_len
        assert value[HANDLES_IDX] is None or isinstance(value[HANDLES_IDX], list)
        assert value[SEND_BUF_IDX] is None or isinstance(value[SEND_BUF_IDX], torch.Tensor)
        if self.gc_send_buf:
            self._release(SEND_BUF_IDX, clear_handles=True)
        self.cache[key] = value
        self._bytes[key] = sum(_tensor_bytes(x) for x in value)

    def get(self, key: int) -> Tuple:
        """Return the tuple under ``key`` without removing it (ep_cache.py:114-124)."""
        assert isinstance(key, int)
        assert isinstance(self.cache[key][RECV_BUF_IDX], torch.Tensor)
        return self.cache[key]

    def contains(self, key: int) -> bool:
        assert isinstance(key, int)
        return self.cache[key] is not None

    # -- garbage collection ---------------------------------------------------
    def _release(self, field: int, clear_handles: bool) -> None:
        for i, entry in enumerate(self.cache):
            if entry is not None and is_completed(entry[HANDLES_IDX]):
                item = list(entry)
                if clear_handles:
                    item[HANDLES_IDX] = None
                self._bytes[i] -= _tensor_bytes(item[field])
                item[field] = None
                self.cache[i] = tuple(item)

    def manual_gc_recv_buf(self) -> None:
        """Drop receive buffers of completed exchanges; a no-op unless the cache
        was built with ``gc_recv_buf`` (ep_cache.py:144-153).  The automatic
        variant of the reference is disabled there (:155-160) and has no
        counterpart here."""
        if self.gc_recv_buf:
            self._release(RECV_BUF_IDX, clear_handles=False)

    def tensors_size(self) -> int:
        """Bytes of all tensors held (ep_cache.py:169-186)."""
        return sum(self._bytes)


class EPSkipCache:
    """One tensor per layer: the un-permuted rows of the slot that conditional
    communication leaves out on skip steps.  ``get`` clears the slot
    (ep_cache.py:188-235)."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.cache: List[Optional[torch.Tensor]] = [None] * capacity

    def clear(self) -> None:
        self.cache = [None] * self.capacity

    def put(self, key: int, tensor: torch.Tensor) -> None:
        assert isinstance(key, int) and isinstance(tensor, torch.Tensor)
        self.cache[key] = tensor

    def get(self, key: int) -> Optional[torch.Tensor]:
        assert isinstance(key, int)
        value, self.cache[key] = self.cache[key], None
        return value

    def contains(self, key: int) -> bool:
        assert isinstance(key, int)
        return self.cache[key] is not None

    def tensors_size(self) -> int:
        return sum(_tensor_bytes(x) for x in self.cache)
