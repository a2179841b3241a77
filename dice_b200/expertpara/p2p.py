"""Set-up and bookkeeping of the NVLink peer-memory exchange (one process per
GPU on one box).

The kernels are in ``csrc/p2p_exchange.cu``; this module owns the buffers each
rank exposes to its peers, maps the peers' buffers through CUDA IPC, and hands
out (slot, sequence number) pairs.  It replaces, for the synchronous exchange,
the reference's ``exchange_token_counts`` / ``global_dispatch`` /
``global_combine`` (``expertpara/ep_fwd.py:214-342``): no NCCL call and no
host synchronisation remain on the per-layer path.

Buffers per rank (``n_slots`` copies, used round-robin so that a peer that is one
call ahead never writes what this rank still reads):

* ``ctrl``  int32: count matrix ``[W][E]`` + three flag arrays ``[W]``
* ``recv``  rows received for this rank's experts, ``capacity_rows x hidden``
* ``back``  expert outputs returned for this rank's tokens, ``max_rows x hidden``
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib

_FLAG_PAD = 64  # ints; keeps the three flag arrays on separate 256-byte lines


class PeerExchange:
    def __init__(self, n_experts: int, hidden: int, dtype: torch.dtype, max_rows: int, capacity_factor: float = 2.0,
                 n_slots: int = 2, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert n_experts % self.world == 0
        self.n_experts, self.hidden, self.dtype = n_experts, hidden, dtype
        self.el = n_experts // self.world
        self.n_slots = n_slots
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = _lib.load()
        self.max_rows = int(max_rows)
        self.calls = 0

        # every rank sizes its receive buffer from the largest sender
        sizes = [None] * self.world
        dist.all_gather_object(sizes, self.max_rows, group=group)
        biggest = max(sizes)
        self.capacity_rows = int(min(self.world * biggest, math.ceil(capacity_factor * biggest)))

        w, e = self.world, n_experts
        self.ctrl_stride = ((w * e + _FLAG_PAD - 1) // _FLAG_PAD + 3) * _FLAG_PAD
        self.flag_base = (w * e + _FLAG_PAD - 1) // _FLAG_PAD * _FLAG_PAD
        self.ctrl = torch.zeros(n_slots * self.ctrl_stride, dtype=torch.int32, device=self.device)
        self.recv = torch.zeros((n_slots, self.capacity_rows, hidden), dtype=dtype, device=self.device)
        self.back = torch.zeros((n_slots, self.max_rows, hidden), dtype=dtype, device=self.device)
        self.meta_ints = self.lib.dice_ep_meta_ints(w, self.el)
        self.meta = torch.zeros((n_slots, self.meta_ints), dtype=torch.int32, device=self.device)
        self.done = torch.zeros(2 * n_slots, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.seq = [0] * n_slots
        torch.cuda.synchronize()

        # every collective below is reached by every rank even when a step fails locally, so that a
        # rank that cannot export or map memory makes ALL ranks give up together instead of hanging
        mine = {"cap": self.capacity_rows, "max_rows": self.max_rows, "err": None}
        try:
            for name in ("ctrl", "recv", "back"):
                mine[name] = self._export(getattr(self, name))
        except Exception as exc:
            mine["err"] = f"rank {self.rank}: {exc}"
        everyone: List[Optional[dict]] = [None] * w
        dist.all_gather_object(everyone, mine, group=group)
        errs = [p["err"] for p in everyone if p["err"]]
        if errs:
            raise RuntimeError("; ".join(errs))
        self.peer_cap = [p["cap"] for p in everyone]
        self.peer_max_rows = [p["max_rows"] for p in everyone]
        base = {}
        self._imported = []
        ok = torch.ones(1, dtype=torch.int32, device=self.device)
        import_err = None
        try:
            for name in ("ctrl", "recv", "back"):
                ptrs = []
                for r, p in enumerate(everyone):
                    if r == self.rank:
                        ptrs.append(getattr(self, name).data_ptr())
                    else:
                        ptrs.append(self._import(*p[name]))
                base[name] = ptrs
        except Exception as exc:
            import_err = exc
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"mapping peer memory failed ({import_err or 'on another rank'})")
        esz = self.recv.element_size()
        self._tables = []
        for slot in range(n_slots):
            c_off = slot * self.ctrl_stride * 4
            t = {
                "matrix": self._table([b + c_off for b in base["ctrl"]]),
                "f_cnt": self._table([b + c_off + (self.flag_base + 0 * _FLAG_PAD) * 4 for b in base["ctrl"]]),
                "f_disp": self._table([b + c_off + (self.flag_base + 1 * _FLAG_PAD) * 4 for b in base["ctrl"]]),
                "f_back": self._table([b + c_off + (self.flag_base + 2 * _FLAG_PAD) * 4 for b in base["ctrl"]]),
                "recv": self._table([b + slot * self.peer_cap[r] * hidden * esz for r, b in enumerate(base["recv"])]),
                "back": self._table([b + slot * self.peer_max_rows[r] * hidden * esz for r, b in enumerate(base["back"])]),
            }
            self._tables.append(t)
        # the smallest receive / return capacity among the peers bounds what this rank may write
        self.min_peer_cap = min(self.peer_cap)
        dist.barrier(group=group)

    # -- IPC ---------------------------------------------------------------------
    def _export(self, t: torch.Tensor):
        handle = (ctypes.c_uint8 * 64)()
        offset = ctypes.c_uint64(0)
        _lib.check(self.lib.dice_ipc_export(t.data_ptr(), handle, ctypes.byref(offset)), "dice_ipc_export")
        return bytes(handle), int(offset.value)

    def _import(self, handle: bytes, offset: int) -> int:
        buf = (ctypes.c_uint8 * 64).from_buffer_copy(handle)
        out = ctypes.c_void_p(0)
        _lib.check(self.lib.dice_ipc_import(buf, offset, ctypes.byref(out)), "dice_ipc_import")
        self._imported.append((out.value, offset))
        return int(out.value)

    def _table(self, ptrs):
        return (ctypes.c_void_p * self.world)(*ptrs)

    # -- per call -------------------------------------------------------------------
    def begin(self):
        """Next (slot, sequence number, tables)."""
        slot = self.calls % self.n_slots
        self.calls += 1
        self.seq[slot] += 1
        return slot, self.seq[slot], self._tables[slot]

    def my_flags_ptr(self, slot: int, which: int) -> int:
        return self.ctrl.data_ptr() + (slot * self.ctrl_stride + self.flag_base + which * _FLAG_PAD) * 4

    def seg_offsets(self, slot: int) -> torch.Tensor:
        """Segments of the receive buffer, (source, slot) order: int32 [W*El + 1]."""
        a = 3 * self.world + 1
        return self.meta[slot, a:a + self.world * self.el + 1]

    def check(self):
        from .. import ops

        ops.check_status(self.status, "peer-memory exchange")


_exchange: Optional[PeerExchange] = None
_enabled = os.environ.get("DICE_EP_P2P", "0") == "1"
_failed = False


def enable(flag: bool = True) -> None:
    """Use the peer-memory exchange for synchronous expert parallelism (falls
    back to NCCL if the peers' memory cannot be mapped)."""
    global _enabled
    _enabled = flag


def enabled() -> bool:
    return _enabled and not _failed


def get_exchange(n_experts: int, hidden: int, dtype: torch.dtype, rows: int) -> Optional[PeerExchange]:
    """The process-wide exchange, created on first use (a collective call: every
    rank reaches it in the same layer call)."""
    global _exchange, _failed
    if not enabled():
        return None
    x = _exchange
    if x is not None:
        if (x.n_experts, x.hidden, x.dtype) != (n_experts, hidden, dtype) or rows > x.max_rows:
            raise RuntimeError("peer-memory exchange was sized for another shape "
                               f"(experts {x.n_experts}, hidden {x.hidden}, {x.dtype}, {x.max_rows} rows)")
        return x
    try:
        factor = float(os.environ.get("DICE_EP_P2P_CAPACITY", "2.0"))
        _exchange = PeerExchange(n_experts, hidden, dtype, max_rows=int(rows * 1.25) + 256, capacity_factor=factor)
    except Exception as exc:  # IPC not permitted in this environment: stay on NCCL, say so once
        _failed = True
        if dist.get_rank() == 0:
            print(f"dice_b200: peer-memory exchange unavailable ({exc}); using NCCL all-to-all", flush=True)
        return None
    return _exchange


def reset() -> None:
    global _exchange, _failed
    _exchange = None
    _failed = False
