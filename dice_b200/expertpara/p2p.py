"""Set-up and bookkeeping of the NVLink peer-memory exchange (one process per
GPU on one box).

The kernels are in ``csrc/p2p_exchange.cu``; this module owns the buffers each
rank exposes to its peers, maps the peers' buffers through CUDA IPC, and hands
out (slot, sequence number) pairs.  It replaces, for the synchronous exchange,
the reference's ``exchange_token_counts`` / ``global_dispatch`` /
``global_combine`` (``expertpara/ep_fwd.py:214-342``): no NCCL call and no
host synchronisation remain on the per-layer path.

Buffers per rank, one set per *slot*.  A layer owns ``n_par`` slots and uses them
in turn, so an exchange launched at one step can still be in flight, or waiting
to be consumed, while the same layer launches the next ones (the displaced
protocol consumes a dispatch one step and its results two steps after launch;
peers are never more than a step ahead, so three slots per layer suffice):

* ``ctrl``  int32: count matrix ``[W][E]`` + three flag arrays (64 words each:
  flags ``[W]`` and, from word 32, the failure marks ``[W]``)
* ``recv``  rows received for this rank's experts, ``capacity_rows x hidden``
* ``back``  expert outputs returned for this rank's tokens, ``max_rows x hidden``

Receive capacity.  The reference has no capacity: ``all_to_all_single`` receives
whatever the router sends (``ep_fwd.py:247-293``).  Here the receive buffers are
allocated once, so ``capacity_rows`` is ``W x`` the largest sender's rows (which
no routing can exceed) whenever all slots then fit into a share of the free
device memory (``DICE_EP_P2P_MEM_FRACTION``, default 0.5), and otherwise as
many rows as that share holds, never fewer than twice the largest sender.  A
routing that still does not fit is detected by every rank in the count exchange
and reported through the device status word (``ops.poll_status``).
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
    def __init__(self, n_experts: int, hidden: int, dtype: torch.dtype, max_rows: int,
                 capacity_factor: Optional[float] = None, n_layers: int = 1, n_par: int = 3, group=None):
        n_slots = n_layers * n_par
        self.n_layers, self.n_par = n_layers, n_par
        self.uses = [0] * n_layers
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
        self._comm = None

        # every rank sizes its receive buffer from the largest sender and the tightest memory, so that all
        # ranks arrive at the same capacity
        sizes = [None] * self.world
        free_bytes = torch.cuda.mem_get_info(self.device)[0]
        dist.all_gather_object(sizes, (self.max_rows, free_bytes), group=group)
        biggest = max(r for r, _ in sizes)
        lossless = self.world * biggest
        if capacity_factor is not None:
            self.capacity_rows = int(min(lossless, math.ceil(capacity_factor * biggest)))
        else:
            share = float(os.environ.get("DICE_EP_P2P_MEM_FRACTION", "0.5")) * min(f for _, f in sizes)
            row_bytes = hidden * torch.empty((), dtype=dtype).element_size()
            fit = int((share / n_slots - self.max_rows * row_bytes) // row_bytes)  # recv + back per slot
            self.capacity_rows = int(min(lossless, max(2 * biggest, fit)))
        self.lossless = self.capacity_rows >= lossless
        # With room for W x the largest sender, every source gets a fixed region of each receive buffer and the
        # exchange needs no count rendezvous (csrc/p2p_exchange.cu); otherwise the sources' blocks are packed and
        # a count exchange tells every source where its block starts.
        self.region_rows = biggest if (self.lossless and os.environ.get("DICE_EP_P2P_REGIONS", "1") != "0") else 0

        w, e = self.world, n_experts
        self.ctrl_stride = ((w * e + _FLAG_PAD - 1) // _FLAG_PAD + 3) * _FLAG_PAD
        self.flag_base = (w * e + _FLAG_PAD - 1) // _FLAG_PAD * _FLAG_PAD
        self.ctrl = torch.zeros(n_slots * self.ctrl_stride, dtype=torch.int32, device=self.device)
        self.recv = torch.zeros((n_slots, self.capacity_rows, hidden), dtype=dtype, device=self.device)
        self.back = torch.zeros((n_slots, self.max_rows, hidden), dtype=dtype, device=self.device)
        self.meta_ints = self.lib.dice_ep_meta_ints(w, self.el)
        self.meta = torch.zeros((n_slots, self.meta_ints), dtype=torch.int32, device=self.device)
        self.done = torch.zeros(2 * n_slots, dtype=torch.int32, device=self.device)
        from .. import ops

        self.status = ops.device_status(self.device)  # shared with the other kernels: polled once per step
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
        self.min_peer_rows = min(self.peer_max_rows)
        a = 4 * self.world + 3  # first of the segment offsets in a meta block
        segs_per_source = self.el + 1 if self.region_rows else self.el
        self.n_seg = self.world * segs_per_source
        self._seg_views = [self.meta[s, a:a + self.n_seg + 1] for s in range(n_slots)]
        self._meta_ptrs = [self.meta[s].data_ptr() for s in range(n_slots)]
        self._done_ptrs = [self.done.data_ptr() + 4 * i for i in range(2 * n_slots)]
        self._recv_views = [self.recv[s] for s in range(n_slots)]
        self.status_ptr = self.status.data_ptr()
        # weight slab of every segment; in the region layout every source's slots are followed by the unused rest
        # of its region, which has no slab (-1: the GEMM skips it)
        per_source = list(range(self.el)) + ([-1] if self.region_rows else [])
        self.seg_slab = [i for _ in range(self.world) for i in per_source]
        self.seg_slab_dev = torch.tensor(self.seg_slab, dtype=torch.int32, device=self.device)
        # finished 256-row blocks of the expert FFN's output (see follow_ffn); None where the kernels have no counters
        self.rows_done = None
        row_bytes = self.hidden * 2
        bulk = os.environ.get("DICE_EP_P2P_BULK", "1") != "0" and row_bytes % 16 == 0 and row_bytes <= 16384
        if self.dtype == torch.bfloat16 and len(self.seg_slab) <= 256 and bulk:  # (the push follows in its bulk form)
            self.rows_done = torch.zeros(self.capacity_rows // 256 + len(self.seg_slab) + 1, dtype=torch.int32,
                                         device=self.device)
        wait_ms = int(os.environ.get("DICE_EP_P2P_WAIT_MS", "0"))
        if wait_ms:  # how long a kernel waits for another rank before it gives up (2000 ms by default)
            from .._lib import check

            check(self.lib.dice_ep_set_wait_limit_ms(wait_ms), "dice_ep_set_wait_limit_ms")
        self._fork = torch.cuda.Event()
        self._fork.record()  # torch creates the CUDA event at its first record; the C side is handed its handle
        self._side_events = [torch.cuda.Event() for _ in range(2 * n_slots)]
        self._ring_events = [torch.cuda.Event() for _ in range(self.FFN_OUT_RING)]
        self._ffn_inter, self._ffn_out, self._ffn_out_event, self._ffn_out_index, self._ffn_next = {}, [], [], {}, 0
        self._comm = torch.cuda.Stream(device=self.device, priority=_side_priority)
        self.comm_raw = self._comm.cuda_stream
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
    def begin(self, layer: int = 0):
        """Next (slot, sequence number, tables) of ``layer``."""
        layer %= self.n_layers
        slot = layer * self.n_par + self.uses[layer] % self.n_par
        self.uses[layer] += 1
        self.calls += 1
        self.seq[slot] += 1
        return slot, self.seq[slot], self._tables[slot]

    def follow_ffn(self, info: "SegInfo", out: torch.Tensor) -> "ReturnedRows":
        """Launch, on the side stream, the return push that follows the expert FFN just launched on the current
        stream with ``rows_done=self.rows_done, first_gemm_done=self._fork`` into ``out``.  The side stream waits
        for the first GEMM, which had the whole GPU; the push then takes the SMs that the second GEMM leaves free.
        The push is launched after its producer, so that it never waits for a kernel the host has yet to launch
        (a first launch may load its module, which can wait for running kernels)."""
        from .._lib import check

        self._comm.wait_event(self._fork)
        stream = self.comm_raw
        tab, slot = info.tab, info.slot
        check(self.lib.dice_ep_return_rows_following(
            out.data_ptr(), self._meta_ptrs[slot], tab["back"], tab["f_back"], self._done_ptrs[2 * slot + 1], self.hidden,
            self.rank, self.world, self.min_peer_rows, self.capacity_rows, info.seq, follow_ctas(),
            self.rows_done.data_ptr(), self.rows_done.numel(), self.seg_slab_dev.data_ptr(), self.n_seg, self.status_ptr,
            stream), "dice_ep_return_rows_following")
        self.note_output_read_on_side(out)
        # no event for the consumer: the push raises this rank's own flag too when all its stores are out, and the
        # combine waits for every source's flag on the device; an event wait would only cut the launch chain
        return ReturnedRows(info, None, beside_ffn=True)

    def fork_to_comm(self) -> int:
        """Order the side stream (on which asynchronous pushes run next to the
        expert FFN) after everything enqueued so far on the current stream;
        returns its raw handle."""
        from ..ops import current_stream_object

        self._fork.record(current_stream_object())
        self._comm.wait_event(self._fork)
        return self.comm_raw

    # -- scratch of the expert FFN over a receive buffer -----------------------------
    # The receive buffer holds `capacity_rows` rows (W x the largest sender when memory allows), of which a
    # routing fills about 1/W.  Allocating the FFN's intermediate and output per call at that size and keeping
    # the outputs alive in the asynchronous caches (two steps x all layers) made the caching allocator thrash on
    # the G/2 shapes.  The exchange therefore owns one intermediate per FFN width and a small ring of output
    # buffers: an output is read by the return push that follows its FFN and is free again long before the ring
    # comes round (the event of that push is waited for all the same).
    FFN_OUT_RING = 4

    def ffn_buffers(self, ffn: int):
        """(intermediate [capacity, ffn], output [capacity, hidden]) for the next expert FFN over a receive buffer."""
        from ..ops import current_stream_object

        inter = self._ffn_inter.get(ffn)
        if inter is None:
            inter = self._ffn_inter[ffn] = torch.empty((self.capacity_rows, ffn), dtype=self.dtype, device=self.device)
        if not self._ffn_out:
            self._ffn_out = [torch.empty((self.capacity_rows, self.hidden), dtype=self.dtype, device=self.device)
                             for _ in range(self.FFN_OUT_RING)]
            self._ffn_out_event = [None] * self.FFN_OUT_RING
            self._ffn_out_index = {t.data_ptr(): i for i, t in enumerate(self._ffn_out)}
            for t in self._ffn_out:
                t.keepalive = None  # the asynchronous caches need not (and must not) count or pin ring buffers
        i = self._ffn_next
        self._ffn_next = (i + 1) % self.FFN_OUT_RING
        ev = self._ffn_out_event[i]
        if ev is not None:  # the side-stream push that last read this buffer
            current_stream_object().wait_event(ev)
            self._ffn_out_event[i] = None
        return inter, self._ffn_out[i]

    def note_output_read_on_side(self, rows_back: torch.Tensor) -> None:
        """A return push on the side stream reads ``rows_back``: if it is a ring buffer, remember where the side
        stream is, so that the buffer's next use waits for this push."""
        i = self._ffn_out_index.get(rows_back.data_ptr()) if self._ffn_out else None
        if i is not None:
            ev = self._ring_events[i]
            ev.record(self._comm)
            self._ffn_out_event[i] = ev

    def record_side_event(self, slot: int, which: int) -> torch.cuda.Event:
        """Mark the side stream's position after a push of ``slot`` (0 dispatch, 1 return)."""
        ev = self._side_events[2 * slot + which]
        ev.record(self._comm)
        return ev

    def my_flags_ptr(self, slot: int, which: int) -> int:
        return self.ctrl.data_ptr() + (slot * self.ctrl_stride + self.flag_base + which * _FLAG_PAD) * 4

    def seg_offsets(self, slot: int) -> torch.Tensor:
        """Segments of the receive buffer, (source, slot) order: int32 [W*El + 1]."""
        return self._seg_views[slot]

    def check(self):
        from .. import ops

        ops.check_status(self.status, "peer-memory exchange")

    def close(self) -> None:
        """Unmap the peers' buffers (all ranks should have stopped using the exchange)."""
        torch.cuda.synchronize(self.device)
        for ptr, offset in self._imported:
            self.lib.dice_ipc_close(ptr, offset)
        self._imported = []


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


def side_push_ctas() -> int:
    """How many CTAs a push may use when it runs on the side stream next to
    the expert FFN (``DICE_EP_P2P_SIDE_CTAS``, default 8; -1 selects the SIMT
    push over all SMs).  The FFN's persistent kernel is told to leave the same
    number of SMs free, so the two never compete for an SM: the push moves its
    rows with the copy unit through shared memory, the GEMM keeps its own SMs
    to itself."""
    return _side_ctas


_side_ctas = int(os.environ.get("DICE_EP_P2P_SIDE_CTAS", "8"))  # read once: this is on the per-layer path
_side_priority = int(os.environ.get("DICE_EP_P2P_SIDE_PRIORITY", "0"))  # CUDA stream priority of the side stream


_side_pushes = False


def note_push(async_op: bool) -> None:
    """Remember whether the exchange is in an asynchronous phase (the last push
    went to the side stream)."""
    global _side_pushes
    _side_pushes = bool(async_op)


def reserve_sms() -> int:
    """SMs the expert FFN should leave free: the side pushes' CTAs while the
    exchange is asynchronous, else none."""
    if not _side_pushes:
        return 0
    n = side_push_ctas()
    return n if n > 0 else 0


_fused_return = os.environ.get("DICE_EP_P2P_FUSED_RETURN", "0") == "1"
_return_follows = os.environ.get("DICE_EP_P2P_RETURN_FOLLOWS", "1") == "1"


def set_return_follows(flag: bool) -> None:
    global _return_follows
    _return_follows = flag


_follow_ctas = int(os.environ.get("DICE_EP_P2P_FOLLOW_CTAS", "16"))
_pair_gemm = os.environ.get("DICE_GEMM_PAIR", "1") != "0"  # only the CTA-pair GEMM counts finished blocks


def follow_ctas() -> int:
    """CTAs (= SMs) of the return push that follows the second expert GEMM.  One SM's copy unit moves about
    30-38 GB/s through shared memory, so hiding a whole return under the second GEMM takes more SMs than a push
    that has a whole FFN to hide under (``side_push_ctas``)."""
    return _follow_ctas


def return_follows() -> bool:
    """Whether, in a synchronous exchange, the return push is launched on the
    side stream together with the expert FFN and sends each chunk of rows as
    soon as the second GEMM has finished the blocks it lies in (the reference
    runs FFN and all-to-all one after the other, ep_fwd.py:375-381)."""
    return _return_follows and _follow_ctas > 0 and _pair_gemm


def set_fused_return(flag: bool) -> None:
    global _fused_return
    _fused_return = flag


def fused_return() -> bool:
    """Whether the second expert GEMM writes its rows straight into the token
    owners' buffers instead of a separate return kernel.  Off by default: the
    epilogue's 64-byte row pieces use NVLink poorly and stall the accumulator
    hand-over (measured: the GEMM loses more than the return kernel costs)."""
    return _fused_return


def get_exchange(n_experts: int, hidden: int, dtype: torch.dtype, rows: int, n_layers: int = 1) -> Optional[PeerExchange]:
    """The process-wide exchange, created on first use (a collective call: every
    rank reaches it in the same layer call).  ``n_layers`` is the number of
    layers that keep exchanges in flight (the capacity given to
    ``ep_cache_init``), 1 when nothing is cached."""
    global _exchange, _failed
    if not enabled():
        return None
    x = _exchange
    if x is not None:
        if (x.n_experts, x.hidden, x.dtype) != (n_experts, hidden, dtype) or rows > x.max_rows or n_layers > x.n_layers:
            raise RuntimeError("peer-memory exchange was sized for another shape "
                               f"(experts {x.n_experts}, hidden {x.hidden}, {x.dtype}, {x.max_rows} rows, "
                               f"{x.n_layers} layers); call ep_cache_init before the first forward and "
                               "p2p.reset() to change shapes")
        return x
    try:
        factor = os.environ.get("DICE_EP_P2P_CAPACITY")
        factor = float(factor) if factor else None
        n_par = int(os.environ.get("DICE_EP_P2P_SLOTS", "3"))
        _exchange = PeerExchange(n_experts, hidden, dtype, max_rows=int(rows * 1.25) + 256, capacity_factor=factor,
                                 n_layers=max(1, n_layers), n_par=n_par)
    except Exception as exc:  # IPC not permitted in this environment: stay on NCCL, say so once
        _failed = True
        if dist.get_rank() == 0:
            print(f"dice_b200: peer-memory exchange unavailable ({exc}); using NCCL all-to-all", flush=True)
        return None
    return _exchange


def reset() -> None:
    """Drop the process-wide exchange (a collective decision: every rank calls it)."""
    global _exchange, _failed, _side_pushes
    if _exchange is not None:
        _exchange.close()
    _exchange = None
    _failed = False
    _side_pushes = False


# ---- stand-ins that travel through the exchange protocol of ep_fwd / diep -------------------


class SegInfo:
    """Plays the part of ``token_counts_global`` for one exchange: which slot and
    sequence number it uses, how many rows this rank sent, and (on the device)
    how the rows it receives are segmented."""

    def __init__(self, xchg: PeerExchange, slot: int, seq: int, tab, rows_sent: int):
        self.xchg, self.slot, self.seq, self.tab, self.rows_sent = xchg, slot, seq, tab, rows_sent

    @property
    def seg_dev(self) -> torch.Tensor:
        return self.xchg.seg_offsets(self.slot)


class PendingRows:
    """Plays the part of ``grouped_dup_inp``: the rows are not gathered into a
    send buffer; the dispatch kernel reads ``inp`` through ``pos`` and writes
    each row into its expert owner's receive buffer."""

    def __init__(self, inp: torch.Tensor, pos: torch.Tensor, seg_offsets: torch.Tensor, k_eff: int, info: SegInfo,
                 on_side: bool = False):
        self.inp, self.pos, self.seg_offsets, self.k_eff, self.info = inp, pos, seg_offsets, k_eff, info
        # the side stream was already ordered after these tensors' producers (by the count exchange in front)
        self.on_side = on_side

    @property
    def keepalive(self) -> torch.Tensor:
        return self.inp


class ReturnedRows:
    """Plays the part of the expert outputs (``grouped_dup_outp``) when the rows
    are already on their way into the token owners' buffers (written by the
    FFN kernel itself, or by a push on the side stream that follows the FFN
    block by block; ``event`` then marks the side stream after that push): the
    combine that follows has nothing left to send."""

    keepalive = None

    def __init__(self, info: SegInfo, event=None, beside_ffn: bool = False):
        self.info = info
        self.event = event
        self.beside_ffn = beside_ffn  # a push on the side stream is still running beside the FFN


class PeerHandle:
    """Work handle of one push: ``wait`` makes the current stream wait for this
    rank's own side-stream work on the exchange (an event) and then (bounded,
    on the device) until every source raised this exchange's flag;
    ``is_completed`` tells whether this rank's own push has left its buffers."""

    def __init__(self, info: SegInfo, which: int, event: Optional[torch.cuda.Event], ordered: bool = False):
        self.info, self.which, self.event = info, which, event
        # behind an FFN that shares the GPU with a push of the side stream the wait kernel is launched in plain
        # stream order, so that neither it nor the kernels after it become resident on the SMs left to the push
        self.ordered = ordered

    def wait(self) -> None:
        from ..ops import _stream

        x = self.info.xchg
        if self.event is not None:
            from ..ops import current_stream_object

            current_stream_object().wait_event(self.event)
        if self.which == 0 and x.region_rows:
            # region layout: the wait for the dispatched rows also derives this exchange's meta block from the
            # counts that came with them
            slot = self.info.slot
            _lib.check(x.lib.dice_ep_wait_dispatch(
                x.my_flags_ptr(slot, 1), x.ctrl.data_ptr() + slot * x.ctrl_stride * 4, x._meta_ptrs[slot], x.rank, x.world,
                x.n_experts, x.region_rows, self.info.seq, x.status.data_ptr(), _stream()), "dice_ep_wait_dispatch")
            return
        _lib.check(x.lib.dice_ep_wait_flags(x.my_flags_ptr(self.info.slot, 1 + self.which), x.world, self.info.seq,
                                            self.which + (2 if self.ordered else 0), x.status.data_ptr(), _stream()),
                   "dice_ep_wait_flags")

    def is_completed(self) -> bool:
        return self.event is None or self.event.query()
