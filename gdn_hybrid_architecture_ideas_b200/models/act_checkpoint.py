"""Activation memory modes of the encoder stack.

  "none"          keep every activation
  "layer"         recompute each layer in the backward (torch checkpoint around one layer)
  "block"         recompute a whole block of layers (one checkpoint per full_attn_interval layers)
  "host"          keep activations, but park the tensors saved for the backward in pinned host memory
  "host_overlap"  the same with the copies on a side stream beside the compute

The host modes use autograd's saved-tensor hooks: packing copies a saved device tensor into a pinned buffer from a pool
keyed by (shape, dtype) and drops the device copy; unpacking copies it back when the backward needs it. The buffer
returns to the pool when autograd drops the handle.

With overlap the copies run on a LANE, a second queue beside the compute:

* forward: the copy to the host is queued behind the compute that produced the tensor and runs while later layers
  compute; the tensor is recorded on the lane so its memory is not handed out again before the copy has read it; at
  most `lead` copies are in flight (the host waits for the oldest before it queues another, else it would run ahead and
  free every saved tensor before one had been copied: no memory saved).
* backward: when a handle is asked for, the copies back of the `lead` handles packed just before it are queued too
  (the backward walks the saved tensors roughly in reverse), so they run while the current node computes; the compute
  waits on the device, not on the host, for a prefetched copy. Nothing assumes the order: a handle that was not
  prefetched copies when asked, one prefetched and never asked for frees its tensor when the handle dies (counters
  `prefetched`, `prefetch_hits`, `prefetch_unused`).

The lane is `CudaLane` (a CUDA stream and events) on a GPU and `EmuLane` elsewhere. `EmuLane` makes the ordering
mistakes of asynchronous copies visible on a CPU: a queued copy does not run until something waits for it; its
destination is filled with NaN until then (a reader that forgot its wait sees NaN, not stale-but-plausible data); a
source that was freed before the copy ran, without having been recorded on the lane, raises `LaneOrderError`; and the
NaN fill of a buffer that goes back to the pool travels through the same queue, so it cannot overtake a copy that still
reads the buffer. Reference: ced/model/act_checkpoint.py:151-775 (HostPool :287, lanes :655-775); there the kept
tensors are the layers' inputs and the layer is recomputed, here the hooks park what the layer saved and nothing is
recomputed.
"""

from __future__ import annotations

import contextlib
import weakref
from collections import defaultdict, deque

import torch
import torch.utils.checkpoint as ckpt

MODES = ("none", "layer", "block", "host", "host_overlap")
MIN_OFFLOAD_BYTES = 1 << 20


def run_checkpointed(fn, x, *extra):
    """fn(x, *extra) recomputed in the backward (non-reentrant checkpoint)."""
    return ckpt.checkpoint(fn, x, *extra, use_reentrant=False)


class LaneOrderError(RuntimeError):
    """A copy on the emulated lane found its source gone: it was freed before the copy ran and never recorded."""


def _poison(t: torch.Tensor) -> None:
    if t.is_floating_point() or t.is_complex():
        t.fill_(float("nan"))
    elif t.dtype == torch.bool:
        t.fill_(True)
    else:
        t.fill_(torch.iinfo(t.dtype).min)


# ---------------------------------------------------------------------------------------------------------------- lanes

class CudaLane:
    """A side stream. A ticket is the event recorded behind a queued copy."""

    def __init__(self, device: torch.device):
        self.device, self.stream = device, torch.cuda.Stream(device)

    def side_waits_compute(self) -> None:
        self.stream.wait_stream(torch.cuda.current_stream(self.device))

    def copy(self, dst: torch.Tensor, src: torch.Tensor):
        with torch.cuda.stream(self.stream):
            dst.copy_(src, non_blocking=True)
            ticket = torch.cuda.Event()
            ticket.record(self.stream)
        return ticket

    def record(self, t: torch.Tensor) -> None:
        if t.is_cuda:
            t.record_stream(self.stream)

    def fill(self, buf: torch.Tensor) -> None:       # pinned buffers are not poisoned on a GPU run (a full host write per use)
        pass

    def compute_waits(self, ticket) -> None:
        torch.cuda.current_stream(self.device).wait_event(ticket)

    def host_waits(self, ticket) -> None:
        ticket.synchronize()

    def drain(self) -> None:
        self.stream.synchronize()


class EmuLane:
    """The side stream of a machine without one: a queue of copies that run only when waited for, in queue order."""

    def __init__(self, device: torch.device | None = None):
        self.device = device
        self.queue: deque = deque()
        self.issued = 0
        self.done = 0
        self.ran_out_of_order = 0

    def side_waits_compute(self) -> None:            # the compute of a CPU run has finished by the time the host gets here
        pass

    def copy(self, dst: torch.Tensor, src: torch.Tensor) -> int:
        _poison(dst)                                   # what a reader sees that does not wait
        self.issued += 1
        self.queue.append(["copy", dst, weakref.ref(src), None, self.issued])
        return self.issued

    def record(self, t: torch.Tensor) -> None:
        """Keep `t` alive for every queued copy that reads it (record_stream's promise)."""
        for op in self.queue:
            if op[0] == "copy" and op[2]() is t:
                op[3] = t

    def fill(self, buf: torch.Tensor) -> None:
        self.issued += 1
        self.queue.append(["fill", buf, None, None, self.issued])

    def _run_through(self, ticket: int) -> None:
        while self.queue and self.queue[0][4] <= ticket:
            kind, dst, src_ref, held, number = self.queue.popleft()
            if kind == "fill":
                _poison(dst)
            else:
                src = held if held is not None else src_ref()
                if src is None:
                    raise LaneOrderError(f"copy {number}: its source was freed before the copy ran and was not recorded on the lane")
                dst.copy_(src)
            self.done = number

    def compute_waits(self, ticket: int) -> None:
        self._run_through(ticket)

    def host_waits(self, ticket: int) -> None:
        self._run_through(ticket)

    def drain(self) -> None:
        self._run_through(self.issued)


# ----------------------------------------------------------------------------------------------------------------- pool

class _Parked:
    """A saved tensor living in a pool buffer; the buffer returns to the pool when autograd drops the handle (after the
    backward used it, or without a use when the graph is freed)."""

    __slots__ = ("pool", "buf", "stored", "index", "back", "back_ticket", "__weakref__")

    def __init__(self, pool, buf, stored, index):
        self.pool, self.buf, self.stored, self.index = pool, buf, stored, index
        self.back, self.back_ticket = None, None

    def __del__(self):
        try:
            self.pool._dropped(self)
        except Exception:       # interpreter shutdown
            pass


class HostPool:
    """Buffers for parked activations.

    overlap   copies on a lane beside the compute (CudaLane on a GPU, EmuLane elsewhere)
    lead      copies to the host in flight at once, and handles prefetched ahead in the backward
    poison    a buffer is filled with NaN when it returns to the pool (default: on for CPU tensors)
    """

    def __init__(self, device: torch.device, overlap: bool = False, lead: int = 2, min_bytes: int = MIN_OFFLOAD_BYTES,
                 poison: bool | None = None, lane=None):
        self.device, self.overlap, self.lead, self.min_bytes = device, bool(overlap), max(1, lead), min_bytes
        self.poison = device.type != "cuda" if poison is None else poison
        self.lane = lane if lane is not None else ((CudaLane(device) if device.type == "cuda" else EmuLane(device)) if overlap else None)
        self.free = defaultdict(list)
        self.in_flight: deque = deque()
        self.live: dict[int, weakref.ref] = {}
        self.count = 0
        self.stats = {"packed": 0, "unpacked": 0, "bytes": 0, "allocated": 0, "kept": 0,
                      "prefetched": 0, "prefetch_hits": 0, "prefetch_unused": 0}

    # -- buffers
    def _take(self, shape, dtype):
        key = (tuple(shape), dtype)
        if self.free[key]:
            return self.free[key].pop()
        self.stats["allocated"] += 1
        return torch.empty(shape, dtype=dtype, device="cpu", pin_memory=self.device.type == "cuda")

    def _give(self, buf):
        if self.poison:
            if self.lane is not None:
                self.lane.fill(buf)      # behind every copy that still reads the buffer
            else:
                _poison(buf)
        self.free[(tuple(buf.shape), buf.dtype)].append(buf)

    def _dropped(self, h: _Parked) -> None:
        self.live.pop(h.index, None)
        if h.back is not None:
            self.stats["prefetch_unused"] += 1
            h.back = None
        self._give(h.buf)

    # -- the hooks
    def pack(self, t: torch.Tensor):
        # Kept as they are: small tensors, parameters, and views into a larger storage (a slice of a flat weight buffer, a
        # column range of an activation): the storage outlives the view, so parking it frees nothing, and code that saved
        # two neighbouring views to address them as one block must get those very views back.
        if not isinstance(t, torch.Tensor) or t.device != self.device or t.numel() * t.element_size() < self.min_bytes or isinstance(t, torch.nn.Parameter) \
                or not t.is_contiguous() or t.untyped_storage().nbytes() != t.numel() * t.element_size():
            self.stats["kept"] += 1
            return ("keep", t)
        buf = self._take(t.shape, t.dtype)
        stored = None
        if self.overlap:
            while len(self.in_flight) >= self.lead:          # bound the copies in flight (and the device memory they pin)
                self.lane.host_waits(self.in_flight.popleft())
            self.lane.side_waits_compute()
            stored = self.lane.copy(buf, t)
            self.lane.record(t)
            self.in_flight.append(stored)
        else:
            buf.copy_(t, non_blocking=False)
        self.stats["packed"] += 1
        self.stats["bytes"] += t.numel() * t.element_size()
        self.count += 1
        h = _Parked(self, buf, stored, self.count)
        self.live[h.index] = weakref.ref(h)
        return h

    def _start_back(self, h: _Parked) -> None:
        """Queue the copy back of `h` on the lane into a new device tensor (made on the compute stream, so the lane first
        waits for the compute to reach this point: whatever used that memory before has finished)."""
        out = torch.empty(h.buf.shape, dtype=h.buf.dtype, device=self.device)
        self.lane.side_waits_compute()
        h.back_ticket = self.lane.copy(out, h.buf)
        self.lane.record(out)
        h.back = out

    def unpack(self, packed):
        if isinstance(packed, tuple):
            return packed[1]
        h = packed
        if not self.overlap:
            out = h.buf.to(self.device).clone() if self.device.type == "cpu" else h.buf.to(self.device)
            self.stats["unpacked"] += 1
            return out
        if h.back is None:
            self._start_back(h)
        else:
            self.stats["prefetch_hits"] += 1
        for j in range(h.index - 1, h.index - 1 - self.lead, -1):     # the ones the backward is likely to ask for next
            ref = self.live.get(j)
            g = ref() if ref is not None else None
            if g is not None and g.back is None:
                self._start_back(g)
                self.stats["prefetched"] += 1
        self.lane.compute_waits(h.back_ticket)       # the device waits; the host goes on
        out, h.back, h.back_ticket = h.back, None, None
        self.stats["unpacked"] += 1
        return out

    def offload(self):
        """Context manager: tensors saved for the backward inside it are parked in the pool."""
        return torch.autograd.graph.saved_tensors_hooks(self.pack, self.unpack)

    def drain(self) -> None:
        """Every queued copy has run (end of a step; tests)."""
        if self.lane is not None:
            self.lane.drain()
        self.in_flight.clear()


def layer_context(mode: str, pool: HostPool | None):
    if mode in ("host", "host_overlap") and pool is not None and torch.is_grad_enabled():
        return pool.offload()
    return contextlib.nullcontext()
