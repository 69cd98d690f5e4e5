"""Activation memory modes of the encoder stack.

  "none"          keep every activation
  "layer"         recompute each layer in the backward (torch checkpoint around one layer)
  "block"         recompute a whole block of layers (one checkpoint per full_attn_interval layers)
  "host"          keep activations, but park the tensors saved for the backward in pinned host memory
  "host_overlap"  the same with the copies on a side stream, overlapped with compute (at most `lead` copies in flight)

The host modes use autograd's saved-tensor hooks: packing copies a saved device tensor into a pinned buffer from a pool
keyed by (shape, dtype) and drops the device copy; unpacking copies it back when the backward needs it and returns the
buffer to the pool. On the CPU (tests) the pool works on ordinary memory and poisons a buffer when it is returned, so
a use after release shows as NaN (reference: ced/model/act_checkpoint.py:151-775, HostPool :287, lanes :655-775).
"""

from __future__ import annotations

import contextlib
from collections import defaultdict, deque

import torch
import torch.utils.checkpoint as ckpt

MODES = ("none", "layer", "block", "host", "host_overlap")
MIN_OFFLOAD_BYTES = 1 << 20


def run_checkpointed(fn, x, *extra):
    """fn(x, *extra) recomputed in the backward (non-reentrant checkpoint)."""
    return ckpt.checkpoint(fn, x, *extra, use_reentrant=False)


class _Parked:
    """A saved tensor living in a pool buffer; the buffer returns to the pool when autograd drops the handle (after the
    backward used it, or without a use when the graph is freed)."""

    __slots__ = ("pool", "buf", "event")

    def __init__(self, pool, buf, event):
        self.pool, self.buf, self.event = pool, buf, event

    def __del__(self):
        try:
            self.pool._give(self.buf)
        except Exception:       # interpreter shutdown
            pass


class HostPool:
    """Buffers for parked activations. `overlap`: copies run on a side stream (CUDA only)."""

    def __init__(self, device: torch.device, overlap: bool = False, lead: int = 2, min_bytes: int = MIN_OFFLOAD_BYTES):
        self.device, self.overlap, self.lead, self.min_bytes = device, overlap and device.type == "cuda", lead, min_bytes
        self.free = defaultdict(list)
        self.in_flight = deque()
        self.stream = torch.cuda.Stream(device) if self.overlap else None
        self.stats = {"packed": 0, "unpacked": 0, "bytes": 0, "allocated": 0, "kept": 0}

    def _take(self, shape, dtype):
        key = (tuple(shape), dtype)
        if self.free[key]:
            return self.free[key].pop()
        self.stats["allocated"] += 1
        return torch.empty(shape, dtype=dtype, device="cpu", pin_memory=self.device.type == "cuda")

    def _give(self, buf):
        if self.device.type != "cuda" and buf.is_floating_point():
            buf.fill_(float("nan"))          # poison: a reader of a released buffer sees NaN
        self.free[(tuple(buf.shape), buf.dtype)].append(buf)

    def pack(self, t: torch.Tensor):
        if not isinstance(t, torch.Tensor) or t.device != self.device or t.numel() * t.element_size() < self.min_bytes or isinstance(t, torch.nn.Parameter) \
                or not t.is_contiguous():
            self.stats["kept"] += 1
            return ("keep", t)
        buf = self._take(t.shape, t.dtype)
        event = None
        if self.overlap:
            while len(self.in_flight) >= self.lead:          # bound the copies in flight (and the device memory they pin)
                self.in_flight.popleft().synchronize()
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                buf.copy_(t, non_blocking=True)
                event = torch.cuda.Event()
                event.record(self.stream)
            t.record_stream(self.stream)
            self.in_flight.append(event)
        else:
            buf.copy_(t, non_blocking=False)
        self.stats["packed"] += 1
        self.stats["bytes"] += t.numel() * t.element_size()
        return _Parked(self, buf, event)

    def unpack(self, packed):
        if isinstance(packed, tuple):
            return packed[1]
        buf, event = packed.buf, packed.event
        if event is not None:
            event.synchronize()
        if self.overlap:
            with torch.cuda.stream(self.stream):
                out = buf.to(self.device, non_blocking=True)
                done = torch.cuda.Event()
                done.record(self.stream)
            torch.cuda.current_stream(self.device).wait_event(done)
            done.synchronize()               # the handle may be dropped (buffer reused) right after: its copy must have left
        else:
            out = buf.to(self.device).clone() if self.device.type == "cpu" else buf.to(self.device)
        self.stats["unpacked"] += 1
        return out

    def offload(self):
        """Context manager: tensors saved for the backward inside it are parked in the pool."""
        return torch.autograd.graph.saved_tensors_hooks(self.pack, self.unpack)


def layer_context(mode: str, pool: HostPool | None):
    if mode in ("host", "host_overlap") and pool is not None and torch.is_grad_enabled():
        return pool.offload()
    return contextlib.nullcontext()
