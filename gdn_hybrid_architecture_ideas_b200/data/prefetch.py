"""Background construction and staging of the next step's batch.

A worker thread builds step N+1's batch on the host while step N runs; on CUDA the batch is then copied from pinned
memory on a side stream and an event orders the training stream after the copy. Reading a staged batch before its
wait is a `PrefetchRace` (reference: ced/train/prefetch.py:49-278)."""

from __future__ import annotations

import threading
import time

import torch


class PrefetchRace(RuntimeError):
    pass


class Staged:
    def __init__(self, batch, event=None):
        self._batch, self._event, self._waited = batch, event, event is None

    def wait(self, stream=None):
        if self._event is not None:
            (stream or torch.cuda.current_stream()).wait_event(self._event)
        self._waited = True
        return self

    @property
    def batch(self):
        if not self._waited:
            raise PrefetchRace("staged batch read before wait()")
        return self._batch


class CudaStage:
    def __init__(self, device):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)

    def stage(self, batch) -> Staged:
        batch = batch.pin()
        with torch.cuda.stream(self.stream):
            dev = batch.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        staged = Staged(dev, ev)
        staged._host = batch  # keep the pinned source alive until the copy has run
        return staged


class EmulatedStage:
    """CPU stand-in with the same ordering contract (tests)."""

    def stage(self, batch) -> Staged:
        s = Staged(batch, None)
        s._waited = False
        s._event = None
        return s


class BatchPrefetcher:
    def __init__(self, build, stage=None):
        """build(step) -> Batch on the host; stage: CudaStage / EmulatedStage / None."""
        self.build, self.stage = build, stage
        self._thread, self._result, self._step = None, None, None
        self.stats = {"build_ms": 0.0, "wait_ms": 0.0}

    def _work(self, step):
        t0 = time.perf_counter()
        try:
            self._result = ("ok", self.build(step))
        except BaseException as e:  # delivered to the training thread by get()
            self._result = ("err", e)
        self.stats["build_ms"] = (time.perf_counter() - t0) * 1e3

    def start(self, step: int) -> None:
        self._step = step
        self._thread = threading.Thread(target=self._work, args=(step,), daemon=True)
        self._thread.start()

    def get(self, step: int):
        if self._thread is None or self._step != step:
            self.start(step)
        t0 = time.perf_counter()
        self._thread.join()
        self.stats["wait_ms"] = (time.perf_counter() - t0) * 1e3
        kind, value = self._result
        self._thread = None
        if kind == "err":
            raise value
        staged = self.stage.stage(value) if self.stage is not None else Staged(value)
        return staged.wait() if not isinstance(self.stage, EmulatedStage) else staged
