"""Checkpoint files: one `torch.save` dict per step under `<run>/checkpoints/step_%08d.pt`, written to a `.tmp`
name and renamed, then an atomically replaced text pointer `latest`; a rolling window of `ckpt_keep` files plus the
pinned `checkpoint_steps` stay on disk (reference: ced/train/trainer.py:3945-4011).

Dict keys (same as the reference's, so files are interchangeable): step, config, model, optimizer, torch_rng,
cuda_rng, python_rng, wandb_run_id, data_state, init_from, resumed_from, and data_parallel under DP.

`AsyncSaver` snapshots the state into one pinned host arena with non-blocking copies and one event, and a background
thread (which makes no CUDA call) serialises it; the file is byte-identical to a synchronous save
(reference: ced/train/async_save.py:66-379).
"""

from __future__ import annotations

import os
import threading
from pathlib import Path

import torch


def step_path(run_dir: Path, step: int) -> Path:
    return Path(run_dir) / "checkpoints" / f"step_{step:08d}.pt"


def latest_path(run_dir: Path) -> Path | None:
    pointer = Path(run_dir) / "checkpoints" / "latest"
    if not pointer.exists():
        return None
    p = Path(run_dir) / "checkpoints" / pointer.read_text().strip()
    return p if p.exists() else None


def write_atomic(state: dict, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(state, tmp)
    os.replace(tmp, path)


def point_latest(path: Path, keep: int, pinned_steps=()) -> None:
    folder = path.parent
    tmp = folder / "latest.tmp"
    tmp.write_text(path.name)
    os.replace(tmp, folder / "latest")
    pinned = {f"step_{int(s):08d}.pt" for s in pinned_steps}
    files = sorted(f for f in folder.glob("step_*.pt"))
    rolling = [f for f in files if f.name not in pinned]
    for old in rolling[:-keep] if keep > 0 else []:
        if old != path:
            old.unlink(missing_ok=True)
            shard_dir = old.with_suffix(".optim")
            if shard_dir.is_dir():
                for f in shard_dir.iterdir():
                    f.unlink()
                shard_dir.rmdir()


def load(path: Path, map_location="cpu") -> dict:
    return torch.load(path, map_location=map_location, weights_only=False)


def load_model(path, device="cpu", dtype=None):
    """(model, train config, step) from a checkpoint file or a run directory (its latest checkpoint): the model is built
    from the checkpoint's own config and takes its weights (evaluation scripts start here)."""
    from .. import config as C
    from ..models import build_model

    p = Path(path)
    if p.is_dir():
        p = latest_path(p)
        if p is None:
            raise FileNotFoundError(f"no checkpoint under {path}")
    state = load(p)
    cfg = C.from_dict(C.TrainConfig, C.checkpoint_config(state["config"]))
    model = build_model(cfg.model)
    model.load_state_dict(state["model"])
    model = model.to(device)
    if dtype is not None:
        model = model.to(dtype)
    return model.eval(), cfg, int(state["step"])


def _tensors(obj, out: list, prefix=()):
    if isinstance(obj, torch.Tensor):
        out.append((prefix, obj))
    elif isinstance(obj, dict):
        for k, v in obj.items():
            _tensors(v, out, prefix + (k,))
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            _tensors(v, out, prefix + (i,))


def _replace(obj, mapping, prefix=()):
    if isinstance(obj, torch.Tensor):
        return mapping[prefix]
    if isinstance(obj, dict):
        return {k: _replace(v, mapping, prefix + (k,)) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_replace(v, mapping, prefix + (i,)) for i, v in enumerate(obj)]
    if isinstance(obj, tuple):
        return tuple(_replace(v, mapping, prefix + (i,)) for i, v in enumerate(obj))
    return obj


class Arena:
    """One pinned host allocation that holds a snapshot of every tensor of a state dict."""

    def __init__(self):
        self.buf: torch.Tensor | None = None

    def snapshot(self, state: dict):
        """Start non-blocking device->host copies of every tensor; returns (host state, event or None)."""
        found: list = []
        _tensors(state, found)
        total = sum(-(-t.numel() * t.element_size() // 64) * 64 for _, t in found)
        if self.buf is None or self.buf.numel() < total:
            self.buf = torch.empty(total, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        mapping, at, any_cuda = {}, 0, False
        for key, t in found:
            nbytes = t.numel() * t.element_size()
            host = self.buf[at:at + nbytes].view(t.dtype).view(t.shape)
            host.copy_(t.detach(), non_blocking=True)
            any_cuda |= t.is_cuda
            mapping[key] = host
            at += -(-nbytes // 64) * 64
        event = None
        if any_cuda:
            event = torch.cuda.Event()
            event.record()
        return _replace(state, mapping), event


class AsyncSaver:
    """At most one write in flight; `commit()` at a later step boundary publishes it (latest pointer, pruning)."""

    def __init__(self):
        self.arena = Arena()
        self._thread: threading.Thread | None = None
        self._pending: tuple | None = None
        self.error: BaseException | None = None

    def busy(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def start(self, state: dict, path: Path, keep: int, pinned) -> None:
        self.wait()
        host_state, event = self.arena.snapshot(state)

        def work():
            try:
                if event is not None:
                    event.synchronize()
                # torch.save refuses differently-typed views of one storage: give every tensor its own (host-side copy,
                # made on this thread; the training thread only paid for the non-blocking device->arena copies)
                found: list = []
                _tensors(host_state, found)
                write_atomic(_replace(host_state, {k: t.clone() for k, t in found}), path)
            except BaseException as e:
                self.error = e

        self._pending = (path, keep, pinned)
        self._thread = threading.Thread(target=work, daemon=True)
        self._thread.start()

    def commit(self, block: bool = False) -> Path | None:
        """Publish a finished write; returns its path, or None if nothing finished (block: wait for it)."""
        if self._pending is None or (self.busy() and not block):
            return None
        self.wait()
        path, keep, pinned = self._pending
        self._pending = None
        if self.error is not None:
            err, self.error = self.error, None
            raise RuntimeError(f"asynchronous checkpoint write of {path} failed") from err
        point_latest(path, keep, pinned)
        return path

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
