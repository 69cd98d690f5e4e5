"""Data-parallel process group: one process per GPU, a tensor group (NCCL on CUDA, gloo on CPU) for gradients and a
gloo host group for the control plane (integer reductions, object gathers, barriers, stop flags).

Contract (reference: ced/train/data_parallel.py:125-301, 492-567): rank r reads rows r*B/W .. (r+1)*B/W - 1 of the
global batch; gradients are SUMmed (the loss is already divided by the global valid-target count); a W-rank run
equals the 1-process run on the same global batch. Environment: GHB_DP_BACKEND (force "gloo"), GHB_DP_WAIT_SECONDS
(host-group timeout, default 7200), GHB_DP_CHECK_EVERY (replica checksum period, 0 = off); the reference's CED_DP_*
spellings are honoured too.
"""

from __future__ import annotations

import datetime
import os
import zlib

import torch
import torch.distributed as dist


def _env(name: str, default: str | None = None) -> str | None:
    return os.environ.get("GHB_" + name, os.environ.get("CED_" + name, default))


class DataParallel:
    def __init__(self, rank: int, world: int, device: torch.device, tensor_group, host_group, backend: str):
        self.rank, self.world, self.device = rank, world, device
        self.tensor_group, self.host_group, self.backend = tensor_group, host_group, backend
        self.check_every = int(_env("DP_CHECK_EVERY", "0"))

    # ---- layout
    @property
    def lead(self) -> bool:
        return self.rank == 0

    def rows(self, batch_size: int) -> tuple[int, int]:
        """(first row, row count) of this rank in a global batch of batch_size rows."""
        if batch_size % self.world:
            raise ValueError(f"data.batch_size {batch_size} is not a multiple of the world size {self.world}")
        per = batch_size // self.world
        return self.rank * per, per

    def check(self, batch_size: int, micro_batch_size: int | None) -> None:
        _, per = self.rows(batch_size)
        if micro_batch_size and per % micro_batch_size:
            raise ValueError(f"micro_batch_size {micro_batch_size} does not divide a rank's {per} rows")

    # ---- host control plane (gloo)
    def sum_host(self, values: list[int]) -> list[int]:
        t = torch.tensor(values, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.host_group)
        return t.tolist()

    def max_host(self, values: list[int]) -> list[int]:
        t = torch.tensor(values, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.host_group)
        return t.tolist()

    def agree(self, *flags: bool) -> tuple[bool, ...]:
        """Every flag OR-ed over ranks: all ranks stop / checkpoint together."""
        return tuple(bool(v) for v in self.max_host([int(bool(f)) for f in flags]))

    def gather_host(self, obj) -> list:
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.host_group)
        return out

    def gather_to_lead(self, obj) -> list | None:
        out = [None] * self.world if self.lead else None
        dist.gather_object(obj, out, dst=0, group=self.host_group)
        return out

    def barrier(self) -> None:
        dist.barrier(group=self.host_group)

    # ---- tensor plane
    def all_reduce_(self, t: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        dist.all_reduce(t, op=op, group=self.tensor_group)
        return t

    def reduce_scatter_(self, out: torch.Tensor, full: torch.Tensor) -> torch.Tensor:
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=self.tensor_group)
        return out

    def all_gather_(self, full: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        dist.all_gather_into_tensor(full, shard, group=self.tensor_group)
        return full

    def max_over_ranks(self, value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.host_group)
        return float(t[0])

    def check_replicas(self, named_tensors) -> None:
        """Raises if any parameter differs between ranks: MAX and MIN of a per-tensor integer checksum must agree."""
        sums = torch.tensor([zlib.crc32(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes())
                             for _, t in named_tensors], dtype=torch.int64)
        hi, lo = sums.clone(), sums.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.host_group)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.host_group)
        bad = (hi != lo).nonzero().flatten().tolist()
        if bad:
            names = [n for n, _ in named_tensors]
            raise RuntimeError(f"data-parallel replicas diverged in {[names[i] for i in bad[:8]]}")

    def close(self) -> None:
        if dist.is_initialized():
            dist.destroy_process_group()


def rank_seed(seed: int, rank: int, step: int = 0) -> int:
    """Per-rank RNG seed re-derivable from (seed, rank, step) after a resume at another world size."""
    return (seed * 1_000_003 + rank * 7919 + step * 104_729 + 17) % (2 ** 63 - 1)


def init(rank: int, world: int, init_method: str = "env://", device: str = "auto", local_rank: int | None = None) -> DataParallel:
    use_cuda = torch.cuda.is_available() and device in ("auto", "cuda") and _env("DP_BACKEND") != "gloo"
    backend = "nccl" if use_cuda else "gloo"
    dev = torch.device("cpu")
    kwargs = {}
    if use_cuda:
        index = (rank if local_rank is None else local_rank) % torch.cuda.device_count()
        torch.cuda.set_device(index)
        dev = torch.device("cuda", index)
        kwargs["device_id"] = dev
    wait = datetime.timedelta(seconds=float(_env("DP_WAIT_SECONDS", "7200")))
    dist.init_process_group(backend, init_method=init_method, rank=rank, world_size=world, **kwargs)
    host = dist.new_group(backend="gloo", timeout=wait)
    return DataParallel(rank, world, dev, dist.group.WORLD, host, backend)


def from_environment(device: str = "auto") -> DataParallel | None:
    """The group torchrun's environment describes, or None for a single process."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None
    return init(int(os.environ["RANK"]), world, "env://", device, int(os.environ.get("LOCAL_RANK", os.environ["RANK"])))
