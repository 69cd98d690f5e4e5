"""ZeRO optimizer-state (stage 1) and gradient (stage 2) sharding over the data-parallel group.

AdamW: the flat buffers are cut into W equal element ranges; rank r keeps moments for range r only, receives the sum
of everybody's gradients for it (reduce-scatter), updates its range of the master weights and the ranks all-gather
the updated weights. Stage 2 differs in when gradients leave: bucket by bucket during backward instead of once at the
end, so only a shard-sized reduced gradient has to persist (new relative to the reference, which stops at stage 1).
Muon needs whole matrices, so its matrices are owned by whole tensor, assigned greedily by size; that is the
reference's ZeRO-1 (ced/train/zero1.py:93-151, 250-264), while the AdamW remainder is range-sharded.

The global gradient norm for clipping is assembled from per-shard sums of squares with one small all-reduce
(zero1.py:293-337). Optimizer state is saved per rank beside the checkpoint and re-sharded by parameter name on load,
so the world size may change across a resume (zero1.py:428-566).
"""

from __future__ import annotations

import torch

from ..train.optim import FlatAdamW, FlatBuffers, param_groups


def assign_owners(sizes: dict[str, int], world: int) -> dict[str, int]:
    """Greedy largest-first assignment of whole tensors to the least-loaded rank."""
    load = [0] * world
    owner = {}
    for name, n in sorted(sizes.items(), key=lambda kv: (-kv[1], kv[0])):
        r = min(range(world), key=lambda i: (load[i], i))
        owner[name] = r
        load[r] += n
    return owner


class ZeroPlan:
    def __init__(self, model, o, dp, stage: str):
        self.model, self.o, self.dp, self.stage = model, o, dp, stage
        self.world, self.rank = dp.world, dp.rank
        self.fused = None

    def build(self, device, lp_dtype):
        groups = param_groups(self.model, self.o)
        self.flat = FlatBuffers(self.model, groups, device, lp_dtype)
        n = self.flat.size
        per = -(-n // (self.world * 1024)) * 1024
        if per * self.world != n:   # grow the buffers so they cut into W equal, 1024-aligned ranges
            self._regrow(per * self.world, device, lp_dtype)
        self.per = per
        self.lo, self.hi = self.rank * per, (self.rank + 1) * per
        if self.o.name == "muon":
            from ..train.muon import MuonWithAdamW

            mats = {s.name: s.numel for s in self.flat.segments if groups[s.group]["kind"] == "muon"}
            self.owner = assign_owners(mats, self.world)
            mine = {n for n, r in self.owner.items() if r == self.rank}
            opt = MuonWithAdamW(self.flat, groups, self.o, (self.lo, self.hi), owned_names=mine)
        else:
            self.owner = {}
            opt = FlatAdamW(self.flat, groups, self.o.betas, self.o.eps, (self.lo, self.hi))
        return self.flat, opt

    def _regrow(self, size: int, device, lp_dtype) -> None:
        f = self.flat
        new = {}
        for name in ("params", "grads", "lp"):
            old = getattr(f, name)
            if old is None:
                new[name] = None
                continue
            new[name] = torch.zeros(size, dtype=old.dtype, device=device)
            new[name][:old.numel()].copy_(old)
        f.rebind(self.model, new["params"], new["grads"], new["lp"])

    def enable_fused(self) -> bool:
        """Switch the step to the peer-memory kernels when symmetric memory is available (CUDA, AdamW, world <= 8)."""
        import os

        from . import fused_comm

        want = os.environ.get("GHB_COMM", "auto")
        if want == "nccl" or self.o.name != "adamw" or not fused_comm.available(self.dp):
            return False
        try:
            self.fused = fused_comm.FusedComm(self.dp, self.flat, self.model, lambda p, g, lp: self.flat.rebind(self.model, p, g, lp))
        except Exception as e:   # no symmetric memory on this system
            # GHB_COMM=nccl is the way to ask for the collective path; falling back silently would let a benchmark
            # report the NCCL step under the fused step's name
            raise RuntimeError(f"the fused peer-memory data-parallel step could not be set up ({type(e).__name__}: {e}); "
                               "set GHB_COMM=nccl to run the NCCL reduce-scatter / all-gather path instead") from e
        return self.fused is not None

    # ------------------------------------------------------------------ the step

    @torch.no_grad()
    def sync_and_step(self, opt, lr: float, max_norm: float, stats: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter gradients, clip by the global norm, update the owned range, all-gather the weights.
        stats: small float64 vector summed over ranks on the way. Returns the global gradient norm."""
        f, dp = self.flat, self.dp
        if getattr(self, "fused", None) is not None:
            dp.all_reduce_(stats)
            return self.fused.step(opt, lr, max_norm)
        shard = f.grads[self.lo:self.hi]
        if self.o.name == "muon":
            dp.all_reduce_(f.grads)      # whole matrices are needed by their owners
        else:
            dp.reduce_scatter_(shard, f.grads)
        sq = shard.double().pow(2).sum() if not shard.is_cuda else _sumsq(shard).double()
        packed = torch.cat([stats, sq.reshape(1)])
        dp.all_reduce_(packed)
        stats.copy_(packed[:-1])
        gnorm = packed[-1].sqrt().float()
        scale = 1.0 if not max_norm or max_norm <= 0 else torch.clamp(max_norm / (gnorm + 1e-6), max=1.0)
        opt.step(lr, scale)
        if self.o.name == "muon":
            self._broadcast_matrices()
        dp.all_gather_(f.params, f.params[self.lo:self.hi].clone())
        f.refresh_lp()
        return gnorm

    def _broadcast_matrices(self) -> None:
        """Muon matrices were updated by their owners outside the range sharding: place each owner's result into the
        range owner's slice so the all-gather distributes it."""
        import torch.distributed as dist

        for name, r in self.owner.items():
            t = self.flat.view(self.flat.params, name)
            dist.broadcast(t, src=r, group=self.dp.tensor_group)

    def gather_master(self) -> None:
        """Master weights are complete on every rank after each step; nothing to do (kept as the hook a
        master-sharded variant needs before a checkpoint)."""

    # ------------------------------------------------------------------ optimizer state I/O

    def optimizer_state(self, opt) -> dict:
        """Full optimizer state assembled on every rank (moments all-gathered), in FlatAdamW.state_dict form."""
        f = self.flat
        full_m = torch.empty(f.size, dtype=torch.float32, device=f.params.device)
        full_v = torch.empty_like(full_m)
        self.dp.all_gather_(full_m, opt.exp_avg)
        self.dp.all_gather_(full_v, opt.exp_avg_sq)
        whole = FlatAdamW.__new__(FlatAdamW)
        whole.flat, whole.groups, whole.betas, whole.eps = f, opt.groups, opt.betas, opt.eps
        whole.lo, whole.hi, whole.exp_avg, whole.exp_avg_sq, whole.steps = 0, f.size, full_m, full_v, opt.steps
        whole.param_groups = opt.param_groups
        sd = FlatAdamW.state_dict(whole)
        if hasattr(opt, "buf"):
            gathered = self.dp.gather_host({n: b.cpu() for n, b in opt.buf.items()})
            sd["muon"] = {n: b for part in gathered for n, b in part.items()}
        return sd

    def load_optimizer_state(self, opt, sd: dict) -> None:
        """Any world size: every rank reads the by-name state and keeps what falls in its range / ownership."""
        f = self.flat
        names = sd.get("names") or [s.name for s in f.segments]
        for index, name in enumerate(names):
            st, s = sd["state"].get(index), f.by_name.get(name)
            if st is None or s is None:
                continue
            a, b = max(s.offset, self.lo), min(s.offset + s.numel, self.hi)
            if b > a:
                opt.exp_avg[a - self.lo:b - self.lo].copy_(st["exp_avg"].reshape(-1)[a - s.offset:b - s.offset])
                opt.exp_avg_sq[a - self.lo:b - self.lo].copy_(st["exp_avg_sq"].reshape(-1)[a - s.offset:b - s.offset])
            opt.steps = int(st["step"])
        for n, b in (sd.get("muon") or {}).items():
            if hasattr(opt, "buf") and n in opt.buf:
                opt.buf[n].copy_(b)


def _sumsq(t: torch.Tensor) -> torch.Tensor:
    from ..ops import native

    return native.sumsq(t)
