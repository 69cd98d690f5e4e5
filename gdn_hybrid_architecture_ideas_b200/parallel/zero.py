"""ZeRO sharding of the optimizer state and of the reduced gradients over the data-parallel group.

The flat buffers are cut into buckets; every bucket is cut into W slices and rank r owns slice r of every bucket: it
receives the sum of everybody's gradients for its slices (reduce-scatter), keeps AdamW moments for them only, updates
them and the ranks all-gather the updated weights.

* `zero1`: one bucket (the whole buffer), reduced after the backward (the reference's stage: ced/train/zero1.py:93-151,
  250-264).
* `zero2`: buckets follow the order in which the backward finishes gradients — the matrices of the last block of layers
  first, the first block's last, then everything else (embedding, norm gains, gates, depth-mix queries: tensors whose
  gradients meet contributions until the end) — and each bucket is reduced as soon as it is final, while the backward of
  earlier layers still runs. After a bucket's reduction only the owner's reduced slice is read again; the full-size
  buffer stays allocated as the workspace the next backward accumulates into (weight-gradient GEMMs add into it in
  place), so what this stage changes is when gradients leave, not the buffer's size. New relative to the reference,
  which stops at stage 1. Muon needs whole matrices, so with Muon both names run the one-bucket form with matrices
  owned by whole tensor, assigned greedily by size, and the AdamW remainder range-sharded.

On CUDA the step runs in the peer-memory kernels (parallel/fused_comm.py); with GHB_COMM=nccl, and on the CPU, as
collectives. The global gradient norm for clipping is assembled from per-shard sums of squares (zero1.py:293-337).
Optimizer state is gathered into the full by-name form for a checkpoint and re-sharded by name on load, so the world
size and the layout may change across a resume (zero1.py:428-566).
"""

from __future__ import annotations

import re

import torch

from ..train.optim import FlatAdamW, FlatBuffers, param_groups

LAST = 1 << 20      # readiness stage of tensors whose gradients are final only when the backward ends
_LAYER = re.compile(r"(?:^|\.)encoder\.layers\.(\d+)\.")


def assign_owners(sizes: dict[str, int], world: int) -> dict[str, int]:
    """Greedy largest-first assignment of whole tensors to the least-loaded rank."""
    load = [0] * world
    owner = {}
    for name, n in sorted(sizes.items(), key=lambda kv: (-kv[1], kv[0])):
        r = min(range(world), key=lambda i: (load[i], i))
        owner[name] = r
        load[r] += n
    return owner


def readiness_stages(model) -> dict[str, int]:
    """Parameter name -> stage of the backward at which its gradient is final. The projection matrices of the layers of
    block b (blocks of `full_attn_interval` layers) are written only by their own layers' backward nodes, which have all
    run once the gradient of the block's input is complete: stage n_blocks - 1 - b, so stage 0 finishes first. Everything
    else (embeddings, norm gains, conv taps, gates, depth-mix readers, which receive gradient from nodes that run after
    the block's input gradient or from several places) is LAST."""
    from ..models.linear import Linear

    enc = getattr(model, "encoder", None)
    block = getattr(enc, "block", 0)
    out = {n: LAST for n, _ in model.named_parameters()}
    if enc is None or block <= 0 or len(enc.layers) % block:
        return out
    n_blocks = len(enc.layers) // block
    mods = dict(model.named_modules())
    for name in out:
        owner, _, leaf = name.rpartition(".")
        m = _LAYER.search(name)
        if m and leaf == "weight" and isinstance(mods.get(owner), Linear):
            out[name] = n_blocks - 1 - int(m.group(1)) // block
    return out


class ZeroPlan:
    def __init__(self, model, o, dp, stage: str):
        self.model, self.o, self.dp, self.stage = model, o, dp, stage
        self.world, self.rank = dp.world, dp.rank
        self.fused = None
        self.bucketed = stage == "zero2" and o.name == "adamw"
        self.armed = False          # the running backward is the step's last: its finished buckets may leave
        self._reduced = set()
        self.early = 0              # buckets reduced from inside a backward so far (monitoring)

    def build(self, device, lp_dtype):
        groups = param_groups(self.model, self.o)
        stages = readiness_stages(self.model) if self.bucketed else {}
        self.flat = FlatBuffers(self.model, groups, device, lp_dtype, order=(lambda n: stages[n]) if self.bucketed else None)
        n = self.flat.size
        per = -(-n // (self.world * 1024)) * 1024
        if per * self.world != n:   # grow the buffers so they cut into W equal, 1024-aligned ranges
            self._regrow(per * self.world, device, lp_dtype)
        self._cut(stages)
        if self.o.name == "muon":
            from ..train.muon import MuonWithAdamW

            mats = {s.name: s.numel for s in self.flat.segments if groups[s.group]["kind"] == "muon"}
            self.owner = assign_owners(mats, self.world)
            mine = {n for n, r in self.owner.items() if r == self.rank}
            opt = MuonWithAdamW(self.flat, groups, self.o, (self.lo, self.hi), owned_names=mine)
        else:
            self.owner = {}
            opt = FlatAdamW(self.flat, groups, self.o.betas, self.o.eps, [(lo, hi) for lo, hi, _ in self.slices if hi > lo] or [(0, 0)])
        if self.bucketed and getattr(self.model, "encoder", None) is not None:
            self.model.encoder.stage_hooks = self
        return self.flat, opt

    def _cut(self, stages: dict) -> None:
        """Buckets (maximal runs of tensors of one readiness stage, in buffer order), this rank's slice of each, and the
        order in which the forward first reads them."""
        f, W = self.flat, self.world
        runs = []                # [lo, hi, stage]
        for s in f.segments:
            st = stages.get(s.name, LAST)
            if runs and runs[-1][2] == st:
                runs[-1][1] = s.offset + s.numel
            else:
                if runs:
                    runs[-1][1] = s.offset
                runs.append([s.offset, s.offset + s.numel, st])
        if not self.bucketed or not runs:
            runs = [[0, f.size, LAST]]
        runs[-1][1] = f.size
        self.buckets = [(lo, hi) for lo, hi, _ in runs]
        self.bucket_stage = [st for _, _, st in runs]
        self.slices, at = [], 0           # (lo, hi, offset in the shard / moment buffers)
        for lo, hi in self.buckets:
            per = -(-(hi - lo) // (W * 1024)) * 1024
            a, b = min(lo + self.rank * per, hi), min(lo + (self.rank + 1) * per, hi)
            self.slices.append((a, b, at))
            at += b - a
        self.owned = at
        self.per = f.size // W
        self.lo, self.hi = (self.slices[0][0], self.slices[0][1]) if len(self.slices) == 1 else (0, 0)
        n_stage = max([st for st in self.bucket_stage if st != LAST], default=-1) + 1
        # the forward reads LAST tensors first (embedding, gains), then block 0's matrices (the highest stage), and so on
        self.update_order = sorted(range(len(self.buckets)), key=lambda i: (-1 if self.bucket_stage[i] == LAST else n_stage - 1 - self.bucket_stage[i], i))

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

    def _fp32_cells(self) -> torch.Tensor | None:
        """One flag per 64 elements: True where every rank needs the fp32 value after an update. A layer matrix with a
        bf16 compute copy is read in fp32 by its owner's optimizer only."""
        from ..models.linear import Linear

        f = self.flat
        if f.lp is None:
            return None
        cells = torch.ones(f.size // 64, dtype=torch.bool)
        mods = dict(self.model.named_modules())
        for s in f.segments:
            owner, _, leaf = s.name.rpartition(".")
            # a low-precision linear quantises its operands from the fp32 master on every rank: it stays complete everywhere
            if leaf == "weight" and isinstance(mods.get(owner), Linear) and _LAYER.search(s.name) and getattr(mods[owner], "weight_lp", None) is not None \
                    and getattr(mods[owner], "precision", "bf16") == "bf16":
                cells[s.offset // 64:(s.offset + s.numel + 63) // 64] = False
        return cells

    def enable_fused(self) -> bool:
        """Switch the step to the peer-memory kernels (CUDA, AdamW, world <= 8) unless GHB_COMM=nccl asks for collectives."""
        import os

        from . import fused_comm

        want = os.environ.get("GHB_COMM", "auto")
        if want == "nccl" or self.o.name != "adamw" or not fused_comm.available(self.dp):
            return False
        try:
            self.fused = fused_comm.FusedComm(self.dp, self.flat, self.model, lambda p, g, lp: self.flat.rebind(self.model, p, g, lp),
                                              self.buckets, self.slices, self.update_order,
                                              self._fp32_cells() if os.environ.get("GHB_COMM_FP32_EVERYWHERE", "0") != "1" else None)
        except Exception as e:   # no symmetric memory on this system
            # GHB_COMM=nccl is the way to ask for the collective path; falling back silently would let a benchmark
            # report the NCCL step under the fused step's name
            raise RuntimeError(f"the fused peer-memory data-parallel step could not be set up ({type(e).__name__}: {e}); "
                               "set GHB_COMM=nccl to run the NCCL reduce-scatter / all-gather path instead") from e
        return True

    # ------------------------------------------------------------------ hooks of the model (models/encoder.py `stage_hooks`)

    def forward_enter(self, block: int) -> None:
        """The forward is about to read block `block`'s matrices: order it after their all-gather."""
        if self.fused is None:
            return
        stage = self._n_stages() - 1 - block
        for i, st in enumerate(self.bucket_stage):
            if st == stage:
                self.fused.wait_bucket(i)

    def backward_done(self, block: int) -> None:
        """The gradient of block `block`'s input is complete: its matrices' gradients are final."""
        if not self.armed:
            return
        stage = self._n_stages() - 1 - block
        for i, st in enumerate(self.bucket_stage):
            if st == stage and i not in self._reduced:
                self.early += 1
                self._reduce(i, last=False)

    def _n_stages(self) -> int:
        return max([st for st in self.bucket_stage if st != LAST], default=-1) + 1

    def before_step(self) -> None:
        """Start of a step on the compute stream: parameters read first (embedding, gains) have landed, and every peer
        has finished reading this rank's gradients of the step before, so they may be zeroed."""
        if self.fused is not None:
            for i, st in enumerate(self.bucket_stage):
                if st == LAST or getattr(getattr(self.model, "encoder", None), "stage_hooks", None) is not self:
                    self.fused.wait_bucket(i)

    def settle(self) -> None:
        """Every parameter is complete on the current stream (before anything that reads parameters outside a training forward)."""
        if self.fused is not None:
            self.fused.wait_all()

    # ------------------------------------------------------------------ the step

    def _reduce(self, i: int, last: bool) -> None:
        if i in self._reduced:
            return
        self._reduced.add(i)
        if self.fused is not None:
            self.fused.reduce_bucket(i, last)
            return
        f, dp = self.flat, self.dp
        lo, hi = self.buckets[i]
        if len(self.buckets) == 1 and self.o.name != "muon" and (hi - lo) % self.world == 0:
            a, b, _ = self.slices[i]
            dp.reduce_scatter_(f.grads[a:b], f.grads[lo:hi])
        else:       # uneven slices (or whole matrices needed): sum the bucket everywhere, the owner reads its slice
            dp.all_reduce_(f.grads[lo:hi])

    @torch.no_grad()
    def sync_and_step(self, opt, lr: float, max_norm: float, stats: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter what the backward has not sent yet, clip by the global norm, update the owned slices,
        all-gather the weights. stats: small float64 vector summed over ranks on the way. Returns the global norm."""
        f, dp = self.flat, self.dp
        pending = [i for i in range(len(self.buckets)) if i not in self._reduced]
        for k, i in enumerate(pending):
            self._reduce(i, last=k == len(pending) - 1)
        self._reduced.clear()
        self.armed = False
        if self.fused is not None:
            dp.all_reduce_(stats)
            gnorm = self.fused.update(opt, lr, max_norm)
            self.fused.wait_bucket(self.update_order[0])      # the norm (and the tensors the next forward reads first) are there
            return gnorm
        own = [(a, b) for a, b, _ in self.slices if b > a]
        sq = sum((_sumsq(f.grads[a:b]).double() if f.grads.is_cuda else f.grads[a:b].double().pow(2).sum()) for a, b in own) \
            if own else torch.zeros((), dtype=torch.float64, device=f.grads.device)
        packed = torch.cat([stats, sq.reshape(1)])
        dp.all_reduce_(packed)
        stats.copy_(packed[:-1])
        gnorm = packed[-1].sqrt().float()
        scale = 1.0 if not max_norm or max_norm <= 0 else torch.clamp(max_norm / (gnorm + 1e-6), max=1.0)
        opt.step(lr, scale)
        if self.o.name == "muon":
            self._broadcast_matrices()
        self._gather(f.params)
        f.refresh_lp()
        return gnorm

    def _gather(self, full: torch.Tensor) -> None:
        """Every rank's owned slices of `full` to every rank, in place."""
        dp = self.dp
        if len(self.buckets) == 1 and full.numel() % self.world == 0 and self.slices[0][1] - self.slices[0][0] == full.numel() // self.world:
            a, b, _ = self.slices[0]
            dp.all_gather_(full, full[a:b].clone())
            return
        mine = torch.zeros_like(full)
        for a, b, _ in self.slices:
            mine[a:b] = full[a:b]
        dp.all_reduce_(mine)
        full.copy_(mine)

    def _broadcast_matrices(self) -> None:
        """Muon matrices were updated by their owners outside the range sharding: place each owner's result into the
        range owner's slice so the all-gather distributes it."""
        import torch.distributed as dist

        for name, r in self.owner.items():
            t = self.flat.view(self.flat.params, name)
            dist.broadcast(t, src=r, group=self.dp.tensor_group)

    def gather_master(self) -> None:
        """Complete fp32 master weights on every rank. After a fused step the fp32 values of the layers' matrices are
        current on their owners only (the bf16 copies are current everywhere); a checkpoint, a replica check or an
        fp32 reader outside training calls this first. A collective: every rank takes part."""
        self.settle()
        if self.fused is not None and self.fused.master_sharded and self.fused.seq > 0:
            self._gather(self.flat.params)

    # ------------------------------------------------------------------ optimizer state I/O

    def _gather_moments(self, shard: torch.Tensor) -> torch.Tensor:
        full = torch.zeros(self.flat.size, dtype=torch.float32, device=self.flat.params.device)
        for a, b, off in self.slices:
            full[a:b] = shard[off:off + b - a]
        self.dp.all_reduce_(full)
        return full

    def optimizer_state(self, opt) -> dict:
        """Full optimizer state assembled on every rank (every rank's moment slices summed into place), in
        FlatAdamW.state_dict form."""
        f = self.flat
        whole = FlatAdamW.__new__(FlatAdamW)
        whole.flat, whole.groups, whole.betas, whole.eps = f, opt.groups, opt.betas, opt.eps
        whole.ranges, whole.lo, whole.hi = [(0, f.size, 0)], 0, f.size
        whole.exp_avg, whole.exp_avg_sq, whole.steps = self._gather_moments(opt.exp_avg), self._gather_moments(opt.exp_avg_sq), opt.steps
        whole.param_groups, whole.torch_order = opt.param_groups, opt.torch_order
        sd = FlatAdamW.state_dict(whole)
        if hasattr(opt, "buf"):
            gathered = self.dp.gather_host({n: b.cpu() for n, b in opt.buf.items()})
            sd["muon"] = {n: b for part in gathered for n, b in part.items()}
        return sd

    def load_optimizer_state(self, opt, sd: dict) -> None:
        """Any world size or layout: every rank reads the by-name state and keeps what falls in its slices / ownership."""
        FlatAdamW.load_state_dict(opt, sd)
        for n, b in (sd.get("muon") or {}).items():
            if hasattr(opt, "buf") and n in opt.buf:
                opt.buf[n].copy_(b)


def _sumsq(t: torch.Tensor) -> torch.Tensor:
    from ..ops import native

    return native.sumsq(t)
