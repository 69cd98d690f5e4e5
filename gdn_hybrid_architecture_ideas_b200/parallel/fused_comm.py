"""Fused data-parallel step over NVLink peer memory: gradient reduce-scatter + global-norm clip + sharded AdamW +
parameter all-gather in the kernels of csrc/comm.cu, in place of NCCL reduce-scatter, a clip pass, an optimizer
launch and an NCCL all-gather (the reference's sequence: ced/train/zero1.py:250-264, 293-337, 354-377).

The flat gradient, fp32 parameter and bf16 parameter buffers live in symmetric memory (every rank maps every peer's
copy); a small signal pad per rank carries the numbered flags and the partial gradient norms. When the allocation
also has an NVSwitch multicast mapping, gradient sums use `multimem.ld_reduce` and parameter writes `multimem.st`;
otherwise plain peer loads and stores. Set GHB_COMM_MULTIMEM=0 to force the peer path (tests that remove a rank must:
a rank that dies while bound to a multicast object faults its peers).

The buffers are cut into buckets and every rank owns one slice of every bucket (parallel/zero.py). All communication
kernels run on one side stream in one job-wide order:

* `reduce_bucket(i)` — called when bucket i's gradients are final on the compute stream (from a backward hook, or after
  the backward): the side stream waits for an event of the compute stream and runs the bucket's reduce kernel on a few
  CTAs, beside the backward of the layers that are still to come;
* `update(...)` — after the last bucket: per bucket, in the order the next forward reads them, AdamW on the owned slice
  and the broadcast of the new values, a wait for every peer's slice, and an event;
* `wait_bucket(i)` — the compute stream waits for bucket i's event: called where the forward first reads the bucket, so
  the all-gather of later layers runs behind the forward of earlier ones.
"""

from __future__ import annotations

import os
import struct

import torch

MAX_RANKS = 8
OVERLAP_CTAS = int(os.environ.get("GHB_COMM_OVERLAP_CTAS", "24"))     # grid of a launch that runs beside compute kernels


def available(dp) -> bool:
    if dp is None or dp.world > MAX_RANKS or dp.device.type != "cuda":
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True


class FusedComm:
    def __init__(self, dp, flat, model, rebind, buckets, slices, update_order, fp32_cells=None):
        """rebind(params, grads, lp): re-homes the model's parameters / gradients / bf16 copies onto new flat buffers.
        buckets: [(lo, hi)] element ranges; slices: this rank's [(lo, hi, offset in the shard / moment buffers)] per
        bucket (hi == lo: nothing owned); update_order: bucket indices in the order the forward reads them;
        fp32_cells: bool tensor, one entry per 64 elements, True where the fp32 value must reach every rank (None: all)."""
        import torch.distributed._symmetric_memory as symm

        from ..ops import native

        self.dp, self.flat = dp, flat
        self.rank, self.world = dp.rank, dp.world
        dev = dp.device
        group = dp.tensor_group
        name = group.group_name
        try:
            symm.enable_symm_mem_for_group(name)
        except Exception:
            pass
        n = flat.size

        def alloc(count, dtype):
            t = symm.empty(count, dtype=dtype, device=dev)
            return t, symm.rendezvous(t, name)

        self.grads, hg = alloc(n, torch.float32)
        self.params, hp = alloc(n, torch.float32)
        self.lp, hl = alloc(n, torch.bfloat16) if flat.lp is not None else (None, None)
        self.pad, hs = alloc(3 * MAX_RANKS + MAX_RANKS, torch.int32)     # flags [3][8] then norms [8] (as fp32 bits)
        self.pad.zero_()
        self.grads.zero_()
        self.params.copy_(flat.params)
        if self.lp is not None:
            self.lp.copy_(flat.lp)
        rebind(self.params, self.grads, self.lp)
        use_mc = os.environ.get("GHB_COMM_MULTIMEM", "1") != "0"

        def mc(h):
            p = int(getattr(h, "multicast_ptr", 0) or 0)
            return p if use_mc else 0

        def ptrs(h, offset_bytes=0):
            got = [int(p) + offset_bytes for p in h.buffer_ptrs]
            return got + [0] * (MAX_RANKS - len(got))

        table = (ptrs(hg) + ptrs(hp) + (ptrs(hl) if hl is not None else [0] * MAX_RANKS) + ptrs(hs) + ptrs(hs, 3 * MAX_RANKS * 4)
                 + [mc(hg), mc(hp), mc(hl) if hl is not None else 0])
        raw = struct.pack(f"<{len(table)}Q", *table)
        assert len(raw) == native.ext().comm_peers_bytes(), (len(raw), native.ext().comm_peers_bytes())
        self.peers = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.multimem = bool(mc(hg))
        self._handles = (hg, hp, hl, hs)
        self.buckets, self.slices, self.update_order = list(buckets), list(slices), list(update_order)
        owned = sum(hi - lo for lo, hi, _ in self.slices)
        self.shard = torch.zeros(max(owned, 8), dtype=torch.float32, device=dev)
        self.acc = torch.zeros(1, dtype=torch.float32, device=dev)
        self.counters = torch.zeros(2, dtype=torch.int32, device=dev)
        self.coef = torch.zeros(2, dtype=torch.float32, device=dev)       # (global gradient norm, clip coefficient) of the step
        self.fp32_map = None
        if fp32_cells is not None and self.lp is not None and not bool(fp32_cells.all()):
            cells = fp32_cells.to(torch.int64)
            cells = torch.cat([cells, cells.new_zeros(-cells.numel() % 32)]).view(-1, 32)
            words = (cells << torch.arange(32, dtype=torch.int64)).sum(1)
            self.fp32_map = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32).to(dev)
        self.master_sharded = self.fp32_map is not None
        self.seq = 0                # optimizer steps taken
        self.reduce_ticket = 0      # reduce launches so far (the same sequence on every rank)
        self.update_ticket = 0      # update launches so far
        self.stream = torch.cuda.Stream(dev)
        self.ready = [None] * len(self.buckets)      # per bucket: event after its update + settle
        self.reduced = set()
        torch.cuda.synchronize(dev)
        dp.barrier()

    # ------------------------------------------------------------------ gradient side
    @torch.no_grad()
    def reduce_bucket(self, i: int, last: bool = False) -> None:
        """Bucket i's gradients are final on the current stream. `last`: the step's last bucket (publishes the norm)."""
        from ..ops import native

        if i in self.reduced:
            return
        self.reduced.add(i)
        cur = torch.cuda.current_stream(self.dp.device)
        done = torch.cuda.Event()
        done.record(cur)
        self.stream.wait_event(done)
        lo, hi, off = self.slices[i]
        self.reduce_ticket += 1
        err = native.err_flag(self.dp.device)
        with torch.cuda.stream(self.stream):
            native.ext().comm_reduce(self.peers, self.rank, self.world, lo, hi - lo, self.shard[off:], self.reduce_ticket,
                                     self.seq + 1 if last else 0, self.acc, self.counters[0:1], err, 0 if last else OVERLAP_CTAS)
        native._count(1)

    # ------------------------------------------------------------------ parameter side
    @torch.no_grad()
    def update(self, opt, lr: float, max_norm: float) -> torch.Tensor:
        """Every bucket has been handed to `reduce_bucket` (the last one with last=True). Launches the updates in
        forward order on the side stream; returns the global gradient norm (a 0-dim view the side stream fills: read it
        after `wait_bucket` of any bucket, or on the side stream)."""
        from ..ops import native

        ext = native.ext()
        self.seq += 1
        err = native.err_flag(self.dp.device)
        opt.steps += 1
        b1, b2 = opt.betas
        starts, wds, lrs = [], [], []
        for gi, g in enumerate(opt.param_groups):
            g["lr"] = lr * g["lr_scale"]
            starts.append(self.flat.group_ranges[gi][0])
            wds.append(g["weight_decay"])
            lrs.append(g["lr"] if g["kind"] == "adamw" else 0.0)
        c1, c2 = 1.0 - b1 ** opt.steps, 1.0 - b2 ** opt.steps
        with torch.cuda.stream(self.stream):
            for k, i in enumerate(self.update_order):
                lo, hi, off = self.slices[i]
                self.update_ticket += 1
                ext.comm_update(self.peers, self.rank, self.world, lo, hi - lo, self.shard[off:], opt.exp_avg[off:], opt.exp_avg_sq[off:],
                                starts, wds, lrs, b1, b2, opt.eps, c1, c2, float(max_norm or 0.0), self.seq, k == 0, self.coef, self.fp32_map,
                                self.update_ticket, self.counters[1:2], err, 0 if k == 0 else 2 * OVERLAP_CTAS)
                ev = torch.cuda.Event()
                ev.record(self.stream)
                self.ready[i] = ev
        native._count(2 * len(self.update_order))
        self.reduced.clear()
        return self.coef[0]

    def wait_bucket(self, i: int) -> None:
        ev = self.ready[i]
        if ev is not None:
            torch.cuda.current_stream(self.dp.device).wait_event(ev)

    def wait_all(self) -> None:
        for i in range(len(self.buckets)):
            self.wait_bucket(i)
