"""Fused data-parallel step over NVLink peer memory: gradient reduce-scatter + global-norm clip + sharded AdamW +
parameter all-gather in the three kernels of csrc/comm.cu, in place of NCCL reduce-scatter, a clip pass, an optimizer
launch and an NCCL all-gather (the reference's sequence: ced/train/zero1.py:250-264, 293-337, 354-377).

The flat gradient, fp32 parameter and bf16 parameter buffers live in symmetric memory (every rank maps every peer's
copy); a small signal pad per rank carries the step-numbered flags and the partial gradient norms. When the
allocation also has an NVSwitch multicast mapping, gradient sums use `multimem.ld_reduce` and parameter writes
`multimem.st`; otherwise plain peer loads and stores. Set GHB_COMM_MULTIMEM=0 to force the peer path (tests that
remove a rank must: a rank that dies while bound to a multicast object faults its peers).
"""

from __future__ import annotations

import os
import struct

import torch

MAX_RANKS = 8


def available(dp) -> bool:
    if dp is None or dp.world > MAX_RANKS or dp.device.type != "cuda":
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True


class FusedComm:
    def __init__(self, dp, flat, model, rebind):
        """rebind(params, grads, lp): re-homes the model's parameters / gradients / bf16 copies onto new flat buffers."""
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
        self.per = n // self.world
        self.lo = self.rank * self.per
        self.shard = torch.zeros(self.per, dtype=torch.float32, device=dev)
        self.acc = torch.zeros(1, dtype=torch.float32, device=dev)
        self.counters = torch.zeros(2, dtype=torch.int32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.seq = 0
        torch.cuda.synchronize(dev)
        dp.barrier()

    @torch.no_grad()
    def step(self, opt, lr: float, max_norm: float) -> torch.Tensor:
        """Gradients in the symmetric buffer are final on this stream. Returns the global gradient norm (0-dim)."""
        from ..ops import native

        ext = native.ext()
        self.seq += 1
        err = native.err_flag(self.dp.device)
        ext.comm_reduce(self.peers, self.rank, self.world, self.lo, self.per, self.shard, self.seq, self.acc, self.counters[0:1], err)
        opt.steps += 1
        b1, b2 = opt.betas
        starts, wds, lrs = [], [], []
        for gi, g in enumerate(opt.param_groups):
            g["lr"] = lr * g["lr_scale"]
            starts.append(self.flat.group_ranges[gi][0])
            wds.append(g["weight_decay"])
            lrs.append(g["lr"] if g["kind"] == "adamw" else 0.0)
        ext.comm_update(self.peers, self.rank, self.world, self.lo, self.per, self.shard, opt.exp_avg, opt.exp_avg_sq, starts, wds, lrs,
                        b1, b2, opt.eps, 1.0 - b1 ** opt.steps, 1.0 - b2 ** opt.steps, float(max_norm or 0.0), self.seq, self.norm,
                        self.counters[1:2], err)
        native._count(3)
        return self.norm[0]
