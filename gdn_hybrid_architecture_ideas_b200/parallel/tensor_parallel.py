"""Tensor parallelism with sequence-parallel norm regions (Megatron-style), for the hybrid stack.

Between the residual stream and a mixer / MLP the tokens are sharded over the ranks ([T / W, d] per rank: norms,
depth mixes and residual adds cost 1 / W); inside, the heads (GDN heads, attention heads, SwiGLU hidden units) are
sharded and every rank sees all tokens. The two boundaries are the collectives:

  column-parallel projection   y = all_gather(x) W_r^T          `ag_gemm`: gather fused into the GEMM's main loop
  row-parallel projection      out = reduce_scatter(h W_r^T)     `gemm_rs`: scatter fused into the GEMM's epilogue

Backward mirrors them (dx = reduce_scatter(dy W_r), dW_r = dy^T all_gather(x); dh = all_gather(dout) W_r,
dW_r = all_gather(dout)^T h); activations are re-gathered in the backward rather than kept.

Two implementations of the same functions: "fused" (csrc/gemm_tp.cu over symmetric memory: the gather's push is one
`multimem.st` per 16 bytes through the NVSwitch multicast mapping of the buffer, the scatter's reduction one
`multimem.ld_reduce`, both inside the GEMM launch, with flags and bounded waits; plain peer stores / loads when the
allocation has no multicast mapping or GHB_COMM_MULTIMEM=0) and "collective" (`torch.distributed`
all_gather_into_tensor / reduce_scatter_tensor around a plain GEMM: the baseline and the CPU / gloo path). The
reference has no tensor parallelism.
"""

from __future__ import annotations

import os
import struct

import torch
import torch.distributed as dist

BF16 = torch.bfloat16
MAXR = 8
CHUNK = 128
N_GATHER_SLOTS = 4
N_STAGE_SLOTS = 2
SEQ_RING = 64          # copy-engine push: sequence-number source words of the gathers in flight
PAD_AG_DONE, PAD_RS_READY, PAD_RS_DONE = 0, 8, 16
_ARGS_FMT = "<8Q8Q8Q5i4x3q2Ii4x8Q5Q2i"


class Gathered:
    """A token-sharded activation placed in a gather slot: `full` is the [T, width] view of this rank's gathered buffer
    (complete once a consuming GEMM has run); `pushed` turns true when the first consumer has sent the local shard."""

    def __init__(self, slot, seq, need, full, shard_rows, width):
        self.slot, self.seq, self.need, self.full, self.shard_rows, self.width = slot, seq, need, full, shard_rows, width
        self.pushed = False
        self.fan = FanIn()


class FanIn:
    """The column-parallel projections that read one gathered input. Each of them owes the input a partial gradient
    dy_i W_i over all tokens, to be reduce-scattered; their sum is one product over the concatenated hidden columns, so
    the backward of every projection but the last to run only leaves (dy_i, W_i) here, and the last one multiplies and
    scatters once: one scatter per input instead of one per projection."""

    __slots__ = ("expected", "left")

    def __init__(self):
        self.expected, self.left = 0, []


class TensorParallel:
    def __init__(self, dp, max_tokens: int, max_width: int, impl: str | None = None):
        """dp: the process-group wrapper (rank, world, device, tensor_group). max_tokens: tokens of a micro-batch over
        all ranks (a multiple of 128 x world); max_width: widest gathered or scattered row (elements)."""
        self.dp = dp
        self.rank, self.world, self.device = dp.rank, dp.world, dp.device
        self.group = dp.tensor_group
        impl = impl or os.environ.get("GHB_TP_IMPL", "fused" if self.device.type == "cuda" else "collective")
        self.impl = impl
        self.max_tokens, self.max_width = max_tokens, max_width
        self.ag_seq = self.rs_seq = 0
        self._cache = {}
        # GHB_TP_MERGE_DX=0: every column-parallel projection scatters its own input gradient (see FanIn)
        self.merge_input_grads = os.environ.get("GHB_TP_MERGE_DX", "1") != "0"
        self.open_fans: set = set()
        if impl != "fused":
            return
        import torch.distributed._symmetric_memory as symm

        from ..ops import native

        if self.world > MAXR or max_tokens % (CHUNK * self.world):
            raise ValueError(f"tensor parallel: {max_tokens} tokens over {self.world} ranks must be a multiple of {CHUNK} per rank")
        name = self.group.group_name
        try:
            symm.enable_symm_mem_for_group(name)
        except Exception:
            pass

        def alloc(count, dtype):
            t = symm.empty(count, dtype=dtype, device=self.device)
            t.zero_()
            return t, symm.rendezvous(t, name)

        n_chunks = max_tokens // CHUNK
        self.gather_buf, hg = alloc(N_GATHER_SLOTS * max_tokens * max_width, BF16)
        self.chunk_flags, hc = alloc(N_GATHER_SLOTS * n_chunks, torch.int32)
        self.stage_buf, hs = alloc(N_STAGE_SLOTS * max_tokens * max_width, BF16)
        self.pad, hp = alloc(native.ext().tp_pad_words(), torch.int32)
        self._handles = (hg, hc, hs, hp)
        self._ptrs = {k: [int(p) for p in h.buffer_ptrs] for k, h in zip("gcsp", self._handles)}
        use_mc = os.environ.get("GHB_COMM_MULTIMEM", "1") != "0"
        self._mc = {k: (int(getattr(h, "multicast_ptr", 0) or 0) if use_mc else 0) for k, h in zip("gs", (hg, hs))}
        self.multimem = bool(self._mc["g"] and self._mc["s"])
        if not self.multimem:
            self._mc = {"g": 0, "s": 0}
        self.owner_counters = torch.zeros(MAXR, dtype=torch.int32, device=self.device)
        self.n_chunks = n_chunks
        self.slot_seq = [0] * N_GATHER_SLOTS
        self.next_slot = 0
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        # CTAs of a launch that push the local shard to the peers. Measured at 2 GPUs (200M, 16 rows): 8 -> 339 ms per step,
        # 32 -> 258, 64 -> 235, 96 -> 244, 128 -> 311 (the GEMM CTAs lose their SMs); 32 was the setting of the 8-GPU runs.
        # With the multicast push a shard leaves the GPU once, whatever the world size: a few CTAs saturate the links.
        default_push = "32" if self.multimem else ("64" if self.world <= 2 else "32")
        # Who moves the bytes between GPUs (measured per boundary with scripts/tp_bench.py, 65536 x 2048 bf16):
        #   GHB_TP_GATHER   "ce": the shard is pushed by the copy engines (device-to-device copies on side streams, each
        #                   followed by a small copy that raises the chunk flags on the peer): no SM is spent and the
        #                   consuming GEMM, which polls the flags chunk by chunk, keeps all of them. Best at 2 ranks; at 8
        #                   the engines carry about 300 GB/s in total, less than the links.
        #                   "threads": a few CTAs of the consuming launch copy with 16-byte loads and stores, ONE multicast
        #                   store per 16 bytes where the buffer is mapped through the switch (the shard leaves this GPU once
        #                   whatever the world size). "tma": those CTAs drive tile loads and tile stores instead (one SM
        #                   keeps about 13 GB/s of remote tile stores in flight: ~60 SMs to fill a link; for comparison).
        #   GHB_TP_SCATTER  "tma": one launch whose epilogue tile-stores each partial tile into its owner's staging slot
        #                   over NVLink; the owner sums the world's tiles from local memory. "ce": one GEMM launch per
        #                   owner's rows, each block carried by a copy engine while the next is multiplied (best at 2
        #                   ranks). "pull": partials stay local and the owner reads them from every rank (through the
        #                   switch's reduction where mapped).
        few = self.world <= 2 or not self.multimem
        self.gather_by = os.environ.get("GHB_TP_GATHER", "ce" if few else "threads")
        self.scatter = os.environ.get("GHB_TP_SCATTER", "ce" if self.world <= 2 else "tma")
        if self.gather_by not in ("ce", "tma", "threads") or self.scatter not in ("ce", "tma", "pull"):
            raise ValueError(f"GHB_TP_GATHER {self.gather_by!r} ('ce', 'tma', 'threads') / GHB_TP_SCATTER {self.scatter!r} ('ce', 'tma', 'pull')")
        if self.gather_by == "tma":
            default_push = "32" if self.world <= 2 else "16"
        self.n_push = int(os.environ.get("GHB_TP_PUSH_CTAS", default_push))
        self.kernel_flags = (0 if self.scatter == "pull" else 1) | (2 if self.gather_by == "tma" else 0)
        self.push_streams = [torch.cuda.Stream(self.device) for _ in range(self.world - 1)]       # one per peer
        self.push_pieces = int(os.environ.get("GHB_TP_PUSH_PIECES", max(1, 8 // self.world)))
        self.seq_words = torch.zeros(SEQ_RING, max_tokens // self.world // CHUNK, dtype=torch.int32, device=self.device)
        self.rs_words = torch.zeros(SEQ_RING, dtype=torch.int32, device=self.device)
        self.parts = None                      # [2][world - 1] blocks of partial rows in flight to their owners
        torch.cuda.synchronize(self.device)
        dp.barrier()

    # ------------------------------------------------------------------ argument table

    def _args(self, mode, slot=0, seq=0, need=0, push=0, axis=0, shard_rows=0, row_elems=0, ld=8, stage_slot=0, out=None):
        n_push = self.n_push if push else 0        # a later consumer of a gather multiplies on every SM
        def peers(key, offset_bytes):
            got = [p + offset_bytes for p in self._ptrs[key]]
            return got + [0] * (MAXR - len(got))

        g_off = slot * self.max_tokens * self.max_width * 2
        c_off = slot * self.n_chunks * 4
        s_off = stage_slot * self.max_tokens * self.max_width * 2
        raw = struct.pack(_ARGS_FMT, *peers("g", g_off), *peers("c", c_off), *peers("p", 0), self.rank, self.world, mode, push, axis,
                          shard_rows, row_elems, ld, seq, need, n_push, *peers("s", s_off), self.done_counter.data_ptr(),
                          self.owner_counters.data_ptr(), (self._mc["g"] + g_off) if self._mc["g"] else 0, (self._mc["s"] + s_off) if self._mc["s"] else 0,
                          0 if out is None else out.data_ptr(), int(out is not None and out.dtype == torch.float32), self.kernel_flags)
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8)

    # ------------------------------------------------------------------ gather handles

    def gather(self, x_shard: torch.Tensor) -> Gathered:
        """x_shard [Ts, width] (bf16 on the fused path). Several GEMMs may consume the same handle; the first one moves
        the data."""
        key = (x_shard.data_ptr(), x_shard._version, tuple(x_shard.shape))
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        Ts, width = x_shard.shape
        T = Ts * self.world
        if self.impl != "fused":
            full = torch.empty(T, width, dtype=x_shard.dtype, device=x_shard.device)
            dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
            g = Gathered(-1, 0, 0, full, Ts, width)
            g.pushed = True
        else:
            from ..ops import native

            if T > self.max_tokens or width > self.max_width or Ts % CHUNK or width % 8:
                raise ValueError(f"tensor parallel gather of [{Ts}, {width}] exceeds the workspace ({self.max_tokens} x {self.max_width})")
            slot = self.next_slot
            self.next_slot = (slot + 1) % N_GATHER_SLOTS
            prev = self.slot_seq[slot]     # released to the peers during the previous gather call (below)
            self.ag_seq += 1
            self.slot_seq[slot] = self.ag_seq
            base = slot * self.max_tokens * self.max_width
            full = self.gather_buf[base:base + T * width].view(T, width)
            full[self.rank * Ts:(self.rank + 1) * Ts].copy_(x_shard)
            g = Gathered(slot, self.ag_seq, prev, full, Ts, width)
            # The slot the NEXT gather will take: everything launched so far has read its contents, so tell the peers now,
            # one gather ahead of its reuse; by the time the peers push into it the word has long arrived.
            nxt, release = self.next_slot, self.slot_seq[self.next_slot]
            if release:
                self._cache = {k: v for k, v in self._cache.items() if v.slot != nxt}
            if self.gather_by == "ce":
                self._push_by_copy_engines(g, release)
            elif release:
                native.ext().tp_signal(self._args(2, seq=release), PAD_AG_DONE, self.pad)
        g.src = x_shard          # keeps the shard's memory alive while the handle is cached: its address cannot be recycled
        if len(self._cache) > 8:
            self._cache.clear()
        self._cache[key] = g
        return g

    def _push_by_copy_engines(self, g: Gathered, release: int) -> None:
        """Queues the push of gather `g` on the side stream: behind the local copy of the shard, behind the word that says
        every peer has released the slot's previous use (a bounded wait in a one-thread kernel on the main stream, which
        also publishes `release`), one data copy and one flag copy per peer and piece."""
        from ..ops import native

        # The flag copies read a ring entry of words holding the sequence number. An entry is rewritten SEQ_RING gathers
        # later; by then its copies have run: this rank's main stream gets there only through GEMMs that needed every
        # peer's later pushes, which the peers queued after GEMMs that needed these flags.
        words = self.seq_words[g.seq % SEQ_RING]
        words.fill_(g.seq)
        args = self._args(0, slot=g.slot, seq=release, need=g.need, shard_rows=g.shard_rows, row_elems=g.width, ld=g.width)
        native.ext().tp_signal(args, PAD_AG_DONE, self.pad, PAD_AG_DONE, native.err_flag(self.device))
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        for st in self.push_streams:
            st.wait_event(ready)
        args = self._args(0, slot=g.slot, seq=g.seq, need=g.need, shard_rows=g.shard_rows, row_elems=g.width, ld=g.width)
        native.ext().tp_push_copies(args, words, self.push_pieces, [st.cuda_stream for st in self.push_streams])
        g.pushed = True

    def _ag_args(self, g: Gathered, axis: int):
        push = 0 if g.pushed else 1
        g.pushed = True
        return self._args(0, slot=g.slot, seq=g.seq, need=g.need, push=push, axis=axis, shard_rows=g.shard_rows, row_elems=g.width, ld=g.width)

    # ------------------------------------------------------------------ the four products

    def ag_gemm(self, g: Gathered, w: torch.Tensor, b_mn: bool = False, out_dtype=BF16) -> torch.Tensor:
        """all_gather(x) w^T ([T, N]); w [N, K], or [K, N] with b_mn."""
        if self.impl != "fused":
            return self._plain(g.full, w, False, b_mn, out_dtype)
        from ..ops import native

        N = w.shape[1] if b_mn else w.shape[0]
        out = torch.empty(g.full.shape[0], N, dtype=out_dtype, device=self.device)
        native.ext().gemm_tp(g.full, w, out, False, b_mn, False, self._ag_args(g, 0), native.err_flag(self.device))
        native._count()
        return out

    def gemm_gathered_k(self, a: torch.Tensor, b: torch.Tensor, g: Gathered, out: torch.Tensor | None = None) -> torch.Tensor:
        """a^T b over all tokens ([cols(a), cols(b)], fp32), a and b stored [T, *]; one of them is `g.full` (a weight gradient
        whose token dimension is gathered)."""
        if self.impl != "fused":
            res = self._plain(a, b, True, True, torch.float32)
            return res if out is None else out.copy_(res)
        from ..ops import native

        if out is None:
            out = torch.empty(a.shape[1], b.shape[1], dtype=torch.float32, device=self.device)
        native.ext().gemm_tp(a, b, out, True, True, False, self._ag_args(g, 1), native.err_flag(self.device))
        native._count()
        return out

    def gemm_rs(self, h: torch.Tensor, w: torch.Tensor, b_mn: bool = False, out_dtype=BF16) -> torch.Tensor:
        """reduce_scatter(h w^T) over token shards ([T / W, N]); h [T, K_r]; w [N, K_r], or [K_r, N] with b_mn."""
        T = h.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        Ts = T // self.world
        if self.impl != "fused":
            if h.is_cuda and h.dtype == BF16:      # the baseline on GPUs: the same bf16 GEMM, then NCCL's reduce-scatter in bf16
                part = self._plain(h, w, False, b_mn, BF16)
                out = torch.empty(Ts, N, dtype=BF16, device=h.device)
            else:
                part = self._plain(h, w, False, b_mn, torch.float32)
                out = torch.empty(Ts, N, dtype=torch.float32, device=h.device)
            dist.reduce_scatter_tensor(out, part.contiguous(), group=self.group)
            return out.to(out_dtype)
        from ..ops import native

        if T > self.max_tokens or N > self.max_width or Ts % CHUNK or N % 8:
            raise ValueError(f"tensor parallel scatter of [{T}, {N}] exceeds the workspace ({self.max_tokens} x {self.max_width})")
        self.rs_seq += 1
        seq, slot = self.rs_seq, self.rs_seq % N_STAGE_SLOTS
        out = torch.empty(Ts, N, dtype=out_dtype if out_dtype in (BF16, torch.float32) else BF16, device=self.device)
        if self.scatter == "ce":
            self._scatter_by_copy_engines(h, w, b_mn, seq, slot, Ts, N, out)
            return out if out.dtype == out_dtype else out.to(out_dtype)
        args = self._args(1, seq=seq, need=max(seq - N_STAGE_SLOTS, 0), shard_rows=Ts, stage_slot=slot, out=out)
        native.ext().gemm_tp(h, w, None, False, b_mn, False, args, native.err_flag(self.device))      # partial tiles, flags and the reduction: one launch
        native._count()
        return out if out.dtype == out_dtype else out.to(out_dtype)

    def _scatter_by_copy_engines(self, h, w, b_mn, seq, slot, Ts, N, out) -> None:
        """h w^T owner by owner, the next rank's rows first and this rank's last: each block of partial rows [Ts, N] is a
        launch of the plain GEMM, and once it is complete a copy engine carries it into its owner's staging slot (at this
        rank's source index) with the call's number behind it, while the next block is multiplied. The reduction launch
        then waits (bounded) for every peer's number, sums the world's blocks from local memory in rank order and tells
        the peers that the slot is read. Before the first block leaves, the peers must have read the slot's previous use
        (bounded wait in a one-thread launch on this stream); that also means this rank's blocks of two calls ago have
        been consumed, so their buffers can be written again."""
        from ..ops import native

        W, r = self.world, self.rank
        e, err = native.ext(), native.err_flag(self.device)
        main = torch.cuda.current_stream(self.device)
        need = max(seq - N_STAGE_SLOTS, 0)
        if need:
            e.tp_signal(self._args(1, seq=0, need=need, shard_rows=Ts), PAD_RS_DONE, self.pad, PAD_RS_DONE, err)
        if self.parts is None or self.parts[0][0].numel() < Ts * N:
            self.parts = [[torch.empty(Ts * N, dtype=BF16, device=self.device) for _ in range(W - 1)] for _ in range(2)]
        word = self.rs_words[seq % SEQ_RING:seq % SEQ_RING + 1]
        word.fill_(seq)
        slot_bytes = slot * self.max_tokens * self.max_width * 2
        block_bytes = Ts * N * 2
        for j in range(1, W):
            d = (r + j) % W
            part = self.parts[seq % 2][j - 1][:Ts * N].view(Ts, N)
            native.gemm(h[d * Ts:(d + 1) * Ts], w, out=part, b_mn=b_mn)
            ready = torch.cuda.Event()
            ready.record(main)
            st = self.push_streams[j - 1]
            st.wait_event(ready)
            e.tp_copy_flagged(self._ptrs["s"][d] + slot_bytes + r * block_bytes, part, block_bytes,
                              self._ptrs["p"][d] + (PAD_RS_READY + r) * 4, word, st.cuda_stream)
        base = slot * self.max_tokens * self.max_width
        own = self.stage_buf[base + r * Ts * N:base + (r + 1) * Ts * N].view(Ts, N)
        native.gemm(h[r * Ts:(r + 1) * Ts], w, out=own, b_mn=b_mn)
        e.tp_reduce(self._args(1, seq=seq, need=need, shard_rows=Ts, stage_slot=slot, out=out), N, err)
        native._count()

    @staticmethod
    def _plain(a, b, a_mn, b_mn, out_dtype):
        """a b^T without communication: the framework's GEMM on CUDA bf16 operands, float math elsewhere."""
        if a.is_cuda and a.dtype == BF16 and b.dtype == BF16:
            from ..ops import native

            return native.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype)
        af = a.float().t() if a_mn else a.float()
        bf = b.float() if b_mn else b.float().t()
        return (af @ bf).to(out_dtype)

    # ------------------------------------------------------------------ replicated parameters

    def check_fans(self) -> None:
        """After a backward: no input may still be waiting for projections whose backward never ran (an output that did
        not reach the loss) — its gradient would be short of the parts left behind. Raises by naming the count."""
        stuck = [f for f in self.open_fans if f.left]
        self.open_fans.clear()
        if stuck:
            for f in stuck:
                f.left, f.expected = [], 0
            raise RuntimeError(f"tensor parallel: {len(stuck)} gathered input(s) received the backward of only some of their column-parallel "
                               "projections; their input gradients were withheld (set GHB_TP_MERGE_DX=0 for models with unused projections)")

    def all_reduce_grads(self, params) -> None:
        """Sum over ranks of the gradients of replicated parameters (each rank saw its own token shard)."""
        self.check_fans()
        grads = [p.grad for p in params if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=self.group)
        at = 0
        for g in grads:
            g.copy_(flat[at:at + g.numel()].view_as(g))
            at += g.numel()


# ---------------------------------------------------------------------------------------------------- autograd


class _ColumnParallel(torch.autograd.Function):
    """y [T, N_r] = all_gather(x) W_r^T for a token shard x [Ts, K]."""

    @staticmethod
    def forward(ctx, x, weight, w_lp, tp):
        x2 = x.reshape(-1, x.shape[-1])
        n = w_lp.shape[0]
        if x.is_cuda:
            from ..ops.native import _pad_rows
            x2, w_lp = x2.to(BF16), _pad_rows(w_lp)       # output rows stay 16-byte aligned for projections with a few outputs
        g = tp.gather(x2)
        y = tp.ag_gemm(g, w_lp, out_dtype=x2.dtype)
        ctx.save_for_backward(x2, w_lp)
        ctx.tp, ctx.xshape, ctx.xdtype, ctx.n = tp, x.shape, x.dtype, n
        ctx.fan = None
        if ctx.needs_input_grad[0] and tp.merge_input_grads:
            ctx.fan = g.fan
            g.fan.expected += 1
            tp.open_fans.add(g.fan)
        return y[:, :n] if n != w_lp.shape[0] else y

    @staticmethod
    def backward(ctx, dy):
        x2, w_lp = ctx.saved_tensors
        tp = ctx.tp
        dy2 = dy.reshape(-1, dy.shape[-1]).to(x2.dtype)
        if ctx.n != w_lp.shape[0]:
            dy2 = torch.nn.functional.pad(dy2, (0, w_lp.shape[0] - ctx.n))
        dy2 = dy2.contiguous()
        fan, dx = ctx.fan, None
        if fan is None:
            if ctx.needs_input_grad[0]:
                dx = tp.gemm_rs(dy2, w_lp, b_mn=True, out_dtype=x2.dtype)
        else:
            fan.left.append((dy2, w_lp))
            if len(fan.left) == fan.expected:          # the last projection of this input: one product, one scatter
                if len(fan.left) == 1:
                    dx = tp.gemm_rs(dy2, w_lp, b_mn=True, out_dtype=x2.dtype)
                else:
                    dx = tp.gemm_rs(torch.cat([d for d, _ in fan.left], dim=1), torch.cat([w for _, w in fan.left], dim=0), b_mn=True, out_dtype=x2.dtype)
                fan.left, fan.expected = [], 0
                tp.open_fans.discard(fan)
        g = tp.gather(x2)
        dw = tp.gemm_gathered_k(dy2, g.full, g)[:ctx.n] if ctx.needs_input_grad[1] else None
        return (None if dx is None else dx.view(ctx.xshape).to(ctx.xdtype)), dw, None, None


class _RowParallel(torch.autograd.Function):
    """out [Ts, N] = reduce_scatter(h W_r^T) for h [T, K_r] (all tokens, this rank's hidden slice)."""

    @staticmethod
    def forward(ctx, h, weight, w_lp, tp):
        h2 = h.reshape(-1, h.shape[-1])
        if h.is_cuda:
            h2 = h2.to(BF16)
        h2 = h2.contiguous()
        out = tp.gemm_rs(h2, w_lp, out_dtype=h2.dtype)
        ctx.save_for_backward(h2, w_lp)
        ctx.tp, ctx.hshape, ctx.hdtype = tp, h.shape, h.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        h2, w_lp = ctx.saved_tensors
        tp = ctx.tp
        g = tp.gather(dout.reshape(-1, dout.shape[-1]).to(h2.dtype).contiguous())
        dh = tp.ag_gemm(g, w_lp, b_mn=True, out_dtype=h2.dtype)
        dw = tp.gemm_gathered_k(g.full, h2, g)
        return dh.view(ctx.hshape).to(ctx.hdtype), dw, None, None


def column_parallel(x, lin, tp):
    from ..ops.native import _w_lp
    w_lp = _w_lp(lin) if x.is_cuda else lin.weight.detach()
    return _ColumnParallel.apply(x, lin.weight, w_lp, tp)


def row_parallel(h, lin, tp):
    from ..ops.native import _w_lp
    w_lp = _w_lp(lin) if h.is_cuda else lin.weight.detach()
    return _RowParallel.apply(h, lin.weight, w_lp, tp)
