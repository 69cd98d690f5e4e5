"""Trainer: builds the model, the flat-buffer optimizer, the data source and the parallel plan from a TrainConfig and
runs the training loop with checkpoints, metrics and clean stops.

One step (reference: ced/train/trainer.py:2823-3362): batch for this rank (pure function of the step) -> micro-batch
loop {pinned H2D, forward to hidden states, fused head + loss, backward into the flat gradient buffer} -> gradient
synchronisation (NCCL all-reduce, or ZeRO reduce-scatter; on CUDA optionally the fused peer-memory kernel that also
applies the update) -> global-norm clip -> optimizer update (+ parameter all-gather under ZeRO) -> metrics.
The loss is sum(valid (ce + z lse^2)) / global valid count, so summing gradients over ranks gives the 1-process step.

Stops: a non-finite loss writes `diverged.json` and raises Diverged (the CLI exits 86; the run directory then refuses
to train); SIGTERM sets a flag that is OR-reduced over ranks each step so all ranks save and leave together
(trainer.py:4361-4404, 4678-4695).
"""

from __future__ import annotations

import json
import math
import random
import signal
import time
from pathlib import Path

import torch

from .. import config as C
from ..data import make_data
from ..data.batch_check import BatchError, check_batch
from ..models import build_model
from . import checkpoint as ckpt
from .fused_head import chunked_ce, fused_linear_ce
from .lr import lr_of
from .optim import build_optimizer, grad_norm

EXIT_DIVERGED = 86


from . import bpb_readout, monitor, periodic_eval, readout


class Diverged(RuntimeError):
    pass


class KernelStatus(RuntimeError):
    """A kernel's bounded wait gave up during the step (the status word was non-zero on some rank)."""


def pick_device(name: str) -> torch.device:
    if name == "auto":
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)


class Trainer:
    def __init__(self, cfg: C.TrainConfig, run_dir: str | Path | None = None, dp=None, device: torch.device | None = None):
        C.require_supported(cfg)
        if cfg.model.mtp.enabled:
            raise ValueError("model.mtp.enabled: the trainer trains the trunk; the drafter head is trained on a frozen trunk "
                             "by models.mtp.train_step (scripts/train_mtp.py)")
        self.cfg, self.dp = cfg, dp
        self.run_dir = Path(run_dir) if run_dir is not None else None
        self.device = device or (dp.device if dp is not None else pick_device(cfg.device))
        self.rank, self.world = (dp.rank, dp.world) if dp is not None else (0, 1)
        self.lead = self.rank == 0
        random.seed(cfg.seed)
        torch.manual_seed(cfg.seed)
        if cfg.tf32 and self.device.type == "cuda":
            torch.backends.cuda.matmul.allow_tf32 = True
        dtype = {"float32": torch.float32, "float64": torch.float64, "bfloat16": torch.bfloat16}[cfg.dtype]
        self.tp = None
        model_cfg = cfg.model
        # A looped middle (models/recur.py): one pass count per optimizer step, drawn from loop.t_choices / t_probs; what it
        # is not built together with is refused here, by key.
        self.looped = bool(cfg.model.loop.recur_layers)
        # The looped encoder-decoder (models/looped_decoder.py): decoder positions in spans from the data, one pass count per
        # optimizer step, the two heads' loss.
        self.slot_decoder = cfg.model.arch == "looped_ced"
        if self.slot_decoder:
            clashes = {"tensor_parallel": cfg.tensor_parallel > 1, "cuda_graphs": cfg.cuda_graphs != "none", "tst.schedule": bool(cfg.tst.schedule),
                       "shape_schedule": bool(cfg.shape_schedule), "loop_switch_step": bool(cfg.loop_switch_step), "freeze_trunk": bool(cfg.freeze_trunk),
                       "optimizer_sharding 'zero2'": cfg.optimizer_sharding == "zero2", "data.kind other than 'synthetic'": cfg.data.kind != "synthetic",
                       "data.loss_mask": cfg.data.loss_mask != "all", "eval.readout_every": bool(cfg.eval.readout_every),
                       "eval.every_steps / eval.bpb_readout_every (the scorers call the one-head stack)": bool(cfg.eval.every_steps or cfg.eval.bpb_readout_every),
                       "activation_checkpoint 'block' / 'host' / 'host_overlap'": cfg.activation_checkpoint in ("block", "host", "host_overlap")}
            hit = [k for k, v in clashes.items() if v]
            if hit:
                raise ValueError(f"model.arch 'looped_ced' is not built together with: {', '.join(hit)}")
        self.gated = cfg.model.loop.pass2_gate != "none"          # a read-only second pass (models/second_pass.py): T = 1 before loop_switch_step, then 2
        self.pass_count = 1
        if self.looped:
            clashes = {"tensor_parallel": cfg.tensor_parallel > 1, "cuda_graphs": cfg.cuda_graphs != "none", "tst.schedule": bool(cfg.tst.schedule),
                       "shape_schedule": bool(cfg.shape_schedule), "loop_switch_step": bool(cfg.loop_switch_step),
                       "optimizer_sharding 'zero2' (its buckets follow one backward pass over the blocks)": cfg.optimizer_sharding == "zero2",
                       "activation_checkpoint 'block'": cfg.activation_checkpoint == "block", "model.fp8.mode": cfg.model.fp8.mode != "none"}
            hit = [k for k, v in clashes.items() if v]
            if hit:
                raise ValueError(f"model.loop.recur_layers (the looped middle) is not built together with: {', '.join(hit)}")
        # A pass count per row (model.loop.t_sampling 'sequence'): the step's rows hold a fixed multiset of counts, and the
        # micro-batches are formed from rows of equal count, micro_batch_by_t[T - 1] rows at a time.
        self._rows_held = None
        by_t = cfg.micro_batch_by_t
        if not isinstance(by_t, list) or any(type(m) is not int or not 1 <= m <= cfg.data.batch_size for m in by_t):
            raise ValueError(f"micro_batch_by_t {by_t!r}: a list of rows per forward by pass count (entry T - 1), each 1 .. data.batch_size ({cfg.data.batch_size})")
        if by_t and not self.looped:
            raise ValueError("micro_batch_by_t is read with a looped middle (model.loop.recur_layers); set micro_batch_size")
        if self.looped and cfg.model.loop.t_sampling == "sequence":
            from ..models.recur import rows_by_count

            if self.world > 1:
                raise ValueError("model.loop.t_sampling 'sequence' (a pass count per row: the step's multiset is dealt over the whole batch) is not built "
                                 "together with data parallelism")
            self._rows_held = rows_by_count(cfg.model.loop, cfg.data.batch_size)
        S = cfg.loop_switch_step
        if type(S) is not int or not 0 <= S < max(cfg.steps, 1):
            raise ValueError(f"loop_switch_step {S!r}: an optimizer step S with 0 <= S < steps ({cfg.steps})")
        if S and not self.gated:
            raise ValueError(f"loop_switch_step {S} switches a gated second pass on (model.loop.pass2_gate 'scalar' with pass2_layers): this model has none")
        if self.gated:
            clashes = {"tensor_parallel": cfg.tensor_parallel > 1, "cuda_graphs": cfg.cuda_graphs != "none", "tst.schedule": bool(cfg.tst.schedule),
                       "shape_schedule": bool(cfg.shape_schedule), "optim.schedule_steps": cfg.optim.schedule_steps is not None,
                       "optim.switch_warmup_steps": bool(cfg.optim.switch_warmup_steps),
                       "optimizer_sharding 'zero2' (its buckets follow one backward pass over the blocks)": cfg.optimizer_sharding == "zero2",
                       "activation_checkpoint 'block' / 'host' / 'host_overlap'": cfg.activation_checkpoint in ("block", "host", "host_overlap")}
            hit = [k for k, v in clashes.items() if v]
            if hit:
                raise ValueError(f"model.loop.pass2_gate (the gated second pass) is not built together with: {', '.join(hit)}")
            if list(cfg.model.loop.t_choices) != [2]:
                raise ValueError(f"model.loop.t_choices {cfg.model.loop.t_choices!r}: the gated second pass trains at T = 2, [2]; T = 1 before a switch-on is loop_switch_step")
        if cfg.tensor_parallel > 1:
            from ..parallel import tp_model

            if dp is None or cfg.tensor_parallel != dp.world:
                raise ValueError("tensor_parallel must equal the number of ranks (one tensor-parallel group per job)")
            if cfg.optimizer_sharding != "replicated" or cfg.tst.schedule:
                raise ValueError("tensor_parallel runs with optimizer_sharding=replicated and without token superposition")
            model_cfg = tp_model.local_model_config(cfg.model, dp.world)
        mup = None
        if cfg.optim.gdn_mup:      # the gates' start with their learning rate (a resume then loads the trained values over it)
            from .optim import gdn_mup_init_

            def mup(m):
                gdn_mup_init_(m, cfg.optim.gdn_mup_base_width)
        if cfg.tensor_parallel > 1:     # the full model's seeded start, cut to this rank (ranks seeding local models would all hold the same draw)
            self.model = tp_model.init_full_then_shard(cfg.model, model_cfg, dp.rank, dp.world, cfg.seed, mup).to(dtype).to(self.device)
        else:
            self.model = build_model(model_cfg).to(dtype).to(self.device)
            if mup is not None:
                mup(self.model)
        if cfg.tensor_parallel > 1:
            from ..parallel.tensor_parallel import TensorParallel

            tokens = (cfg.micro_batch_size or cfg.data.batch_size) * cfg.data.seq_len
            width = max(cfg.model.d_model, cfg.model.ffn_hidden // dp.world)
            self.tp = TensorParallel(dp, tokens, width)
            tp_model.apply(self.model, self.tp)
        self.model.encoder.activation_checkpoint = cfg.activation_checkpoint
        self.autocast = cfg.autocast == "bfloat16"
        native = self.device.type == "cuda"
        from .. import ops

        self.native = native and ops.mode() == "native"
        lp = torch.bfloat16 if (self.native and self.autocast) else None
        self.sharding = cfg.optimizer_sharding if self.world > 1 else "replicated"
        if cfg.micro_batch_size is not None and dp is not None and self.tp is None:
            dp.check(cfg.data.batch_size, cfg.micro_batch_size)
        # The Copy-Paste head (models/cp_head.py): the loss is the mixture's cross entropy; with freeze_trunk the head alone
        # trains on a finished trunk (train/freeze_trunk.py): every tensor outside cp_head.* takes no gradient and an update of
        # learning-rate scale 0, and its bytes are checked against a digest.
        self._cp = getattr(self.model, "cp_head", None)
        self._trainable = None
        self.trunk_guard = None
        if self._cp is not None:
            clashes = {"tensor_parallel": cfg.tensor_parallel > 1, "cuda_graphs": cfg.cuda_graphs != "none", "tst.schedule": bool(cfg.tst.schedule),
                       "shape_schedule": bool(cfg.shape_schedule), "head_impl 'fused' (the mixture runs on the chunked head: set head_impl 'chunked')": cfg.head_impl == "fused"}
            if cfg.model.cp_head.pointer_input == "shared":     # a recomputed layer returns no key set, and with it no head query and key
                clashes["activation_checkpoint (pointer_input 'shared' reads the shared layer's key set: set it 'none')"] = cfg.activation_checkpoint != "none"
            if cfg.model.cp_head.train_mode == "addon":        # the two clips are one process's
                clashes.update({"data parallelism (train_mode 'addon')": self.world > 1, "freeze_trunk (train_mode 'addon')": bool(cfg.freeze_trunk)})
            hit = [k for k, v in clashes.items() if v]
            if hit:
                raise ValueError(f"model.cp_head is not built together with: {', '.join(hit)}")
        if cfg.freeze_trunk:
            clashes = {"no model.cp_head.enabled (the part that trains)": self._cp is None, "no init_from (a frozen random trunk trains a head on nothing)": not cfg.init_from,
                       "data parallelism": dp is not None, "activation_checkpoint": cfg.activation_checkpoint != "none",
                       "optimizer_sharding": cfg.optimizer_sharding != "replicated", "wgrad_accum 'fp32'": cfg.wgrad_accum == "fp32",
                       "log_zero_wgrad_every": bool(cfg.log_zero_wgrad_every), "model.encoder.gdn_qmix_select_step": bool(cfg.model.encoder.gdn_qmix_select_step)}
            hit = [k for k, v in clashes.items() if v]
            if hit:
                raise ValueError(f"freeze_trunk is not built with: {', '.join(hit)}")
            self._trainable = lambda name: name.startswith("cp_head.")
        self.flat, self.optimizer, self.zero = self._build_optimizer(lp)
        if cfg.freeze_trunk:
            from .freeze_trunk import TrunkGuard

            self.trunk_guard = TrunkGuard(self.model, ("cp_head.",))       # requires_grad False outside the head; digests taken when the trunk is loaded
        self.capacity = self.model.capacity(cfg.data.seq_len) if self.slot_decoder else None
        self.data = make_data(cfg.data, cfg.model.vocab_size, self.capacity)
        self.tst = None
        if cfg.tst.schedule:
            from .tst import TSTPlan

            self.tst = TSTPlan(cfg.tst, self.data, cfg.model.vocab_size, cfg.data.batch_size, cfg.seed)
        if cfg.data.loss_mask != "all" and (cfg.data.kind != "shards" or cfg.tst.schedule or cfg.shape_schedule):
            raise ValueError(f"data.loss_mask {cfg.data.loss_mask!r} reads per-token flags of a shard set: it needs data.kind 'shards' and is "
                             "not built together with tst.schedule or shape_schedule")
        self.shape = None
        if cfg.shape_schedule:       # rows per step and row length by phases of the run's tokens
            from .shape_schedule import ShapeSchedule

            if cfg.tst.schedule or cfg.tensor_parallel > 1 or cfg.cuda_graphs != "none" or cfg.data_prefetch:
                raise ValueError("shape_schedule changes the batch shape between phases: not built together with tst.schedule, "
                                 "tensor_parallel, cuda_graphs or data_prefetch")
            self.shape = ShapeSchedule(cfg.shape_schedule, cfg.steps, cfg.data.batch_size, cfg.data.seq_len, cfg.micro_batch_size, cfg.shape_lr)
            bad = [p.rows for p in self.shape.phases if p.rows % self.world]
            if bad:
                raise ValueError(f"shape_schedule: rows per step {bad} must divide over the {self.world} data-parallel ranks")
        import os

        self._nvtx = os.environ.get("GHB_NVTX", "0") == "1"      # named ranges around the step's phases for a profiler timeline
        self._wandb = None
        self.total_steps = cfg.steps if self.shape is None else self.shape.total_steps      # optimizer steps of the run
        self.step = 0
        self.wandb_run_id = None
        self.init_info = self.resume_info = None
        self._stop = False
        self._saver = ckpt.AsyncSaver() if cfg.ckpt_async else None
        self._last_ckpt_time = time.time()
        self._pinned = None
        self.last_metrics: dict = {}
        self.h2d_bytes = self.d2h_bytes = 0
        if self.run_dir is not None and self.lead:
            self.run_dir.mkdir(parents=True, exist_ok=True)
        if cfg.init_from:
            self.init_from_checkpoint(cfg.init_from)
        if self.native:
            from ..ops import native as _native_ops

            _native_ops.WGRAD_INTO_MAIN = cfg.wgrad_accum == "fp32"
        self.zero_wgrad = None
        if cfg.log_zero_wgrad_every:
            from .zero_wgrad import ZeroWgradMonitor

            self.zero_wgrad = ZeroWgradMonitor(self.model)
        # qmix's static top-2 query mix (models/qmix_select.py): the choice is made at the start of step S from one extra
        # forward of the step's first micro-batch (reference: ced/train/trainer.py:1860-1876, 2420-2455).
        self._qmix = self.model.encoder if cfg.model.encoder.gdn_qmix_select_step else None
        self._qmix_chosen = None
        if self._qmix is not None:
            what = "model.encoder.gdn_qmix_select_step"
            if self.dp is not None or self.tp is not None:
                raise ValueError(f"{what} is not built with data or tensor parallelism: the choice is one process's statistic over its own rows")
            if cfg.activation_checkpoint in ("block", "host", "host_overlap"):
                raise ValueError(f"{what} is not built with activation_checkpoint {cfg.activation_checkpoint!r}: 'none' or 'layer'")
            if cfg.cuda_graphs != "none":
                raise ValueError(f"{what} is not built with cuda_graphs {cfg.cuda_graphs!r}: the choice is a host read and changes the captured forward")
            if cfg.freeze_trunk:
                raise ValueError(f"{what} is not built with freeze_trunk: the choice writes one of the trunk's tensors in a step")
        # The checkpoint cross-read (models/ccr.py): tensor ops on one process; the gates' floor is a clamp after each step.
        from ..models import ccr as ccr_mod

        self._ccr_floor = None
        if ccr_mod.on(cfg.model):
            what = "model.encoder.gdn_ccr_spacing"
            if self.tp is not None:
                raise ValueError(f"{what} is not built with tensor parallelism: a reader's heads read its source's states on the same rank only")
            if cfg.cuda_graphs != "none":
                raise ValueError(f"{what} is not built with cuda_graphs {cfg.cuda_graphs!r}")
            if cfg.activation_checkpoint not in ccr_mod.CHECKPOINT_MODES:
                raise ValueError(f"{what} runs with activation_checkpoint {ccr_mod.CHECKPOINT_MODES}, not {cfg.activation_checkpoint!r}: "
                                 "the record stays on the device and is an input and output of a layer's call")
            if cfg.model.encoder.gdn_ccr_gate_floor:
                if cfg.optim.zero_gate_decay != "none":
                    raise ValueError(f"model.encoder.gdn_ccr_gate_floor {cfg.model.encoder.gdn_ccr_gate_floor!r} is built with optim.zero_gate_decay "
                                     "'none': weight decay would pull a gate at its floor below it before the clamp")
                if self.zero is not None:
                    raise ValueError("model.encoder.gdn_ccr_gate_floor is not built with optimizer sharding: the clamp writes the whole parameter")
                self._ccr_floor = self.model.encoder
        self._readout = None
        readout.check_readout_config(cfg)
        self._probe_readout = readout.Readout(self) if cfg.eval.readout_every else None      # the sample is read (and checked) before the run trains
        self.prefetch = None
        if cfg.data_prefetch:
            from ..data.prefetch import BatchPrefetcher

            self.prefetch = BatchPrefetcher(self.batch_at)
        self.graphs = None
        if cfg.cuda_graphs != "none":
            from .cuda_graphs import GraphRunner

            e = cfg.model.encoder
            tensor_op_arms = [name for on, name in (
                (e.attention.normalizer != "softmax", "attention.normalizer 'asentmax'"), (e.gdn.kda.decay != "scalar", "gdn.kda.decay 'channel'"),
                (e.gdn.erase.mode != "none", "gdn.erase.mode 'eda'"), (e.gdn.dprod.n_h != 1, "gdn.dprod.n_h >= 2"),
                (e.attn_res == "ldm", "attn_res 'ldm'")) if on]
            if tensor_op_arms:      # their rules run as eager tensor ops (recompute inside, chunk loops): not captured
                raise ValueError(f"cuda_graphs {cfg.cuda_graphs!r} is not built with {', '.join(tensor_op_arms)}: these arms run as "
                                 "tensor ops outside the captured step; train them with cuda_graphs 'none'")

            self.graphs = GraphRunner(self)
            if self.zero is not None:      # a captured micro-batch cannot launch per-bucket reductions from its hooks
                self.model.encoder.stage_hooks = None

    # ------------------------------------------------------------------ construction

    def _build_optimizer(self, lp):
        cfg = self.cfg
        zero = None
        if self.sharding in ("zero1", "zero2"):
            from ..parallel.zero import ZeroPlan

            zero = ZeroPlan(self.model, cfg.optim, self.dp, self.sharding)
            flat, opt = zero.build(self.device, lp)
            if self.device.type == "cuda":
                zero.enable_fused()
        else:
            flat, opt = build_optimizer(self.model, cfg.optim, self.device, lp, trainable=self._trainable)
        return flat, opt, zero

    # ------------------------------------------------------------------ data

    def batch_at(self, step: int):
        if self.shape is not None:
            from ..data.synthetic import short_rows

            sh = self.shape.at(step)
            per = sh.rows // self.world
            return short_rows(self.data, sh.first_row + self.rank * per, per, sh.seq_len, self.cfg.data.seq_len)
        B = self.cfg.data.batch_size
        first, count = self.dp.rows(B) if (self.dp is not None and self.tp is None) else (0, B)   # tensor-parallel ranks share the rows
        src_step = step - self.cfg.data_start_step      # a stage on a new shard set starts its stream at its own first update
        if self.tst is not None:
            return self.tst.batch_at(src_step, first, count)
        return self.data.batch(src_step, first, count)

    def lr_at(self, step: int) -> float:
        """The schedule's LR of optimizer step `step`: under a batch-shape schedule read at the step's token clock (and
        divided by the phase's steps per reference step in "rows" mode), so warm-up and decay sit where they are in tokens."""
        if self.shape is None:
            return lr_of(self.cfg, step)
        from .lr import lr_schedule

        sh = self.shape.at(min(step, self.shape.total_steps - 1))
        total = self.cfg.steps if self.cfg.optim.schedule_steps is None else self.cfg.optim.schedule_steps
        return lr_schedule(self.cfg.optim, total, sh.clock) * sh.lr_scale

    def _global_counts(self, batch) -> tuple[int, int]:
        """(valid targets over all ranks, bad-batch flag over all ranks) from one host reduction."""
        bad = 0
        try:
            check_batch(batch, self.cfg.model.vocab_size)
        except BatchError as e:
            bad, self._bad = 1, e
        n = int(_scored(batch).sum()) if batch.multi_valid is None else int(batch.multi_valid.any(-1).sum())
        if self.slot_decoder:       # the two heads' own counts: valid targets at the kept slots, and at the other positions
            from ..models.looped_decoder import select_slots

            kept = select_slots(batch.dec_mask, self.capacity).kept
            heads = [int((batch.target_valid & kept).sum()), int((batch.target_valid & ~kept).sum())]
            if self.dp is not None:
                n, bad, *heads = self.dp.sum_host([n, bad, *heads])
            self._head_counts = heads
            return n, bad
        if self.dp is not None and self.tp is None:
            n, bad = self.dp.sum_host([n, bad])
        return n, bad

    def _two_head_micro(self, mb, n_global):
        """The looped encoder-decoder's micro-batch: (its share of the batch loss, the decoder head's CE sum)."""
        from ..models.looped_decoder import two_head_loss

        cfg = self.cfg
        draft = cfg.model.loop.draft_loss_weight
        with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast and not self.native):
            out = self.model(mb.tokens, mb.doc_ids, mb.dec_mask, T=self.pass_count, capacity=self.capacity, return_hidden=True, return_drafts=draft > 0)
        n_dec, n_aux = (max(c, 1) for c in self._head_counts)
        share = mb.tokens.shape[0] / cfg.data.batch_size           # a routed FFN's balance term counts at the micro-batch's share of the rows
        loss, sums = two_head_loss(self.model, out, mb.targets, mb.target_valid, float(n_global), float(n_dec), float(n_aux), cfg.loss.z_loss,
                                   cfg.loss.aux_weight, cfg.loss.normalization, draft, share)
        for k, v in sums.items():
            self._head_sums[k] = self._head_sums.get(k, 0) + v
        self._head_sums["dropped"] = self._head_sums.get("dropped", 0) + out.n_dropped.sum()
        return loss, sums["ce_dec"] / n_dec

    # ------------------------------------------------------------------ one step

    def _micro_loss(self, mb, n_global):
        """n_global: the number of valid targets over all ranks (int), or a 0-dim device tensor holding its inverse
        (CUDA-graph replay: the normaliser must not be baked into the graph)."""
        cfg = self.cfg
        if self.slot_decoder:
            return self._two_head_micro(mb, n_global)
        inv = n_global if isinstance(n_global, torch.Tensor) else 1.0 / n_global
        z = cfg.loss.z_loss
        s = mb.tokens.shape[2] if mb.tokens.dim() == 3 else 1
        kw = {}
        if s > 1 and cfg.tst.gdn_resolution_gates != "none":
            kw.update(gdn_scale=s, gdn_beta_power=cfg.tst.gdn_resolution_gates == "E")
        if s > 1 and cfg.tst.token_scale_rope:
            kw.update(rope_scale=s)
        if self.looped or self.gated:
            kw.update(T=self.pass_count)
        if self.gated and self.pass_count == 2 and self.model.schedule is not None and self.model.schedule.unscored is not None:
            kw.update(scored=_scored(mb))        # pass counts by segment (models/pass_counts.py): a target that does not count runs pass 1 only
        ac = torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast and not self.native)
        with ac:
            out = self.model(mb.tokens, mb.doc_ids, return_hidden=True, single_doc=mb.single_doc, **kw)
        hidden = out.hidden_aux
        if mb.multi_targets is not None:
            from .tst import bag_weights

            w = bag_weights(s).to(hidden.device)
            targets = mb.multi_targets
            a = mb.multi_valid.to(torch.float32) * w * inv
            b = mb.multi_valid.any(-1).to(torch.float32) * (z * inv)
        else:
            targets = mb.targets
            valid = _scored(mb).to(torch.float32)
            if self.tp is not None:        # the hidden states are this rank's token shard: score the same tokens
                per = targets.numel() // self.tp.world
                cut = slice(self.tp.rank * per, (self.tp.rank + 1) * per)
                targets, valid = targets.reshape(-1)[cut][None], valid.reshape(-1)[cut][None]
            a, b = valid * inv, valid * (z * inv)
        if self._cp is not None and not self._cp.gated:       # the pointer's own loss beside p_LM's (models/cp_head.py, train_mode 'aux')
            from ..models.cp_head import aux_terms, terms

            if mb.multi_targets is not None:
                raise ValueError("model.cp_head is built for one target a position")
            with torch.autocast(self.device.type, enabled=False):
                l_aux, at_sink = aux_terms(terms(self._cp, hidden, mb.tokens, targets, mb.doc_ids, checkpoint=True, pointer=out.cp_pointer))
            aux = (l_aux * valid).sum() * (self._cp.cfg.aux_weight * inv)
            self._cp_aux = ((l_aux.detach() * valid).sum() / valid.sum().clamp_min(1.0), (at_sink.to(valid.dtype) * valid).sum() / valid.sum().clamp_min(1.0))
        elif self._cp is not None and self._cp.cfg.train_mode == "addon":      # the head's own term beside p_LM's loss, nothing of the trunk in its graph
            from ..models.cp_head import addon_loss

            if mb.multi_targets is not None:
                raise ValueError("model.cp_head is built for one target a position")
            aux, ce_mix, lam = addon_loss(self.model, hidden, targets, mb.tokens, mb.doc_ids, valid * inv, cfg.head_chunk, out.cp_pointer)
            self._cp_lambda = (lam * valid).sum() / valid.sum().clamp_min(1.0)
            self._cp_mix = (ce_mix * valid).sum() / valid.sum().clamp_min(1.0)
        elif self._cp is not None:
            from ..models.cp_head import mixture_loss

            if mb.multi_targets is not None:
                raise ValueError("model.cp_head is built for one target a position")
            loss, ce, lam = mixture_loss(self.model, hidden, targets, mb.tokens, mb.doc_ids, a, b, cfg.head_chunk, out.cp_pointer)
            self._cp_lambda = (lam * valid).sum() / valid.sum().clamp_min(1.0)
            return loss, (ce * valid).sum().detach()
        W = self.model.head_weight()
        if cfg.head_impl == "fused":
            loss, ce, _ = fused_linear_ce(hidden, W, targets, a, b, cfg.head_chunk, self.model.head_weight_lp, cfg.loss.ce_form, cfg.head_precision)
            ce_sum = (ce.detach() if mb.multi_targets is not None else ce.detach()).sum()
        else:
            loss, ce_sum = chunked_ce(hidden, W, targets, a, b, ce_form=cfg.loss.ce_form, precision=cfg.head_precision)
            ce_sum = ce_sum.detach()
        if self._cp is not None and (not self._cp.gated or self._cp.cfg.train_mode == "addon"):
            loss = loss + aux.to(loss.dtype)
        return loss, ce_sum

    def device_step(self, batch, n_global: int, lr: float | None = None) -> torch.Tensor:
        """The device part of a step on a batch already on the device: zero gradients, micro-batch loop (forward,
        fused head + loss, backward), gradient synchronisation, clip, update. Returns a device tensor
        (loss, ce sum, gradient norm, kernel status word); nothing is read back to the host here."""
        cfg = self.cfg
        lr = self.lr_at(self.step) if lr is None else lr
        if self.trunk_guard is not None:
            self.trunk_guard.check_loaded()
        if self.zero is not None:
            self.zero.before_step()     # the last step's first-read parameters have landed; peers are done with its gradients
        self.flat.grads.zero_()
        rows = batch.tokens.shape[0]
        micro = cfg.micro_batch_size or rows
        if self.shape is not None:      # the config's TOKENS per forward/backward, whatever the phase's row length
            sh = self.shape.at(self.step)
            per_rank = cfg.micro_batch_size or max(1, cfg.data.batch_size // self.world)
            micro = max(1, min(rows, per_rank * cfg.data.seq_len // sh.seq_len))
            while rows % micro:
                micro -= 1
        if rows % micro and not cfg.micro_batch_by_t:
            raise ValueError(f"micro_batch_size {micro} does not divide this rank's {rows} rows")
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        ce_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        if self.looped and cfg.micro_batch_by_t and self._rows_held is None:
            micro = self.micro_rows(self.pass_count)
        plan = [(lo, self.pass_count) for lo in range(0, rows, micro)] if self._rows_held is None else self.row_plan(self.step)
        for at, (lo, passes) in enumerate(plan):
            if self._rows_held is None:
                mb = batch if micro >= rows else _slice(batch, lo, min(lo + micro, rows))
            else:       # the rows of one pass count: a gather by an index that goes to the device once
                mb, self.pass_count = _rows(batch, torch.tensor(lo, dtype=torch.long).to(self.device, non_blocking=True)), passes
            if self._qmix is not None and at == 0 and self.step >= cfg.model.encoder.gdn_qmix_select_step:
                from ..models import qmix_select

                if qmix_select.pending(self._qmix):      # once: the extra forward is discarded, nothing runs backward
                    self._qmix_chosen = {"step": self.step, **qmix_select.choose(self._qmix, lambda: self._micro_loss(mb, max(n_global, 1)))}
            if self.graphs is not None:
                loss, ce = self.graphs.micro(mb, n_global)
                loss_sum += loss
            else:
                with monitor.nvtx_range("forward", self._nvtx):
                    loss, ce = self._micro_loss(mb, max(n_global, 1))
                if self.zero is not None:       # gradients are final after the last micro-batch: its finished buckets may leave
                    self.zero.armed = at == len(plan) - 1
                with monitor.nvtx_range("backward", self._nvtx):
                    loss.backward()
                loss_sum += loss.detach().float()
            ce_sum += ce.float()
        stats = torch.stack([loss_sum, ce_sum]).double()
        nvtx_sync = monitor.nvtx_range("grad_sync+optimizer", self._nvtx)
        nvtx_sync.__enter__()
        if self.zero is not None:
            gnorm = self.zero.sync_and_step(self.optimizer, lr, cfg.optim.grad_clip, stats)
        elif self.tp is not None:
            from ..parallel import tp_model

            self.tp.all_reduce_grads(tp_model.replicated_parameters(self.model))
            self.dp.all_reduce_(stats)
            sq = torch.stack([sum((p.grad.float() ** 2).sum() for p in self.model.parameters() if p.grad is not None and getattr(p, "tp_sharded", False)),
                              sum((p.grad.float() ** 2).sum() for p in self.model.parameters() if p.grad is not None and not getattr(p, "tp_sharded", False))])
            part = sq[0:1].clone()
            self.dp.all_reduce_(part)
            gnorm = (part[0] + sq[1]).sqrt()
            self.optimizer.step(lr, _clip_coef(gnorm, cfg.optim.grad_clip))
        else:
            if self.dp is not None:
                self.dp.all_reduce_(self.flat.grads)
                self.dp.all_reduce_(stats)
            if self.trunk_guard is not None and (self.step == 0 or (cfg.log_every and self.step % cfg.log_every == 0)):
                self.trunk_guard.check_grads()
            if cfg.log_every and self.step % cfg.log_every == 0:      # per-family gradient norms before clipping (whole gradients are here)
                self._family_norms = monitor.family_grad_norms(self.flat)
            gnorm = grad_norm(self.flat)
            if self._cp is not None and self._cp.cfg.train_mode == "addon":
                # two clips: the trunk and the LM head by their own norm (the model's without the head), the head by its own; the
                # optimizer applies the trunk's factor to everything, so the head's gradients are scaled to theirs first
                own = [p.grad for n, p in self.model.named_parameters() if n.startswith("cp_head.") and p.grad is not None]
                head_norm = torch.stack([g.double().pow(2).sum() for g in own]).sum().sqrt().float()
                gnorm = (gnorm.double().pow(2) - head_norm.double().pow(2)).clamp_min(0).sqrt().float()
                ratio = _clip_coef(head_norm, cfg.optim.grad_clip) / _clip_coef(gnorm, cfg.optim.grad_clip)
                for g in own:
                    g.mul_(ratio.to(g.dtype) if isinstance(ratio, torch.Tensor) else ratio)
                self._cp_grad_norm = head_norm
            self.optimizer.step(lr, _clip_coef(gnorm, cfg.optim.grad_clip))
        if not cfg.freeze_trunk and self.model.encoder.scalar_form != "none":
            if self.zero is not None:
                self.zero.settle()
            self.model.encoder.project_layer_scalars()      # the span-bounded residual scalars back into their range
        if self._ccr_floor is not None and not cfg.freeze_trunk:
            from ..models.ccr import floor_gates_

            floor_gates_(self._ccr_floor)                   # the cross-read gates back to at least their floor
            self.flat.refresh_lp()
        nvtx_sync.__exit__(None, None, None)
        self.step += 1
        from .. import ops

        status = ops.status_word(self.device).to(torch.float32).reshape(())      # kernels' bounded waits report here (0 = clean)
        out = torch.stack([stats[0].float(), stats[1].float(), gnorm.float(), status])
        fam, self._family_norms = getattr(self, "_family_norms", None), None
        return out if fam is None else torch.cat([out, fam.float()])

    def micro_rows(self, passes: int) -> int:
        """Rows per forward / backward at a pass count: micro_batch_by_t's entry (its last beyond the list), else micro_batch_size."""
        by_t = self.cfg.micro_batch_by_t
        return by_t[min(passes, len(by_t)) - 1] if by_t else (self.cfg.micro_batch_size or self.cfg.data.batch_size)

    def row_passes(self, step: int):
        """The pass count of every row of the step's batch (t_sampling 'sequence'; None otherwise): a function of (seed, step)."""
        from ..models.recur import row_pass_counts

        return None if self._rows_held is None else row_pass_counts(self._rows_held, self.cfg.seed, step)

    def row_plan(self, step: int) -> list:
        from ..models.recur import micro_plan

        return micro_plan(self.row_passes(step), self.micro_rows)

    def train_step(self) -> dict:
        """One full training step through the public path: build this rank's batch (a pure function of the step),
        copy it from pinned host memory to the device, run `device_step`, read (loss, ce, grad norm) back."""
        cfg = self.cfg
        t0 = time.perf_counter()
        step = self.step
        tst_event = self.tst.switch(self, step) if self.tst is not None else None     # a later phase's first step starts with the switch
        if self.prefetch is not None:          # the batch was built by the background thread while the last step ran
            batch = self.prefetch.get(step).batch
            self.prefetch.start(step + 1)
        else:
            batch = self.batch_at(step)
        n_global, bad = self._global_counts(batch)
        if bad:
            self._halt_bad_batch(step)
        if self.looped or self.slot_decoder:
            from ..models.recur import pass_count_for_step

            self.pass_count = pass_count_for_step(cfg.model.loop, cfg.seed, step)
            self._head_sums = {}
        if self.gated:
            self.pass_count = 1 if step < cfg.loop_switch_step else 2
        lr = self.lr_at(step)
        if self.tst is not None:
            factor = self.tst.lr_factor(step)
            if factor is not None:
                lr = lr * factor
        if self.device.type == "cuda":
            batch = batch.pin()
        self.h2d_bytes = batch.h2d_bytes()
        dev_batch = batch.to(self.device)
        host = self.device_step(dev_batch, n_global, lr).cpu()      # the step's one device->host read
        self.d2h_bytes = host.numel() * host.element_size()
        loss_v, ce_v, gn_v, status = (float(x) for x in host[:4])
        self._check_kernel_status(int(status), step)
        seconds = time.perf_counter() - t0
        s = batch.tokens.shape[2] if batch.tokens.dim() == 3 else 1
        n_tokens = cfg.data.batch_size * cfg.data.seq_len * s
        if self.shape is not None:
            n_tokens = self.shape.at(step).rows * self.shape.at(step).seq_len
        m = {"step": step, "loss": loss_v, "ce_dec": ce_v, "lr": lr, "grad_norm": gn_v, "n_targets": n_global,
             "step_seconds": seconds, "tokens_per_s": n_tokens / seconds}
        if self.device.type == "cuda":
            m["peak_alloc_gib"] = torch.cuda.max_memory_allocated(self.device) / 2 ** 30
        if self._cp is not None and not self._cp.gated:
            m["cp_aux"], m["cp_aux_sink"] = (float(x) for x in self._cp_aux)      # the step's last micro-batch: the mean auxiliary CE, the share of targets at the sink
        if self._cp is not None and self._cp.cfg.train_mode == "addon":
            m["ce_mix"], m["cp_grad_norm"] = float(self._cp_mix), float(self._cp_grad_norm)      # grad_norm above is the trunk's and the LM head's
        if self._cp is not None and self._cp.gated and cfg.log_every and step % cfg.log_every == 0:
            m["cp_lambda"] = float(self._cp_lambda)          # the mean copy weight at the scored targets of the step's last micro-batch
            if self._cp.cfg.qk_norm:
                gains = (1.0 + self._cp.qk_gain.detach().float()).tolist()          # one a pointer head
                m["cp_qk_gain"] = gains[0] if len(gains) == 1 else gains
        if self.gated:
            m["T"] = self.pass_count
            if cfg.log_every and step % cfg.log_every == 0:
                m["pass2_alpha"] = float(self.model.alpha())
                if self.pass_count == 2 and getattr(self.model, "last_loop_usage", None) is not None:
                    m["loop_usage"] = float(self.model.last_loop_usage)
                if self.pass_count == 2 and self.model.schedule is not None:      # the share of positions at each pass count in the step's last micro-batch
                    c = self.model.last_counts
                    m["pass_counts"] = {str(k): float((c == k).float().mean()) for k in range(1, self.model.n_passes + 1)}
        if self.slot_decoder:       # the heads' mean CE over their own counts (one more host read of a few scalars)
            m["T"] = self.pass_count
            n_dec, n_aux = (max(c, 1) for c in self._head_counts)
            for k, v in self._head_sums.items():
                m[k] = float(v) / (n_aux if k == "ce_aux" else 1 if k in ("moe_balance", "dropped") else n_dec)
        if self.looped:
            m["T"] = self.pass_count
            if self._rows_held is not None:
                m["T_rows"] = self.row_passes(step)
                m["T"] = sum(m["T_rows"]) / len(m["T_rows"])
            inj = self.model.encoder.recur_injection
            if inj is not None and cfg.log_every and step % cfg.log_every == 0:
                m["recur_injection"] = inj.summary()
            if self.model.encoder.recur_mix is not None:
                m["recur_mix"] = float(self.model.encoder.recur_mix.detach())
        if tst_event is not None:
            m["tst_switch"] = tst_event
        if host.numel() > 4:        # a logging step: gradient norm per parameter family, the depth-mix readers' state
            m.update({f"grad_norm/{n}": float(v) for n, v in zip(monitor.family_names(), host[4:])})
            readers = monitor.depth_reader_summary(self.model)
            if readers:
                m["depth_readers"] = readers
            cross = monitor.ccr_summary(self.model)
            if cross:
                m["ccr"] = cross
        if cfg.log_stream_rms_every and self.step % cfg.log_stream_rms_every == 0:
            if self._qmix is not None:
                self._qmix.qmix_record = {}
            try:
                with torch.no_grad(), monitor.StreamRMS(self.model) as rms:
                    probe = _slice(dev_batch, 0, 1)
                    self.model(probe.tokens, probe.doc_ids, return_hidden=True, single_doc=probe.single_doc)
            finally:
                if self._qmix is not None:
                    record, self._qmix.qmix_record = self._qmix.qmix_record, None
            m["stream_rms"] = rms.values()
            if self._qmix is not None:      # each query mix's token-mean weights as the layer uses them now, on the probe row
                from ..models import qmix_select

                m["qmix_weights"] = qmix_select.weights_metrics(self._qmix, record)
        if self._qmix_chosen is not None:
            m["qmix_selection"], self._qmix_chosen = self._qmix_chosen, None
        if self.zero_wgrad is not None and self.step % cfg.log_zero_wgrad_every == 0:
            m.update(self.zero_wgrad.summary())
        self.last_metrics = m
        if not math.isfinite(loss_v):
            self._halt_diverged(m)
        if self.dp is not None and self.dp.check_every and self.step % self.dp.check_every == 0:
            if self.zero is not None:
                self.zero.gather_master()
            self.dp.check_replicas(list(self.model.named_parameters()))
        return m

    # ------------------------------------------------------------------ loop

    def fit(self, until_step: int | None = None) -> None:
        cfg = self.cfg
        if self.run_dir is not None and (self.run_dir / "diverged.json").exists():
            raise Diverged(f"{self.run_dir} is marked diverged: start a new run directory")
        end = self.total_steps if until_step is None else min(self.total_steps, until_step)
        old = None
        try:
            old = signal.signal(signal.SIGTERM, self._request_stop)
        except ValueError:  # not the main thread
            pass
        self._jsonl({"event": "start", "step": self.step, "world": self.world, "device": str(self.device),
                     "params": sum(p.numel() for p in self.model.parameters())})
        if self.lead and cfg.wandb.mode != "disabled":
            self._wandb = monitor.WandbLogger(cfg.wandb, self.wandb_run_id, C.to_dict(cfg), directory=self.run_dir)
            self.wandb_run_id = self._wandb.run_id
        try:
            while self.step < end:
                m = self.train_step()
                if self.lead:
                    if "tst_switch" in m:
                        self._jsonl({"event": "tst_switch", **m["tst_switch"]})
                    self._jsonl(m)
                    if cfg.log_every and (m["step"] % cfg.log_every == 0 or self.step == end):
                        print(f"step {m['step']:6d} loss {m['loss']:.4f} lr {m['lr']:.2e} gnorm {m['grad_norm']:.3f} "
                              f"{m['tokens_per_s']:.0f} tok/s", flush=True)
                if bpb_readout.due(cfg, self.step):
                    if self._readout is None:
                        self._readout = bpb_readout.BpbReadout(self)
                    scores = self._readout.run()
                    if self.lead and scores:
                        self._jsonl({"event": "bpb_readout", "step": self.step, **scores})
                if self._probe_readout is not None and readout.readout_due(cfg, self.step, end):
                    record = self._probe_readout.run(self)
                    if record is not None:
                        self._jsonl(record)
                if periodic_eval.due(cfg, self.step):
                    scores = periodic_eval.run_eval_sets(self)
                    if self.lead:
                        self._jsonl({"event": "eval", "step": self.step, **{f"eval/{k}/bpb": v["bpb"] for k, v in scores.items()}})
                due = self._ckpt_due(end)
                stop = self._stop
                if self.dp is not None:
                    stop, due = self.dp.agree(stop, due)
                if self._saver is not None:
                    self._saver.commit()
                if due or stop:
                    self.save_checkpoint(sync=stop or self.step == end)
                if self._wandb is not None:      # after the save: logging can never hold up a checkpoint
                    self._wandb.log(m, self.step)
                if stop:
                    break
        finally:
            if self._wandb is not None:
                self._wandb.finish()
                self._wandb = None
            if self._saver is not None:
                self._saver.commit(block=True)
            if old is not None:
                signal.signal(signal.SIGTERM, old)

    def _request_stop(self, *_):
        self._stop = True

    def _ckpt_due(self, end: int) -> bool:
        cfg = self.cfg
        if self.run_dir is None:
            return False
        if self.step == end or self.step in cfg.checkpoint_steps:
            return True
        if cfg.ckpt_every_steps and self.step % cfg.ckpt_every_steps == 0:
            return True
        if cfg.ckpt_every_minutes and time.time() - self._last_ckpt_time > 60.0 * cfg.ckpt_every_minutes:
            return True
        return False

    # ------------------------------------------------------------------ failure paths

    def _halt_diverged(self, m: dict):
        if self.run_dir is not None and self.lead:
            (self.run_dir / "diverged.json").write_text(json.dumps({"step": m["step"], "loss": str(m["loss"])}))
            self._jsonl({"event": "diverged", **{k: (str(v) if isinstance(v, float) and not math.isfinite(v) else v) for k, v in m.items()}})
        raise Diverged(f"non-finite loss at step {m['step']}")

    def _check_kernel_status(self, code: int, step: int) -> None:
        """A kernel whose bounded wait gave up (a late or lost rank, a protocol error) returns early and leaves partial
        output behind, so the step that read it is void: every rank learns of any rank's code (MAX over the host group)
        and all raise together, before metrics, checkpoints or another step."""
        if self.dp is not None:
            code = int(self.dp.max_host([code])[0])
        if code:
            from .. import ops

            ops.clear_status(self.device)
            if self.run_dir is not None and self.lead:
                self._jsonl({"event": "kernel_status", "step": step, "code": code})
            raise KernelStatus(f"step {step}: a kernel reported status {code} (a bounded wait gave up); the step's update is not trustworthy "
                               "and no checkpoint is written")

    def _halt_bad_batch(self, step: int):
        info = {"rank": self.rank, "error": str(getattr(self, "_bad", "")), "rows": getattr(getattr(self, "_bad", None), "rows", [])}
        infos = self.dp.gather_host(info) if self.dp is not None else [info]
        if self.run_dir is not None and self.lead:
            self._jsonl({"event": "bad_batch", "step": step, "ranks": [i for i in infos if i["error"]]})
        raise BatchError(f"bad batch at step {step}: {[i for i in infos if i['error']]}")

    def _jsonl(self, record: dict) -> None:
        if self.run_dir is None or not self.lead or not self.cfg.metrics_jsonl:
            return
        with open(self.run_dir / "metrics.jsonl", "a") as f:
            f.write(json.dumps(record) + "\n")

    # ------------------------------------------------------------------ checkpoints

    def data_state(self) -> dict:
        d = self.cfg.data
        state = {"kind": d.kind, "seed": d.seed, "seq_len": d.seq_len, "batch_size": d.batch_size}
        if d.kind == "shards":
            state["fingerprint"] = self.data.fingerprint()
            if d.loss_mask != "all":      # the mask and the identity of the span / flag files it read: a resume on others is refused
                state["loss_mask"] = d.loss_mask
                state["loss_spans"] = self.data.loss_spans_state
        if self.cfg.data_start_step:
            state["data_start_step"] = self.cfg.data_start_step
        if self.tst is not None:
            state.update(self.tst.data_state())
        return state

    def state_dict(self) -> dict:
        if self.zero is not None:
            self.zero.gather_master()      # fp32 masters that live on their owners only, to every rank (collective)
        model_state = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        optim_state = self.optimizer.state_dict() if self.zero is None else self.zero.optimizer_state(self.optimizer)
        if self.tp is not None:     # the checkpoint holds the FULL model and its moments: every rank's slices meet on the lead
            from ..parallel import tp_model

            cpu = lambda d: {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
            opt_cpu = {**optim_state, "state": {i: cpu(st) for i, st in optim_state["state"].items()}}
            parts = self.dp.gather_to_lead((cpu(model_state), opt_cpu))
            if self.lead:
                model_state = tp_model.merge_state_dicts([m for m, _ in parts], self.cfg.model)
                optim_state = tp_model.merge_optimizer_states([o for _, o in parts], self.cfg.model)
        state = {
            "step": self.step, "config": C.to_dict(self.cfg),
            "model": model_state,
            "optimizer": optim_state,
            "torch_rng": torch.get_rng_state(),
            "cuda_rng": torch.cuda.get_rng_state_all() if self.device.type == "cuda" and self.dp is None else None,
            "python_rng": random.getstate(), "wandb_run_id": self.wandb_run_id, "data_state": self.data_state(),
            "init_from": self.init_info, "resumed_from": self.resume_info,
        }
        if self.dp is not None:
            state["data_parallel"] = {"world_size": self.world, "sharding": self.sharding}
        if self.trunk_guard is not None:        # a checkpoint whose trunk is not the start's is not written
            self.trunk_guard.check_values()
            state["freeze_trunk"] = {"trunk_sha256": self.trunk_guard.summary(), "tensors": len(self.trunk_guard.frozen)}
        return state

    def save_checkpoint(self, sync: bool = True) -> Path | None:
        if self.run_dir is None:
            return None
        path = ckpt.step_path(self.run_dir, self.step)
        state = self.state_dict()   # collective under ZeRO: every rank takes part
        if self.lead:
            if self._saver is not None and not sync:
                self._saver.start(state, path, self.cfg.ckpt_keep, self.cfg.checkpoint_steps)
            else:
                if self._saver is not None:
                    self._saver.commit(block=True)
                ckpt.write_atomic(state, path)
                ckpt.point_latest(path, self.cfg.ckpt_keep, self.cfg.checkpoint_steps)
        if self.dp is not None:
            self.dp.barrier()
        self._last_ckpt_time = time.time()
        return path

    def load_state_dict(self, state: dict, check_config: bool = True, weights_only: bool = False) -> None:
        if check_config:
            saved = C.checkpoint_config(state["config"])
            diff = C.config_differences(C.to_dict(C.from_dict(C.TrainConfig, saved)), C.to_dict(self.cfg))
            if diff:
                raise ValueError(f"the checkpoint was written by a run with a different config: {diff}")
        if self.tp is not None:     # checkpoints hold the full model: keep this rank's slices
            from ..parallel import tp_model

            state = {**state, "model": tp_model.shard_state_dict(state["model"], self.cfg.model, self.rank, self.world)}
            if not weights_only:
                state["optimizer"] = tp_model.shard_optimizer_state(state["optimizer"], self.cfg.model, self.rank, self.world)
        with torch.no_grad():
            own = self.model.state_dict()
            missing = [k for k in own if k not in state["model"]]
            if missing and not weights_only:
                raise KeyError(f"checkpoint lacks parameters {missing[:6]}")
            for k, v in state["model"].items():
                if k in own:
                    own[k].copy_(v)
        if self.cfg.model.encoder.gdn_qmix_select_step:     # the layers' form follows the loaded buffers
            from ..models import qmix_select

            qmix_select.sync_static(self.model.encoder)
        self.flat.refresh_lp()
        if weights_only:
            return
        if self.trunk_guard is not None:        # a resume: the file's trunk must hash to its record
            self.trunk_guard.take_digests()
            want = (state.get("freeze_trunk") or {}).get("trunk_sha256")
            if want != self.trunk_guard.summary():
                raise ValueError("freeze_trunk: the checkpoint's trunk does not hash to its record (the file was changed after the save, or was not written by a frozen-trunk run)")
        if self.zero is not None:
            self.zero.load_optimizer_state(self.optimizer, state["optimizer"])
        else:
            self.optimizer.load_state_dict(state["optimizer"])
        self.step = int(state["step"])
        torch.set_rng_state(state["torch_rng"])
        random.setstate(state["python_rng"])
        if state.get("cuda_rng") is not None and self.device.type == "cuda" and self.dp is None:
            torch.cuda.set_rng_state_all(state["cuda_rng"])
        self.wandb_run_id = state.get("wandb_run_id")
        if state.get("data_state") and state["data_state"] != self.data_state():
            raise ValueError(f"the checkpoint's data stream {state['data_state']} is not this run's {self.data_state()}")

    def resume_from_checkpoint(self, path: str | Path | None = None) -> bool:
        """Resume from `path`, or from the run directory's latest checkpoint; False when there is none."""
        p = Path(path) if path is not None else (ckpt.latest_path(self.run_dir) if self.run_dir is not None else None)
        if p is None:
            return False
        self.load_state_dict(ckpt.load(p))
        self.resume_info = {"path": str(p), "step": self.step}
        return True

    # What a run that CONTINUES another run's checkpoint (`resume_from`) may differ in from its source, besides the fields
    # that select an implementation: its own length and bookkeeping; under `stage: continue` also the decay's share, the
    # shard set and where the data stream starts; under `precision_switch` also the low-precision recipes
    # (reference: ced/config.py:2160-2215, ced/train/trainer.py:905-1076).
    BRANCH_FREE = ("steps", "checkpoint_steps", "resume_from", "eval", "wandb")
    STAGE_FREE = ("optim.decay_fraction", "data.shard_dir", "data.extra_shard_dirs", "data.loss_mask", "stage", "data_start_step")
    PRECISION_FREE = ("model.nvfp4", "model.fp8", "precision_switch")

    def continue_from(self, path: str | Path) -> None:
        """Start this NEW run from another run's checkpoint: its whole training state (weights, optimizer state, step
        counter, RNG states). Strict: the source's config must be this one apart from the fields above, its data this
        run's (unless the stage brings a new shard set), and the two LR schedules must agree on every update the source
        has made, so that the run is the run this config would have trained from its own start."""
        cfg = self.cfg
        if cfg.stage not in ("none", "continue"):
            raise ValueError(f"stage {cfg.stage!r}: 'none' or 'continue'")
        if cfg.precision_switch and cfg.stage != "continue":
            raise ValueError("precision_switch is read with stage 'continue'")
        if cfg.data_start_step and cfg.stage != "continue":
            raise ValueError("data_start_step is read with stage 'continue'")
        state = ckpt.load(Path(path))
        src = C.from_dict(C.TrainConfig, C.checkpoint_config(state["config"]))
        free = self.BRANCH_FREE + (self.STAGE_FREE if cfg.stage == "continue" else ()) + (self.PRECISION_FREE if cfg.precision_switch else ())
        diff = [d for d in C.config_differences(C.to_dict(src), C.to_dict(cfg)) if not any(d == f or d.startswith(f + ".") for f in free)]
        if diff:
            raise ValueError(f"resume_from: the source run's config differs from this one in {diff}"
                             + ("" if cfg.stage == "continue" else " (stage 'continue' frees the decay share, the shard set and data_start_step)"))
        S = int(state["step"])
        from .lr import lr_of as lr_fn

        moved = [k for k in range(S) if lr_fn(src, k) != lr_fn(cfg, k)]
        if moved:
            raise ValueError(f"resume_from: the source trained update {moved[0]} at LR {lr_fn(src, moved[0])}, this config's schedule gives "
                             f"{lr_fn(cfg, moved[0])}: the schedules must agree on every update the source has made")
        new_data = cfg.stage == "continue" and (src.data.shard_dir != cfg.data.shard_dir or src.data.extra_shard_dirs != cfg.data.extra_shard_dirs)
        if new_data and cfg.data_start_step != S:
            raise ValueError(f"stage 'continue' on a new shard set starts its stream at this run's first update: data_start_step must be {S}")
        if not new_data and cfg.data_start_step not in (0, src.data_start_step):
            raise ValueError("data_start_step: 0 (or the source's own) when the shard set is the source's: the stream goes on where the source is")
        if new_data or cfg.precision_switch:
            state = {**state, "data_state": None}
        self.load_state_dict(state, check_config=False)
        self.resume_info = {"path": str(path), "step": self.step, "stage": cfg.stage,
                            "precision": [C.to_dict(src.model.fp8)["mode"] + "/" + C.to_dict(src.model.nvfp4)["mode"],
                                          C.to_dict(cfg.model.fp8)["mode"] + "/" + C.to_dict(cfg.model.nvfp4)["mode"]]}

    def init_from_checkpoint(self, path: str | Path) -> None:
        """Weights only, from another run; parameters the file lacks keep their initial values."""
        state = ckpt.load(Path(path))
        self.load_state_dict(state, check_config=False, weights_only=True)
        self.init_info = {"path": str(path), "step": int(state.get("step", 0))}
        own = set(self.model.state_dict())
        self.init_info["grown"] = sorted(own - set(state["model"]))          # tensors the source lacks keep their own start (a head added to a finished trunk)
        if getattr(self, "trunk_guard", None) is not None:
            self.trunk_guard.take_digests()
            self.init_info["trunk_sha256"] = self.trunk_guard.summary()


def _scored(batch) -> torch.Tensor:
    """The targets that count in the loss: inside their document and, under a per-token loss mask, kept by it."""
    return batch.target_valid if batch.loss_mask is None else batch.target_valid & batch.loss_mask


def _slice(batch, lo: int, hi: int):
    from ..data.synthetic import Batch

    def cut(t):
        return t[lo:hi] if isinstance(t, torch.Tensor) else t
    return Batch(tokens=cut(batch.tokens), targets=cut(batch.targets), target_valid=cut(batch.target_valid),
                 doc_ids=cut(batch.doc_ids), dec_mask=cut(batch.dec_mask), multi_targets=cut(batch.multi_targets),
                 multi_valid=cut(batch.multi_valid), loss_mask=cut(batch.loss_mask), single_doc=batch.single_doc)


def _rows(batch, index: torch.Tensor):
    """The batch's rows `index` (a device LongTensor, ascending), gathered."""
    from ..data.synthetic import Batch

    def take(t):
        return t.index_select(0, index) if isinstance(t, torch.Tensor) else t
    return Batch(tokens=take(batch.tokens), targets=take(batch.targets), target_valid=take(batch.target_valid),
                 doc_ids=take(batch.doc_ids), dec_mask=take(batch.dec_mask), multi_targets=take(batch.multi_targets),
                 multi_valid=take(batch.multi_valid), loss_mask=take(batch.loss_mask), single_doc=batch.single_doc)


def _clip_coef(norm: torch.Tensor, max_norm: float):
    """min(1, max_norm / (norm + 1e-6)) as a 0-dim tensor (no host sync); 1.0 when clipping is off."""
    if not max_norm or max_norm <= 0:
        return 1.0
    return torch.clamp(max_norm / (norm + 1e-6), max=1.0)
