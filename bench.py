#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the 200M full hybrid (bf16, AdamW, seq 4096, 16 rows per GPU, synthetic
uniform token ids, random-init weights) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by torchrun (one rank per GPU, NCCL); this file reads RANK / LOCAL_RANK / WORLD_SIZE. Rank 0 prints
ONE JSON line. `value` is device-timed (CUDA events around K steps whose inputs are already on the device, max over
ranks); `e2e.value` times K calls of the public `Trainer.train_step()` — batch construction, the pinned host->device
copy of the step's inputs and the device->host read of the step's loss included. `--impl reference` runs the
unmodified reference package installed under baseline/_ref through its own Trainer on the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = "200m-full-hybrid"
SEQ_LEN = 4096
ROWS_PER_GPU = 16
VOCAB = 32768


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="200m", help="model size preset (the headline is 200m)")
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--rows", type=int, default=ROWS_PER_GPU, help="rows per GPU per step")
    ap.add_argument("--sharding", default="auto", help="replicated | zero1 | zero2 | auto (zero2 when N > 1)")
    ap.add_argument("--comm", default="auto", help="fused | nccl | auto")
    ap.add_argument("--graphs", action="store_true", help="replay the micro-batch as a CUDA graph after warm-up")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "tp"],
                    help="tp: tensor parallel over all ranks with a sequence-parallel stream (--rows is then the whole job's rows per step)")
    ap.add_argument("--tp-impl", default="fused", choices=["fused", "collective"], help="tp: fused peer-memory GEMMs or NCCL collectives around plain GEMMs")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "mxfp8", "nvfp4"],
                    help="GEMM precision of the layers' projections: bf16 (the headline), block-scaled MXFP8 on the tensor cores, or the NVFP4 recipe")
    ap.add_argument("--mode", default="train", choices=["train", "decode"], help="decode: static-cache greedy decode tokens/s")
    ap.add_argument("--kv", default="gqa", choices=["gqa", "grid"], help="decode: KV sharing of the attention layers")
    ap.add_argument("--prompt", type=int, default=32768, help="decode: prompt length")
    ap.add_argument("--batch", type=int, default=64, help="decode: rows per GPU")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi samples of SM clocks and throttle reasons while the timed region runs (rank 0 only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, enabled: bool):
        self.proc, self.path = None, None
        if not enabled:
            return
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, n_gpus: int) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) >= n_gpus:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def max_over_ranks(value: float, dp) -> float:
    return value if dp is None else dp.max_over_ranks(value)


def baseline_number():
    try:
        pub = json.loads((ROOT / "BASELINE.json").read_text()).get("published") or {}
        return pub.get("train_tokens_per_s")
    except Exception:
        return None


# ---------------------------------------------------------------------------------------------------------- ours

def run_ours(args) -> dict:
    import torch

    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    dp = data_parallel.from_environment()
    world = 1 if dp is None else dp.world
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torchrun --nproc-per-node {args.gpus}")
    cfg = C.TrainConfig(model=C.hybrid_model_config(args.size, full=True))
    if args.precision == "mxfp8":
        cfg.model.fp8.mode, cfg.model.fp8.scaling = "linears", "mxfp8"
    elif args.precision == "nvfp4":
        cfg.model.nvfp4.mode = "all_linears"
    tp = args.parallelism == "tp" and world > 1
    job_rows = args.rows if tp else args.rows * world
    cfg.data = C.DataConfig(kind="uniform", seq_len=args.seq_len, batch_size=job_rows, seed=1)
    cfg.micro_batch_size = args.rows
    if tp:
        cfg.tensor_parallel = world
        os.environ["GHB_TP_IMPL"] = args.tp_impl
    cfg.steps, cfg.seed, cfg.dtype, cfg.autocast, cfg.head_impl = 10 ** 6, 1, "float32", "bfloat16", "fused"
    cfg.head_chunk = 4096      # positions per chunk of logits: fills the SMs in the head's input-gradient GEMM (2048: 64 tiles)
    cfg.optim.name, cfg.optim.warmup_steps = "adamw", 100
    cfg.metrics_jsonl, cfg.log_every, cfg.ckpt_every_steps, cfg.ckpt_every_minutes = False, 0, 0, 0.0
    cfg.optimizer_sharding = ("zero2" if world > 1 and not tp else "replicated") if args.sharding == "auto" else args.sharding
    if args.comm != "auto":
        os.environ["GHB_COMM"] = args.comm
    if args.graphs:
        cfg.cuda_graphs = "microbatch"
    trainer = Trainer(cfg, None, dp)
    dev = trainer.device
    for _ in range(args.warmup):
        trainer.train_step()
    # ---- device-timed region: inputs resident on the device, no host read inside
    batches = [trainer.batch_at(trainer.step + i).pin().to(dev) for i in range(args.steps)]
    counts = [trainer._global_counts(trainer.batch_at(trainer.step + i))[0] for i in range(args.steps)]
    torch.cuda.synchronize()
    if dp is not None:
        dp.barrier()
    sampler = ClockSampler(dp is None or dp.lead)
    ops.reset_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for b, n in zip(batches, counts):
        trainer.device_step(b, n)
    end.record()
    torch.cuda.synchronize()
    launches = ops.launch_count()
    if dp is not None:
        dp.barrier()
    dev_ms = max_over_ranks(start.elapsed_time(end), dp) / args.steps
    # ---- end-to-end region: the public train_step (batch build, pinned H2D, D2H loss read) every step
    torch.cuda.synchronize()
    if dp is not None:
        dp.barrier()
    start.record()
    for _ in range(args.steps):
        m = trainer.train_step()
    end.record()
    torch.cuda.synchronize()
    if dp is not None:
        dp.barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(end), dp) / args.steps
    clocks = sampler.stop(world)
    ops.check_status()          # a bounded wait that gave up inside a kernel voids the run
    tokens = job_rows * args.seq_len
    base = baseline_number()
    zero = trainer.zero
    value = tokens / (dev_ms / 1e3)
    out = {
        "metric": "train tokens/s/box, 200M hybrid", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong" if tp else "weak",
        "vs_baseline": (value / base) if base and not tp else None, "dtype": args.precision, "data": "synthetic",
        "config": {"model": MODEL if args.size == "200m" else args.size, "global_batch": job_rows,
                   "seq_len": args.seq_len,
                   "parallelism": (f"tp{world}-sp-{args.tp_impl}" if tp else f"dp{world}" + ("" if world == 1 else f"-{cfg.optimizer_sharding}")),
                   "optimizer": "adamw", "vocab": VOCAB, "l2": "per-step working set (GBs of activations) >> 126 MB L2",
                   "comm": os.environ.get("GHB_COMM", "auto"), "fused": bool(zero is not None and zero.fused is not None),
                   "multimem": bool(zero is not None and zero.fused is not None and zero.fused.multimem),
                   "cuda_graphs": cfg.cuda_graphs, "loss": m["loss"],
                   **({"tp_gather": getattr(trainer.tp, "gather_by", None), "tp_scatter": getattr(trainer.tp, "scatter", None),
                       "tp_multimem": bool(getattr(trainer.tp, "multimem", False))} if tp and trainer.tp is not None else {})},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": trainer.h2d_bytes, "d2h_bytes_per_step": trainer.d2h_bytes},
        "gpu_launches": launches, "impl": "ours",
    }
    if dp is not None:
        dp.close()
    return out


# ---------------------------------------------------------------------------------------------------------- decode

def run_decode(args) -> dict:
    """Greedy decode with the CUDA-graph static-cache engine: `batch` rows per GPU (data-parallel replicas), a
    `prompt`-token uniform random prompt, `steps` timed generated tokens per row after `warmup` untimed ones."""
    import torch

    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.infer.engine import DecodeEngine
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.ops import native
    from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel
    from gdn_hybrid_architecture_ideas_b200.train.optim import build_optimizer

    dp = data_parallel.from_environment()
    world = 1 if dp is None else dp.world
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    torch.manual_seed(1)
    cfg = C.hybrid_model_config(args.size, full=True, kv=args.kv)
    model = build_model(cfg).to(dev)
    flat, _ = build_optimizer(model, C.OptimConfig(), dev, torch.bfloat16)      # bf16 weight copies for the GEMMs
    B, P = args.batch, args.prompt
    eng = DecodeEngine(model, B, P + 2 * args.steps + args.warmup + 8)      # device-timed and end-to-end loops both generate `steps` tokens
    g = torch.Generator().manual_seed(1 + (0 if dp is None else dp.rank))
    prompts = torch.randint(0, VOCAB, (B, P), generator=g).pin_memory().to(dev, non_blocking=True)
    t0 = time.time()
    eng.prefill(prompts)
    torch.cuda.synchronize()
    prefill_s = time.time() - t0
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    if dp is not None:
        dp.barrier()
    sampler = ClockSampler(dp is None or dp.lead)
    native.reset_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        eng.step()
    end.record()
    torch.cuda.synchronize()
    dev_ms = max_over_ranks(start.elapsed_time(end), dp) / args.steps
    # end to end: the step's result (next token ids) is read back to the host every step and fed from pinned memory
    host = torch.empty(B, dtype=torch.long).pin_memory()
    start.record()
    for _ in range(args.steps):
        nxt = eng.step()
        host.copy_(nxt, non_blocking=False)
        eng.tokens.copy_(host, non_blocking=True)
    end.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(start.elapsed_time(end), dp) / args.steps
    native.check_status()
    clocks = sampler.stop(world)
    out = {"metric": "decode tokens/s at 32k context", "value": B * world / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"model": MODEL + ("-grid4x4" if args.kv == "grid" else "-gqa4"), "batch_per_gpu": B, "prompt": P, "parallelism": f"dp{world}",
                      "cache_gib": eng.cache_bytes() / 2 ** 30, "prefill_s": prefill_s, "l2": "KV cache read per step >> 126 MB L2",
                      "graph_kernels_per_step": "one CUDA graph replay"},
           "clocks": clocks, "e2e": {"value": B * world / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
           "gpu_launches": args.steps, "impl": "ours"}
    if dp is not None:
        dp.close()
    return out


# ---------------------------------------------------------------------------------------------------------- reference

def reference_config(args, world: int, micro: int) -> dict:
    """The same model and step as `run_ours`, in the reference's own config keys; implementation switches are the
    ones its shipped 200M base config uses (compiled layers, flex attention, fused head, TF32), except the GDN kernel:
    its Triton kernel refuses value dim 256, so the layer runs its own chunked PyTorch path."""
    attn = dict(n_q_heads=16, n_kv_heads=4, head_dim=64, gate="elementwise", qk_norm=True, rope_fraction=0.25,
                rope_theta=1e7, rope_max_distance=2048, backend=os.environ.get("GHB_REF_ATTENTION", "flex"))
    gdn = dict(n_k_heads=8, n_v_heads=8, k_head_dim=128, v_head_dim=256, conv_kernel=4, init="fla", kernel="chunked",
               chunk_size=64, output_gate="sigmoid", input_dtype="bfloat16")
    enc = dict(n_layers=16, full_attn_interval=4, attention=attn, gdn=gdn, nope_global_layers=[3], attn_res="block_entry",
               gdn_write_mix="layer", gdn_write_variant="qmix")
    model = dict(arch="control", vocab_size=VOCAB, tie_embeddings=True, d_model=1024, ffn_hidden=2816, init_std=0.02,
                 encoder=enc)
    data = dict(kind="synthetic", seq_len=args.seq_len, batch_size=args.rows * world, doc_len_min=args.seq_len + 1,
                doc_len_max=args.seq_len + 1, seed=1)
    optim = dict(name="adamw", warmup_steps=100)
    return dict(model=model, data=data, optim=optim, steps=10 ** 6, seed=1, dtype="float32", autocast="bfloat16",
                micro_batch_size=micro, tf32=True, deterministic=False, metrics_jsonl=False, log_every=10 ** 9,
                ckpt_every_steps=10 ** 9, ckpt_every_minutes=10 ** 9, compile=os.environ.get("GHB_REF_COMPILE", "all"),
                head_select=True, head_impl="fused", device="auto")


def run_reference(args) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "ced").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-deps --target baseline/_ref <reference checkout>/code)"}
    sys.path.insert(0, str(ref))
    try:
        import torch
        import ced.config as RC
        from ced.train import data_parallel as rdp
        from ced.train.trainer import Trainer as RefTrainer
    except Exception as e:  # the package does not import here
        return {"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {str(e)[:160]}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    dp = rdp.from_environment() if int(os.environ.get("WORLD_SIZE", "1")) > 1 else None
    world = 1 if dp is None else dp.world
    micro, err = args.rows, None
    while micro >= 1:
        try:
            cfg = RC.from_dict(RC.TrainConfig, reference_config(args, world, micro))
            run_dir = tempfile.mkdtemp(prefix="refrun_")
            trainer = RefTrainer(cfg, run_dir, dp=dp)
            for _ in range(args.warmup):
                trainer.train_step()
            break
        except torch.cuda.OutOfMemoryError as e:
            err, trainer = e, None
            torch.cuda.empty_cache()
            micro //= 2
    else:
        return {"impl": "reference", "unavailable": f"reference ran out of memory at every micro-batch size: {str(err)[:120]}"}
    torch.cuda.synchronize()
    if dp is not None:
        dp.barrier()
    sampler = ClockSampler(dp is None or dp.lead)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        m = trainer.train_step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    if dp is not None:
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
    ms /= args.steps
    clocks = sampler.stop(world)
    tokens = args.rows * world * args.seq_len
    value = tokens / (ms / 1e3)
    loss = m.get("loss") if isinstance(m, dict) else None
    out = {"metric": "train tokens/s/box, 200M hybrid", "value": value, "unit": "tokens/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"model": MODEL, "global_batch": args.rows * world, "seq_len": args.seq_len,
                      "parallelism": f"dp{world}", "optimizer": "adamw", "micro_batch": micro,
                      "compile": os.environ.get("GHB_REF_COMPILE", "all"),
                      "attention": os.environ.get("GHB_REF_ATTENTION", "flex"), "gdn": "chunked (torch)", "loss": loss},
           "clocks": clocks, "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's train_step is end to end"},
           "impl": "reference"}
    if dp is not None:
        dp.close()
    return out


def run_reference_decode(args) -> dict:
    """The reference's own batched greedy generation (ced/eval/recall_ruler_gen.py `generate_greedy_batched`: chunked
    prefill through its cached forward, caches that grow by concatenation, one `extend` per token) on the same model,
    batch, prompt length and number of generated tokens. Its decode engine proper is batch 1 and refuses depth mixing,
    the GDN mixes and grid KV, so this is the path its evaluations use at batch > 1. The rate is its own
    `decode_steps` / `decode_s` (a host clock between device synchronisations, as the function reports it)."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "ced").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-deps --target baseline/_ref <reference checkout>/code)"}
    sys.path.insert(0, str(ref))
    import torch
    import ced.config as RC
    from ced.eval.recall_ruler_gen import generate_greedy_batched
    from ced.model.control import build_model as ref_build

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    args_t = argparse.Namespace(**{**vars(args), "rows": 1})
    mcfg = reference_config(args_t, 1, 1)["model"]
    mcfg["encoder"]["attention"]["backend"] = os.environ.get("GHB_REF_DECODE_ATTENTION", "reference")     # the cached forward's own attention
    if args.kv == "grid":
        mcfg["encoder"]["attention"].update(kv_sharing="grid", n_kv_heads=1, grid_rows=4, grid_cols=4, row_dim=32, col_dim=32)
    torch.manual_seed(1)
    model = ref_build(RC.from_dict(RC.ModelConfig, mcfg)).to(dev).eval()
    g = torch.Generator().manual_seed(1 + rank)
    B, P = args.batch, args.prompt
    prompts = torch.randint(0, VOCAB, (B, P), generator=g).tolist()
    sampler = ClockSampler(rank == 0)
    n_new = args.steps + args.warmup + 1
    _, stats = generate_greedy_batched(model, prompts, n_new, prefill_rows=int(os.environ.get("GHB_REF_PREFILL_ROWS", "2")), autocast_dtype=torch.bfloat16)
    clocks = sampler.stop(world)
    ms = 1e3 * stats["decode_s"] / max(1, stats["decode_steps"])
    if world > 1:
        import torch.distributed as dist

        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        dist.destroy_process_group()
    value = B * world / (ms / 1e3)
    return {"metric": "decode tokens/s at 32k context", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": stats["decode_steps"], "warmup": 0,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": MODEL + ("-grid4x4" if args.kv == "grid" else "-gqa4"), "batch_per_gpu": B, "prompt": P, "parallelism": f"dp{world}",
                       "prefill_s": stats["prefill_s"], "path": "generate_greedy_batched (prefill / extend, concatenated caches)",
                       "timing": "the function's own decode_s / decode_steps (host clock between synchronisations)"},
            "clocks": clocks, "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's loop reads every token back to the host"},
            "impl": "reference"}


def main():
    args = parse()
    t0 = time.time()
    try:
        if args.mode == "decode":
            out = run_reference_decode(args) if args.impl == "reference" else run_decode(args)
        else:
            out = run_reference(args) if args.impl == "reference" else run_ours(args)
    except Exception as e:
        if args.impl != "reference":
            raise
        out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    if int(os.environ.get("RANK", "0")) == 0:
        out["wall_s"] = round(time.time() - t0, 1)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
