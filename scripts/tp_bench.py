"""Times the tensor-parallel boundaries in isolation, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port 29731 \
        scripts/tp_bench.py --tokens 65536 --width 2048 --shard 768

For each of all-gather -> GEMM, GEMM -> reduce-scatter and the weight gradient over gathered tokens it runs the fused
kernels (`--impl fused`, default both) and the collective baseline (NCCL around the framework's GEMM) on the same
shapes, CUDA events on the launching stream, maximum over ranks, and prints one JSON line per (op, impl) with the wire
bytes per rank, the FLOPs per rank and the fraction of the roofline max(FLOPs / GEMM peak, bytes / link bandwidth).
Peaks are read from MEASURED_PEAKS.json beside the package when present (else 1.4 PFLOP/s sustained); the link figure
is the measured 770 GB/s per direction.
"""

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel, tensor_parallel as tpm  # noqa: E402

LINK_BYTES_S = 770e9


def peak_flops() -> float:
    f = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(f.read_text())["bf16_tflops_sustained"]) * 1e12
    except Exception:
        return 1.4e15


def timed(dp, fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dp.barrier()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([beg.elapsed_time(end) / iters], device=dp.device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=dp.tensor_group)
    return float(ms)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=65536, help="tokens over all ranks")
    p.add_argument("--width", type=int, default=2048, help="model width (the gathered / scattered row)")
    p.add_argument("--shard", type=int, default=768, help="this rank's slice of the hidden width")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["both", "fused", "collective"], default="both")
    p.add_argument("--ops", default="ag_gemm,gemm_rs,wgrad")
    a = p.parse_args()
    dp = data_parallel.from_environment()
    W, dev = dp.world, dp.device
    T, d, n = a.tokens, a.width, a.shard
    Ts = T // W
    peak = peak_flops()
    bf = torch.bfloat16
    shards = [torch.randn(Ts, d, device=dev, dtype=bf) for _ in range(4)]       # distinct inputs: every call gathers anew
    w_col = torch.randn(n, d, device=dev, dtype=bf) * d ** -0.5
    h = torch.randn(T, n, device=dev, dtype=bf)
    w_row = torch.randn(d, n, device=dev, dtype=bf) * n ** -0.5
    dy = torch.randn(T, n, device=dev, dtype=bf)
    full = torch.randn(T, d, device=dev, dtype=bf)
    wire = (W - 1) / W * T * d * 2                                               # bytes in (gather) or out (scatter) per rank
    flops = {k: 2.0 * T * d * n for k in ("ag_gemm", "gemm_rs", "wgrad", "gemm_col", "gemm_row")}
    impls = ["fused", "collective"] if a.impl == "both" else [a.impl]
    for impl in impls:
        tp = tpm.TensorParallel(dp, max_tokens=T, max_width=max(d, n, 512), impl=impl)
        turn = [0]

        def ag():
            turn[0] += 1
            tp._cache.clear()
            return tp.ag_gemm(tp.gather(shards[turn[0] % 4]), w_col)

        def rs():
            return tp.gemm_rs(h, w_row)

        def wg():
            turn[0] += 1
            tp._cache.clear()
            g = tp.gather(shards[turn[0] % 4])
            return tp.gemm_gathered_k(dy, g.full, g)

        def gather_only():                                                       # the baseline's collective alone
            turn[0] += 1
            tp._cache.clear()
            return tp.gather(shards[turn[0] % 4])

        def plain_col():                                                         # the products without any communication
            return tp._plain(full, w_col, False, False, bf)

        def plain_row():
            return tp._plain(h, w_row, False, False, bf)

        table = {"ag_gemm": ag, "gemm_rs": rs, "wgrad": wg}
        extra = []
        if impl == "collective":
            table.update(all_gather=gather_only, gemm_col=plain_col, gemm_row=plain_row)
            extra = ["all_gather", "gemm_col", "gemm_row"]
        for op in [o for o in a.ops.split(",") if o in table] + extra:
            tp._cache.clear()
            ms = timed(dp, table[op], a.iters, a.warmup)
            fl = flops.get(op, 0.0)
            target = max(fl / peak, 0.0 if op.startswith("gemm_col") or op == "gemm_row" else wire / LINK_BYTES_S) * 1e3
            if dp.lead:
                print(json.dumps({"op": op, "impl": impl, "world": W, "tokens": T, "d": d, "n": n, "ms": round(ms, 4),
                                  "wire_MB_per_rank": round(wire / 1e6, 1), "gflop_per_rank": round(fl / 1e9, 1),
                                  "roofline_ms": round(target, 4), "fraction_of_roofline": round(target / ms, 3),
                                  "gather": getattr(tp, "gather_by", None), "scatter": getattr(tp, "scatter", None)}), flush=True)
        if impl == "fused":
            from gdn_hybrid_architecture_ideas_b200.ops import native
            torch.cuda.synchronize()
            native.check_status()
        del tp
    dp.barrier()
    dp.close()


if __name__ == "__main__":
    main()
