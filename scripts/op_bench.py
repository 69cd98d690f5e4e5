"""Time one hot op of the package in isolation (forward and backward), CUDA events after warm-up.

    python scripts/op_bench.py attention --B 2 --L 4096 --cap 1024
    python scripts/op_bench.py gdn --B 2 --L 4096
    python scripts/op_bench.py gdn_prep --B 2 --L 4096
    python scripts/op_bench.py gemm --M 65536 --N 1024 --K 1024 --layout nt
    python scripts/op_bench.py rmsnorm --rows 65536 --d 1024

Prints one JSON line per op with milliseconds per call and the achieved rate against the op's algorithmic FLOPs or
bytes. `--iters 1 --warmup 0` gives a run short enough to capture under a profiler. Inputs are larger than the L2
cache at the default sizes; an L2 flush (a 256 MB write) runs between timed calls.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.ops import attention_native, gdn_native, native  # noqa: E402

BF16 = torch.bfloat16


def timed(fn, iters, warmup):
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    native.check_status()
    return total / max(iters, 1)


def bench_attention(a):
    B, L, Hq, Hkv, hd = a.B, a.L, a.Hq, a.Hkv, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda h: torch.randn(B, L, h, hd, device="cuda", generator=g).to(BF16).requires_grad_()
    q, k, v = mk(Hq), mk(Hkv), mk(Hkv)
    capped = a.cap >= 0
    qf, kf = (mk(Hq), mk(Hkv)) if capped else (None, None)
    doc = pos = None
    if a.doc_len:
        idx = torch.arange(L, device="cuda")
        doc = (idx // a.doc_len).to(torch.int32)[None].expand(B, L).contiguous()
        pos = (idx % a.doc_len).to(torch.int32)[None].expand(B, L).contiguous()
    out = {}

    def fwd():
        out["o"] = attention_native._Attention.apply(q, k, v, qf, kf, doc, pos, a.cap if capped else None)

    ms_f = timed(fwd, a.iters, a.warmup)
    do = torch.randn_like(out["o"])

    def bwd():
        out["o"].backward(do, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    span = min(a.doc_len, L) if a.doc_len else L
    pairs = B * Hq * (L // span) * span * (span + 1) / 2          # visible (query, key) pairs
    f_fwd, f_bwd = 4 * pairs * hd, 10 * pairs * hd
    return {"op": "attention", "B": B, "L": L, "Hq": Hq, "Hkv": Hkv, "cap": a.cap, "doc_len": a.doc_len, "fwd_ms": ms_f, "bwd_ms": ms_b,
            "fwd_tflops": f_fwd / ms_f / 1e9, "bwd_tflops": f_bwd / ms_b / 1e9}


def bench_gdn(a):
    B, L, H, dk, dv = a.B, a.L, a.H, 128, a.dv
    g_ = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g_)
    q = (torch.nn.functional.normalize(rn(B, L, H, dk), dim=-1) * dk ** -0.5).to(BF16).requires_grad_()
    k = torch.nn.functional.normalize(rn(B, L, H, dk), dim=-1).to(BF16).requires_grad_()
    v = rn(B, L, H, dv).to(BF16).requires_grad_()
    g = (-torch.rand(B, L, H, device="cuda", generator=g_) * 0.5).requires_grad_()
    beta = torch.rand(B, L, H, device="cuda", generator=g_).requires_grad_()
    start = torch.zeros(B, L, dtype=torch.bool, device="cuda")
    out = {}

    def fwd():
        out["o"], _ = gdn_native.delta_rule(q, k, v, g, beta, start, None, 64, False)

    ms_f = timed(fwd, a.iters, a.warmup)
    do = torch.randn_like(out["o"])

    def bwd():
        out["o"].backward(do, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    return {"op": "gdn", "B": B, "L": L, "H": H, "dv": dv, "fwd_ms": ms_f, "bwd_ms": ms_b}


def bench_gemm(a):
    """--layout nt: y = x W^T (forward); nn: dx = dy W (W stored [K, N]); tn: dW = dy^T x (both stored [K, *], fp32 out)."""
    M, N, K = a.M, a.N, a.K
    if a.layout == "nt":
        x = torch.randn(M, K, device="cuda").to(BF16)
        w = torch.randn(N, K, device="cuda").to(BF16)
        ours, lib = (lambda: native.gemm(x, w)), (lambda: torch.matmul(x, w.t()))
    elif a.layout == "nn":
        x = torch.randn(M, K, device="cuda").to(BF16)
        w = torch.randn(K, N, device="cuda").to(BF16)
        ours, lib = (lambda: native.gemm(x, w, b_mn=True)), (lambda: torch.matmul(x, w))
    else:
        x = torch.randn(K, M, device="cuda").to(BF16)
        w = torch.randn(K, N, device="cuda").to(BF16)
        out = torch.empty(M, N, device="cuda")
        ours, lib = (lambda: native.gemm(x, w, out=out, a_mn=True, b_mn=True)), (lambda: torch.matmul(x.t(), w))
    ms = timed(ours, a.iters, a.warmup)
    ms_lib = timed(lib, a.iters, a.warmup)
    fl = 2.0 * M * N * K
    return {"op": "gemm", "layout": a.layout, "M": M, "N": N, "K": K, "ms": ms, "tflops": fl / ms / 1e9, "cublas_ms": ms_lib,
            "cublas_tflops": fl / ms_lib / 1e9}


def bench_gemm_mx(a):
    """MXFP8: the quantise kernel on an [M, K] bf16 activation (both block orientations from one read) and the block-scaled
    product y = x_q W_q^T, against the bf16 kernel on the same shape."""
    M, N, K = a.M, a.N, a.K
    x = torch.randn(M, K, device="cuda").to(BF16)
    w = torch.randn(N, K, device="cuda") * 0.02
    xq, xs, _, _ = native.mx_quantize(x, True, False)
    wq, ws, _, _ = native.mx_quantize(w, True, False)
    wl = w.to(BF16)
    ms = timed(lambda: native.gemm_mx(xq, xs, wq, ws), a.iters, a.warmup)
    ms_bf16 = timed(lambda: native.gemm(x, wl), a.iters, a.warmup)
    ms_q1 = timed(lambda: native.mx_quantize(x, True, False), a.iters, a.warmup)
    ms_q2 = timed(lambda: native.mx_quantize(x, True, True), a.iters, a.warmup)
    fl = 2.0 * M * N * K
    return {"op": "gemm_mx", "M": M, "N": N, "K": K, "ms": ms, "tflops": fl / ms / 1e9, "bf16_kernel_ms": ms_bf16, "bf16_kernel_tflops": fl / ms_bf16 / 1e9,
            "quantise_rowwise_ms": ms_q1, "quantise_rowwise_gbs": M * K * 3 / ms_q1 / 1e6, "quantise_both_ms": ms_q2,
            "quantise_both_gbs": M * K * 4 / ms_q2 / 1e6}


def bench_gdn_prep(a):
    from gdn_hybrid_architecture_ideas_b200 import ops
    B, L, hk, hv, dk, dv = a.B, a.L, a.H, a.H, 128, a.dv
    C = 2 * hk * dk + hv * dv
    u = torch.randn(B, L, C, device="cuda").to(BF16).requires_grad_()
    w = (torch.rand(C, 4, device="cuda") - 0.5).requires_grad_()
    doc = torch.zeros(B, L, dtype=torch.long, device="cuda")
    out = {}

    def fwd():
        out["y"] = ops.gdn_prep(u, doc, w, hk, hv, dk, dv, single_doc=True, packed=True)[0]

    ms_f = timed(fwd, a.iters, a.warmup)
    dy = torch.randn_like(out["y"])

    def bwd():
        out["y"].backward(dy, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    n = B * L * C
    return {"op": "gdn_prep", "B": B, "L": L, "C": C, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_gbs": n * 4 / ms_f / 1e6, "bwd_gbs": n * 6 / ms_b / 1e6}


def bench_rmsnorm(a):
    from gdn_hybrid_architecture_ideas_b200 import ops
    x = torch.randn(a.rows, a.d, device="cuda", requires_grad=True)
    w = torch.zeros(a.d, device="cuda", requires_grad=True)
    out = {}

    def fwd():
        out["y"] = ops.rmsnorm(x, w, 1e-6, out_dtype=BF16)

    ms_f = timed(fwd, a.iters, a.warmup)
    dy = torch.randn_like(out["y"])

    def bwd():
        out["y"].backward(dy, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    n = a.rows * a.d
    return {"op": "rmsnorm", "rows": a.rows, "d": a.d, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_gbs": n * 6 / ms_f / 1e6, "bwd_gbs": n * 10 / ms_b / 1e6}


def bench_depth_mix(a):
    from gdn_hybrid_architecture_ideas_b200 import ops
    rows, d, n = a.rows, a.d, a.sources
    srcs = [torch.randn(1, rows, d, device="cuda", requires_grad=True) for _ in range(n)]
    q = (torch.randn(d, device="cuda") * 0.1).requires_grad_()
    gain = torch.zeros(d, device="cuda", requires_grad=True)
    out = {}

    def fwd():
        out["y"] = ops.depth_mix(srcs, q, gain, 1e-6)

    ms_f = timed(fwd, a.iters, a.warmup)
    dy = torch.randn_like(out["y"])

    def bwd():
        out["y"].backward(dy, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    nb = rows * d * 4
    return {"op": "depth_mix", "rows": rows, "d": d, "sources": n, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_gbs": nb * (n + 1) / ms_f / 1e6,
            "bwd_gbs": nb * (2 * n + 1) / ms_b / 1e6}


def bench_swiglu(a):
    rows, f = a.rows, a.ffn
    gu = torch.randn(rows, 2 * f, device="cuda").to(BF16).requires_grad_()
    out = {}

    def fwd():
        out["y"] = native._SiluMul.apply(gu)

    ms_f = timed(fwd, a.iters, a.warmup)
    dy = torch.randn_like(out["y"])

    def bwd():
        out["y"].backward(dy, retain_graph=True)

    ms_b = timed(bwd, a.iters, a.warmup)
    nb = rows * f * 2
    return {"op": "swiglu", "rows": rows, "ffn": f, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_gbs": nb * 3 / ms_f / 1e6, "bwd_gbs": nb * 5 / ms_b / 1e6}


def bench_lm_head(a):
    rows, d, V = a.rows, a.d, a.vocab
    h = torch.randn(rows, d, device="cuda").to(BF16).requires_grad_()
    W = (torch.randn(V, d, device="cuda") * 0.02).requires_grad_()
    t = torch.randint(0, V, (rows, 1), device="cuda")
    w = torch.full((rows, 1), 1.0 / rows, device="cuda")
    b = torch.zeros(rows, device="cuda")
    ms = timed(lambda: native.fused_linear_ce(h, W, t, w, b, a.chunk)[0].backward(), a.iters, a.warmup)
    return {"op": "lm_head", "rows": rows, "d": d, "vocab": V, "chunk": a.chunk, "fwd_bwd_ms": ms, "tflops": 6.0 * rows * d * V / ms / 1e9}


def bench_adamw(a):
    n = a.numel
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=BF16)
    ms = timed(lambda: native.adamw_(p, g, m, v, lp, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0), a.iters, a.warmup)
    return {"op": "adamw", "numel": n, "ms": ms, "gbs": n * 30 / ms / 1e6}


def bench_decode_attention(a):
    from gdn_hybrid_architecture_ideas_b200.ops import native as nat
    B, T, Hq, Hkv, hd = a.B, a.L, a.Hq, a.Hkv, 64
    q = torch.randn(B, Hq, hd, device="cuda")
    k = torch.randn(B, T, Hkv, hd, device="cuda").to(BF16)
    v = torch.randn(B, T, Hkv, hd, device="cuda").to(BF16)
    lens = torch.full((B,), T, dtype=torch.int32, device="cuda")
    rot = 16
    ang = torch.arange(max(a.cap, 1) + 1, device="cuda")[:, None] * (1e7 ** (-torch.arange(rot // 2, device="cuda") / (rot // 2)))[None]
    cos_t, sin_t = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    out = torch.empty(B, Hq, hd, device="cuda", dtype=BF16)
    splits = 16
    po = torch.empty(B, Hq, splits, hd, device="cuda")
    pml = torch.empty(B, Hq, splits, 2, device="cuda")
    if a.kv == "grid":      # 4 x 4 grid of 32-channel components: 256 cached channels per token, scored from the raw components
        assert Hq == 16, "the grid kernel serves 16 query heads"
        kg = torch.randn(B, T, 256, device="cuda").to(BF16)
        vg = torch.randn(B, T, 256, device="cuda").to(BF16)
        gain = torch.ones(64, device="cuda")
        splits = max(16, min(256, 592 // max(B, 1)))
        po = torch.empty(B, Hq, splits, hd, device="cuda")
        pml = torch.empty(B, Hq, splits, 2, device="cuda")
        ms = timed(lambda: nat.ext().decode_attention_grid(q, kg, vg, lens, None, cos_t, sin_t, gain, out, po, pml, rot, a.cap, splits, hd ** -0.5, 1e-6),
                   a.iters, a.warmup)
        return {"op": "decode_attention", "kv": "grid4x4", "B": B, "T": T, "Hq": Hq, "ms": ms, "gbs": 2 * B * T * 256 * 2 / ms / 1e6}
    ms = timed(lambda: nat.ext().decode_attention(q, k, v, lens, None, cos_t, sin_t, out, po, pml, rot, a.cap, splits, hd ** -0.5), a.iters, a.warmup)
    nb = 2 * B * T * Hkv * hd * 2
    return {"op": "decode_attention", "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "ms": ms, "gbs": nb / ms / 1e6}


def main():
    p = argparse.ArgumentParser()
    p.add_argument("op", choices=["attention", "gdn", "gdn_prep", "gemm", "gemm_mx", "rmsnorm", "depth_mix", "swiglu", "lm_head", "adamw", "decode_attention"])
    p.add_argument("--kv", choices=["gqa", "grid"], default="gqa", help="decode_attention: grouped KV heads or the 4 x 4 grid's raw components")
    p.add_argument("--sources", type=int, default=4)
    p.add_argument("--ffn", type=int, default=2816)
    p.add_argument("--vocab", type=int, default=32768)
    p.add_argument("--chunk", type=int, default=2048, help="lm_head: positions per chunk of logits")
    p.add_argument("--numel", type=int, default=1 << 28)
    p.add_argument("--layout", choices=["nt", "nn", "tn"], default="nt")
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--B", type=int, default=2)
    p.add_argument("--L", type=int, default=4096)
    p.add_argument("--Hq", type=int, default=16)
    p.add_argument("--Hkv", type=int, default=16)
    p.add_argument("--H", type=int, default=8)
    p.add_argument("--dv", type=int, default=256)
    p.add_argument("--cap", type=int, default=-1)
    p.add_argument("--doc-len", type=int, default=0)
    p.add_argument("--M", type=int, default=65536)
    p.add_argument("--N", type=int, default=1024)
    p.add_argument("--K", type=int, default=1024)
    p.add_argument("--rows", type=int, default=65536)
    p.add_argument("--d", type=int, default=1024)
    a = p.parse_args()
    res = {"attention": bench_attention, "gdn": bench_gdn, "gdn_prep": bench_gdn_prep, "gemm": bench_gemm, "gemm_mx": bench_gemm_mx, "rmsnorm": bench_rmsnorm,
           "depth_mix": bench_depth_mix, "swiglu": bench_swiglu, "lm_head": bench_lm_head, "adamw": bench_adamw,
           "decode_attention": bench_decode_attention}[a.op](a)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
