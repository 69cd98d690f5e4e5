"""Worker of the tensor-parallel tests (one process per rank under torchrun). argv[1]: output path; argv[2]: 'fused'
(CUDA kernels over symmetric memory, checked against the collective implementation in the same process) or
'collective' (gloo / NCCL collectives, checked against one process's dense math)."""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from gdn_hybrid_architecture_ideas_b200.models.linear import Linear  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel, tensor_parallel as tpm  # noqa: E402


def main():
    mode = sys.argv[2]
    dp = data_parallel.from_environment()
    W, r, dev = dp.world, dp.rank, dp.device
    cuda = dev.type == "cuda"
    dt = torch.bfloat16 if cuda else torch.float32
    Ts, K, N, Kr = (256, 512, 384, 256) if cuda else (8, 16, 12, 8)
    T = Ts * W
    g = torch.Generator().manual_seed(11)
    x_full = torch.randn(T, K, generator=g)
    w_col = torch.randn(W, N, K, generator=g) * K ** -0.5          # rank r owns w_col[r] (column-parallel output slice)
    w_small = torch.randn(W, 4, K, generator=g) * K ** -0.5        # a projection with 4 outputs per rank
    h_full = torch.randn(T, W * Kr, generator=g)
    w_row = torch.randn(N, W * Kr, generator=g) * (W * Kr) ** -0.5
    dy_col = torch.randn(T, W * N, generator=g)
    dout = torch.randn(T, N, generator=g)
    results = {}
    impls = ["collective", "fused"] if mode == "fused" else ["collective"]
    for impl in impls:
        tp = tpm.TensorParallel(dp, max_tokens=T, max_width=max(K, N, W * 0 + Kr, 512), impl=impl)
        out = []
        for rep in range(3):                       # several rounds: gather and staging slots are reused
            x = x_full[r * Ts:(r + 1) * Ts].to(dev, dt).requires_grad_()
            lin = Linear(K, N).to(dev)
            lin.weight.data.copy_(w_col[r])
            small = Linear(K, 4).to(dev)
            small.weight.data.copy_(w_small[r])
            y = tpm.column_parallel(x, lin, tp)
            ys = tpm.column_parallel(x, small, tp)
            (y.float() * dy_col[:, r * N:(r + 1) * N].to(dev)).sum().backward(retain_graph=True)
            ys.float().sum().backward()
            h = h_full[:, r * Kr:(r + 1) * Kr].to(dev, dt).requires_grad_()
            row = Linear(Kr, N).to(dev)
            row.weight.data.copy_(w_row[:, r * Kr:(r + 1) * Kr])
            o = tpm.row_parallel(h, row, tp)
            (o.float() * dout[r * Ts:(r + 1) * Ts].to(dev)).sum().backward()
            out = [t.detach().float().cpu().clone() for t in (y, ys, x.grad, lin.weight.grad, small.weight.grad, o, h.grad, row.weight.grad)]
        # the two projections of one input scatter their input gradient once, and a projection whose output never reached
        # the loss is reported instead of silently shortening the gradient
        calls, plain_rs = [0], tp.gemm_rs

        def counted(*a, **k):
            calls[0] += 1
            return plain_rs(*a, **k)
        tp.gemm_rs = counted
        x = x_full[r * Ts:(r + 1) * Ts].to(dev, dt).requires_grad_()
        (tpm.column_parallel(x, lin, tp).float().sum() + tpm.column_parallel(x, small, tp).float().sum()).backward()
        assert calls[0] == 1 and x.grad is not None, calls
        tp.check_fans()
        x = x_full[r * Ts:(r + 1) * Ts].to(dev, dt).requires_grad_()
        y, _unused = tpm.column_parallel(x, lin, tp), tpm.column_parallel(x, small, tp)
        y.float().sum().backward()
        try:
            tp.check_fans()
            raise AssertionError("an input whose projections did not all run backward was not reported")
        except RuntimeError as err:
            assert "withheld" in str(err)
        tp.gemm_rs = plain_rs
        if cuda:
            from gdn_hybrid_architecture_ideas_b200.ops import native
            torch.cuda.synchronize()
            native.check_status()
        results[impl] = out
    if mode == "collective":                       # dense single-process math on the same numbers
        wc = w_col.reshape(W * N, K)
        y_all = x_full @ wc.t()
        dx_all = dy_col @ wc + torch.ones(T, 4 * W) @ w_small.reshape(4 * W, K)
        o_all = h_full @ w_row.t()
        want = [y_all[:, r * N:(r + 1) * N], x_full @ w_small[r].t(), dx_all[r * Ts:(r + 1) * Ts], dy_col[:, r * N:(r + 1) * N].t() @ x_full,
                torch.ones(T, 4).t() @ x_full, o_all[r * Ts:(r + 1) * Ts], (dout @ w_row)[:, r * Kr:(r + 1) * Kr], dout.t() @ h_full[:, r * Kr:(r + 1) * Kr]]
        results["dense"] = want
    torch.save(results, f"{sys.argv[1]}.{r}")
    dp.barrier()
    dp.close()


if __name__ == "__main__":
    main()
