"""Each sm_100a kernel against the plain PyTorch fp32 statement of the same op, forward and backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, atol, rtol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3e} (bound {bound.max().item():.3e}), worst ratio {(err / bound).max().item():.2f}"


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 1024, 1024), (304, 200, 264), (128, 16, 1024), (1024, 4112, 1024), (4096, 2816, 1024)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_layouts(M, N, K, layout):
    from gdn_hybrid_architecture_ideas_b200.ops import native

    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g).to(_dev(), torch.bfloat16)
    b = torch.randn(N, K, generator=g).to(_dev(), torch.bfloat16)
    want = a.float() @ b.float().T
    if layout == "nt":
        got = native.gemm(a, b, out_dtype=torch.float32)
    elif layout == "nn":      # b stored [K, N]
        got = native.gemm(a, b.T.contiguous(), b_mn=True, out_dtype=torch.float32)
    else:                     # both stored with the reduction dimension outermost
        got = native.gemm(a.T.contiguous(), b.T.contiguous(), a_mn=True, b_mn=True, out_dtype=torch.float32)
    native.check_status()
    _close(got, want, 2e-3 * K ** 0.5, 1e-3, f"gemm {layout} {M}x{N}x{K}")
    got16 = native.gemm(a, b)
    _close(got16, want, 2e-2 * K ** 0.5, 1e-2, "bf16 out")
    acc = torch.ones(M, N, device=_dev())
    native.gemm(a, b, out=acc, accumulate=True)
    _close(acc, want + 1, 2e-3 * K ** 0.5, 1e-3, "accumulate")
    native.check_status()


def test_gemm_split_k():
    """Few output tiles and a long reduction: the reduction is sliced across CTAs and meets in the fp32 output."""
    from gdn_hybrid_architecture_ideas_b200.ops import native

    M, N, K = 256, 384, 16384
    g = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn(K, M, generator=g).to(_dev(), torch.bfloat16)      # stored [K, M]: the weight-gradient layout
    b = torch.randn(K, N, generator=g).to(_dev(), torch.bfloat16)
    want = a.float().T @ b.float()
    got = native.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    _close(got, want, 2e-3 * K ** 0.5, 1e-3, "split-k store")
    acc = torch.full((M, N), 2.0, device=_dev())
    native.gemm(a, b, out=acc, a_mn=True, b_mn=True, accumulate=True)
    _close(acc, want + 2, 2e-3 * K ** 0.5, 1e-3, "split-k accumulate")
    wide = torch.zeros(M, N + 8, device=_dev())                        # a strided output (row stride > N) stays intact outside N
    native.gemm(a, b, out=wide[:, :N], a_mn=True, b_mn=True)
    _close(wide[:, :N], want, 2e-3 * K ** 0.5, 1e-3, "split-k strided")
    assert float(wide[:, N:].abs().max()) == 0.0
    native.check_status()


@pytest.mark.parametrize("dual", [True, False])
def test_input_mixes_kernel(dual):
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    g = torch.Generator().manual_seed(3)
    mk = lambda: torch.randn(3, 50, 256, generator=g).to(_dev(), torch.bfloat16)
    x, ya, yb = mk(), mk(), mk()
    la, lb = torch.tensor([0.3], device=_dev()), torch.tensor([-0.7], device=_dev())
    leaves = [t.clone().requires_grad_() for t in (x, ya, la, yb, lb)]
    refs = [t.clone().float().requires_grad_() for t in (x, ya, la, yb, lb)]
    oa, ob = native.input_mixes(leaves[0], leaves[1], leaves[2], leaves[3] if dual else None, leaves[4] if dual else None)
    ra, rb = ref.input_mixes(refs[0], refs[1], refs[2], refs[3] if dual else None, refs[4] if dual else None)
    _close(oa, ra, 2e-2, 1e-2, "write mix")
    ga, gb = torch.randn_like(ra), torch.randn_like(ra)
    if dual:
        _close(ob, rb, 2e-2, 1e-2, "query mix")
        (oa.float() * ga + ob.float() * gb).sum().backward()
        (ra * ga + rb * gb).sum().backward()
    else:
        assert ob is None
        (oa.float() * ga).sum().backward()
        (ra * ga).sum().backward()
    for name, a, b in zip(("dx", "dya", "dla", "dyb", "dlb"), leaves, refs):
        if b.grad is None:
            assert a.grad is None
            continue
        scale = float(b.grad.abs().max())
        _close(a.grad, b.grad, 2e-2 * max(scale, 1.0), 2e-2, name)
    native.check_status()


def test_split_linear_kernel():
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.models.linear import Linear

    lin = Linear(256, 640).to(_dev())
    g = torch.Generator().manual_seed(4)
    xa = torch.randn(2, 70, 256, generator=g).to(_dev(), torch.bfloat16).requires_grad_()
    xb = torch.randn(2, 70, 256, generator=g).to(_dev(), torch.bfloat16).requires_grad_()
    y = ops.split_linear(xa, xb, lin, 128)
    want = torch.cat([xa.float() @ lin.weight[:128].T, xb.float() @ lin.weight[128:].T], dim=-1)
    _close(y, want, 3e-2, 2e-2, "split linear")
    go = torch.randn_like(want).to(torch.bfloat16).float()
    y.backward(go.to(y.dtype))
    got = (xa.grad.clone(), xb.grad.clone(), lin.weight.grad.clone())
    xa.grad = xb.grad = lin.weight.grad = None
    want.backward(go)
    for name, a, b in zip(("dxa", "dxb", "dw"), got, (xa.grad, xb.grad, lin.weight.grad)):
        _close(a, b, 1e-1, 3e-2, name)


def test_linear_autograd():
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.models.linear import Linear

    lin = Linear(512, 384).to(_dev())
    x = torch.randn(4, 96, 512, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, lin)
    w = lin.weight.detach().to(torch.bfloat16).float()
    _close(y, x.detach().float() @ w.T, 2e-2, 1e-2)
    gy = torch.randn_like(y)
    y.backward(gy)
    _close(x.grad, gy.float() @ w, 3e-2, 2e-2)
    _close(lin.weight.grad, gy.float().reshape(-1, 384).T @ x.detach().float().reshape(-1, 512), 5e-2, 2e-2)


@pytest.mark.parametrize("d,in_dt,gate", [(1024, torch.float32, None), (64, torch.bfloat16, None), (256, torch.bfloat16, "sigmoid"),
                                         (256, torch.float32, "silu"), (512, torch.float32, None), (2048, torch.float32, None)])
def test_rmsnorm_family(d, in_dt, gate):
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    rows = 333
    x = torch.randn(rows, d, device=_dev()).to(in_dt).requires_grad_()
    w = (torch.randn(d, device=_dev()) * 0.1).requires_grad_()
    z = torch.randn(rows, d, device=_dev()).to(torch.bfloat16).requires_grad_() if gate else None
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    zr = z.detach().float().requires_grad_() if gate else None
    if gate:
        y = native.gated_rmsnorm(x, z, w, 1e-6, gate, out_dtype=torch.float32)
        yr = ref.gated_rmsnorm(xr, zr, wr, 1e-6, gate)
    else:
        y = native.rmsnorm(x, w, 1e-6, out_dtype=torch.float32)
        yr = ref.rmsnorm(xr, wr, 1e-6)
    tol = 2e-2 if in_dt == torch.bfloat16 else 1e-5
    _close(y, yr, tol, tol, "fwd")
    gy = torch.randn_like(yr)
    y.backward(gy), yr.backward(gy)
    _close(x.grad, xr.grad, 3e-2 if in_dt == torch.bfloat16 else 1e-4, 2e-2 if in_dt == torch.bfloat16 else 1e-4, "dx")
    _close(w.grad, wr.grad, 2e-3 * rows ** 0.5, 1e-3, "dw")
    if gate:
        _close(z.grad, zr.grad, 3e-2, 2e-2, "dz")


def test_norm_add():
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    rows, d = 257, 1024
    resid = torch.randn(rows, d, device=_dev(), requires_grad=True)
    br = torch.randn(rows, d, device=_dev()).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(d, device=_dev()) * 0.1).requires_grad_()
    y = native.norm_add(resid, br, w, 1e-6, 0.5)
    r2, b2, w2 = resid.detach().clone().requires_grad_(), br.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = r2 + 0.5 * ref.rmsnorm(b2, w2, 1e-6)
    _close(y, yr, 1e-5, 1e-5)
    gy = torch.randn_like(yr)
    y.backward(gy), yr.backward(gy)
    _close(resid.grad, r2.grad, 0, 0)
    _close(br.grad, b2.grad, 2e-2, 2e-2)
    _close(w.grad, w2.grad, 5e-2, 1e-3)


def test_swiglu_mlp():
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.models.mlp import SwiGLU

    m = SwiGLU(256, 704).to(_dev())
    x = torch.randn(3, 100, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = m(x)
    ops.set_mode("reference")
    try:
        xr = x.detach().float().requires_grad_()
        mr = SwiGLU(256, 704).to(_dev())
        mr.load_state_dict(m.state_dict())
        yr = mr(xr)
    finally:
        ops.set_mode("native")
    _close(y, yr, 3e-2, 3e-2)
    gy = torch.randn_like(yr)
    y.backward(gy.to(y.dtype)), yr.backward(gy)
    _close(x.grad, xr.grad, 5e-2, 5e-2)
    for a, b in zip(m.parameters(), mr.parameters()):
        _close(a.grad, b.grad, 1e-1, 5e-2)


@pytest.mark.parametrize("single,L", [(True, 200), (False, 200), (False, 2100)])
def test_gdn_prep(single, L):
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    B, hk, hv, dk, dv = 2, 2, 2, 128, 256
    C = 2 * hk * dk + hv * dv
    u = torch.randn(B, L, C, device=_dev()).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(C, 4, device=_dev()) * 0.5).requires_grad_()
    doc = torch.zeros(B, L, dtype=torch.long, device=_dev())
    if not single:
        doc[0, 50:] = 1
        doc[0, 51:] = 2
        doc[1, 199:] = 3
        doc[1, L - 1:] = 4
    q, k, v, hist, _ = native.gdn_prep(u, doc, w, hk, hv, dk, dv, single_doc=single)
    ur, wr = u.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    qr, kr, vr, histr, _ = ref.gdn_prep(ur, doc, wr, hk, hv, dk, dv)
    for a, b, n in ((q, qr, "q"), (k, kr, "k"), (v, vr, "v")):
        _close(a, b, 1e-2, 2e-2, n)
    gq, gk, gv = torch.randn_like(qr), torch.randn_like(kr), torch.randn_like(vr)
    torch.autograd.backward([q, k, v], [gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype)])
    torch.autograd.backward([qr, kr, vr], [gq, gk, gv])
    _close(u.grad, ur.grad, 5e-2, 5e-2, "du")
    _close(w.grad, wr.grad, 0.5, 3e-2, "dw")


@pytest.mark.parametrize("n,d", [(2, 1024), (5, 1024), (4, 512), (3, 2048)])
def test_depth_mix(n, d):
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    rows = 97
    src = [torch.randn(2, rows, d, device=_dev()).requires_grad_() for _ in range(n)]
    qy = (torch.randn(d, device=_dev()) * 0.2).requires_grad_()
    gn = (torch.randn(d, device=_dev()) * 0.1).requires_grad_()
    y = native.depth_mix(src, qy, gn, 1e-6)
    src2 = [s.detach().clone().requires_grad_() for s in src]
    q2, g2 = qy.detach().clone().requires_grad_(), gn.detach().clone().requires_grad_()
    yr = ref.depth_mix(src2, q2, g2, 1e-6)
    _close(y, yr, 1e-4, 1e-4)
    gy = torch.randn_like(yr)
    y.backward(gy), yr.backward(gy)
    for a, b in zip(src, src2):
        _close(a.grad, b.grad, 1e-4, 1e-3, "dsrc")
    _close(qy.grad, q2.grad, 1e-3, 1e-3, "dq")
    _close(gn.grad, g2.grad, 1e-3, 1e-3, "dgain")


@pytest.mark.parametrize("s,V", [(1, 4096), (4, 4096), (1, 1000)])
def test_fused_linear_ce(s, V):
    from gdn_hybrid_architecture_ideas_b200.train.fused_head import _FusedLinearCE, fused_linear_ce

    n, d = 700, 256
    h = torch.randn(n, d, device=_dev()).to(torch.bfloat16).requires_grad_()
    W = (torch.randn(V, d, device=_dev()) * 0.05).requires_grad_()
    t = torch.randint(0, V, (n, s), device=_dev())
    a = torch.rand(n, s, device=_dev()) / n
    a[5] = 0
    b = a.sum(1) * 1e-2
    loss, ce, lse = fused_linear_ce(h, W, t, a, b, 256)
    loss.backward()
    hr = h.detach().float().requires_grad_()
    Wr = W.detach().to(torch.bfloat16).float().requires_grad_()
    lossr, cer, lser = _FusedLinearCE.apply(hr, Wr, t, a, b, 256)
    lossr.backward()
    _close(loss, lossr, 1e-3, 1e-3, "loss")
    _close(lse, lser, 2e-3, 1e-3, "lse")
    _close(h.grad, hr.grad, 2e-5, 5e-2, "dh")
    _close(W.grad, Wr.grad, 2e-5, 5e-2, "dW")


def test_adamw_and_sumsq():
    from gdn_hybrid_architecture_ideas_b200.ops import native

    n = 1 << 20
    p = torch.randn(n, device=_dev())
    g = torch.randn(n, device=_dev())
    m, v = torch.zeros(n, device=_dev()), torch.zeros(n, device=_dev())
    lp = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ref_p.grad = g * 0.5
        opt.step()
        native.adamw_(p, g, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, torch.tensor(0.5, device=_dev()))
    _close(p, ref_p.detach(), 1e-6, 1e-5)
    _close(lp, p, 1e-2, 1e-2)
    _close(native.sumsq(g), g.double().pow(2).sum(), 1.0, 1e-5)


@pytest.mark.parametrize("L,cap,docs,Hq,Hkv,ramp", [(256, None, False, 4, 2, False), (384, 100, False, 4, 1, False), (300, 64, True, 2, 2, False),
                                                    (512, 200, True, 8, 2, False), (1024, None, True, 2, 1, False), (1024, 300, False, 2, 1, True),
                                                    (640, None, False, 2, 2, True)])
def test_attention_kernels(L, cap, docs, Hq, Hkv, ramp):
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    B, hd = 2, 64
    g = torch.Generator().manual_seed(L + Hq)
    def mk(h):
        return (torch.randn(B, L, h, hd, generator=g) * 0.7).to(_dev(), torch.bfloat16)
    q, qf, k, kf, v = mk(Hq), mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv)
    if ramp:      # key norms grow along the row, so later key tiles raise the row maxima by many powers of two
        grow = torch.linspace(0.2, 9.0, L, device=_dev())[None, :, None, None]
        k, kf = (k.float() * grow).to(torch.bfloat16), (kf.float() * grow).to(torch.bfloat16)
    doc = torch.zeros(B, L, dtype=torch.long, device=_dev())
    if docs:
        doc[0, L // 3:] = 1
        doc[0, L // 3 + 5:] = 2
        doc[1, L - 7:] = 4
    idx = torch.arange(L, device=_dev())[None].expand(B, L)
    start = torch.where(torch.cat([torch.ones(B, 1, dtype=torch.bool, device=_dev()), doc[:, 1:] != doc[:, :-1]], 1), idx, torch.zeros_like(idx)).cummax(1).values
    pos = idx - start
    leaves = [t.clone().requires_grad_() for t in (q, k, v, qf, kf)]
    o = native.attention(leaves[0], leaves[1], leaves[2], doc, leaves[3] if cap else None, leaves[4] if cap else None, cap, pos, single_doc=not docs)
    native.check_status()
    refs = [t.float().requires_grad_() for t in (q, k, v, qf, kf)]
    orf = ref.attention(refs[0], refs[1], refs[2], idx, doc, idx, doc, None, refs[3] if cap else None, refs[4] if cap else None, cap)
    _close(o, orf, 2e-2, 2e-2, "o")
    go = torch.randn_like(orf)
    o.backward(go.to(o.dtype))
    orf.backward(go)
    native.check_status()
    names = ["dq", "dk", "dv", "dq_far", "dk_far"]
    for n, a, b in zip(names, leaves, refs):
        if b.grad is None:
            continue
        _close(a.grad, b.grad, 4e-2, 4e-2, n)


@pytest.mark.parametrize("L,dv,H,docs,with_state,rep,beta_max", [(128, 128, 2, False, False, 1, 1), (256, 256, 2, True, True, 1, 1),
                                                                  (200, 256, 1, True, False, 1, 1), (192, 128, 4, True, False, 2, 1),
                                                                  (256, 256, 2, True, True, 1, 2)])
def test_gdn_delta_rule_kernels(L, dv, H, docs, with_state, rep, beta_max):
    from gdn_hybrid_architecture_ideas_b200.ops import gdn_native, native, reference as ref

    B, dk = 2, 128
    g_ = torch.Generator().manual_seed(L + dv)
    q = torch.nn.functional.normalize(torch.randn(B, L, H // rep, dk, generator=g_), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(B, L, H // rep, dk, generator=g_), dim=-1)
    v = torch.randn(B, L, H, dv, generator=g_)
    g = -torch.rand(B, L, H, generator=g_) * 0.5
    beta = torch.rand(B, L, H, generator=g_) * beta_max      # 2: write strengths past 1 (negative eigenvalues)
    S0 = torch.randn(B, H, dk, dv, generator=g_) * 0.1 if with_state else None
    start = torch.zeros(B, L, dtype=torch.bool)
    if docs:
        start[0, 70] = True
        start[1, 3] = True
        start[1, L - 2] = True
    dev = _dev()
    leaves = [t.to(dev).to(torch.bfloat16 if i < 3 else torch.float32).requires_grad_() for i, t in enumerate((q, k, v, g, beta))]
    S0d = S0.to(dev).requires_grad_() if with_state else None
    o, S = gdn_native.delta_rule(*leaves, start.to(dev), S0d, 64, need_state=with_state)
    native.check_status()
    refs = [t.detach().float().requires_grad_() for t in leaves]
    S0r = S0.to(dev).requires_grad_() if with_state else torch.zeros(B, H, dk, dv, device=dev)
    orf, Sr = ref.chunked_delta_rule(refs[0].repeat_interleave(rep, dim=2), refs[1].repeat_interleave(rep, dim=2), *refs[2:], start.to(dev), S0r, 64)
    slack = beta_max                # the inverse's entries reach about beta_max: bf16 rounds them at that absolute error
    _close(o, orf, 2e-2 * slack, 3e-2, "o")
    go = torch.randn_like(orf)
    if with_state:
        _close(S, Sr, 2e-2 * slack, 3e-2, "S")
        gS = torch.randn_like(Sr) * 0.1
        torch.autograd.backward([o, S], [go.to(o.dtype), gS])
        torch.autograd.backward([orf, Sr], [go, gS])
        _close(S0d.grad, S0r.grad, 3e-2 * slack, 5e-2, "dS0")
    else:
        o.backward(go.to(o.dtype))
        orf.backward(go)
    native.check_status()
    for n, a, b in zip(("dq", "dk", "dv", "dg", "dbeta"), leaves, refs):
        scale = b.grad.abs().max().item()
        _close(a.grad, b.grad, 3e-2 * scale * slack, 5e-2, n)


def test_cuda_graph_training_matches_eager():
    """Replaying the captured micro-batch (forward, head, backward) trains like the eager step."""
    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.ops import native
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    def run(graphs):
        model = C.hybrid_model_config("60m", full=True)
        model.encoder.n_layers, model.encoder.nope_global_layers, model.vocab_size = 4, (0,), 4096
        cfg = C.TrainConfig(model=model, data=C.DataConfig(kind="synthetic", seq_len=256, batch_size=4, seed=5), steps=100, seed=7)
        cfg.autocast, cfg.head_impl, cfg.metrics_jsonl, cfg.log_every, cfg.micro_batch_size = "bfloat16", "fused", False, 0, 2
        cfg.optim.warmup_steps, cfg.optim.lr, cfg.cuda_graphs = 1, 1e-4, graphs
        t = Trainer(cfg, None, None)
        losses = [t.train_step()["loss"] for _ in range(6)]
        native.check_status()
        return losses, t.flat.params.detach().clone(), t

    l0, p0, _ = run("none")
    l1, p1, t1 = run("microbatch")
    assert t1.graphs.graph is not None and t1.graphs.seen == 12
    assert max(abs(a - b) for a, b in zip(l0, l1)) < 2e-2, (l0, l1)
    diff = (p0 - p1).abs()
    assert diff.max().item() < 1e-3 and diff.mean().item() < 2e-5, (diff.max().item(), diff.mean().item())


def test_wgrad_accumulates_into_main_grad():
    """`wgrad_accum: fp32`: the weight-gradient GEMM adds into the parameter's fp32 main gradient; autograd gets none."""
    from gdn_hybrid_architecture_ideas_b200.models.linear import Linear
    from gdn_hybrid_architecture_ideas_b200.ops import native

    lin = Linear(256, 384).to(_dev())
    x = torch.randn(200, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(200, 384, device=_dev(), dtype=torch.bfloat16)
    lin(x).backward(go)
    want = lin.weight.grad.clone()
    lin.weight.grad = None
    lin.weight.main_grad = torch.full_like(want, 0.5)
    native.WGRAD_INTO_MAIN = True
    try:
        for _ in range(2):
            lin(x).backward(go)
    finally:
        native.WGRAD_INTO_MAIN = False
    assert lin.weight.grad is None
    _close(lin.weight.main_grad, 2 * want + 0.5, 2e-2 * float(want.abs().max()), 1e-2, "main grad")
    native.check_status()


@pytest.mark.parametrize("gate,cap,frac,docs", [("elementwise", 64, 0.25, True), ("none", None, 0.5, False), ("elementwise", None, 0.0, False)])
def test_attention_layer_fused_prep(gate, cap, frac, docs):
    """The layer with the fused q / k preparation (norm + rotations + far copies, output gate) against the same layer
    run in float32 through the PyTorch statements."""
    import copy

    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.config import AttentionConfig
    from gdn_hybrid_architecture_ideas_b200.models.attention import GatedAttention
    from gdn_hybrid_architecture_ideas_b200.models.sequence import sequence_context
    from gdn_hybrid_architecture_ideas_b200.ops import native

    torch.manual_seed(11)
    B, L, d = 2, 320, 256
    cfg = AttentionConfig(n_q_heads=4, n_kv_heads=2, head_dim=64, gate=gate, rope_fraction=frac, rope_max_distance=cap, rope_theta=10000.0)
    layer = GatedAttention(d, cfg, 1e-6).to(_dev())
    with torch.no_grad():
        layer.q_norm.weight.normal_(0, 0.2)
        layer.k_norm.weight.normal_(0, 0.2)
    oracle = copy.deepcopy(layer).float()
    layer = layer.to(torch.bfloat16)
    for p, q in zip(layer.parameters(), oracle.parameters()):
        q.data.copy_(p.data.float())
    doc = torch.zeros(B, L, dtype=torch.long, device=_dev())
    if docs:
        doc[0, 100:] = 1
        doc[1, 37:] = 1
        doc[1, 250:] = 2
    x = torch.randn(B, L, d, device=_dev()).to(torch.bfloat16)
    go = torch.randn(B, L, d, device=_dev()).to(torch.bfloat16)
    xa = x.clone().requires_grad_(True)
    xb = x.float().requires_grad_(True)
    ctx, _ = sequence_context(doc)
    assert layer.fused_prep_ok(xa)
    y, keys = layer(xa, ctx)
    y.backward(go)
    native.check_status()
    ops.set_mode("reference")
    try:
        ctx2, _ = sequence_context(doc)
        y2, keys2 = oracle(xb, ctx2)
        y2.backward(go.float())
    finally:
        ops.set_mode("native")
    _close(keys.k, keys2.k, 3e-2, 2e-2, "k")
    if cap is not None:
        _close(keys.k_far, keys2.k_far, 3e-2, 2e-2, "k_far")
    scale = y2.abs().max().item()
    _close(y, y2, 3e-2 * scale, 3e-2, "y")
    _close(xa.grad, xb.grad, 4e-2 * xb.grad.abs().max().item(), 3e-2, "dx")
    for (n, p), q in zip(layer.named_parameters(), oracle.parameters()):
        assert p.grad is not None, n
        _close(p.grad, q.grad, 4e-2 * q.grad.abs().max().item() + 1e-3, 3e-2, f"d{n}")


@pytest.mark.parametrize("n,Q,d", [(2, 7, 1024), (4, 3, 1024), (3, 2, 512), (5, 8, 2048)])
def test_depth_mix_multi(n, Q, d):
    """Q readers over the same sources in one kernel against the PyTorch statement of each reader; one output is left
    without a gradient (a reader whose mix is not used downstream)."""
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    torch.manual_seed(n * 10 + Q)
    rows = (3, 70)
    srcs = [(torch.randn(*rows, d, device=_dev()) * (1 + i)).requires_grad_() for i in range(n)]
    qs = [(torch.randn(d, device=_dev()) * 0.1).requires_grad_() for _ in range(Q)]
    gs = [(torch.randn(d, device=_dev()) * 0.1).requires_grad_() for _ in range(Q)]
    outs = native.depth_mix_multi(srcs, list(zip(qs, gs)), 1e-6)
    native.check_status()
    rs = [s.detach().clone().requires_grad_() for s in srcs]
    rq = [q.detach().clone().requires_grad_() for q in qs]
    rg = [g.detach().clone().requires_grad_() for g in gs]
    want = [ref.depth_mix(rs, q, g, 1e-6) for q, g in zip(rq, rg)]
    for a, b in zip(outs, want):
        _close(a, b, 1e-4, 1e-4, "mix")
    go = [torch.randn_like(o) for o in outs]
    used = range(Q - 1)           # the last reader's output gets no gradient
    torch.autograd.backward([outs[i] for i in used], [go[i] for i in used])
    torch.autograd.backward([want[i] for i in used], [go[i] for i in used])
    native.check_status()
    for a, b in zip(srcs, rs):
        _close(a.grad, b.grad, 2e-4 * b.grad.abs().max().item(), 1e-3, "dsrc")
    for i in used:
        _close(qs[i].grad, rq[i].grad, 2e-3 * rq[i].grad.abs().max().item(), 2e-3, "dquery")
        _close(gs[i].grad, rg[i].grad, 2e-3 * rg[i].grad.abs().max().item() + 1e-6, 2e-3, "dgain")
    assert qs[Q - 1].grad is None or float(qs[Q - 1].grad.abs().max()) == 0.0


def test_prenorm_passthrough():
    """(RMSNorm(x), x) as one node: the two gradients of x are summed inside the norm's backward kernel."""
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    torch.manual_seed(5)
    x = torch.randn(4, 300, 1024, device=_dev()).requires_grad_()
    w = (torch.randn(1024, device=_dev()) * 0.1).requires_grad_()
    y, xp = ops.prenorm(x, w, 1e-6)
    assert y.dtype == torch.bfloat16 and xp.data_ptr() == x.data_ptr()
    gy, gx = torch.randn_like(y), torch.randn_like(x)
    torch.autograd.backward([y, xp], [gy, gx])
    native.check_status()
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-6)
    torch.autograd.backward([yr, xr * 1.0], [gy.float(), gx])
    _close(y, yr, 2e-2, 1e-2, "y")
    _close(x.grad, xr.grad, 2e-2, 1e-2, "dx")
    _close(w.grad, wr.grad, 5e-2 * wr.grad.abs().max().item(), 2e-2, "dw")
    x2 = x.detach().clone().requires_grad_()
    y2, xp2 = ops.prenorm(x2, w, 1e-6)
    xp2.backward(gx)                       # only the pass-through is used
    assert torch.equal(x2.grad, gx)


@pytest.mark.parametrize("s,V", [(1, 4096), (3, 32768)])
def test_ce_grad_fixed_form(s, V):
    """The fixed cross-entropy in the CE kernel against the PyTorch statement, with rows collapsed onto their target (the
    argmax column) and onto another column."""
    from gdn_hybrid_architecture_ideas_b200.ops import native
    from gdn_hybrid_architecture_ideas_b200.train import fused_head as FH

    torch.manual_seed(V + s)
    n = 64
    logits = (torch.randn(n, V, device=_dev()) * 2).contiguous()
    t = torch.randint(0, V, (n, s), device=_dev())
    logits[0, t[0, 0]] += 40.0
    logits[1, (t[1, 0] + 1) % V] += 40.0
    if s > 1:
        t[2, 1] = t[2, 0]
    a = torch.rand(n, s, device=_dev())
    a[3, 0] = 0.0
    b = torch.rand(n, device=_dev()) * 0.01
    grad = torch.empty(n, V, dtype=torch.bfloat16, device=_dev())
    ce = torch.empty(n, device=_dev())
    lse = torch.empty(n, device=_dev())
    native.ext().ce_grad(logits, t, a, b, grad, ce, lse, True)
    native.check_status()
    wce, wlse, wg = FH._ce_grad_chunk(logits.double(), t, a.double(), b.double(), fixed=True)
    _close(lse, wlse, 1e-4, 1e-5, "lse")
    _close(ce, wce, 1e-4, 1e-4, "ce")
    _close(grad, wg, 1e-5, 1e-2, "grad")
    b0 = torch.zeros_like(b)
    native.ext().ce_grad(logits, t, a, b0, grad, ce, lse, True)
    tiny = grad[0, t[0, 0]].float().item()
    want0 = FH._ce_grad_chunk(logits.double(), t, a.double(), b0.double(), fixed=True)[2][0, t[0, 0]].item()
    assert abs(tiny - want0) <= 2e-2 * abs(want0), (tiny, want0)
    if s == 1:
        assert want0 < 0 and abs(want0) < 1e-8, want0          # -a sigmoid(L'): tiny, not zero
    native.ext().ce_grad(logits, t, a, b0, grad, ce, lse, False)
    if s == 1:
        assert abs(grad[0, t[0, 0]].float().item()) < 1e-6      # the standard form's softmax_t - 1 has rounded away (to a few fp32 ulps of a)


@pytest.mark.parametrize("s", [1, 4])
def test_embedding_kernels(s):
    """Gather (bags: mean of the rows) and the scatter-add backward against torch."""
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    torch.manual_seed(s)
    V, d, B, L = 1000, 1024, 3, 257
    w = torch.randn(V, d, device=_dev(), requires_grad=True)
    tok = torch.randint(0, V, (B, L) if s == 1 else (B, L, s), device=_dev())
    tok[0, :5] = 7                       # repeated ids: their gradients add up
    out = native.embedding(tok, w)
    wr = w.detach().clone().requires_grad_()
    want = ref.embedding(tok, wr)
    _close(out, want, 1e-6, 1e-6, "rows")
    g = torch.randn_like(want)
    out.backward(g)
    want.backward(g)
    native.check_status()
    _close(w.grad, wr.grad, 1e-5, 1e-5, "table gradient")


@pytest.mark.parametrize("Hk,Hv,dv", [(2, 2, 128), (2, 4, 256)])
def test_gdn_decode_step_kernel(Hk, Hv, dv):
    """One cached token of the gated delta rule on the in-place step kernel against the per-token recurrence, over a few
    steps, with a row that starts a new document."""
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    torch.manual_seed(Hv)
    B, dk = 5, 128
    S = torch.randn(B, Hv, dk, dv, device=_dev()) * 0.1
    Sr = S.clone()
    buf = S
    for step in range(3):
        q = torch.nn.functional.normalize(torch.randn(B, 1, Hk, dk, device=_dev()), dim=-1) * dk ** -0.5
        k = torch.nn.functional.normalize(torch.randn(B, 1, Hk, dk, device=_dev()), dim=-1)
        v = torch.randn(B, 1, Hv, dv, device=_dev())
        g = -torch.rand(B, 1, Hv, device=_dev())
        beta = torch.rand(B, 1, Hv, device=_dev()) * 2
        start = torch.zeros(B, 1, dtype=torch.bool, device=_dev())
        start[1, 0] = step == 1
        with torch.no_grad():
            o, S = ops.delta_rule(q.bfloat16(), k.bfloat16(), v.bfloat16(), g, beta, start, S, inplace_state=True)
            rep = Hv // Hk
            qr, kr = (t.bfloat16().float().repeat_interleave(rep, dim=2) for t in (q, k))
            orf, Sr = ref.delta_rule_recurrence(qr, kr, v.bfloat16().float(), g, beta, start, Sr)
        native.check_status()
        assert S is buf                      # updated in place
        _close(o, orf, 2e-2, 2e-2, f"o at step {step}")
        _close(S, Sr, 1e-5, 1e-5, f"S at step {step}")
    with torch.no_grad():
        o2, S2 = ops.delta_rule(q.bfloat16(), k.bfloat16(), v.bfloat16(), g, beta, start, S)
    assert S2 is not S


@pytest.mark.parametrize("L", [1, 2, 70])
def test_gdn_prep_with_history(L):
    """A chunk that continues cached rows (K - 1 cached inputs with their document ids, -1 where none) on the prep kernel
    against the PyTorch statement."""
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.ops import native, reference as ref

    torch.manual_seed(L)
    B, hk, hv, dk, dv = 3, 2, 2, 128, 256
    C = 2 * hk * dk + hv * dv
    u = torch.randn(B, L, C, device=_dev()).to(torch.bfloat16)
    w = torch.randn(C, 4, device=_dev()) * 0.5
    hist = torch.randn(B, 3, C, device=_dev()).to(torch.bfloat16)
    hist_doc = torch.tensor([[5, 5, 5], [-1, -1, 4], [2, 3, 3]], device=_dev())
    doc = torch.tensor([[5], [4], [4]], device=_dev()).expand(B, L).contiguous()
    if L > 2:
        doc = doc.clone()
        doc[0, L // 2:] = 6
    with torch.no_grad():
        qkv, h, hd = ops.gdn_prep(u, doc, w, hk, hv, dk, dv, hist, hist_doc, packed=True)
        q, k, v, hr, hdr = ref.gdn_prep(u.float(), doc, w, hk, hv, dk, dv, hist.float(), hist_doc)
    native.check_status()
    want = torch.cat([q.flatten(2), k.flatten(2), v.flatten(2)], dim=-1)
    assert qkv.shape == want.shape
    _close(qkv, want, 1e-2, 2e-2, "qkv")
    assert torch.equal(hd, hdr) and torch.equal(h.float(), hr)


@pytest.mark.parametrize("arm", ["block", "heads", "token", "scalars", "canon", "negeig", "shapes"])
def test_experimental_arms_on_the_device(arm):
    """Each experimental arm, forward and backward on the CUDA kernels under bf16 autocast, against the same model on the
    PyTorch statements: loss and gradient norm agree within bf16 noise."""
    from gdn_hybrid_architecture_ideas_b200 import config as C, ops
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.ops import native

    torch.manual_seed(3)
    cfg = C.hybrid_model_config("60m", full=arm in ("heads", "token"))
    cfg.encoder.n_layers, cfg.encoder.nope_global_layers, cfg.vocab_size = 8, (1,), 2048
    cfg.encoder.attention.rope_max_distance = 96
    e = cfg.encoder
    if arm == "block":
        e.attn_res = "block"
    if arm == "heads":
        e.attn_res_heads, e.gdn_write_mix, e.gdn_write_variant = 4, "none", "none"
    if arm == "token":
        e.attn_res_query, e.gdn_write_mix, e.gdn_write_variant = "token", "none", "none"
    if arm == "scalars":
        e.layer_scalars = "skip_x0_span"
    if arm == "canon":
        e.canon_kernel, e.canon_init = 4, "uniform"
    if arm == "negeig":
        e.gdn.negeig.beta_max = 2
    if arm == "shapes":
        e.gdn_shape_by_layer = {0: (2, 4, 128), 3: (4, 4, 128)}
    model = build_model(cfg).cuda()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    B, L = 2, 384
    tok = torch.randint(0, 2048, (B, L), device="cuda")
    doc = torch.zeros(B, L, dtype=torch.long, device="cuda")
    doc[1, 200:] = 1

    def run():
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(tok, doc)
        loss = torch.nn.functional.cross_entropy(out.logits[:, :-1].flatten(0, 1).float(), tok[:, 1:].flatten())
        loss.backward()
        gn = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in model.parameters() if p.grad is not None))
        return loss.item(), gn.item()

    la, ga = run()
    native.check_status()
    ops.set_mode("reference")
    try:
        lb, gb = run()
    finally:
        ops.set_mode("native")
    assert abs(la - lb) < 2e-2 * abs(lb), (la, lb)
    assert abs(ga - gb) < 8e-2 * gb, (ga, gb)
