"""Block-scaled formats: bytes and values equal the reference's emulations; quantised linears train (finite, close to
bf16) and are inactive in evaluation mode."""

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import build_model
from gdn_hybrid_architecture_ideas_b200.ops import lowp
from tests.helpers import random_rows


def _samples():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(48, 100, generator=g) * torch.logspace(-6, 4, 48)[:, None]
    x[0, :32] = 0
    x[1, 5] = float("inf")
    x[2, 7] = float("nan")
    x[3] *= 1e30
    return x


def test_mxfp8_bytes_equal_reference(reference):
    import ced.model.mxfp8 as rmx

    x = _samples()
    for dim in (-1, 0):
        q, b = lowp.mx_quantize(x, dim)
        rq, rb = rmx.quantize(x, dim)
        assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8)) and torch.equal(b, rb)
        d, rd = lowp.mx_dequantize(q, b, dim), rmx.dequantize(rq, rb, dim)
        assert torch.equal(torch.nan_to_num(d, nan=7.0), torch.nan_to_num(rd, nan=7.0))


def test_nvfp4_values_equal_reference(reference):
    import ced.model.nvfp4 as rnv

    g = torch.Generator().manual_seed(4)
    x = torch.randn(40, 70, generator=g) * 3
    assert torch.equal(lowp.nvfp4_fake(x), rnv.fake_quantize(x))
    assert torch.equal(lowp.nvfp4_fake(x, block_2d=True), rnv.fake_quantize(x, block_2d=True))
    assert torch.equal(lowp.rht_matrix(), rnv.rht_matrix())
    assert torch.equal(lowp.rht_tokens(x, lowp.rht_matrix()), rnv.rht_tokens(x, rnv.rht_matrix()))
    torch.manual_seed(9)
    a = lowp.nvfp4_fake(x, stochastic=True)
    torch.manual_seed(9)
    b = rnv.fake_quantize(x, stochastic=True)
    assert torch.equal(a, b)


@pytest.mark.parametrize("scaling", ["mxfp8", "rowwise", "tensorwise"])
def test_fp8_linear_matches_reference(reference, scaling):
    import ced.model.fp8 as rfp8

    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 20, 64, generator=g, requires_grad=True)
    w = (torch.randn(96, 64, generator=g) * 0.1).requires_grad_()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    kind = "mxfp8" if scaling == "mxfp8" else "fp8_" + scaling
    y = lowp.Recipe(kind).emulated_linear(x, w)
    yr = rfp8.FP8LinearFunction.apply(x2, w2, scaling, torch.float32)
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-5)
    gy = torch.randn(3, 20, 96, generator=g)
    y.backward(gy), yr.backward(gy)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5, rtol=1e-4)
    assert torch.allclose(w.grad, w2.grad, atol=1e-4, rtol=1e-4)


def test_quartet2_linear_equals_the_reference_draw_for_draw(reference):
    """The Quartet II recipe: the four-over-six forward quantiser value for value; the backward (one sign vector a call, MS-EDEN
    with stochastic scale roundings) bit for bit under the same seed; the estimator's error against the exact products; the
    stochastic block scales unbiased around the corrected scale."""
    import ced.model.nvfp4 as rnv

    g = torch.Generator().manual_seed(6)
    x = torch.randn(3, 40, 72, generator=g, requires_grad=True)
    w = (torch.randn(48, 72, generator=g) * 0.05).requires_grad_()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    a = torch.rand(4000, generator=g) * 7
    assert torch.equal(lowp.e2m1_round_away(a), rnv.e2m1_round_away(a)) and float(lowp.e2m1_round_away(torch.tensor([0.25, 0.75, 2.5, 5.0, 9.0])).sum()) == 0.5 + 1 + 3 + 6 + 6
    for four in (True, False):
        v, sd = lowp.q2_rtn_quantize(x.detach().reshape(-1, 72), four)
        rv, rsd = rnv.quartet2_rtn_quantize(x.detach().reshape(-1, 72), four)
        assert torch.equal(v, rv) and torch.equal(sd, rsd) and torch.equal(v.bfloat16().float(), v)          # operands exact in bf16
    y = lowp.Recipe("quartet2").emulated_linear(x, w)
    yr = rnv.Quartet2LinearFunction.apply(x2, w2, rnv.hadamard_matrix(128) / 128 ** 0.5, torch.float32)
    assert torch.equal(y, yr)
    gy = torch.randn(3, 40, 48, generator=g)
    torch.manual_seed(11)
    y.backward(gy)
    torch.manual_seed(11)
    yr.backward(gy)
    assert torch.equal(x.grad, x2.grad) and torch.equal(w.grad, w2.grad)
    exact_dx, exact_dw = gy @ w.detach(), gy.reshape(-1, 48).t() @ x.detach().reshape(-1, 72)
    assert (x.grad - exact_dx).norm() / exact_dx.norm() < 0.3 and (w.grad - exact_dw).norm() / exact_dw.norm() < 0.3
    c = torch.tensor([[0.3], [17.0], [100.0]])
    down, up = lowp.e4m3_neighbours(c)
    assert (down <= c).all() and (c <= up).all() and torch.equal(lowp.e4m3_neighbours(torch.tensor([16.0]))[0], torch.tensor([16.0]))
    t = torch.randn(64, 256, generator=g)
    T = lowp.q2_hadamard()
    draws = torch.stack([lowp.q2_eden_quantize(t, T, torch.rand(64, 16, generator=g))[0] for _ in range(200)]).mean(0)
    v0, s0 = lowp.q2_eden_quantize(t, T, torch.full((64, 16), 0.5))
    rot = lowp.q2_rotate(t, T)
    assert ((draws * s0 - rot).norm() / rot.norm()) < ((v0 * s0 - rot).norm() / rot.norm())            # averaging the draws approaches the rotated tensor
    assert (T @ T.t() - torch.eye(128)).abs().max() < 1e-6


@pytest.mark.parametrize("which", ["mxfp8", "nvfp4", "quartet2"])
def test_quantised_model_trains_and_evaluates_in_high_precision(which):
    cfg = C.tiny_control_config()
    cfg.d_model, cfg.ffn_hidden = 64, 192
    if which == "mxfp8":
        cfg.fp8.mode, cfg.fp8.scaling = "linears", "mxfp8"
    else:
        cfg.nvfp4.mode = "all_linears"
        cfg.nvfp4.recipe = "nvidia" if which == "nvfp4" else "quartet2"
    if which == "quartet2":
        bad = C.tiny_control_config()
        bad.nvfp4.mode, bad.nvfp4.recipe, bad.nvfp4.rht = "all_linears", "quartet2", False
        with pytest.raises(ValueError, match="quartet2"):
            build_model(bad)
    torch.manual_seed(0)
    m = build_model(cfg)
    plain = C.tiny_control_config()
    torch.manual_seed(0)
    base = build_model(plain)
    quantised = [n for n, mod in m.named_modules() if getattr(mod, "precision", "bf16") != "bf16"]
    assert quantised and not any(n.endswith(("in_proj_a", "in_proj_b")) for n in quantised)
    tok, doc = random_rows(2, 32)
    m.eval(), base.eval()
    assert torch.equal(m(tok, doc).logits, base(tok, doc).logits)          # evaluation runs in high precision
    m.train(), base.train()
    a, b = m(tok, doc).logits, base(tok, doc).logits
    rel = ((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt()).item()
    assert torch.isfinite(a).all() and rel < (0.6 if which == "mxfp8" else 1.5), rel
    a.logsumexp(-1).sum().backward()
    assert all(torch.isfinite(p.grad).all() for p in m.parameters() if p.grad is not None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [-1, 0])
def test_mxfp8_kernel_equals_emulation(dtype, dim):
    """The MXFP8 round-trip kernel gives, value for value, what the tensor-op emulation gives (which equals the reference byte
    for byte): ragged block counts, zero blocks, tiny and huge magnitudes, blocks holding inf or NaN."""
    from gdn_hybrid_architecture_ideas_b200 import ops

    g = torch.Generator().manual_seed(3)
    x = torch.randn(203, 150, generator=g) * torch.exp(torch.randn(203, 150, generator=g) * 4)
    x[5, :40] = 0.0
    x[:40, 7] = 0.0
    x[9, 3] = 3e38
    x[10, 100] = 1e-41
    x[11, 64] = float("inf")
    x[100, 11] = float("nan")
    x = x.to("cuda").to(dtype).contiguous()
    got = lowp.mx_fake(x, dim)
    ops.set_mode("reference")
    try:
        want = lowp.mx_fake(x, dim)
    finally:
        ops.set_mode("native")
    assert got.dtype == torch.bfloat16 and want.dtype == torch.float32
    same = (got.float() == want) | (torch.isnan(got.float()) & torch.isnan(want))
    assert bool(same.all()), f"{int((~same).sum())} values differ; first at {torch.nonzero(~same)[0].tolist()}"
    assert bool(torch.isnan(want).any()) and bool((want == 0).any())


# ---------------------------------------------------------------------------------------------------- block-scaled tensor-core path

def _mx_inputs(R, C, seed, dtype=torch.float32, wide=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(R, C, generator=g)
    if wide:      # magnitudes over many binades, a zero block, an infinity and a NaN
        x = x * torch.logspace(-5, 3, R)[:, None]
        x[0, :32] = 0
        x[1, 5] = float("inf")
        x[2, 40] = float("nan")
    return x.to(dtype).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(256, 384), (160, 128), (4096, 1024)])
def test_mx_quantise_kernel_bytes_equal_emulation(dtype, shape):
    """The quantise kernel's E4M3 bytes and E8M0 exponents, in both block orientations, equal the tensor-op emulation's."""
    from gdn_hybrid_architecture_ideas_b200.ops import native

    R, C = shape
    x = _mx_inputs(R, C, 11, dtype)
    qr, sr, qc, sc = native.mx_quantize(x, True, True)
    wq, wb = lowp.mx_quantize(x.float().cpu(), -1)
    assert torch.equal(qr.cpu(), wq.view(torch.uint8))
    assert torch.equal(lowp.mx_cells_to_rows(sr.cpu(), R, C), wb)
    tq, tb = lowp.mx_quantize(x.float().cpu().t().contiguous(), -1)      # blocks along R of x = blocks along the last dim of x^T
    assert torch.equal(qc.cpu(), tq.view(torch.uint8))
    assert torch.equal(lowp.mx_cells_to_rows(sc.cpu(), C, R), tb)


@pytest.mark.gpu
@pytest.mark.parametrize("mnk", [(256, 256, 256), (384, 128, 1024), (4096, 2816, 1024), (6400, 640, 512), (160, 96, 256)])
def test_mx_gemm_equals_dequantised_product(mnk):
    """The block-scaled product equals the fp32 product of the dequantised operands (same values, other summation order)."""
    from gdn_hybrid_architecture_ideas_b200.ops import native

    M, N, K = mnk
    a, b = _mx_inputs(M, K, 21, wide=False), _mx_inputs(N, K, 22, wide=False) * 0.05
    a = a * torch.logspace(-2, 2, M, device="cuda")[:, None]
    aq, asf, _, _ = native.mx_quantize(a, True, False)
    bq, bsf, _, _ = native.mx_quantize(b, True, False)
    got = native.gemm_mx(aq, asf, bq, bsf, out_dtype=torch.float32)
    ad = lowp.mx_dequantize(aq.view(lowp.E4M3), lowp.mx_cells_to_rows(asf, M, K))
    bd = lowp.mx_dequantize(bq.view(lowp.E4M3), lowp.mx_cells_to_rows(bsf, N, K))
    want = ad.double() @ bd.double().t()
    torch.cuda.synchronize()
    native.check_status()
    err = (got.double() - want).abs().max() / want.abs().max()
    assert err < 1e-5, err
    got16 = native.gemm_mx(aq, asf, bq, bsf)
    assert (got16.double() - want).abs().max() / want.abs().max() < 1e-2
    acc = torch.ones(M, N, device="cuda")
    native.gemm_mx(aq, asf, bq, bsf, out=acc, accumulate=True)
    assert ((acc.double() - 1) - want).abs().max() / want.abs().max() < 1e-5


@pytest.mark.gpu
def test_mx_linear_equals_emulated_linear():
    """Forward, input gradient and weight gradient of the tensor-core MXFP8 linear against the emulated recipe in fp32."""
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(4, 128, 256, generator=g)).cuda().to(torch.bfloat16).requires_grad_()
    w = (torch.randn(384, 256, generator=g) * 0.05).cuda().requires_grad_()
    dy = torch.randn(4, 128, 384, generator=g).cuda().to(torch.bfloat16)
    y = lowp._MxLinear.apply(x, w)
    y.backward(dy)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    y2 = lowp._LowpLinear.apply(x2, w2, lowp.Recipe("mxfp8"), False)
    y2.backward(dy)
    for got, want, tol in ((y, y2, 1e-2), (x.grad, x2.grad, 1e-2), (w.grad, w2.grad, 1e-4)):
        scale = want.float().abs().max()
        assert (got.float() - want.float()).abs().max() / scale < tol


@pytest.mark.gpu
def test_mx_quantise_and_gemm_timing_smoke():
    """The 200M model's widest projection shape runs clean through quantise + product (status word stays 0)."""
    from gdn_hybrid_architecture_ideas_b200.ops import native

    x = torch.randn(8192, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(5632, 1024, device="cuda") * 0.02
    xq, xs, _, _ = native.mx_quantize(x)
    wq, ws, _, _ = native.mx_quantize(w)
    y = native.gemm_mx(xq, xs, wq, ws)
    torch.cuda.synchronize()
    native.check_status()
    want = x.float() @ w.t()
    assert (y.float() - want).abs().max() / want.abs().max() < 0.1
