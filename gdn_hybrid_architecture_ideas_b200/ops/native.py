"""CUDA path of the op layer: `torch.autograd.Function`s over the in-tree sm_100a extension `_native.so`.

Precision policy (the reference's "float32 master weights + bfloat16 autocast", ced/train/trainer.py:1241-1886, made
explicit): GEMM operands are bfloat16 with fp32 accumulation; the residual stream, norm statistics, softmaxes, the
loss and the optimizer are fp32. A Linear reads its bfloat16 shadow weight (`weight_lp`, refreshed by the fused
AdamW kernel) when one exists, else casts the master weight.

Importing this module on a machine with a GPU but without the built extension raises: there is no silent fallback.
"""

from __future__ import annotations

import importlib.util
from pathlib import Path

import torch

from . import reference as ref

_SO = Path(__file__).resolve().parent.parent / "_native.so"
_ext = None
_launches = 0
_err = {}


def ext():
    global _ext
    if _ext is None:
        if not _SO.exists():
            raise RuntimeError(f"native extension {_SO} is not built: run `python -m gdn_hybrid_architecture_ideas_b200.build`")
        spec = importlib.util.spec_from_file_location("_native", _SO)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ext = mod
    return _ext


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def err_flag(device) -> torch.Tensor:
    """Per-device int32 status word the tensor-core kernels write when a bounded wait gives up (0 = clean)."""
    key = torch.device(device).index or 0
    if key not in _err:
        _err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err[key]


def check_status(device=None) -> None:
    """Raises if any kernel reported a protocol timeout since the last check (one host read)."""
    for key, flag in _err.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise RuntimeError(f"sm_100a kernel reported status {code} on cuda:{key} (a bounded wait gave up)")


BF16 = torch.bfloat16


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == BF16 else t.to(BF16)


# ------------------------------------------------------------------------------------------------------------ GEMM

def gemm(a, b, out=None, a_mn=False, b_mn=False, accumulate=False, out_dtype=BF16):
    """out = a b^T (+ out): a [M,K] (or [K,M] with a_mn), b [N,K] (or [K,N] with b_mn), bf16 operands."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    ext().gemm(a, b, out, a_mn, b_mn, accumulate, err_flag(a.device))
    _count()
    return out


def mx_quantize(x2: torch.Tensor, rowwise: bool = True, colwise: bool = False):
    """MXFP8 operands of x2 [R, C] (fp32 or bf16; R, C multiples of 32) from one read: (q_row [R, C] E4M3 bytes with blocks
    along C, its scale cells) and / or (q_col [C, R], the transpose with blocks along R, its scale cells), each None when
    not asked for. Scale cells are in the tensor core's layout (csrc/gemm_mx.cu); rows padded to 128 are zero."""
    R, C = x2.shape
    e = ext()
    dev = x2.device

    def pair(rows, k):
        q = torch.empty(rows, k, dtype=torch.uint8, device=dev)
        n = e.mx_scale_bytes(rows, k)
        sf = torch.zeros(n, dtype=torch.uint8, device=dev) if rows % 128 or k % 128 else torch.empty(n, dtype=torch.uint8, device=dev)
        return q, sf
    qr, sr = pair(R, C) if rowwise else (None, None)
    qc, sc = pair(C, R) if colwise else (None, None)
    e.mx_quantize(x2, qr, sr, qc, sc)
    _count()
    return qr, sr, qc, sc


def gemm_mx(a, sfa, b, sfb, out=None, accumulate=False, out_dtype=BF16):
    """out = a b^T (+ out) on the block-scaled tensor-core path: a [M, K], b [N, K] E4M3 bytes with their scale cells."""
    if out is None:
        out = torch.empty(a.shape[0], b.shape[0], dtype=out_dtype, device=a.device)
    ext().gemm_mx(a, sfa, b, sfb, out, accumulate, err_flag(a.device))
    _count()
    return out


def _w_lp(lin) -> torch.Tensor:
    lp = getattr(lin, "weight_lp", None)
    return lp if lp is not None else lin.weight.detach().to(BF16)


def _pad_rows(w: torch.Tensor, mult: int = 8) -> torch.Tensor:
    """Weight [N, K] zero-padded to a multiple of `mult` rows (projections with a handful of outputs, such as the
    per-head decay and beta gates, get 16-byte-aligned output rows this way)."""
    n = w.shape[0]
    if n % mult == 0:
        return w
    out = torch.zeros(-(-n // mult) * mult, w.shape[1], dtype=w.dtype, device=w.device)
    out[:n] = w
    return out


# `wgrad_accum: fp32`: weight-gradient GEMMs add straight into the parameter's fp32 main gradient (the epilogue's
# accumulate mode) and autograd receives no weight gradient, instead of producing a tensor that autograd then adds
# (reference: ced/train/wgrad_accum.py:87-369).
WGRAD_INTO_MAIN = False


def _wgrad(dy2, x2, weight, n):
    main = getattr(weight, "main_grad", None) if WGRAD_INTO_MAIN else None
    if main is not None and main.dtype == torch.float32 and main.shape[0] == n and dy2.shape[1] == n:
        gemm(dy2, x2, out=main, a_mn=True, b_mn=True, accumulate=True)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)[:n]


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, w_lp):
        x2 = _bf16(x).reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        n = w_lp.shape[0]
        w_lp = _pad_rows(w_lp)
        y = gemm(x2, w_lp)
        ctx.save_for_backward(x2, w_lp)
        ctx.xshape, ctx.xdtype, ctx.n, ctx.weight = x.shape, x.dtype, n, weight
        if n != w_lp.shape[0]:
            y = y[:, :n]
        return y.reshape(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        x2, w_lp = ctx.saved_tensors
        dy2 = _bf16(dy).reshape(-1, dy.shape[-1])
        if ctx.n != w_lp.shape[0]:
            dy2 = torch.nn.functional.pad(dy2, (0, w_lp.shape[0] - ctx.n))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w_lp, b_mn=True).view(ctx.xshape)           # dy [M,N] . W [N,K]
            if ctx.xdtype != BF16:
                dx = dx.to(ctx.xdtype)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy2, x2, ctx.weight, ctx.n)          # dy^T [N,M] . x [M,K]
        return dx, dw, None


def linear(x, lin):
    if getattr(lin, "precision", "bf16") != "bf16" and lin.training:
        from . import lowp

        return lowp.native_linear(x, lin)
    return _Linear.apply(x, lin.weight, _w_lp(lin))


class _SplitLinear(torch.autograd.Function):
    """u = [xa W[:n]^T | xb W[n:]^T]: two row ranges of one weight project two inputs into one output buffer (the q/k/v
    projection of a GDN layer whose query and write inputs differ). The GEMMs write into and read from column ranges of
    the [rows, N] buffers directly (row stride N), so neither direction copies a slice."""

    @staticmethod
    def forward(ctx, xa, xb, weight, w_lp, n):
        a2 = _bf16(xa).reshape(-1, xa.shape[-1]).contiguous()
        b2 = _bf16(xb).reshape(-1, xb.shape[-1]).contiguous()
        N = w_lp.shape[0]
        out = torch.empty(a2.shape[0], N, dtype=BF16, device=xa.device)
        gemm(a2, w_lp[:n], out=out[:, :n])
        gemm(b2, w_lp[n:], out=out[:, n:])
        ctx.save_for_backward(a2, b2, w_lp)
        ctx.n, ctx.shapes, ctx.dtypes = n, (xa.shape, xb.shape), (xa.dtype, xb.dtype)
        return out.view(*xa.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        a2, b2, w_lp = ctx.saved_tensors
        n = ctx.n
        dy2 = _bf16(dy).reshape(-1, dy.shape[-1]).contiguous()
        dxa = gemm(dy2[:, :n], w_lp[:n], b_mn=True).view(ctx.shapes[0])
        dxb = gemm(dy2[:, n:], w_lp[n:], b_mn=True).view(ctx.shapes[1])
        dw = torch.empty(w_lp.shape, dtype=torch.float32, device=dy.device)
        gemm(dy2[:, :n], a2, out=dw[:n], a_mn=True, b_mn=True)
        gemm(dy2[:, n:], b2, out=dw[n:], a_mn=True, b_mn=True)
        da, db = ctx.dtypes
        return (dxa if da == BF16 else dxa.to(da)), (dxb if db == BF16 else dxb.to(db)), dw, None, None


def split_linear(xa, xb, lin, n):
    if getattr(lin, "precision", "bf16") != "bf16" and lin.training or lin.weight.shape[0] % 8 or n % 8:
        from ..models.linear import RowView
        N = lin.weight.shape[0]
        return torch.cat([linear(xa, RowView(lin, 0, n)), linear(xb, RowView(lin, n, N))], dim=-1)
    return _SplitLinear.apply(xa, xb, lin.weight, _w_lp(lin), n)


class _DualLerp(torch.autograd.Function):
    """(x + la (ya - x), x + lb (yb - x)) in fp32, rounded to bf16; la, lb one-element fp32 parameters. yb None: the
    first only."""

    @staticmethod
    def forward(ctx, x, ya, la, yb, lb):
        xc, yac = _bf16(x).contiguous(), _bf16(ya).contiguous()
        ybc = None if yb is None else _bf16(yb).contiguous()
        laf = la.detach().float().reshape(1)
        lbf = None if yb is None else lb.detach().float().reshape(1)
        oa = torch.empty_like(xc)
        ob = None if yb is None else torch.empty_like(xc)
        ext().dual_lerp_fwd(xc, yac, ybc, laf, lbf, oa, ob)
        _count()
        ctx.save_for_backward(xc, yac, ybc, laf, lbf)
        ctx.meta = (x.dtype, ya.dtype, None if yb is None else yb.dtype, la.dtype, la.shape, None if yb is None else lb.dtype)
        if yb is None:
            ob = oa.new_zeros(0)
            ctx.mark_non_differentiable(ob)
        return oa, ob

    @staticmethod
    def backward(ctx, ga, gb):
        xc, yac, ybc, laf, lbf = ctx.saved_tensors
        xd, yad, ybd, lad, lshape, lbd = ctx.meta
        dual = ybc is not None
        gac = _bf16(ga).contiguous()
        gbc = _bf16(gb).contiguous() if dual else None
        dx, dya = torch.empty_like(xc), torch.empty_like(xc)
        dyb = torch.empty_like(xc) if dual else None
        dl = torch.zeros(2, dtype=torch.float32, device=xc.device)
        ext().dual_lerp_bwd(gac, gbc, xc, yac, ybc, laf, lbf, dx, dya, dyb, dl)
        _count()
        return (dx.to(xd), dya.to(yad), dl[0].reshape(lshape).to(lad), dyb.to(ybd) if dual else None,
                dl[1].reshape(lshape).to(lbd) if dual else None)


def input_mixes(x, y_write, lam_write, y_read=None, lam_read=None):
    if lam_write.numel() != 1 or x.numel() % 4 or (y_read is not None and lam_read.numel() != 1):
        return ref.input_mixes(x, y_write, lam_write, y_read, lam_read)
    oa, ob = _DualLerp.apply(x, y_write, lam_write, y_read, lam_read)
    return oa, (ob if y_read is not None else None)


# ------------------------------------------------------------------------------------------------------------ norms

class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, out_dtype, z, gate, resid, scale):
        xc = x.contiguous()
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        rstd = torch.empty(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device)
        zc = None if z is None else _bf16(z).contiguous()
        ext().rmsnorm_fwd(xc, weight, zc, gate, None if resid is None else resid.contiguous(), y, rstd, eps, scale)
        _count()
        ctx.save_for_backward(xc, weight, rstd, zc)
        ctx.gate, ctx.scale, ctx.has_resid = gate, scale, resid is not None
        ctx.zdtype = None if z is None else z.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, weight, rstd, zc = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype not in (BF16, torch.float32):
            dy = dy.float()
        dx = torch.empty_like(xc)
        dz = torch.empty_like(zc) if zc is not None else None
        dw = torch.zeros_like(weight)
        ext().rmsnorm_bwd(dy, xc, weight, zc, ctx.gate, rstd, None, dx, dz, dw, ctx.scale)
        _count()
        if dz is not None and ctx.zdtype != BF16:
            dz = dz.to(ctx.zdtype)
        return dx, dw, None, None, dz, None, (dy if ctx.has_resid else None), None


class _PreNorm(torch.autograd.Function):
    """(RMSNorm(x), x): the normed branch input and the stream passed through. The stream has two readers in a Peri-LN
    layer (the branch's norm and the residual add); as one node their two gradients meet inside the norm's backward kernel
    (dx = norm backward + the pass-through gradient) instead of in a separate accumulation pass over the stream."""

    @staticmethod
    def forward(ctx, x, weight, eps, out_dtype):
        xc = x.contiguous()
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        rstd = torch.empty(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device)
        ext().rmsnorm_fwd(xc, weight, None, 0, None, y, rstd, eps, 1.0)
        _count()
        ctx.save_for_backward(xc, weight, rstd)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dpass):
        xc, weight, rstd = ctx.saved_tensors
        if dy is None:
            return dpass, None, None, None
        dy = dy.contiguous()
        if dy.dtype not in (BF16, torch.float32):
            dy = dy.float()
        dx = torch.empty_like(xc)
        dw = torch.zeros_like(weight)
        ext().rmsnorm_bwd(dy, xc, weight, None, 0, rstd, None if dpass is None else dpass.contiguous().float(), dx, None, dw, 1.0)
        _count()
        return dx, dw, None, None


def prenorm(x, weight, eps):
    """(RMSNorm(x) in bf16, x passed through) as one autograd node; x float32."""
    return _PreNorm.apply(x, weight, eps, BF16)


def _norm_ok(x, weight) -> bool:
    return x.dtype in (BF16, torch.float32) and weight.dtype == torch.float32 and x.shape[-1] % 4 == 0 and x.shape[-1] <= 2048


def rmsnorm(x, weight, eps, out_dtype=None):
    if not _norm_ok(x, weight):
        return ref.rmsnorm(x, weight, eps, out_dtype)
    return _RMSNorm.apply(x, weight, eps, out_dtype or BF16, None, 0, None, 1.0)


def gated_rmsnorm(x, z, weight, eps, gate, out_dtype=None):
    if not _norm_ok(x, weight):
        return ref.gated_rmsnorm(x, z, weight, eps, gate, out_dtype)
    return _RMSNorm.apply(x, weight, eps, out_dtype or BF16, z, 1 if gate == "silu" else 2, None, 1.0)


def norm_add(resid, branch, weight, eps, scale):
    """resid + scale * rmsnorm(branch) in fp32, one pass."""
    if not _norm_ok(branch, weight) or resid.dtype != torch.float32:
        return resid + scale * ref.rmsnorm(branch, weight, eps)
    return _RMSNorm.apply(branch, weight, eps, torch.float32, None, 0, resid, float(scale))


# ------------------------------------------------------------------------------------------------------------ MLP

class _SiluMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        f = gu.shape[-1] // 2
        h = torch.empty(*gu.shape[:-1], f, dtype=BF16, device=gu.device)
        ext().silu_mul_fwd(gu, h)
        _count()
        ctx.save_for_backward(gu)
        return h

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        dgu = torch.empty_like(gu)
        ext().silu_mul_bwd(_bf16(dh).contiguous(), gu, dgu)
        _count()
        return dgu


class _CatLinear(torch.autograd.Function):
    """y = x [W1; W2]^T as one GEMM when the two shadow weights are adjacent in the flat buffer (else two GEMMs into
    one output), returning the concatenated [.., n1 + n2] activations; gradients go to each weight separately."""

    @staticmethod
    def forward(ctx, x, w1, w2, lp1, lp2):
        x2 = _bf16(x).reshape(-1, x.shape[-1]).contiguous()
        n1, n2 = lp1.shape[0], lp2.shape[0]
        out = torch.empty(x2.shape[0], n1 + n2, dtype=BF16, device=x.device)
        adjacent = (lp1.data_ptr() + lp1.numel() * 2 == lp2.data_ptr() and lp1.is_contiguous() and lp2.is_contiguous()
                    and lp1.untyped_storage().data_ptr() == lp2.untyped_storage().data_ptr())     # views of one flat buffer
        if adjacent:
            wcat = torch.as_strided(lp1, (n1 + n2, lp1.shape[1]), (lp1.shape[1], 1))
            gemm(x2, wcat, out=out)
        else:
            wcat = None
            gemm(x2, lp1, out=out[:, :n1])
            gemm(x2, lp2, out=out[:, n1:])
        ctx.save_for_backward(x2, lp1, lp2)
        ctx.adjacent, ctx.xshape, ctx.xdtype = adjacent, x.shape, x.dtype
        return out.view(*x.shape[:-1], n1 + n2)

    @staticmethod
    def backward(ctx, dy):
        x2, lp1, lp2 = ctx.saved_tensors
        n1, n2 = lp1.shape[0], lp2.shape[0]
        dy2 = _bf16(dy).reshape(-1, n1 + n2).contiguous()
        if ctx.adjacent:
            wcat = torch.as_strided(lp1, (n1 + n2, lp1.shape[1]), (lp1.shape[1], 1))
            dx = gemm(dy2, wcat, b_mn=True)
        else:
            dx = gemm(dy2[:, :n1], lp1, b_mn=True, out_dtype=torch.float32)
            gemm(dy2[:, n1:], lp2, b_mn=True, out=dx, accumulate=True)
            dx = dx.to(BF16)
        dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dx = dx.view(ctx.xshape)
        return (dx if ctx.xdtype == BF16 else dx.to(ctx.xdtype)), dw[:n1], dw[n1:], None, None


def swiglu_mlp(x, w_gate, w_up, w_down):
    if any(getattr(m, "precision", "bf16") != "bf16" and m.training for m in (w_gate, w_up, w_down)):
        return linear(torch.nn.functional.silu(linear(x, w_gate)) * linear(x, w_up), w_down)
    gu = _CatLinear.apply(x, w_gate.weight, w_up.weight, _w_lp(w_gate), _w_lp(w_up))
    return linear(_SiluMul.apply(gu), w_down)


# ------------------------------------------------------------------------------------------------------------ GDN prep / gates

class _GdnPrep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u_pre, doc32, conv_weight, L, nq, qscale):
        u = _bf16(u_pre).contiguous()
        out = torch.empty_like(u)
        ext().gdn_prep_fwd(u, doc32, conv_weight, out, L, nq, qscale)
        _count()
        ctx.save_for_backward(u, doc32, conv_weight)
        ctx.meta = (L, nq, qscale, u_pre.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        u, doc32, w = ctx.saved_tensors
        L, nq, qscale, dt = ctx.meta
        du = torch.empty_like(u)
        dw = torch.zeros_like(w)
        ext().gdn_prep_bwd(u, doc32, w, _bf16(dout).contiguous(), du, dw, L, nq, qscale)
        _count()
        return (du if dt == BF16 else du.to(dt)), None, dw, None, None, None


def gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv, single_doc=False, packed=False):
    B, L, C = u_pre.shape
    ok = dk == 128 and (hv * dv) % 128 == 0 and conv_weight.shape[1] == 4 and conv_weight.dtype == torch.float32
    if not ok:
        q, k, v, h, hd = ref.gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv)
        return (torch.cat([q.flatten(2), k.flatten(2), v.flatten(2)], dim=-1), h, hd) if packed else (q, k, v, h, hd)
    doc32 = None if single_doc else doc.to(torch.int32).contiguous()
    out = _GdnPrep.apply(u_pre, doc32, conv_weight, L, hk * dk, dk ** -0.5)
    nq = hk * dk
    if packed:
        K = conv_weight.shape[1]
        return out, u_pre[:, L - (K - 1):], doc[:, L - (K - 1):]
    q = out[..., :nq].view(B, L, hk, dk)
    k = out[..., nq:2 * nq].view(B, L, hk, dk)
    v = out[..., 2 * nq:].view(B, L, hv, dv)
    K = conv_weight.shape[1]
    return q, k, v, u_pre[:, L - (K - 1):], doc[:, L - (K - 1):]


def gdn_prep_cached(u_pre, doc, conv_weight, hk, hv, dk, dv, hist, hist_doc, packed=False):
    """`gdn_prep` of a chunk that continues cached rows: the K - 1 cached inputs (and their document ids; -1 where there is
    none) are placed in front of the chunk, the same kernel runs over the longer rows and the first K - 1 outputs are
    dropped. The document mask keeps taps of other documents (and of the empty history) out."""
    K = conv_weight.shape[1]
    full = torch.cat([hist.to(u_pre.dtype), u_pre], dim=1)
    full_doc = torch.cat([hist_doc, doc], dim=1)
    out = gdn_prep(full, full_doc, conv_weight, hk, hv, dk, dv, False, packed)
    head, (h, hd) = out[:-2], out[-2:]
    return (*(t[:, K - 1:] for t in head), h, hd)


def gdn_gates(a_lin, b_lin, A_log, dt_bias):
    """Tiny (B, L, Hv) elementwise maths in fp32; left to the framework's elementwise kernels."""
    g = -torch.exp(A_log) * torch.nn.functional.softplus(a_lin.float() + dt_bias)
    return g, torch.sigmoid(b_lin.float())


class _Embedding(torch.autograd.Function):
    """Rows of the table (bags: the mean of their rows). The backward adds the row gradients into a zeroed table gradient
    with vector reductions (or straight into the parameter's accumulation buffer when weight gradients accumulate there)."""

    @staticmethod
    def forward(ctx, tokens, weight):
        ids = tokens.reshape(-1, tokens.shape[2] if tokens.dim() == 3 else 1).contiguous()
        out = torch.empty(*tokens.shape[:2], weight.shape[1], dtype=torch.float32, device=weight.device)
        ext().embedding_fwd(ids, weight.detach().contiguous(), out)
        _count()
        ctx.save_for_backward(ids)
        ctx.weight = weight
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        main = getattr(w, "main_grad", None) if WGRAD_INTO_MAIN else None
        if main is not None and main.dtype == torch.float32 and main.shape == w.shape and main.is_contiguous():
            ext().embedding_bwd(ids, g.contiguous().float(), main)
            _count()
            return None, None
        dw = torch.zeros_like(w, dtype=torch.float32)
        ext().embedding_bwd(ids, g.contiguous().float(), dw)
        _count()
        return None, dw.to(w.dtype)


def embedding(tokens, weight):
    if weight.dtype != torch.float32 or weight.shape[1] % 4 or tokens.dim() not in (2, 3) or torch.are_deterministic_algorithms_enabled():
        return ref.embedding(tokens, weight)
    return _Embedding.apply(tokens, weight)


# ------------------------------------------------------------------------------------------------------------ depth mix

class _DepthMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, gain, eps, *sources):
        srcs = [s.contiguous() for s in sources]
        ueff = (query * (1.0 + gain)).contiguous()
        out = torch.empty_like(srcs[0])
        rows = out.numel() // out.shape[-1]
        alpha = torch.empty(rows, len(srcs), dtype=torch.float32, device=out.device)
        rnorm = torch.empty_like(alpha)
        ext().depth_mix_fwd(srcs, ueff, out, alpha, rnorm, eps)
        _count()
        ctx.save_for_backward(query, gain, ueff, alpha, rnorm, *srcs)
        return out

    @staticmethod
    def backward(ctx, dh):
        query, gain, ueff, alpha, rnorm, *srcs = ctx.saved_tensors
        dsrc = [torch.empty_like(s) for s in srcs]
        du = torch.zeros_like(ueff)
        ext().depth_mix_bwd(srcs, dsrc, ueff, dh.contiguous().float(), alpha, rnorm, du)
        _count()
        return (du * (1.0 + gain), du * query, None, *dsrc)


def depth_mix(sources, query, gain, eps):
    d = sources[0].shape[-1]
    if len(sources) > 8 or d % 512 or d > 2048 or any(s.dtype != torch.float32 for s in sources):
        return ref.depth_mix(sources, query, gain, eps)
    return _DepthMix.apply(query, gain, eps, *sources)


class _DepthMixMulti(torch.autograd.Function):
    """Q readers over the same n sources in one pass: args = n sources, Q queries, Q key-norm gains; returns Q mixes."""

    @staticmethod
    def forward(ctx, eps, n, *args):
        Q = (len(args) - n) // 2
        srcs = [s.contiguous() for s in args[:n]]
        queries, gains = args[n:n + Q], args[n + Q:]
        ueff = torch.stack([q.float() * (1.0 + g.float()) for q, g in zip(queries, gains)]).contiguous()
        outs = [torch.empty_like(srcs[0]) for _ in range(Q)]
        rows = srcs[0].numel() // srcs[0].shape[-1]
        alpha = torch.empty(rows, Q, n, dtype=torch.float32, device=ueff.device)
        vu = torch.empty_like(alpha)
        rnorm = torch.empty(rows, n, dtype=torch.float32, device=ueff.device)
        ext().depth_mix_multi_fwd(srcs, ueff, outs, alpha, rnorm, vu, eps)
        _count()
        ctx.save_for_backward(ueff, alpha, rnorm, vu, *srcs, *queries, *gains)
        ctx.n, ctx.Q = n, Q
        return tuple(outs)

    @staticmethod
    def backward(ctx, *dhs):
        n, Q = ctx.n, ctx.Q
        ueff, alpha, rnorm, vu, *rest = ctx.saved_tensors
        srcs, queries, gains = rest[:n], rest[n:n + Q], rest[n + Q:]
        dsrc = [torch.empty_like(s) for s in srcs]
        du = torch.zeros_like(ueff)
        ext().depth_mix_multi_bwd(list(srcs), dsrc, ueff, [None if g is None else g.contiguous().float() for g in dhs], alpha, rnorm, vu, du)
        _count()
        dq = [(du[i] * (1.0 + gains[i].float())).to(queries[i].dtype) for i in range(Q)]
        dg = [(du[i] * queries[i].float()).to(gains[i].dtype) if gains[i].numel() == du[i].numel() else (du[i] * queries[i].float()).sum().reshape(gains[i].shape).to(gains[i].dtype)
              for i in range(Q)]
        return (None, None, *dsrc, *dq, *dg)


def depth_mix_multi(sources, readers, eps):
    """readers: [(query, gain)]. One kernel for all of them when the shapes fit, else one mix per reader."""
    d = sources[0].shape[-1]
    if len(sources) > 8 or len(readers) > 8 or d % 512 or d > 2048 or any(s.dtype != torch.float32 for s in sources):
        return [depth_mix(sources, q, g, eps) for q, g in readers]
    return list(_DepthMixMulti.apply(eps, len(sources), *sources, *[q for q, _ in readers], *[g for _, g in readers]))


# ------------------------------------------------------------------------------------------------------------ fused head + CE

class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, a, b, chunk, w_lp, fixed=False):
        d = hidden.shape[-1]
        h = _bf16(hidden).reshape(-1, d).contiguous()
        n, V = h.shape[0], w_lp.shape[0]
        t = targets.reshape(n, -1).contiguous()
        a2 = a.reshape(n, -1).float().contiguous()
        b1 = b.reshape(-1).float().contiguous()
        ce = torch.empty(n, dtype=torch.float32, device=h.device)
        lse = torch.empty_like(ce)
        dh = torch.empty(n, d, dtype=BF16, device=h.device)
        dW = torch.zeros(V, d, dtype=torch.float32, device=h.device)
        logits = torch.empty(min(chunk, n), V, dtype=torch.float32, device=h.device)
        grad = torch.empty(min(chunk, n), V, dtype=BF16, device=h.device)
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            m = hi - lo
            gemm(h[lo:hi], w_lp, out=logits[:m])
            ext().ce_grad(logits[:m], t[lo:hi], a2[lo:hi], b1[lo:hi], grad[:m], ce[lo:hi], lse[lo:hi], fixed)
            _count()
            gemm(grad[:m], w_lp, out=dh[lo:hi], b_mn=True)
            gemm(grad[:m], h[lo:hi], out=dW, a_mn=True, b_mn=True, accumulate=True)
        loss = ce.sum() + (b1 * lse * lse).sum()
        ctx.save_for_backward(dh, dW)
        ctx.meta = (hidden.dtype, hidden.shape, weight.dtype)
        ctx.mark_non_differentiable(ce, lse)
        return loss, ce, lse

    @staticmethod
    def backward(ctx, g_loss, g_ce, g_lse):
        dh, dW = ctx.saved_tensors
        hd, hs, wd = ctx.meta
        return (dh * g_loss).to(hd).reshape(hs), (dW * g_loss).to(wd), None, None, None, None, None, None


def fused_linear_ce(hidden, weight, targets, a, b, chunk, weight_lp=None, fixed=False):
    w_lp = weight_lp if weight_lp is not None else weight.detach().to(BF16)
    return _FusedLinearCE.apply(hidden, weight, targets, a, b, chunk, w_lp, fixed)


def lm_loss_sums(hidden, weight, targets, weights=None, z_loss=0.0, weight_lp=None):
    n = hidden.reshape(-1, hidden.shape[-1]).shape[0]
    t = targets.reshape(n, -1)
    a = torch.ones_like(t, dtype=torch.float32) if weights is None else weights.reshape(n, -1).float()
    a = a * (t >= 0)
    b = a.sum(1) * z_loss
    loss, ce, _ = fused_linear_ce(hidden, weight, t, a, b, 2048, weight_lp)
    return loss, ce.sum()


# ------------------------------------------------------------------------------------------------------------ optimizer

def adamw_(p, g, m, v, lp, lr, b1, b2, eps, wd, c1, c2, grad_scale):
    gs_t, gs_h = (grad_scale.reshape(1).float(), 1.0) if isinstance(grad_scale, torch.Tensor) else (None, float(grad_scale))
    ext().adamw(p, g, m, v, lp, lr, b1, b2, eps, wd, c1, c2, gs_t, gs_h)
    _count()


def sumsq(x):
    _count()
    return ext().sumsq(x)


def cast_bf16_(x, y):
    ext().cast_bf16(x, y)
    _count()


# ------------------------------------------------------------------------------------------------------------ sequence mixers

def delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, is_doc_start, S0, need_state):
    from . import gdn_native
    return gdn_native.delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, is_doc_start, S0, need_state)


def delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size, need_state):
    from . import gdn_native

    return gdn_native.delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size, need_state)


def attention(q, k, v, doc, q_far, k_far, cap, pos=None, single_doc=False):
    from . import attention_native

    return attention_native.attention(q, k, v, doc, q_far, k_far, cap, pos, single_doc)
