"""Block-scaled low-precision formats and the linears that train with them.

Formats (byte-compatible with the reference's emulations, which are the oracle: ced/model/mxfp8.py:86-188,
ced/model/nvfp4.py:169-250, ced/model/fp8.py:159-344):

* MXFP8: E4M3 elements in blocks of 32 along the reduction dimension with one E8M0 exponent per block, chosen by the
  round-up rule on amax / 448; a block holding a non-finite value becomes all NaN with exponent 0xFF.
* NVFP4: E2M1 elements in blocks of 16 with an E4M3 block scale and one fp32 tensor scale (s_enc = 6 * 448 / amax);
  weights in 16 x 16 blocks; gradients rounded stochastically; Wgrad operands through a 16 x 16 random Hadamard
  transform over 16-token segments (sign vector from seed 2509).
* FP8 rowwise / tensorwise: E4M3 (E5M2 for tensorwise gradients) with a power-of-two scale per row / per tensor.

A quantised linear keeps its master weight in high precision and quantises both operands of each of its three GEMMs
from the high-precision tensors, along that GEMM's reduction dimension. MXFP8 linears run on the block-scaled
tensor-core kernel (`tcgen05.mma.kind::mxf8f6f4.block_scale`, csrc/gemm_mx.cu) over E4M3 bytes and E8M0 scale cells
written by one quantise kernel per tensor; the other recipes (and shapes the kernel does not take) run on the bf16
tcgen05 kernel over the dequantised operands: every E4M3 / E2M1 value times its power-of-two (or E4M3) scale is exact
in bfloat16, so the products equal the block-scaled products and only the accumulation order differs. Quantised paths
are active in training mode only; evaluation is bf16.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2
E4M3_MAX, E5M2_MAX, E2M1_MAX = 448.0, 57344.0, 6.0
MX_BLOCK, NV_BLOCK = 32, 16
RHT_SEED = 2509


# ------------------------------------------------------------------------------------------------------------ MXFP8

def e8m0_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Biased E8M0 exponent (int32, 0..255) of blocks with largest magnitude amax: the exponent of amax / 448 rounded
    UP to a power of two (a nonzero mantissa bumps it), infinities saturate to 254, NaN gives 255."""
    v = amax.float() * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=amax.device)
    bits = v.view(torch.int32)
    e, m = (bits >> 23) & 0xFF, bits & 0x7FFFFF
    bump = (m > 0) & (e != 254) & ((e != 0) | (m > 0x400000))
    b = e + bump.to(torch.int32)
    b = torch.where((e == 255) & (m == 0), torch.full_like(b, 254), b)
    return torch.where((e == 255) & (m != 0), torch.full_like(b, 255), b)


def _pow2(bits_exp: torch.Tensor, zero_code: int) -> torch.Tensor:
    bits = torch.where(bits_exp == zero_code, torch.full_like(bits_exp, 0x00400000), bits_exp << 23)
    return bits


def mx_quantize(t: torch.Tensor, dim: int = -1):
    """(q, b): q float8_e4m3fn of t's shape, b uint8 exponents with ceil(n / 32) entries along dim."""
    x = t.float().movedim(dim, -1)
    n = x.shape[-1]
    pad = (-n) % MX_BLOCK
    if pad:
        x = F.pad(x, (0, pad))
    xb = x.reshape(*x.shape[:-1], -1, MX_BLOCK)
    a = xb.abs()
    amax = torch.where(torch.isnan(a), torch.zeros_like(a), a).amax(-1)
    b = e8m0_exponent(amax)
    inv_bits = torch.where(b == 254, torch.full_like(b, 0x00400000), (254 - b) << 23)
    inv_bits = torch.where(b == 255, torch.full_like(b, 0x7FFFFFFF), inv_bits)
    y = (xb * inv_bits.view(torch.float32)[..., None]).clamp(-E4M3_MAX, E4M3_MAX)
    bad = ~torch.isfinite(xb).all(-1)
    y = torch.where(bad[..., None], torch.full_like(y, float("nan")), y)
    b = torch.where(bad, torch.full_like(b, 255), b)
    q = y.to(E4M3).reshape(*xb.shape[:-2], -1)[..., :n].movedim(-1, dim).contiguous()
    return q, b.to(torch.uint8).movedim(-1, dim).contiguous()


def mx_dequantize(q: torch.Tensor, b: torch.Tensor, dim: int = -1, dtype=torch.float32) -> torch.Tensor:
    n = q.shape[dim]
    bi = b.to(torch.int32)
    bits = torch.where(bi == 0, torch.full_like(bi, 0x00400000), bi << 23)
    bits = torch.where(bi == 255, torch.full_like(bi, 0x7FFFFFFF), bits)
    s = bits.view(torch.float32).movedim(dim, -1)
    s = s.unsqueeze(-1).expand(*s.shape, MX_BLOCK).reshape(*s.shape[:-1], -1)[..., :n].movedim(-1, dim)
    return (q.float() * s).to(dtype)


def mx_fake(t: torch.Tensor, dim: int = -1, dtype=torch.float32) -> torch.Tensor:
    """Quantise to MXFP8 along `dim` and multiply back. A 2-D CUDA tensor goes through one kernel that reads the input once
    and writes the values as bfloat16 (exact for E4M3 times a power of two); everything else through the tensor ops."""
    if t.is_cuda and t.dim() == 2 and t.dtype in (torch.float32, torch.bfloat16) and t.is_contiguous() and dim in (-1, 0, 1):
        from . import use_native

        if use_native(t):
            from . import native

            out = torch.empty(t.shape, dtype=torch.bfloat16, device=t.device)
            native.ext().mx_fake(t.detach(), out, dim == 0)
            native._count()
            return out
    q, b = mx_quantize(t, dim)
    return mx_dequantize(q, b, dim, dtype)


# ------------------------------------------------------------------------------------------------------------ NVFP4

def e2m1_round(a: torch.Tensor, u: torch.Tensor | None = None) -> torch.Tensor:
    """Magnitudes a >= 0 onto {0, .5, 1, 1.5, 2, 3, 4, 6}: nearest-even, or stochastic with u ~ U[0, 1); saturates at 6."""
    step = torch.where(a < 2.0, 0.5, torch.where(a < 4.0, 1.0, 2.0)).to(a.dtype)
    t = a / step
    n = torch.round(t) if u is None else torch.floor(t + u)
    return torch.clamp(n * step, max=E2M1_MAX)


def nvfp4_fake(x: torch.Tensor, stochastic: bool = False, block_2d: bool = False, generator=None) -> torch.Tensor:
    """The dequantised NVFP4 tensor (float32, x's shape): element = e2m1 * e4m3 block scale * fp32 tensor scale."""
    x32 = x.float()
    shape = x32.shape
    pn = (-shape[-1]) % NV_BLOCK
    if block_2d:
        pm = (-shape[-2]) % NV_BLOCK
        xp = F.pad(x32, (0, pn, 0, pm)) if (pn or pm) else x32
        M, N = xp.shape[-2:]
        blocks = xp.reshape(*xp.shape[:-2], M // NV_BLOCK, NV_BLOCK, N // NV_BLOCK, NV_BLOCK)
        amax_b = blocks.abs().amax(dim=(-3, -1), keepdim=True)
    else:
        xp = F.pad(x32, (0, pn)) if pn else x32
        blocks = xp.reshape(*xp.shape[:-1], -1, NV_BLOCK)
        amax_b = blocks.abs().amax(dim=-1, keepdim=True)
    amax = x32.abs().amax()
    s_enc = torch.where(amax > 0, torch.clamp((E2M1_MAX * E4M3_MAX) / amax, max=torch.finfo(torch.float32).max), torch.ones_like(amax))
    s_dec = 1.0 / s_enc
    scales = torch.clamp(amax_b / E2M1_MAX * s_enc, max=E4M3_MAX).to(E4M3).float()
    live = scales > 0
    enc_b = torch.where(live, 1.0 / (torch.where(live, scales, torch.ones_like(scales)) * s_dec), torch.zeros_like(scales))
    scaled = blocks * enc_b
    mag = scaled.abs()
    u = torch.rand(mag.shape, device=mag.device, generator=generator) if stochastic else None
    v = torch.copysign(e2m1_round(mag, u), scaled) * scales
    if block_2d:
        v = v.reshape(*v.shape[:-4], v.shape[-4] * NV_BLOCK, v.shape[-2] * NV_BLOCK)[..., :shape[-2], :shape[-1]]
    else:
        v = v.reshape(*v.shape[:-2], -1)[..., :shape[-1]]
    return v * s_dec


def hadamard(n: int = NV_BLOCK) -> torch.Tensor:
    h = torch.ones(1, 1)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def rht_matrix(seed: int = RHT_SEED) -> torch.Tensor:
    """T = diag(s) H_16 / 4 with one seeded sign vector (orthogonal)."""
    g = torch.Generator().manual_seed(seed)
    s = torch.randint(0, 2, (NV_BLOCK,), generator=g).float() * 2 - 1
    return s[:, None] * hadamard(NV_BLOCK) / math.sqrt(NV_BLOCK)


def rht_tokens(t2d: torch.Tensor, transform: torch.Tensor | None) -> torch.Tensor:
    """(M, n) -> (n, M'): transposed, M zero-padded to a multiple of 16, each 16-token segment times the transform."""
    t = t2d.float().t()
    pad = (-t.shape[-1]) % NV_BLOCK
    if pad:
        t = F.pad(t, (0, pad))
    if transform is None:
        return t
    n, m = t.shape
    return torch.matmul(t.reshape(n, m // NV_BLOCK, NV_BLOCK), transform.to(t.device)).reshape(n, m)


# ------------------------------------------------------------------------------------------------------------ FP8 scalings

def fp8_scale(amax: torch.Tensor, fmax: float, pow2: bool) -> torch.Tensor:
    """fmax / max(amax, 1e-12) formed in float64 and rounded to float32; with pow2 rounded down to a power of two by
    clearing the mantissa bits (torchao's rowwise rule). Per-tensor scaling keeps the full value (delayed-scaling recipe)."""
    s = (fmax / amax.double().clamp(min=1e-12)).float()
    return (s.view(torch.int32) & 0x7F800000).view(torch.float32) if pow2 else s


def fp8_fake(t: torch.Tensor, dim: int | None, dtype=E4M3) -> torch.Tensor:
    """Per-row (dim = the reduction dimension, power-of-two scale) or per-tensor (dim None, exact scale) FP8, dequantised."""
    fmax = E4M3_MAX if dtype == E4M3 else E5M2_MAX
    x = t.float()
    amax = x.abs().amax() if dim is None else x.abs().amax(dim=dim, keepdim=True)
    s = fp8_scale(amax, fmax, pow2=dim is not None)
    return (x * s).clamp(-fmax, fmax).to(dtype).float() * s.reciprocal()


# ------------------------------------------------------------------------------------------------------------ recipes

@dataclass
class Recipe:
    """How one linear quantises the operands of its three GEMMs. kind: "mxfp8", "fp8_rowwise", "fp8_tensorwise", "nvfp4"."""

    kind: str
    stochastic: bool = True
    rht: bool = True
    weight_2d: bool = True

    def operands(self, which: str, x2, w, dy2=None):
        """(A, B) dequantised operands (float32) of GEMM `which`: "fprop" y = A B^T, "dgrad" dx = A B, "wgrad" dW = A^T-form
        returned as (dy-operand [n, M], x-operand [k, M]) so that dW = A B^T."""
        k = self.kind
        if k == "mxfp8":
            if which == "fprop":
                return mx_fake(x2, -1), mx_fake(w, -1)
            if which == "dgrad":
                return mx_fake(dy2, -1), mx_fake(w, 0)
            return mx_fake(dy2, 0).t(), mx_fake(x2, 0).t()
        if k == "fp8_rowwise":
            if which == "fprop":
                return fp8_fake(x2, -1), fp8_fake(w, -1)
            if which == "dgrad":
                return fp8_fake(dy2, -1), fp8_fake(w.t(), -1).t()
            return fp8_fake(dy2.t(), -1), fp8_fake(x2.t(), -1)
        if k == "fp8_tensorwise":
            if which == "fprop":
                return fp8_fake(x2, None), fp8_fake(w, None)
            if which == "dgrad":
                return fp8_fake(dy2, None, E5M2), fp8_fake(w, None)
            return fp8_fake(dy2, None, E5M2).t(), fp8_fake(x2, None).t()
        if k == "nvfp4":
            if which == "fprop":
                return nvfp4_fake(x2), nvfp4_fake(w, block_2d=self.weight_2d)
            if which == "dgrad":
                wq = nvfp4_fake(w, block_2d=True) if self.weight_2d else nvfp4_fake(w.t()).t()
                return nvfp4_fake(dy2, stochastic=self.stochastic), wq
            T = rht_matrix() if self.rht else None
            return nvfp4_fake(rht_tokens(dy2, T), stochastic=self.stochastic), nvfp4_fake(rht_tokens(x2, T))
        raise ValueError(f"unknown low-precision recipe {k!r}")

    # the op layer's two entry points
    def emulated_linear(self, x, weight):
        return _LowpLinear.apply(x, weight, self, False)


def recipe_for(cfg, name: str) -> Recipe:
    """The recipe the model config assigns to the linear called `name`."""
    if cfg.fp8.mode != "none":
        kind = "mxfp8" if cfg.fp8.scaling == "mxfp8" else "fp8_" + cfg.fp8.scaling
        return Recipe(kind)
    nv = cfg.nvfp4
    if any(name.endswith(k) or k in name for k in nv.fp8_names):
        return Recipe("mxfp8")
    return Recipe("nvfp4", stochastic=nv.stochastic_rounding, rht=nv.rht, weight_2d=nv.weight_2d)


def _mm(a, b_t, native_gemm: bool, out_dtype):
    """a [M, K] . b_t [N, K]^T. On the device path the dequantised operands go through the tcgen05 bf16 GEMM (their values are
    exact in bf16); otherwise a float32 matmul."""
    if native_gemm:
        from . import native

        K = a.shape[1]
        pad = (-K) % 8
        if pad:
            a, b_t = F.pad(a, (0, pad)), F.pad(b_t, (0, pad))
        return native.gemm(a.to(torch.bfloat16).contiguous(), native._pad_rows(b_t.to(torch.bfloat16).contiguous()),
                           out_dtype=torch.float32)[:, :b_t.shape[0]].to(out_dtype)
    return (a.float() @ b_t.float().t()).to(out_dtype)


class _LowpLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, recipe: Recipe, native_gemm: bool):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        a, b = recipe.operands("fprop", x2, weight)
        out_dtype = x.dtype if x.dtype != torch.float32 or not native_gemm else torch.bfloat16
        y = _mm(a, b, native_gemm, out_dtype)
        ctx.save_for_backward(x2, weight)
        ctx.recipe, ctx.native_gemm, ctx.xshape = recipe, native_gemm, x.shape
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        r = ctx.recipe
        dy2 = dy.reshape(-1, weight.shape[0])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            a, b = r.operands("dgrad", x2, weight, dy2)
            dx = _mm(a, b.t(), ctx.native_gemm, x2.dtype).reshape(ctx.xshape)
        if ctx.needs_input_grad[1]:
            a, b = r.operands("wgrad", x2, weight, dy2)
            dw = _mm(a, b, ctx.native_gemm, torch.float32)[:, :weight.shape[1]].to(weight.dtype)
        return dx, dw, None, None


def mx_cells_to_rows(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Scale cells in the tensor core's layout -> exponents [rows, k / 32] (the inverse of the quantise kernel's placement:
    cell [row tile][k tile] of 512 bytes, byte (row % 32) * 16 + (row % 128 // 32) * 4 + block % 4)."""
    rt, kt = -(-rows // 128), -(-k // 128)
    cells = sf[:rt * kt * 512].view(rt, kt, 32, 4, 4)          # [row tile][k tile][row % 32][row // 32 % 4][block % 4]
    return cells.permute(0, 3, 2, 1, 4).reshape(rt * 128, kt * 4)[:rows, :k // 32]


class _MxLinear(torch.autograd.Function):
    """A linear whose three GEMMs run on the block-scaled MXFP8 tensor-core kernel. Each activation is quantised once, in
    both block orientations from one read (x: along features for the forward, along tokens for the weight gradient; dy
    likewise), the weight once per orientation; the forward keeps x's token-blocked transpose for the backward instead
    of x itself. Same quantisation points as the emulation (reference: ced/model/fp8.py:223-291)."""

    @staticmethod
    def forward(ctx, x, weight):
        from . import native

        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.dtype not in (torch.float32, torch.bfloat16):
            x2 = x2.float()
        need_w = ctx.needs_input_grad[1]
        xq, xs, xtq, xts = native.mx_quantize(x2, True, need_w)
        wq, ws, wtq, wts = native.mx_quantize(weight.detach(), True, ctx.needs_input_grad[0])
        y = native.gemm_mx(xq, xs, wq, ws)
        ctx.save_for_backward(xtq, xts, wtq, wts)
        ctx.xshape, ctx.xdtype, ctx.weight = x.shape, x.dtype, weight
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import native

        xtq, xts, wtq, wts = ctx.saved_tensors
        n = ctx.weight.shape[0]
        dy2 = dy.reshape(-1, n)
        if dy2.dtype not in (torch.float32, torch.bfloat16):
            dy2 = dy2.float()
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        gq, gs, gtq, gts = native.mx_quantize(dy2, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm_mx(gq, gs, wtq, wts).view(ctx.xshape)
            if ctx.xdtype != torch.bfloat16:
                dx = dx.to(ctx.xdtype)
        if ctx.needs_input_grad[1]:
            main = getattr(ctx.weight, "main_grad", None) if native.WGRAD_INTO_MAIN else None
            if main is not None and main.dtype == torch.float32:
                native.gemm_mx(gtq, gts, xtq, xts, out=main, accumulate=True)
            else:
                dw = native.gemm_mx(gtq, gts, xtq, xts, out_dtype=torch.float32).to(ctx.weight.dtype)
        return dx, dw


def mx_native_ok(x, weight) -> bool:
    """Shapes the block-scaled kernel takes: every reduction dimension (features in, features out, tokens) a multiple of 128."""
    tokens = x.numel() // x.shape[-1]
    return weight.shape[0] % 128 == 0 and weight.shape[1] % 128 == 0 and tokens % 128 == 0 and weight.dtype in (torch.float32, torch.bfloat16)


def native_linear(x, lin):
    """Device path of a quantised linear in training mode: MXFP8 on the block-scaled tensor-core kernel where the shapes
    allow, every other recipe (and odd shapes) on the bf16 kernel over the dequantised operands."""
    import os

    if lin.lowp.kind == "mxfp8" and mx_native_ok(x, lin.weight) and os.environ.get("GHB_MX_GEMM", "native") == "native":
        return _MxLinear.apply(x, lin.weight)
    return _LowpLinear.apply(x, lin.weight, lin.lowp, True)
