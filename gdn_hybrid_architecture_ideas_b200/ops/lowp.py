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
from typing import NamedTuple

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


# ------------------------------------------------------------------------------------------------------------ Quartet II
# `model.nvfp4.recipe: quartet2` (Panferov et al., arXiv 2601.22813, Algorithm 1). Forward: activations and weights in 1 x 16
# blocks along the dot product, round to nearest with ties AWAY from zero, and "four over six": every block is quantised
# with its largest magnitude mapped to 6 and to 4 and keeps the one with the smaller squared error (6 on a tie); tensor
# decode scale amax / 256 / 6. Backward: each operand of Dgrad and Wgrad (the gradient and the forward's QUANTISED weight and
# activation) is re-quantised with MS-EDEN along its GEMM's dot product: one random Hadamard transform over 128-element
# segments with ONE fresh sign vector a backward call (it cancels in each product), tensor scale amax / 255.99 / g with
# g = 6 / (17/16 * 0.93), round to nearest, the per-block correction S = <x', x'> / <x', q>, and the corrected block scale
# rounded STOCHASTICALLY to an E4M3 neighbour so that its expectation is S * scale. A quantised tensor is kept as (v, s_dec):
# v = element x block scale (exact in bf16), the tensor scale applied to the GEMM's output
# (reference: ced/model/nvfp4.py:296-449, 508-552).

Q2_FWD_SCALES_MAX, Q2_BWD_SCALES_MAX, Q2_BWD_GRID_MAX, Q2_RHT = 256.0, 255.99, 6.0 / ((17.0 / 16.0) * 0.93), 128
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


class Quantized(NamedTuple):
    """A quantised tensor as the GEMM takes it: `values` = element x block scale (exact in bf16) and the tensor's decode scale."""

    values: torch.Tensor
    scale: torch.Tensor

    def dequant(self) -> torch.Tensor:
        return self.values * self.scale


def _constant(values, like: torch.Tensor) -> torch.Tensor:
    return torch.tensor(values, dtype=like.dtype, device=like.device)


def e2m1_round_away(a: torch.Tensor) -> torch.Tensor:
    """Magnitudes a >= 0 onto the E2M1 grid, ties away from zero, saturating at 6: the grid point whose cell, cut at the
    midpoints and closed below, holds a (one search over seven thresholds; exact)."""
    grid = _constant(E2M1_GRID, a)
    return grid[torch.bucketize(a, (grid[1:] + grid[:-1]) / 2, right=True)]


def _signed_grid(t: torch.Tensor) -> torch.Tensor:
    return torch.copysign(e2m1_round_away(t.abs()), t)


def _block_view(t: torch.Tensor, n: int) -> torch.Tensor:
    """(..., K) -> (..., K' / n, n) in float32, K zero-padded up to a multiple of n."""
    t = t.float()
    short = -t.shape[-1] % n
    return (F.pad(t, (0, short)) if short else t).unflatten(-1, (-1, n))


def _tensor_scale(t: torch.Tensor, denominator: tuple) -> torch.Tensor:
    """amax / denominator / grid max as the reference divides (two divisions), 1 for a tensor of zeros."""
    top = t.abs().amax()
    return torch.where(top > 0, top / denominator[0] / denominator[1], torch.ones_like(top))


def _e4m3_or_one(s: torch.Tensor) -> torch.Tensor:
    """s (>= 0) rounded to E4M3 (saturating); 1 where that underflows to zero, so that such a block quantises to zeros."""
    stored = s.clamp(max=E4M3_MAX).to(E4M3).float()
    return stored.masked_fill(stored == 0, 1.0)


def q2_rtn_quantize(x: torch.Tensor, four_over_six: bool = True) -> Quantized:
    """The forward quantiser along x's last dimension. Under four-over-six both candidates of every block (largest magnitude
    on 6, on 4) are formed side by side along a leading axis and the one with the smaller squared error is kept (6 on a tie)."""
    blocks = _block_view(x, NV_BLOCK)
    s_dec = _tensor_scale(x.float(), (Q2_FWD_SCALES_MAX if four_over_six else E4M3_MAX, E2M1_MAX))
    peak = blocks.abs().amax(dim=-1, keepdim=True)
    on_six = peak / E2M1_MAX / s_dec
    tried = torch.stack([on_six, peak / E2M1_MAX * 1.5 / s_dec]) if four_over_six else on_six.unsqueeze(0)
    scales = _e4m3_or_one(tried)
    cell = scales * s_dec
    grid = _signed_grid(blocks / cell)
    kept = grid[0] * scales[0]
    if four_over_six:
        miss = (blocks - grid * cell).square().sum(-1, keepdim=True)
        kept = torch.where(miss[1] < miss[0], grid[1] * scales[1], kept)
    return Quantized(kept.flatten(-2)[..., :x.shape[-1]], s_dec)


def q2_rotate(t2d: torch.Tensor, transform: torch.Tensor) -> torch.Tensor:
    """(R, K) -> (R, K'): every n-segment of each row times the (n x n) transform, K zero-padded to a multiple of n."""
    return (_block_view(t2d, transform.shape[0]) @ transform.float()).flatten(-2)


def e4m3_neighbours(c: torch.Tensor):
    """(down, up): the E4M3 values around c >= 0, both c itself when c is one. Two searches in the table of the 127
    finite non-negative codes."""
    table = torch.arange(0x7F, dtype=torch.uint8, device=c.device).view(E4M3).to(c.dtype)
    c = c.clamp(max=E4M3_MAX)
    below = torch.bucketize(c, table, right=True) - 1                       # the last code <= c
    above = torch.bucketize(c, table, right=False).clamp(max=table.numel() - 1)      # the first code >= c
    return table[below], table[above]


def q2_eden_quantize(t2d: torch.Tensor, transform: torch.Tensor, u: torch.Tensor | None = None) -> Quantized:
    """MS-EDEN along K of t2d (R, K): the dequantised ROTATED tensor is values * scale. u (R, K' / 16) ~ U[0, 1)
    decides each block scale's rounding (drawn here from the device's global generator when None)."""
    rotated = q2_rotate(t2d, transform)
    blocks = rotated.unflatten(-1, (-1, NV_BLOCK))
    s_dec = _tensor_scale(rotated, (Q2_BWD_SCALES_MAX, Q2_BWD_GRID_MAX))
    scale = _e4m3_or_one(blocks.abs().amax(dim=-1, keepdim=True) / Q2_BWD_GRID_MAX / s_dec)
    unit = blocks / (scale * s_dec)
    grid = _signed_grid(unit)
    # the correction <x', x'> / <x', q> of the block (1 for a block that quantised to zeros), folded into its scale
    own, cross = (unit * unit).sum(-1, keepdim=True), (unit * grid).sum(-1, keepdim=True)
    empty = cross == 0
    wanted = scale * (own / cross.masked_fill(empty, 1.0)).masked_fill(empty, 1.0)
    down, up = e4m3_neighbours(wanted)
    width = up - down
    chance_up = ((wanted - down) / width.masked_fill(width <= 0, 1.0)).masked_fill(width <= 0, 0.0)
    if u is None:
        u = torch.rand_like(own[..., 0])
    return Quantized((grid * torch.where(u.unsqueeze(-1) < chance_up, up, down)).flatten(-2), s_dec)


def q2_hadamard() -> torch.Tensor:
    return hadamard(Q2_RHT) / math.sqrt(Q2_RHT)


class _Quartet2Linear(torch.autograd.Function):
    """Draws of a backward call, in this order from the device's global generator: the 128 signs, then the scale roundings of
    dy and W^T (Dgrad), dy^T and x^T (Wgrad)."""

    @staticmethod
    def forward(ctx, x, weight, native_gemm: bool):
        xq, wq = q2_rtn_quantize(x.flatten(0, -2)), q2_rtn_quantize(weight)
        y = _mm(xq.values, wq.values, native_gemm, torch.float32) * (xq.scale * wq.scale)
        stored = torch.bfloat16 if native_gemm else xq.values.dtype
        ctx.save_for_backward(xq.values.to(stored), xq.scale, wq.values.to(stored), wq.scale)
        ctx.native_gemm, ctx.like_x, ctx.like_w = native_gemm, (x.shape, x.dtype), weight.dtype
        to = torch.bfloat16 if native_gemm and x.dtype == torch.float32 else x.dtype
        return y.to(to).unflatten(0, x.shape[:-1])

    @staticmethod
    def backward(ctx, dy):
        x_values, x_scale, w_values, w_scale = ctx.saved_tensors
        (x_shape, x_dtype), rows = ctx.like_x, dy.flatten(0, -2)
        flips = torch.where(torch.rand(Q2_RHT, device=dy.device) < 0.5, 1.0, -1.0)
        turn = flips.unsqueeze(1) * q2_hadamard().to(dy.device)

        def product(left, right, carried):
            """left @ right^T with both sides re-quantised along the dot product; carried: the forward scale the stored side lacks."""
            lq, rq = q2_eden_quantize(left, turn), q2_eden_quantize(right, turn)
            return _mm(lq.values, rq.values, ctx.native_gemm, torch.float32) * (lq.scale * rq.scale * carried)

        dx = dw = None
        if ctx.needs_input_grad[0]:             # dx = dy W: the dot product over the output features
            dx = product(rows, w_values.float().t(), w_scale).view(x_shape).to(x_dtype)
        if ctx.needs_input_grad[1]:             # dW = dy^T x: the dot product over the tokens
            dw = product(rows.t(), x_values.float().t(), x_scale).to(ctx.like_w)
        return dx, dw, None


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
        if self.kind == "quartet2":
            return _Quartet2Linear.apply(x, weight, False)
        return _LowpLinear.apply(x, weight, self, False)


def recipe_for(cfg, name: str) -> Recipe:
    """The recipe the model config assigns to the linear called `name`."""
    if cfg.fp8.mode != "none":
        kind = "mxfp8" if cfg.fp8.scaling == "mxfp8" else "fp8_" + cfg.fp8.scaling
        return Recipe(kind)
    nv = cfg.nvfp4
    if any(name.endswith(k) or k in name for k in nv.fp8_names):
        return Recipe("mxfp8")
    if nv.recipe == "quartet2":
        return Recipe("quartet2")
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
    if lin.lowp.kind == "quartet2":
        return _Quartet2Linear.apply(x, lin.weight, True)
    return _LowpLinear.apply(x, lin.weight, lin.lowp, True)
