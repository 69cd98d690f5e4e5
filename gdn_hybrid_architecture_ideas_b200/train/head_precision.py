"""The precision of the LM head's three matmuls in the training loss (`head_precision`).

  "fp32"  float32 operands (float64 for float64 inputs): the reference statement.
  "bf16"  every operand of the three products is rounded once to bfloat16 (round to nearest even),
              logits = bf16(h) bf16(W)^T,   dh = bf16(G) bf16(W),   dW += bf16(G)^T bf16(h),
          and the products are accumulated in the compute dtype (float32; float64 for float64 inputs, the exact form of the
          same function the tests use) into outputs of that dtype. Softmax, log-sum-exp, CE, z-loss and the logit gradient G
          are computed in the compute dtype from those logits; G is rounded only as an operand of the two backward products.
          A product of two bfloat16 numbers is exact in float32, so this is: exact products of the rounded operands, summed
          in float32.

On a GPU the native fused head IS the "bf16" form (bf16 operands into the tcgen05 GEMM, fp32 accumulators, fp32 softmax in
the CE kernel) whatever the key says; the key selects the form of the PyTorch statements (the CPU path, and the oracle the
GPU tests compare with). Scores never read it: evaluation runs the float32 head. Reference: ced/train/head_precision.py.
"""

from __future__ import annotations

import torch

PRECISIONS = ("fp32", "bf16")


def check_head_precision(precision: str) -> str:
    if precision not in PRECISIONS:
        raise ValueError(f"head_precision {precision!r}: one of {PRECISIONS} ('fp32': float32 operands; 'bf16': operands rounded to "
                         "bfloat16, float32 accumulation and float32 softmax / CE)")
    return precision


def round_operand(x: torch.Tensor, precision: str) -> torch.Tensor:
    """x as an operand of a head product: itself for "fp32", rounded through bfloat16 (same dtype back) for "bf16"."""
    return x if precision == "fp32" else x.to(torch.bfloat16).to(x.dtype)


def mm_acc(a: torch.Tensor, b: torch.Tensor, precision: str) -> torch.Tensor:
    """a @ b with the operands of `precision`, accumulated in a's dtype (the compute dtype)."""
    return round_operand(a, precision) @ round_operand(b, precision)


def addmm_acc_(acc: torch.Tensor, a: torch.Tensor, b: torch.Tensor, precision: str) -> torch.Tensor:
    """acc += a @ b, in place."""
    return acc.addmm_(round_operand(a, precision), round_operand(b, precision))


class _HeadLinear(torch.autograd.Function):
    """logits = h W^T at a head precision, with dh and dW formed from the rounded logit gradient as the module docstring says."""

    @staticmethod
    def forward(ctx, h, W, precision):
        ctx.save_for_backward(h, W)
        ctx.precision = precision
        return mm_acc(h, W.t(), precision)

    @staticmethod
    def backward(ctx, g):
        h, W = ctx.saved_tensors
        p = ctx.precision
        lead = g.reshape(-1, g.shape[-1])
        return mm_acc(g, W, p), mm_acc(lead.t(), h.reshape(-1, h.shape[-1]), p), None


def head_linear(h: torch.Tensor, W: torch.Tensor, precision: str = "fp32") -> torch.Tensor:
    """h (..., d) in the compute dtype, W (V, d) -> logits (..., V)."""
    check_head_precision(precision)
    if precision == "fp32":
        return torch.nn.functional.linear(h, W)
    return _HeadLinear.apply(h, W, precision)
