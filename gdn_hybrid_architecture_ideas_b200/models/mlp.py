"""Dense feed-forward blocks: SwiGLU `w_down(silu(w_gate x) * w_up x)` and ReLU-squared, bias-free
(reference: ced/model/mlp.py:12-60). On CUDA the gate and up projections run as one tcgen05 GEMM whose epilogue
applies the activation (`ops.swiglu_mlp`)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class SwiGLU(nn.Module):
    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.w_gate = Linear(d_model, hidden)
        self.w_up = Linear(d_model, hidden)
        self.w_down = Linear(hidden, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.swiglu_mlp(x, self.w_gate, self.w_up, self.w_down)


class ReLU2(nn.Module):
    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.w_up = Linear(d_model, hidden)
        self.w_down = Linear(hidden, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w_down(F.relu(self.w_up(x)).square())


def dense_ffn(d_model: int, hidden: int, activation: str) -> nn.Module:
    if activation == "swiglu":
        return SwiGLU(d_model, hidden)
    if activation == "relu2":
        return ReLU2(d_model, hidden)
    raise ValueError(f"ffn_activation {activation!r}: 'swiglu' or 'relu2'")


class RoutedSwiGLU(nn.Module):
    """Mixture of SwiGLU experts with top-k routing per token. The gates are the router's softmax over experts, kept at
    the k largest and renormalised; the output is the gate-weighted sum of the chosen experts. Tokens are dispatched:
    each expert runs only on the tokens routed to it (a gather, the expert's three GEMMs, a scatter-add), which equals
    running every expert on every token and weighting by the gates (`forward_dense`, the statement the reference uses:
    ced/model/mlp.py:61-109). Routing statistics accumulate over calls since `reset_stats()`:
    balance_loss = n_experts * sum_e (share of routed slots to e) * (mean router probability of e) (1 when uniform),
    z_loss = mean over tokens of logsumexp(router logits)^2."""

    def __init__(self, d_model: int, n_experts: int, top_k: int, expert_hidden: int):
        super().__init__()
        self.n_experts, self.top_k = n_experts, top_k
        self.router = Linear(d_model, n_experts)
        self.experts = nn.ModuleList(SwiGLU(d_model, expert_hidden) for _ in range(n_experts))
        self.reset_stats()

    def reset_stats(self) -> None:
        self._chosen, self._prob, self._n, self._z = 0.0, 0.0, 0.0, 0.0

    def balance_loss(self) -> torch.Tensor:
        frac = self._chosen / (self._n * self.top_k)
        return self.n_experts * (frac * (self._prob / self._n)).sum()

    def z_loss(self) -> torch.Tensor:
        return self._z / self._n

    def gates(self, x: torch.Tensor, valid: torch.Tensor | None = None) -> torch.Tensor:
        logits = torch.nn.functional.linear(x, self.router.weight.to(x.dtype))
        probs = torch.softmax(logits.to(torch.promote_types(logits.dtype, torch.float32)), dim=-1)
        top_p, top_i = probs.topk(self.top_k, dim=-1)
        g = torch.zeros_like(probs).scatter(-1, top_i, top_p / top_p.sum(-1, keepdim=True))
        w = torch.ones(x.shape[:-1], dtype=probs.dtype, device=x.device) if valid is None else valid.to(probs.dtype)
        dims = tuple(range(probs.dim() - 1))
        self._chosen = self._chosen + ((g > 0).to(probs.dtype) * w[..., None]).sum(dim=dims)
        self._prob = self._prob + (probs * w[..., None]).sum(dim=dims)
        self._n = self._n + w.sum().clamp(min=1)
        self._z = self._z + (torch.logsumexp(logits.to(probs.dtype), dim=-1).pow(2) * w).sum()
        return g

    def forward(self, x: torch.Tensor, valid: torch.Tensor | None = None) -> torch.Tensor:
        g = self.gates(x, valid)
        flat, gf = x.reshape(-1, x.shape[-1]), g.reshape(-1, self.n_experts)
        out = torch.zeros_like(flat)
        for e, expert in enumerate(self.experts):
            rows = torch.nonzero(gf[:, e] > 0).squeeze(-1)
            if rows.numel():
                y = expert(flat.index_select(0, rows).unsqueeze(0)).squeeze(0)
                out = out.index_add(0, rows, gf[rows, e].to(x.dtype)[:, None] * y)
        return out.view_as(x)

    def forward_dense(self, x: torch.Tensor, valid: torch.Tensor | None = None) -> torch.Tensor:
        g = self.gates(x, valid)
        return sum(g[..., e:e + 1].to(x.dtype) * expert(x) for e, expert in enumerate(self.experts))
