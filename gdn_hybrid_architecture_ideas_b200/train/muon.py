"""Muon for hidden 2-D matrices with AdamW for everything else, on the flat buffers.

Muon: Nesterov momentum (0.95), then the momentum matrix is orthogonalised by 5 Polar-Express iterations in bfloat16
(X <- X / (||X|| * 1.01 + 1e-7); A = X X^T; B = b A + c A^2; X <- a X + B X, per-step (a, b, c)), and the weight moves
by W <- W (1 - lr wd) - lr * 0.2 * sqrt(max(m, n)) * O (reference: ced/train/muon.py:30-128). Whole matrices are
needed, so under sharding a matrix belongs to one rank (ZeRO-1 by whole tensor, parallel/zero.py).
"""

from __future__ import annotations

import torch

from .optim import FlatAdamW, FlatBuffers

# Polar Express coefficients (Amsel et al., arXiv 2505.16932), safety-scaled as in the public reference code.
_PE = [(8.28721201814563, -23.595886519098837, 17.300387312530933),
       (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
       (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
       (3.3184196573706015, -2.488488024314874, 0.51004894012372),
       (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
       (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
       (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
       (1.875, -1.25, 0.375)]
# the paper's listing evaluates p(x / 1.01) for every tuple but the last
_PE = [(a / 1.01, b / 1.01 ** 3, c / 1.01 ** 5) for a, b, c in _PE[:-1]] + [_PE[-1]]


def polar_express(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate orthogonal factor of G (m, n), iterated in bfloat16 on the wide orientation."""
    X = G.to(torch.bfloat16)
    tall = X.shape[0] > X.shape[1]
    if tall:
        X = X.T
    X = X / (X.norm() * 1.01 + 1e-7)
    for a, b, c in (_PE[min(i, len(_PE) - 1)] for i in range(steps)):
        A = X @ X.T
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return (X.T if tall else X).to(G.dtype)


class MuonWithAdamW(FlatAdamW):
    def __init__(self, flat: FlatBuffers, groups, o, shard=None, owned_names: set | None = None):
        super().__init__(flat, groups, o.betas, o.eps, shard)
        self.momentum, self.nesterov, self.ns_steps = o.muon_momentum, o.muon_nesterov, o.muon_ns_steps
        self.owned_names = owned_names  # None: every matrix (replicated); else this rank's matrices (ZeRO-1)
        self.mats = [s for s in flat.segments if groups[s.group]["kind"] == "muon"]
        self.buf = {s.name: torch.zeros(s.shape, dtype=torch.float32, device=flat.params.device) for s in self.mats
                    if owned_names is None or s.name in owned_names}

    @torch.no_grad()
    def step(self, lr: float, grad_scale=1.0) -> None:
        super().step(lr, grad_scale, kinds=("adamw",))
        for s in self.mats:
            if s.name not in self.buf:
                continue
            g = self.flat.view(self.flat.grads, s.name) * grad_scale
            wd = self.param_groups[s.group]["weight_decay"]
            m = self.buf[s.name].mul_(self.momentum).add_(g)
            upd = polar_express(g.add(m, alpha=self.momentum) if self.nesterov else m, self.ns_steps)
            W = self.flat.view(self.flat.params, s.name)
            W.mul_(1.0 - lr * wd).add_(upd, alpha=-lr * 0.2 * max(s.shape) ** 0.5)
            if self.flat.lp is not None:
                self.flat.view(self.flat.lp, s.name).copy_(W)

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["muon"] = {n: b.clone() for n, b in self.buf.items()}
        return sd

    def load_state_dict(self, sd: dict) -> None:
        super().load_state_dict(sd)
        for n, b in (sd.get("muon") or {}).items():
            if n in self.buf:
                self.buf[n].copy_(b)

    def reset_moments(self) -> None:
        super().reset_moments()
        for b in self.buf.values():
            b.zero_()
