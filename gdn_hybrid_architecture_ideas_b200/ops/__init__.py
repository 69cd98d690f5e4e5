"""Op layer: every model op has a pure-PyTorch statement (`ops.reference`) and, for CUDA tensors, a hand-written
sm_100a kernel behind a `torch.autograd.Function` (`ops.native`).

Dispatch rule: a CUDA input runs the native kernel unless the process set `GHB_KERNELS=reference` (debug switch, used
to produce oracle values on the GPU). A CUDA input with the extension missing raises: there is no silent fallback.
CPU inputs always run the reference statement (the gloo/CPU path and the tests' oracle).
"""

from __future__ import annotations

import os

import torch

from . import reference as ref

_MODE = os.environ.get("GHB_KERNELS", "native")


def set_mode(mode: str) -> None:
    """"native" (default) or "reference": which implementation CUDA tensors use."""
    global _MODE
    assert mode in ("native", "reference"), mode
    _MODE = mode


def mode() -> str:
    return _MODE


def use_native(x: torch.Tensor) -> bool:
    return x.is_cuda and _MODE == "native"


def _native():
    from . import native
    return native


def rmsnorm(x, weight, eps, out_dtype=None):
    if use_native(x):
        return _native().rmsnorm(x, weight, eps, out_dtype)
    return ref.rmsnorm(x, weight, eps, out_dtype)


def prenorm(x, weight, eps):
    """(RMSNorm(x), x): the branch input and the stream for the residual add. On CUDA one autograd node, so the stream's
    two gradients are summed inside the norm's backward kernel."""
    if use_native(x) and x.dtype == torch.float32 and weight.dtype == torch.float32 and x.shape[-1] % 4 == 0 and x.shape[-1] <= 2048 \
            and torch.is_grad_enabled() and x.requires_grad:
        return _native().prenorm(x, weight, eps)
    return rmsnorm(x, weight, eps), x


def gated_rmsnorm(x, z, weight, eps, gate, out_dtype=None):
    if use_native(x):
        return _native().gated_rmsnorm(x, z, weight, eps, gate, out_dtype)
    return ref.gated_rmsnorm(x, z, weight, eps, gate, out_dtype)


def _tp_linear(x, lin):
    from ..parallel import tensor_parallel as tpm
    tp = lin.tp
    if lin.tp_mode == "column":
        return tpm.column_parallel(x, lin, tp).view(*tp.batch_shape, -1)
    return tpm.row_parallel(x, lin, tp).unsqueeze(0)


def linear(x, lin):
    if getattr(lin, "tp_mode", None) is not None:
        return _tp_linear(x, lin)
    if use_native(x):
        return _native().linear(x, lin)
    if getattr(lin, "precision", "bf16") != "bf16" and lin.training:
        return lin.lowp.emulated_linear(x, lin.weight)
    return ref.linear(x, lin)


def split_linear(xa, xb, lin, n):
    """[lin.rows(0, n)(xa) | lin.rows(n, N)(xb)]: two row ranges of one projection reading two inputs."""
    if getattr(lin, "tp_mode", None) is not None:
        return torch.cat([linear(xa, lin.rows(0, n)), linear(xb, lin.rows(n, lin.weight.shape[0]))], dim=-1)
    if use_native(xa):
        return _native().split_linear(xa, xb, lin, n)
    return torch.cat([linear(xa, lin.rows(0, n)), linear(xb, lin.rows(n, lin.weight.shape[0]))], dim=-1)


def input_mixes(x, y_write, lam_write, y_read=None, lam_read=None):
    """The write (and query) input of a GDN layer with mixes: x + lam (y - x) per mix."""
    if use_native(x) and x.dtype == torch.bfloat16:
        return _native().input_mixes(x, y_write, lam_write, y_read, lam_read)
    return ref.input_mixes(x, y_write, lam_write, y_read, lam_read)


def swiglu_mlp(x, w_gate, w_up, w_down):
    if getattr(w_gate, "tp_mode", None) is not None:
        return linear(torch.nn.functional.silu(linear(x, w_gate)) * linear(x, w_up), w_down)
    if use_native(x):
        return _native().swiglu_mlp(x, w_gate, w_up, w_down)
    return linear(torch.nn.functional.silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv, hist=None, hist_doc=None, single_doc=False, packed=False):
    """(q, k, v, conv history, its document ids); packed: (qkv, history, ids) with qkv = [q | k | v] per token, the
    layout `delta_rule_packed` reads."""
    if use_native(u_pre) and hist is None:
        return _native().gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv, single_doc, packed)
    if use_native(u_pre) and u_pre.dtype == torch.bfloat16:
        return _native().gdn_prep_cached(u_pre, doc, conv_weight, hk, hv, dk, dv, hist, hist_doc, packed)
    q, k, v, h, hd = ref.gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv, hist, hist_doc)
    if packed:
        return torch.cat([q.flatten(2), k.flatten(2), v.flatten(2)], dim=-1), h, hd
    return q, k, v, h, hd


def gdn_gates(a_lin, b_lin, A_log, dt_bias, scale=1, beta_power=False):
    if use_native(a_lin) and scale == 1:
        return _native().gdn_gates(a_lin, b_lin, A_log, dt_bias)
    return ref.gdn_gates(a_lin, b_lin, A_log, dt_bias, scale, beta_power)


def delta_rule(q, k, v, g, beta, is_doc_start, S0, kernel="chunked", chunk_size=64, need_state=True, inplace_state=False):
    """(o, S_final). q,k (B,L,Hk,dk) with Hv a multiple of Hk: value head j reads key head j // (Hv/Hk).
    inplace_state: a single cached token may update S0 in place and return it (the decode engine's static buffers)."""
    if use_native(q) and q.shape[1] > 1:
        return _native().delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size, need_state)
    if use_native(q):
        from . import gdn_native
        if gdn_native.step_ok(q, v, S0):
            return gdn_native.delta_rule_step(q, k, v, g, beta, is_doc_start, S0, inplace_state)
    rep = v.shape[2] // q.shape[2]
    if rep > 1:
        q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    out_dtype = v.dtype
    if q.is_cuda:      # a cached step on the device: the recurrence runs in fp32 on the fp32 state
        q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if S0 is None:
        S0 = q.new_zeros(q.shape[0], v.shape[2], q.shape[-1], v.shape[-1])
    elif q.is_cuda:
        S0 = S0.float()
    if q.is_cuda:
        o, S = (ref.delta_rule_recurrence if (kernel == "recurrence" or q.shape[1] == 1) else ref.chunked_delta_rule)(
            q, k, v, g, beta, is_doc_start, S0, *(() if (kernel == "recurrence" or q.shape[1] == 1) else (chunk_size,)))
        return o.to(out_dtype), S
    if kernel == "recurrence" or q.shape[1] == 1:
        return ref.delta_rule_recurrence(q, k, v, g, beta, is_doc_start, S0)
    return ref.chunked_delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size)


def delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, is_doc_start, S0, kernel="chunked", chunk_size=64, need_state=True, inplace_state=False):
    """`delta_rule` on the packed [q | k | v] tensor of `gdn_prep(packed=True)`: on the CUDA kernels the whole rule is
    one autograd node whose gradient returns packed the same way."""
    B, L, _ = qkv.shape
    if use_native(qkv) and L > 1 and kernel != "recurrence":
        from . import gdn_native
        if gdn_native.packed_ok(qkv, hk, hv, dk, dv, chunk_size):
            return _native().delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, is_doc_start, S0, need_state)
    nq = hk * dk
    q, k, v = qkv[..., :nq].view(B, L, hk, dk), qkv[..., nq:2 * nq].view(B, L, hk, dk), qkv[..., 2 * nq:].view(B, L, hv, dv)
    return delta_rule(q, k, v, g, beta, is_doc_start, S0, kernel=kernel, chunk_size=chunk_size, need_state=need_state, inplace_state=inplace_state)


def attention(q, k, v, q_idx, q_doc, k_idx, k_doc, k_ok=None, q_far=None, k_far=None, cap=None, self_aligned=False, q_pos=None,
              single_doc=False):
    """self_aligned: queries and keys are the same positions of the same rows (a training forward without a cache),
    which is the case the fused training kernel covers."""
    if use_native(q) and self_aligned:
        return _native().attention(q, k, v, q_doc, q_far, k_far, cap, q_pos, single_doc)
    return ref.attention(q, k, v, q_idx, q_doc, k_idx, k_doc, k_ok, q_far, k_far, cap)


def norm_add(resid, branch, weight, eps, scale):
    """resid + scale * rmsnorm(branch): the Peri-LN residual update."""
    if use_native(branch):
        return _native().norm_add(resid, branch, weight, eps, scale)
    return resid + scale * ref.rmsnorm(branch, weight, eps)


_cpu_status = torch.zeros(1, dtype=torch.int32)


def status_word(device) -> torch.Tensor:
    """The per-device int32 word that kernels write when a bounded wait gives up (0 = clean). On the CPU a process-wide
    word with the same contract (nothing writes it but tests and host-side fault injection)."""
    if torch.device(device).type == "cuda":
        return _native().err_flag(device)
    return _cpu_status


def clear_status(device) -> None:
    status_word(device).zero_()


def check_status() -> None:
    """Raises if any device's status word is non-zero (one host read per device), and clears it."""
    code = int(_cpu_status.item())
    if code:
        _cpu_status.zero_()
        raise RuntimeError(f"status {code} reported on the CPU status word")
    if torch.cuda.is_available():
        _native().check_status()


def launch_count() -> int:
    """Kernels of this framework launched since the last reset (bench.py reports it)."""
    from . import native
    return native.launch_count()


def reset_launch_count() -> None:
    from . import native
    native.reset_launch_count()


def depth_mix(sources, query, gain, eps):
    if use_native(sources[0]):
        return _native().depth_mix(sources, query, gain, eps)
    return ref.depth_mix(sources, query, gain, eps)


def depth_mix_multi(sources, readers, eps):
    """Several depth-mix readers [(query, key-norm gain)] over the same sources: a list of mixes, one per reader."""
    if use_native(sources[0]) and len(sources) > 1:
        return _native().depth_mix_multi(sources, readers, eps)
    return [depth_mix(sources, q, g, eps) for q, g in readers]


def embedding(tokens, weight):
    if use_native(weight):
        return _native().embedding(tokens, weight)
    return ref.embedding(tokens, weight)


def lm_loss_sums(hidden, weight, targets, weights=None, z_loss=0.0, weight_lp=None):
    if use_native(hidden):
        return _native().lm_loss_sums(hidden, weight, targets, weights, z_loss, weight_lp)
    return ref.lm_loss_sums(hidden, weight, targets, weights, z_loss)
