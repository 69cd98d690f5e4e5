"""Static-cache batched decode engine with a CUDA-graph step.

The reference's engine (ced/infer/engine.py:148-755) is batch 1, has no CUDA graph and refuses block-entry mixing,
the GDN write/query mixes, grid KV and the ssmax temperature; its feature-complete path is `prefill` / `extend` with
caches that grow by `torch.cat` (ced/eval/recall_ruler_gen.py:130-216). This engine covers every model feature at any
batch size with fixed-shape state:

* attention layers: key/value caches [B, max_len, Hkv, hd] allocated once. Keys are stored normed and UNROTATED; the
  decode kernel applies the rotation by min(distance, cap) while scoring (csrc/decode.cu), so the distance cap needs
  no second key copy. Grid KV layers cache the RAW row / column components [B, max_len, 1, width] (the reference's
  cache, ced/model/attention.py:943-1030: a 4 x 4 grid of 32-channel components holds 256 channels per token, the
  same bytes as 4 grouped KV heads); the key norm over the assembled head and the rotation are applied while scoring,
  on the GPU inside the grid decode kernel.
* GDN layers: the recurrent state S [B, Hv, dk, dv] (fp32) and the K-1 conv inputs, updated in place.
* one decode step (embedding -> all layers -> final norm -> head -> argmax) is captured in a CUDA graph on static
  input/output buffers; per-row lengths live on the device and advance inside the graph.

Prefill runs the training forward (flash attention + chunked GDN kernels) over whole prompts, a few rows at a time,
and copies the resulting caches into the static buffers. Oracle for tests: `HybridLM.prefill` / `extend`.
"""

from __future__ import annotations

import torch

from .. import ops
from .arena import GuardedBuffers
from ..models.attention import assemble_grid
from ..models.encoder import apply_layer_scalars
from ..models.gdn import READ_MIX_VARIANTS, GDNState
from ..models.rope import apply_rope, rotary_dims
from ..models.sequence import SeqContext


class DecodeEngine:
    def __init__(self, model, batch: int, max_len: int, device=None, splits: int | None = None, use_graph: bool = True):
        self.model = model.eval()
        self.cfg = model.cfg
        self.B, self.T = batch, max_len
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.native = self.device.type == "cuda" and ops.mode() == "native"
        self.use_graph = use_graph and self.device.type == "cuda"
        dev, B, T = self.device, batch, max_len
        # every static buffer sits between guard bands (infer/arena.py); `check_guards()` after a run finds a write past an end
        self.buffers = GuardedBuffers(dev)
        z = self.buffers.zeros
        self.lens = z("lens", B, torch.int32)                   # cached positions per row
        self.doc_start = z("doc_start", B, torch.int32)         # start of each row's current document
        self.doc_id = z("doc_id", B, torch.long)
        self.tokens = z("tokens", B, torch.long)                # static input of the step
        self.next_tokens = z("next_tokens", B, torch.long)      # static output of the step
        self.logits = z("logits", (B, self.cfg.vocab_size), torch.float32)
        self.layers = []
        if self.cfg.arch != "control":
            raise ValueError(f"the decode engine runs the hybrid stack (model.arch 'control'); arch {self.cfg.arch!r} generates through the model's own "
                             "cached forward (LoopedCED.generate)")
        if self.cfg.encoder.attn_res in ("block", "ldm"):
            raise ValueError(f"the decode engine walks the plain and the block-entry stacks; model.encoder.attn_res {self.cfg.encoder.attn_res!r} "
                             "generates through the model's cached forward (eval.generate)")
        if self.cfg.loop.recur_layers:
            raise ValueError("the decode engine walks every layer once; a looped middle (model.loop.recur_layers) generates through the "
                             "model's cached forward (eval.generate)")
        if self.cfg.loop.pass2_gate != "none":
            raise ValueError("the decode engine runs one pass; a gated second pass (model.loop.pass2_gate) generates through the model's "
                             "cached forward (eval.generate)")
        if self.cfg.encoder.gdn_ccr_spacing:
            raise ValueError("the decode engine keeps one state a GDN layer; the checkpoint cross-read (model.encoder.gdn_ccr_spacing) "
                             "generates through the model's cached forward (eval.generate)")
        if self.cfg.encoder.attn_res_query != "static":
            raise ValueError("the decode engine's block-entry reads are the static ones; model.encoder.attn_res_query 'token' "
                             "generates through the model's cached forward (eval.generate)")
        if self.cfg.encoder.gdn.kda.decay != "scalar" or self.cfg.encoder.gdn.erase.mode != "none" or self.cfg.encoder.gdn.dprod.n_h != 1:
            raise ValueError("the decode engine's GDN step kernel reads one decay a value head and one write a token: gdn.kda.decay "
                             "'channel', gdn.erase.mode 'eda' and gdn.dprod.n_h >= 2 generate "
                             "through the model's cached forward (eval.generate)")
        if self.cfg.encoder.attention.normalizer != "softmax":
            raise ValueError("the decode engine's attention kernel is the softmax one; attention.normalizer 'asentmax' generates "
                             "through the model's cached forward (eval.generate)")
        if self.cfg.encoder.canon_kernel:
            raise ValueError("the decode engine does not keep a Canon layer's input history (model.encoder.canon_kernel): "
                             "generate through the model's cached forward (eval.generate)")
        kv_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        for li, layer in enumerate(model.encoder.layers):
            m = layer.mixer
            if layer.kind == "attention":
                c = m.cfg
                heads, width = (1, m.grid.width) if m.grid is not None else (c.n_kv_heads, c.head_dim)
                rot = rotary_dims(c.head_dim, c.rope_fraction)
                n_ang = (m.cap + 1) if m.cap is not None else max_len
                st = {"k": z(f"layer{li}.k", (B, T, heads, width), kv_dtype),
                      "v": z(f"layer{li}.v", (B, T, heads, width), kv_dtype), "rot": rot, "heads": heads}
                if rot:
                    inv = c.rope_theta ** (-torch.arange(0, rot, 2, dtype=torch.float64, device=dev) / rot)
                    ang = torch.arange(n_ang, dtype=torch.float64, device=dev)[:, None] * inv
                    st["cos"], st["sin"] = ang.cos().float().contiguous(), ang.sin().float().contiguous()
                else:
                    st["cos"] = st["sin"] = torch.zeros(1, 1, device=dev)
                self.layers.append(st)
            else:
                g = m.cfg
                self.layers.append({"S": z(f"layer{li}.S", (B, g.n_v_heads, g.k_head_dim, g.v_head_dim), torch.float32),
                                    "conv": z(f"layer{li}.conv", (B, g.conv_kernel - 1, m.conv_channels), kv_dtype),
                                    "conv_doc": self.buffers.full(f"layer{li}.conv_doc", (B, g.conv_kernel - 1), -1, torch.long)})
        hq = max((l.mixer.cfg.n_q_heads for l in model.encoder.layers if l.kind == "attention"), default=1)
        self.splits = splits or max(1, min(64, (148 * 2) // max(1, B)))
        grid_layers = any(l.kind == "attention" and l.mixer.grid is not None for l in model.encoder.layers)
        scratch_splits = self.splits * (4 if grid_layers else 1)
        self.part_o = z("part_o", B * hq * scratch_splits * 64, torch.float32)
        self.part_ml = z("part_ml", B * hq * scratch_splits * 2, torch.float32)
        self.native_grid = True     # False: score grid layers through the assembled-heads statement (oracle of the grid kernel)
        self.graph = None
        self._host_len = 0          # host-side mirror of the (equal) row lengths: guards the static capacity before each launch

    def check_guards(self) -> None:
        """After a run: no static buffer was written past either end (raises `arena.GuardOverrun` naming it)."""
        self.buffers.check()

    # ------------------------------------------------------------------ sizes

    def cache_bytes(self) -> int:
        n = 0
        for st in self.layers:
            n += sum(t.numel() * t.element_size() for t in st.values() if isinstance(t, torch.Tensor))
        return n

    # ------------------------------------------------------------------ prefill

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, doc_ids: torch.Tensor | None = None, rows_per_pass: int = 4) -> torch.Tensor:
        """tokens (B, P): the prompts (equal length). Fills the caches and returns the first generated token (B,)."""
        B, P = tokens.shape
        assert B == self.B and P < self.T
        if doc_ids is None:
            doc_ids = torch.zeros_like(tokens)
        first = []
        for lo in range(0, B, rows_per_pass):
            hi = min(B, lo + rows_per_pass)
            single = bool((doc_ids[lo:hi] == doc_ids[lo:hi, :1]).all())
            out = self.model(tokens[lo:hi], doc_ids[lo:hi], return_cache=True, return_hidden=True, single_doc=single)
            h_last = out.hidden_aux[:, -1]
            logits = torch.nn.functional.linear(h_last.float(), self.model.head_weight().float())
            first.append(logits.argmax(-1))
            for st, layer, cache in zip(self.layers, self.model.encoder.layers, out.cache.encoder):
                if layer.kind == "attention":
                    m = layer.mixer
                    if m.grid is not None:      # raw components, as the model's own cache holds them
                        kn, v = cache.k, cache.v
                    else:
                        v = cache.v
                        if cache.k_far is not None or st["rot"] == 0:
                            kn = cache.k_far if cache.k_far is not None else cache.k
                        else:       # rotated keys without a cap: undo the rotation
                            kn = _unrotate(cache.k, doc_ids[lo:hi], m.cfg)
                    st["k"][lo:hi, :P] = kn.to(st["k"].dtype)
                    st["v"][lo:hi, :P] = v.to(st["v"].dtype)
                else:
                    st["S"][lo:hi] = cache.S.float()
                    st["conv"][lo:hi] = cache.conv_input.to(st["conv"].dtype)
                    st["conv_doc"][lo:hi] = cache.conv_doc
            d = doc_ids[lo:hi]
            start = torch.where(d == d[:, -1:], torch.arange(P, device=d.device)[None], torch.full_like(d, P)).min(1).values
            self.doc_start[lo:hi] = start.to(torch.int32)
            self.doc_id[lo:hi] = d[:, -1]
        self.lens.fill_(P)
        self._host_len = P
        nxt = torch.cat(first)
        self.tokens.copy_(nxt)
        return nxt

    # ------------------------------------------------------------------ one step

    def _attention_step(self, layer, st, h, pos):
        """h (B, 1, d) normed input; pos (B,) position of the new token inside its document."""
        m, c = layer.mixer, layer.mixer.cfg
        B, hq, hd = self.B, c.n_q_heads, c.head_dim
        gate = None
        if c.gate == "elementwise":
            q, gate = m.q_proj(h).view(B, 1, hq, 2 * hd).chunk(2, dim=-1)
        else:
            q = m.q_proj(h).view(B, 1, hq, hd)
            if m.g_proj is not None:
                gate = m.g_proj(h).view(B, 1, hq, 1)
        qn = m.q_norm(q.contiguous(), out_dtype=torch.float32) if hasattr(m.q_norm, "weight") else q.float()
        f = m.query_factor(pos[:, None], torch.float32)
        if f is not None:
            qn = qn * f
        if m.grid is not None:
            kw = m.grid.width
            k_new, v_new = m.k_proj(h).view(B, 1, 1, kw), m.v_proj(h).view(B, 1, 1, kw)
        else:
            k_new = m.k_norm(m.k_proj(h).view(B, 1, c.n_kv_heads, hd)) if hasattr(m.k_norm, "weight") else m.k_proj(h).view(B, 1, c.n_kv_heads, hd)
            v_new = m.v_proj(h).view(B, 1, c.n_kv_heads, hd)
        rows = torch.arange(B, device=h.device)
        at = self.lens.long()
        st["k"][rows, at] = k_new[:, 0].to(st["k"].dtype)
        st["v"][rows, at] = v_new[:, 0].to(st["v"].dtype)
        cap = m.cap if m.cap is not None else -1
        if m.grid is not None:
            g = m.grid
            normed = hasattr(m.k_norm, "weight")
            if self.native and self.native_grid and (g.rows, g.cols, g.row_dim, g.col_dim, g.heads_per_cell, g.depth) == (4, 4, 32, 32, 1, 0) and st["rot"] <= 32:
                from ..ops import native

                o = torch.empty(B, hq, hd, dtype=torch.bfloat16, device=h.device)
                splits = self.splits * 4          # one CTA serves all 16 heads of a split: four times the splits fill the same grid
                # (the norm's gain is stored zero-centred: the kernel takes 1 + w)
                native.ext().decode_attention_grid(qn.view(B, hq, hd).contiguous(), st["k"].view(B, self.T, kw), st["v"].view(B, self.T, kw),
                                                   (self.lens + 1).contiguous(), self.doc_start, st["cos"], st["sin"],
                                                   (1.0 + m.k_norm.weight.float()) if normed else None, o, self.part_o, self.part_ml, st["rot"], cap, splits,
                                                   hd ** -0.5, m.k_norm.eps if normed else 0.0)
                native._count(2)
                return m.output(o.view(B, 1, hq, hd).to(h.dtype) if gate is None else o.view(B, 1, hq, hd).to(gate.dtype), gate)
            # other grid shapes and the CPU: assemble the heads from the cached components, then the plain statement
            kk = m.k_norm(assemble_grid(st["k"], g).float())
            o = _decode_attention_reference(qn.view(B, hq, hd), kk, assemble_grid(st["v"], g), self.lens + 1, self.doc_start, st["cos"], st["sin"], st["rot"], cap)
            return m.output(o.view(B, 1, hq, hd).to(h.dtype) if gate is None else o.view(B, 1, hq, hd).to(gate.dtype), gate)
        if self.native and hd == 64:
            from ..ops import native

            o = torch.empty(B, hq, hd, dtype=torch.bfloat16, device=h.device)
            native.ext().decode_attention(qn.view(B, hq, hd).contiguous(), st["k"], st["v"], (self.lens + 1).contiguous(), self.doc_start, st["cos"], st["sin"], o,
                                          self.part_o, self.part_ml, st["rot"], cap, self.splits, hd ** -0.5)
            native._count(2)
            o = o.view(B, 1, hq, hd)
        else:
            o = _decode_attention_reference(qn.view(B, hq, hd), st["k"], st["v"], self.lens + 1, self.doc_start, st["cos"], st["sin"], st["rot"], cap)
            o = o.view(B, 1, hq, hd).to(h.dtype)
        return m.output(o.to(h.dtype) if gate is None else o.to(gate.dtype), gate)

    def _step_impl(self) -> None:
        model = self.model
        B = self.B
        enc = model.encoder
        pos = (self.lens - self.doc_start).long()
        idx = self.lens.long()[:, None]
        ctx = SeqContext(idx=idx, doc=self.doc_id[:, None], pos=pos[:, None], is_doc_start=torch.zeros(B, 1, dtype=torch.bool, device=self.device))
        ctx.memo["inplace_state"] = True       # the GDN step kernel updates this engine's static state buffers in place
        x = model.embed_tokens(self.tokens[:, None])
        S = enc.block
        sources = [x]
        n = len(enc.layers)
        scalars = enc.layer_scalar_args(x)
        for i, (layer, st) in enumerate(zip(enc.layers, self.layers)):
            if enc.block_entry and i % S == 0:
                start = x if i == 0 else layer.attn_res.entry(sources)
                x = start
            x_in = x
            h = layer.mixer_in_norm(x)
            if layer.kind == "gdn":
                arms = getattr(layer, "gdn_arms", None)
                kw = {}
                if arms is not None:
                    xw = layer.mixer_in_norm(arms.write_query(sources) if arms.write_query is not None else sources[0])
                    xr = None
                    if arms.variant in READ_MIX_VARIANTS:
                        xr = xw if arms.qmix_query is None else layer.mixer_in_norm(arms.read_mix(sources))
                    kw = dict(arms=arms, x_write=xw, x_read=xr)
                state = GDNState(conv_input=st["conv"], conv_doc=st["conv_doc"], S=st["S"])
                mixed, new = layer.mixer(h, ctx, state, **kw)
                if new.S is not st["S"]:          # the step kernel updated the buffer in place
                    st["S"].copy_(new.S)
                st["conv"].copy_(new.conv_input.to(st["conv"].dtype))
                st["conv_doc"].copy_(new.conv_doc)
            else:
                mixed = self._attention_step(layer, st, h, pos)
            x = ops.norm_add(x, mixed, layer.mixer_out_norm.weight, layer.mixer_out_norm.eps, layer.residual_scale)
            x = ops.norm_add(x, layer.mlp(layer.mlp_in_norm(x)), layer.mlp_out_norm.weight, layer.mlp_out_norm.eps, layer.residual_scale)
            if scalars is not None:
                x = apply_layer_scalars(x, x_in, *scalars[i])
            if enc.block_entry and i % S == S - 1:
                sources = sources + [x - start]
        if enc.block_entry:
            x = enc.layers[n - 1].attn_res.out(sources)
        hidden = model.final_norm(x)[:, 0]
        w = model.head_weight_lp if (self.native and model.head_weight_lp is not None) else model.head_weight()
        if self.native:
            from ..ops import native

            native.gemm(hidden.to(torch.bfloat16).contiguous(), w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16), out=self.logits)
        else:
            self.logits.copy_(torch.nn.functional.linear(hidden.float(), w.float()))
        self.next_tokens.copy_(self.logits.argmax(-1))
        self.tokens.copy_(self.next_tokens)
        self.lens.add_(1)

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Consume `self.tokens`, append it to the caches, return the next token of every row (B,) (a static buffer)."""
        if self._host_len + 1 > self.T:
            raise RuntimeError(f"decode cache is full: {self._host_len} positions cached, capacity {self.T}")
        self._host_len += 1
        if not self.use_graph:
            self._step_impl()
            return self.next_tokens
        if self.graph is None:
            self._capture()
        self.graph.replay()
        return self.next_tokens

    def _capture(self) -> None:
        """Warm up on a side stream, then capture one step. State touched by the warm-up steps is restored before the
        capture, and the captured step itself is not run by capture."""
        if self._host_len + 2 > self.T:
            raise RuntimeError("the capture's two warm-up steps need two free cache positions")
        snap = self._snapshot()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step_impl()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._restore(snap)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_impl()
        self._restore(snap)

    def _snapshot(self):
        snap = {"lens": self.lens.clone(), "tokens": self.tokens.clone(), "gdn": []}
        for st in self.layers:
            if "S" in st:
                snap["gdn"].append((st["S"].clone(), st["conv"].clone(), st["conv_doc"].clone()))
        return snap

    def _restore(self, snap) -> None:
        self.lens.copy_(snap["lens"])
        self.tokens.copy_(snap["tokens"])
        it = iter(snap["gdn"])
        for st in self.layers:
            if "S" in st:
                S, c, d = next(it)
                st["S"].copy_(S), st["conv"].copy_(c), st["conv_doc"].copy_(d)

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, new_tokens: int, doc_ids: torch.Tensor | None = None) -> torch.Tensor:
        """Greedy continuation: (B, new_tokens) token ids (the first comes from the prefill)."""
        out = [self.prefill(prompts, doc_ids).clone()]
        for _ in range(new_tokens - 1):
            out.append(self.step().clone())
        return torch.stack(out, dim=1)


def _unrotate(k, doc_ids, cfg):
    """Keys rotated at their document positions back to the unrotated normed keys."""
    B, P = doc_ids.shape
    idx = torch.arange(P, device=k.device)[None].expand(B, P)
    starts = torch.cat([torch.ones(B, 1, dtype=torch.bool, device=k.device), doc_ids[:, 1:] != doc_ids[:, :-1]], 1)
    begin = torch.where(starts, idx, torch.zeros_like(idx)).cummax(1).values
    return apply_rope(k, -(idx - begin), cfg.rope_fraction, cfg.rope_theta)


def _decode_attention_reference(q, k, v, lens, doc_start, cos_t, sin_t, rot, cap):
    """PyTorch statement of csrc/decode.cu: q (B,Hq,hd) fp32 unrotated; k, v (B,T,Hkv,hd); returns (B,Hq,hd) fp32."""
    B, Hq, hd = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    t = torch.arange(T, device=q.device)[None]
    qpos = (lens.long() - 1)[:, None]
    allow = (t <= qpos) & (t >= doc_start.long()[:, None])
    kf = k.float()
    if rot:
        d = (qpos - t).clamp(min=0)
        if cap >= 0:
            d = d.clamp(max=cap)
        d = d.clamp(max=cos_t.shape[0] - 1)
        c, s = cos_t[d][:, :, None, :], sin_t[d][:, :, None, :]
        half = rot // 2
        x1, x2 = kf[..., :half], kf[..., half:rot]
        kf = torch.cat([x1 * c + x2 * s, x2 * c - x1 * s, kf[..., rot:]], dim=-1)
    rep = Hq // Hkv
    kk = kf.repeat_interleave(rep, dim=2)
    vv = v.float().repeat_interleave(rep, dim=2)
    sc = torch.einsum("bhd,bthd->bht", q.float(), kk) * hd ** -0.5
    sc = sc.masked_fill(~allow[:, None], float("-inf"))
    return torch.einsum("bht,bthd->bhd", torch.softmax(sc, -1), vv)
