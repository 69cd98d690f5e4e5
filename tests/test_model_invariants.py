"""Behavioural invariants of the model, in float64 on the CPU so nothing hides behind a tolerance: causality of outputs
and of gradients, isolation of packed documents, teacher-forced logits equal cached generation token by token and in
random chunks, grid-shared keys equal ordinary multi-head attention with the assembled weights (values and gradient
sums), and the zero-initialised mixes start as the plain model.
(The reference's suites of the same names: tests/test_causality.py, test_cache_consistency.py, test_grid_kv.py,
test_export_components.py.)"""

import copy

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import build_model
from gdn_hybrid_architecture_ideas_b200.models.attention import assemble_grid, grid_spec
from tests.helpers import make_model, random_rows

L = 48


def _grid(cfg, rows, cols, rd, cd, depth=0, dd=0):
    a = cfg.encoder.attention
    a.kv_sharing, a.n_kv_heads, a.grid_rows, a.grid_cols, a.row_dim, a.col_dim = "grid", 1, rows, cols, rd, cd
    a.grid_depth, a.depth_dim = depth, dd
    a.n_q_heads, a.head_dim = rows * cols * max(depth, 1), rd + cd + dd
    return cfg


def _variants():
    full = C.tiny_full_config
    plain = C.tiny_control_config
    out = {"control": plain(), "full": full(), "grid_2x2": _grid(full(), 2, 2, 8, 8), "grid_2x4": _grid(full(), 2, 4, 8, 8),
           "grid_2x2x2": _grid(plain(), 2, 2, 8, 4, 2, 4)}
    untied = full()
    untied.tie_embeddings = False
    out["untied"] = untied
    nocap = full()
    nocap.encoder.attention.rope_max_distance = None
    out["nocap"] = nocap
    return out


VARIANTS = _variants()


def _chunked(model, tokens, docs, boundaries):
    edges = [0, *boundaries, tokens.shape[1]]
    out, pieces = None, []
    for a, b in zip(edges[:-1], edges[1:]):
        out = model.prefill(tokens[:, a:b], docs[:, a:b]) if out is None else model.extend(tokens[:, a:b], docs[:, a:b], None, out.cache)
        pieces.append(out.logits)
    return torch.cat(pieces, dim=1)


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_future_token_does_not_change_past_outputs(name):
    model = make_model(copy.deepcopy(VARIANTS[name])).eval()
    tokens, docs = random_rows(2, L, model.cfg.vocab_size, seed=1)
    with torch.no_grad():
        base = model(tokens, docs).logits
        for j in (1, 7, 20, 33, L - 1):
            changed = tokens.clone()
            changed[:, j] = (changed[:, j] + 1 + j) % model.cfg.vocab_size
            out = model(changed, docs).logits
            assert torch.equal(out[:, :j], base[:, :j]), f"outputs before {j} changed"
            assert not torch.equal(out[:, j:], base[:, j:]), "the change had no effect at all (the test is vacuous)"


@pytest.mark.parametrize("name", ["control", "full", "grid_2x2"])
def test_gradients_do_not_flow_from_future_inputs(name):
    """d logits[t] / d (embedding output at s) is exactly zero for every s > t: catches leaks through gathers, masks or
    the chunked recurrences that a forward-only check could miss."""
    model = make_model(copy.deepcopy(VARIANTS[name]))
    tokens, docs = random_rows(1, L, model.cfg.vocab_size, seed=3)
    captured = {}
    embed_tokens = model.embed_tokens

    def keep(tok):
        out = embed_tokens(tok)
        out.retain_grad()
        captured["h"] = out
        return out

    model.embed_tokens = keep
    try:
        for t in (0, 9, 24, 40):
            model.zero_grad(set_to_none=True)
            logits = model(tokens, docs).logits
            logits[:, t].sum().backward()
            grad = captured["h"].grad
            assert torch.count_nonzero(grad[:, t + 1:]) == 0, f"future inputs influence position {t}"
            assert torch.count_nonzero(grad[:, : t + 1]) > 0
    finally:
        model.embed_tokens = embed_tokens


@pytest.mark.parametrize("name", ["control", "full", "grid_2x2"])
def test_packed_documents_are_isolated(name):
    """A document packed after another gives the outputs it gives alone: attention masks, GDN state and conv window
    resets, document-relative rotary positions."""
    model = make_model(copy.deepcopy(VARIANTS[name])).eval()
    tokens, _ = random_rows(1, L, model.cfg.vocab_size, seed=4, docs=False)
    split = 19
    docs = torch.zeros(1, L, dtype=torch.long)
    docs[:, split:] = 1
    with torch.no_grad():
        packed = model(tokens, docs).logits
        first = model(tokens[:, :split], torch.zeros(1, split, dtype=torch.long)).logits
        second = model(tokens[:, split:], torch.zeros(1, L - split, dtype=torch.long)).logits
    torch.testing.assert_close(packed[:, :split], first, rtol=0, atol=1e-10)
    torch.testing.assert_close(packed[:, split:], second, rtol=0, atol=1e-10)


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_teacher_forced_equals_token_by_token(name):
    model = make_model(copy.deepcopy(VARIANTS[name])).eval()
    tokens, docs = random_rows(2, L, model.cfg.vocab_size, seed=10)
    with torch.no_grad():
        teacher = model(tokens, docs).logits
        stepwise = _chunked(model, tokens, docs, list(range(1, L)))
    torch.testing.assert_close(stepwise, teacher, rtol=0, atol=1e-10)


@pytest.mark.parametrize("seed", [0, 1, 2])
@pytest.mark.parametrize("name", ["full", "grid_2x4"])
def test_teacher_forced_equals_random_chunked_prefill(name, seed):
    model = make_model(copy.deepcopy(VARIANTS[name])).eval()
    tokens, docs = random_rows(2, L, model.cfg.vocab_size, seed=20 + seed)
    g = torch.Generator().manual_seed(seed)
    boundaries = sorted(torch.randperm(L - 1, generator=g)[:5].add(1).tolist())
    with torch.no_grad():
        torch.testing.assert_close(_chunked(model, tokens, docs, boundaries), model(tokens, docs).logits, rtol=0, atol=1e-10)


def test_greedy_generation_matches_teacher_forced_rescoring():
    from gdn_hybrid_architecture_ideas_b200.eval.generate import generate_greedy_batched

    model = make_model(C.tiny_full_config()).eval()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (30, 30)]
    new = generate_greedy_batched(model, prompts, 12)
    full = torch.tensor([p + n for p, n in zip(prompts, new)])
    with torch.no_grad():
        rescored = model(full, torch.zeros_like(full)).logits[:, 29:29 + 12].argmax(-1)
    assert torch.equal(rescored, torch.tensor(new))


@pytest.mark.parametrize("name", ["grid_2x2", "grid_2x4", "grid_2x2x2"])
def test_grid_keys_equal_multi_head_attention_with_the_assembled_weights(name):
    """Grid sharing is ordinary multi-head attention whose per-head key / value projections are assembled from the
    component projections: same logits, and the component weights' gradients are the SUMS of the assembled heads'."""
    cfg = copy.deepcopy(VARIANTS[name])
    grid_model = make_model(cfg)
    a = cfg.encoder.attention
    spec = grid_spec(a)
    mha_cfg = copy.deepcopy(cfg)
    m = mha_cfg.encoder.attention
    m.kv_sharing, m.n_kv_heads = "gqa", a.n_q_heads
    m.grid_rows = m.grid_cols = m.row_dim = m.col_dim = m.grid_depth = m.depth_dim = 0
    mha = make_model(mha_cfg)
    state = {k: v.clone() for k, v in grid_model.state_dict().items()}
    d = cfg.d_model
    for key in list(state):
        if key.endswith(("mixer.k_proj.weight", "mixer.v_proj.weight")) and state[key].shape[0] == spec.width:
            comp = state[key].t().reshape(1, d, 1, spec.width)                 # each input channel's components as a "token"
            state[key] = assemble_grid(comp, spec).reshape(d, spec.n_heads * spec.head_dim).t().contiguous()
    mha.load_state_dict(state)
    tokens, docs = random_rows(2, L, cfg.vocab_size, seed=7)
    lg, lm = grid_model(tokens, docs).logits, mha(tokens, docs).logits
    torch.testing.assert_close(lg, lm, rtol=0, atol=1e-10)
    w = torch.randn(lg.shape, generator=torch.Generator().manual_seed(8), dtype=lg.dtype)
    (lg * w).sum().backward()
    (lm * w).sum().backward()
    named_g, named_m = dict(grid_model.named_parameters()), dict(mha.named_parameters())
    checked = 0
    for key, p in named_g.items():
        if key.endswith(("mixer.k_proj.weight", "mixer.v_proj.weight")) and p.shape[0] == spec.width:
            full = named_m[key].grad.t().reshape(d, spec.n_heads, spec.head_dim)        # per assembled head
            # scatter the heads' gradients back onto the components they were copied from
            index = assemble_grid(torch.arange(spec.width, dtype=torch.float64).reshape(1, 1, 1, spec.width), spec).long().reshape(spec.n_heads, spec.head_dim)
            want = torch.zeros(d, spec.width, dtype=full.dtype).index_add_(1, index.reshape(-1), full.reshape(d, -1))
            torch.testing.assert_close(p.grad.t(), want, rtol=0, atol=1e-9)
            checked += 1
        elif not key.endswith(("mixer.k_proj.weight", "mixer.v_proj.weight")):
            torch.testing.assert_close(p.grad, named_m[key].grad, rtol=0, atol=1e-9)
    assert checked >= 2


def test_grid_cache_holds_raw_components():
    """The cached keys / values of a grid layer are the raw components: width = sum(count x dim), one head."""
    cfg = copy.deepcopy(VARIANTS["grid_2x4"])
    model = make_model(cfg).eval()
    tokens, docs = random_rows(1, 12, cfg.vocab_size, seed=9)
    with torch.no_grad():
        cache = model.prefill(tokens, docs).cache
    spec = grid_spec(cfg.encoder.attention)
    shapes = [tuple(c.k.shape) for c, layer in zip(cache.encoder, model.encoder.layers) if layer.kind == "attention"]
    assert shapes and all(s == (1, 12, 1, spec.width) for s in shapes), shapes
    assert spec.width == 2 * 8 + 4 * 8 and spec.n_heads * spec.head_dim == 8 * 16          # 48 cached channels for 128 assembled


def test_the_mixes_start_as_the_plain_model():
    """The GDN write / query mixes are zero-initialised gates: with the shared parameters equal and the extra ones zero,
    the mixed model computes the logits of the model with block-entry mixing alone."""
    base = C.tiny_full_config()
    base.encoder.gdn_write_mix, base.encoder.gdn_write_variant = "none", "none"
    plain = make_model(base, perturbed=True)
    mixed = make_model(C.tiny_full_config(), perturbed=True)
    shared = dict(plain.named_parameters())
    with torch.no_grad():
        for n, p in mixed.named_parameters():
            if n in shared:
                p.copy_(shared[n])
            else:
                p.zero_()
    tokens, docs = random_rows(2, L, 256, seed=3)
    with torch.no_grad():
        torch.testing.assert_close(mixed(tokens, docs).logits, plain(tokens, docs).logits, rtol=0, atol=1e-10)
