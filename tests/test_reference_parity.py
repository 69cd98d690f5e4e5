"""The model equals the reference implementation on CPU in float64: state-dict keys and initial values with the same
seed, logits, parameter gradients, and cached generation; parameter counts of the published 200M / 60M entries."""

import copy

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import build_model
from tests.helpers import REFERENCE, random_rows


def _pair(reference, cfg):
    import ced.config as RC
    from ced.model.control import build_model as ref_build

    torch.manual_seed(0)
    mine = build_model(cfg).double()
    torch.manual_seed(0)
    theirs = ref_build(RC.from_dict(RC.ModelConfig, C.to_dict(cfg))).double()
    return mine, theirs


@pytest.mark.parametrize("preset", ["full", "control", "grid", "negeig", "skip_x0", "skip_x0_span", "x0", "skip", "canon", "canon_uniform", "gdn_shapes", "heads", "block_every", "token_query", "asentmax", "kda", "kda_floor", "erase", "kda_erase", "dprod", "dprod_b1", "dprod_layers", "dprod_heads", "dprod_mixed", "dprod_lowrank", "dprod_prev", "dprod_perm", "dprod_perm_random", "dprod_rot",
                                    "write_head", "dprod_noconv", "dprod_stride", "dprod_stride_all", "dprod_xmean", "dprod_kvmean", "dprod_xmean_b1", "ldm"])
def test_state_dict_forward_backward(reference, preset):
    scalars = preset in ("skip_x0", "skip_x0_span", "x0", "skip")     # not built together with the depth mixing
    cfg = C.tiny_control_config() if preset in ("control", "gdn_shapes") or scalars or preset.startswith(("canon", "kda", "erase", "dprod")) else C.tiny_full_config()
    if preset == "grid":
        a = cfg.encoder.attention
        a.kv_sharing, a.n_kv_heads, a.grid_rows, a.grid_cols, a.row_dim, a.col_dim = "grid", 1, 2, 2, 8, 8
    if preset == "negeig":
        cfg.encoder.gdn.negeig.beta_max = 2
    if scalars:
        cfg.encoder.layer_scalars = preset
    if preset == "write_head":                 # the write mix with one lambda a key head and a value head
        cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "head", "none"
    if preset == "block_every":
        cfg.encoder.attn_res = "block"
        cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "none", "none"
    if preset == "ldm":
        cfg.encoder.attn_res, cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "ldm", "none", "none"
        cfg.encoder.ldm_groups, cfg.encoder.ldm_key_dim, cfg.encoder.ldm_hidden = 4, 4, 6
    if preset.startswith("dprod"):
        cfg.encoder.gdn.dprod.n_h = 2 if preset == "dprod" else 3
        if preset == "dprod_layers":           # GDN ordinals 0 and 3 carry the extra step; the others are the plain layer
            cfg.encoder.gdn.dprod.layers = (0, 3)
        if preset == "dprod_heads":            # the first key group of every layer carries it
            cfg.encoder.gdn.dprod.heads = 2
        if preset == "dprod_mixed":
            d = cfg.encoder.gdn.dprod
            d.n_h, d.layers, d.heads, d.heads_by_layer = 3, (1, 2, 5), 2, {2: (2, 3), 5: (0, 1, 2, 3)}
            cfg.encoder.gdn.kernel, cfg.encoder.gdn.chunk_size = "chunked", 16
        if preset in ("dprod_lowrank", "dprod_prev", "dprod_perm", "dprod_perm_random", "dprod_rot"):      # the second step made from the first
            d = cfg.encoder.gdn.dprod
            d.n_h, d.key, d.value, d.conv = 2, preset.split("_")[1], "v1", False
            if preset == "dprod_lowrank":
                d.rank = 4
            if preset == "dprod_perm_random":
                d.perm = "random"
                cfg.encoder.gdn.kernel, cfg.encoder.gdn.chunk_size = "chunked", 16
        sparse = {"dprod_noconv": {}, "dprod_stride": {"stride": 4}, "dprod_stride_all": {"stride": 4, "first_beta": "all", "chunked": True},
                  "dprod_xmean": {"stride": 8, "summary": "xmean"}, "dprod_kvmean": {"stride": 8, "summary": "kvmean", "chunked": True},
                  "dprod_xmean_b1": {"stride": 3, "summary": "xmean", "beta_max": 1, "chunked": True}}
        if preset in sparse:                   # the second step on a subset of the tokens (cached cuts fall inside groups)
            d = cfg.encoder.gdn.dprod
            d.n_h, d.conv = 2, False
            for k, v in sparse[preset].items():
                if k == "chunked":
                    cfg.encoder.gdn.kernel, cfg.encoder.gdn.chunk_size = "chunked", 16
                else:
                    setattr(d, k, v)
        if preset == "dprod_b1":
            cfg.encoder.gdn.dprod.beta_max, cfg.encoder.gdn.dprod.beta_init = 1, 0.95
    if preset.endswith("erase"):
        cfg.encoder.gdn.erase.mode, cfg.encoder.gdn.erase.rank = "eda", 4
    if preset.startswith("kda"):
        cfg.encoder.gdn.kda.decay = "channel"
        if preset == "kda_floor":
            k = cfg.encoder.gdn.kda
            k.proj, k.rank, k.floor_channels, k.floor_min, k.floor_max = "per_head", 4, 3, 8.0, 512.0
    if preset == "asentmax":
        a = cfg.encoder.attention
        a.normalizer, a.temperature, a.rope_max_distance = "asentmax", "fixed", None
        cfg.encoder.nope_global_layers = ()
    if preset == "token_query":
        cfg.encoder.attn_res_query, cfg.encoder.attn_res_heads = "token", 2
        cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "none", "none"
    if preset == "heads":
        cfg.encoder.attn_res_heads = 4
        cfg.encoder.gdn_write_mix, cfg.encoder.gdn_write_variant = "none", "none"
    if preset == "gdn_shapes":
        cfg.encoder.gdn_shape_by_layer = {1: (1, 2, 8), 4: (2, 2, 16)}
    if preset.startswith("canon"):
        cfg.encoder.canon_kernel = 4
        cfg.encoder.canon_init = "uniform" if preset == "canon_uniform" else "zeros"
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd)
    assert all(torch.equal(sd[k], rsd[k]) for k in sd), "initial values differ under the same seed"
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 48)
    a, b = mine(tok, doc).logits, theirs(tok, doc).logits
    assert (a - b).abs().max() < 1e-10
    ga = torch.autograd.grad(a.logsumexp(-1).sum(), list(mine.parameters()))
    gb = torch.autograd.grad(b.logsumexp(-1).sum(), list(theirs.parameters()))
    assert max((x - y).abs().max() for x, y in zip(ga, gb)) < 1e-9
    out = mine.prefill(tok[:, :17], doc[:, :17])
    parts, cache = [out.logits], out.cache
    for s, e in ((17, 18), (18, 31), (31, 48)):
        out = mine.extend(tok[:, s:e], doc[:, s:e], None, cache)
        cache = out.cache
        parts.append(out.logits)
    assert (torch.cat(parts, 1) - a).abs().max() < 1e-10


PINS = {  # (total, non-embedding) of the reference's published run entries (reference: tests/test_run_entry.py)
    ("arch-s5qmix-200m.yaml", "s5qmix200-s1"): (267_769_564, 218_617_564),
    ("ladder-200m-base.yaml", "base200-s1"): (306_533_556, 208_229_556),
    ("fminus200-nomix.yaml", "fminus200-nomix-s1"): (267_714_228, 218_562_228),
}


@pytest.mark.parametrize("key", list(PINS))
def test_published_parameter_counts(reference, key):
    import yaml

    runs = yaml.safe_load((REFERENCE / "runs" / key[0]).read_text())
    entry = next(e for e in runs["runs"] if e["name"] == key[1])
    cfg = C.load_yaml(REFERENCE / entry["config"])
    for s in entry["set"]:
        C.apply_override(cfg, s)
    with torch.device("meta"):
        m = build_model(cfg.model)
    total = sum(p.numel() for p in m.parameters())
    emb = sum(p.numel() for n, p in m.named_parameters() if n.endswith("embed.weight"))
    assert (total, total - emb) == PINS[key]


def test_every_reference_run_file_parses(reference):
    import yaml

    seen = 0
    for path in sorted((REFERENCE / "runs").glob("*.yaml")):
        runs = yaml.safe_load(path.read_text())
        for entry in runs.get("runs", []):
            cfg = C.load_yaml(REFERENCE / entry["config"])
            for s in entry.get("set", []):
                C.apply_override(cfg, s.replace("${RUN_ROOT}", "/tmp").replace("${DATA_ROOT}", "/tmp"))
            C.unsupported_options(cfg)   # parses and classifies; experimental arms are reported, not crashed on
            seen += 1
    assert seen > 20


def test_mtp_head_matches_reference(reference):
    """The drafter head on a frozen trunk: same state-dict keys and start under the same seed, same head output and
    gradients, the trunk untouched by the key."""
    import ced.config as RC
    from ced.model import mtp as rmtp
    from ced.model.sequence import sequence_context as ref_context

    from gdn_hybrid_architecture_ideas_b200.models import mtp
    from gdn_hybrid_architecture_ideas_b200.models.sequence import sequence_context

    cfg = C.tiny_control_config()
    plain, _ = _pair(reference, cfg)
    cfg.mtp.enabled = True
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and any(k.startswith("mtp.") for k in sd)
    assert all(torch.equal(sd[k], rsd[k]) for k in sd)
    assert all(torch.equal(v, sd[k]) for k, v in plain.state_dict().items()), "the key changed the trunk's start"
    tok, doc = random_rows(2, 40)
    targets = torch.cat([tok[:, 1:], tok[:, :1]], 1)
    valid = torch.cat([doc[:, 1:] == doc[:, :-1], torch.zeros(2, 1, dtype=torch.bool)], 1)
    head = mtp.freeze_trunk(mine)
    rmtp.freeze_trunk(theirs)
    assert len(head) == len(rmtp.mtp_parameter_names(theirs))
    ha, hb = mtp.trunk_hidden(mine, tok, doc), rmtp.trunk_hidden(theirs, tok, doc)
    assert (ha - hb).abs().max() < 1e-10
    ya, _ = mine.mtp(ha, targets, mine.embed, sequence_context(doc)[0])
    yb, _ = theirs.mtp(hb, targets, theirs.embed, ref_context(doc, None)[0])
    assert (ya - yb).abs().max() < 1e-10
    t2a, v2a = mtp.mtp_targets(targets, valid)
    t2b, v2b = rmtp.mtp_targets(targets, valid)
    assert torch.equal(t2a, t2b) and torch.equal(v2a, v2b)
    ga = torch.autograd.grad(mine.mtp.out_norm(ya).pow(3).sum(), head)
    gb = torch.autograd.grad(theirs.mtp.out_norm(yb).pow(3).sum(), [p for n, p in theirs.named_parameters() if n.startswith("mtp.")])
    assert max((x - y).abs().max() for x, y in zip(ga, gb)) < 1e-9
    mtp.assert_trunk_frozen(mine)
    opt = torch.optim.AdamW(head, lr=3e-3)
    first = mtp.train_step(mine, opt, tok, doc, targets, valid)
    for _ in range(30):
        last = mtp.train_step(mine, opt, tok, doc, targets, valid)
    assert last["loss"] < first["loss"] and last["positions"] == int(v2a.sum())
    ctx = sequence_context(doc[:, :1])[0]
    drafts, _ = mtp.draft(mine, ha[:, :1], targets[:, :1], ctx, depth=3)
    assert drafts.shape == (2, 3)


def test_fixed_cross_entropy_matches_reference(reference):
    """loss.ce_form "fixed": the chunk gradient (one target and bags) equals the reference's in-place forms and autograd of
    its per-term definition; at a margin where softmax_t - 1 rounds to zero the target gradient keeps its value."""
    from ced.train import ce_fix as R

    from gdn_hybrid_architecture_ideas_b200.train import fused_head as FH

    g = torch.Generator().manual_seed(0)
    n, V, K = 12, 50, 3
    logits = torch.randn(n, V, generator=g, dtype=torch.float64) * 3
    logits[0, 7] += 60.0           # a collapsed row: its target is the argmax by a wide margin
    logits[1, 3] += 60.0           # a collapsed row whose target is NOT the argmax
    t1 = torch.randint(0, V, (n, 1), generator=g)
    t1[0, 0], t1[1, 0] = 7, 9
    a1 = torch.rand(n, 1, generator=g, dtype=torch.float64)
    b = torch.rand(n, generator=g, dtype=torch.float64) * 0.01
    ce, lse, grad = FH._ce_grad_chunk(logits.clone(), t1, a1, b, fixed=True)
    want = logits.clone()
    rce, rlse = torch.empty(n, dtype=torch.float64), torch.empty(n, dtype=torch.float64)
    R.ce_grad_fixed_torch(want, t1[:, 0], a1[:, 0], b, rce, rlse)
    assert (grad - want).abs().max() < 1e-12 and (ce - a1[:, 0] * rce).abs().max() < 1e-12 and (lse - rlse).abs().max() < 1e-12
    assert abs(float(grad[0].sum() - 2 * b[0] * lse[0])) < 1e-12                 # the row sums to the z-loss part
    g_fix = FH._ce_grad_chunk(logits.clone(), t1, a1, torch.zeros_like(b), fixed=True)[2]
    g_std = FH._ce_grad_chunk(logits.clone(), t1, a1, torch.zeros_like(b))[2]
    assert g_std[0, 7] == 0 and -1e-15 < g_fix[0, 7] < 0 and abs(float(g_fix[0].sum())) < 1e-30      # tiny, not zero, and the row sums to zero
    z = logits.clone().requires_grad_()
    rc, rl = R.fixed_ce_lse(z, t1[:, 0])
    ((a1[:, 0] * rc).sum() + (b * rl * rl).sum()).backward()
    assert (grad - z.grad).abs().max() < 1e-12
    tk = torch.randint(0, V, (n, K), generator=g)
    tk[2, 1] = tk[2, 0]            # a token twice in a bag
    tk[0, 0] = 7
    ak = torch.rand(n, K, generator=g, dtype=torch.float64)
    ce, lse, grad = FH._ce_grad_chunk(logits.clone(), tk, ak, b, fixed=True)
    z = logits.clone().requires_grad_()
    rc, rl = R.fixed_multi_ce_lse(z, tk)
    ((ak * rc).sum() + (b * rl * rl).sum()).backward()
    assert (grad - z.grad).abs().max() < 1e-11 and (ce - (ak * rc).sum(1)).abs().max() < 1e-11
    h = torch.randn(n, 16, generator=g, dtype=torch.float64, requires_grad=True)
    W = torch.randn(V, 16, generator=g, dtype=torch.float64, requires_grad=True)
    la, _, _ = FH.fused_linear_ce(h, W, tk, ak, b, 5, ce_form="fixed")
    ga = torch.autograd.grad(la, [h, W])
    lb, _ = FH.chunked_ce(h, W, tk, ak, b, chunk=5, ce_form="fixed")
    gb = torch.autograd.grad(lb, [h, W])
    assert abs(float(la - lb)) < 1e-10 and max((x - y).abs().max() for x, y in zip(ga, gb)) < 1e-10
    with pytest.raises(ValueError):
        FH.fused_linear_ce(h, W, tk, ak, b, 5, ce_form="other")


def test_entmax15_is_the_simplex_projection():
    """p = [x - tau]_+^2 sums to one over the allowed entries; tau agrees with a bisection solve; a row without an
    allowed entry is zero; the masked entries get exactly zero and no gradient."""
    from gdn_hybrid_architecture_ideas_b200.ops.reference import entmax15

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(5, 7, 33, generator=g, dtype=torch.float64) * 2).requires_grad_()
    allow = torch.rand(5, 7, 33, generator=g) < 0.7
    allow[0, 0] = False
    allow[1, 1] = False
    allow[1, 1, 4] = True
    p = entmax15(x, allow)
    s = p.sum(-1)
    assert torch.equal(s[0, 0], torch.zeros((), dtype=torch.float64)) and (p[~allow] == 0).all()
    rows = allow.any(-1)
    assert (s[rows] - 1).abs().max() < 1e-12
    assert p[1, 1, 4] == 1
    xm = torch.where(allow, x.detach(), torch.full_like(x, -1e9))
    lo, hi = xm.amax(-1, keepdim=True) - 1.0, xm.amax(-1, keepdim=True)
    for _ in range(80):
        mid = (lo + hi) / 2
        big = (xm - mid).clamp(min=0).square().sum(-1, keepdim=True) > 1
        lo, hi = torch.where(big, mid, lo), torch.where(big, hi, mid)
    want = (xm - lo).clamp(min=0).square()
    assert (p.detach() - want)[rows].abs().max() < 1e-9
    (p * torch.randn(p.shape, generator=g, dtype=torch.float64)).sum().backward()
    assert (x.grad[~allow] == 0).all() and torch.isfinite(x.grad).all()


def test_entmax_attention_chunks_equal_one_pass():
    from gdn_hybrid_architecture_ideas_b200.ops.reference import entmax_attention

    g = torch.Generator().manual_seed(5)
    B, L, H, Hk, D = 2, 37, 4, 2, 8
    q, k, v = (torch.randn(B, L, h, D, generator=g, dtype=torch.float64, requires_grad=True) for h in (H, Hk, Hk))
    idx = torch.arange(L)[None].expand(B, L)
    doc = torch.zeros(B, L, dtype=torch.long)
    doc[1, 20:] = 1
    w = torch.randn(B, L, H, D, generator=g, dtype=torch.float64)
    outs = []
    for chunk in (64, 8):
        o = entmax_attention(q, k, v, idx, doc, idx, doc, chunk=chunk)
        grads = torch.autograd.grad((o * w).sum(), (q, k, v))
        outs.append((o.detach(), *grads))
    for a, b in zip(*outs):
        assert (a - b).abs().max() < 1e-12


def _tiny_train_cfg():
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config(seq_len=48, batch_size=4), steps=6, seed=3)
    cfg.optim.warmup_steps, cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.head_impl, cfg.log_every, cfg.device = 2, 0, False, "chunked", 1000, "cpu"
    return cfg


def test_checkpoints_cross_between_the_trainers(reference, tmp_path):
    """The checkpoint format is shared: a file written by the reference's Trainer loads into this Trainer (weights and
    AdamW moments, so the next update is the reference's next update on the same batch), and a file written here loads
    into the reference's Trainer."""
    import ced.config as RC
    from ced.train.trainer import Trainer as RefTrainer

    from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    cfg = _tiny_train_cfg()
    ref_cfg = RC.from_dict(RC.TrainConfig, C.to_dict(cfg))
    theirs = RefTrainer(ref_cfg, str(tmp_path / "ref"))
    for _ in range(2):
        theirs.train_step()
    ref_path = theirs.save_checkpoint()
    state = ckpt.load(ref_path)
    mine = Trainer(cfg, tmp_path / "mine")
    mine.load_state_dict(state, check_config=False)
    assert mine.step == 2
    sd, rsd = mine.model.state_dict(), theirs.model.state_dict()
    assert all(torch.equal(sd[k], rsd[k]) for k in rsd)
    # the moments came along: one more update of each trainer on ONE batch (given to both) lands on the same weights
    batch = mine.batch_at(2)
    n = int(batch.target_valid.sum())
    mine.device_step(batch, n, lr=1e-3)
    ref_opt = theirs.optimizer
    for g in ref_opt.param_groups:
        g["lr"] = 1e-3 * g.get("lr_scale", 1.0)
    theirs.model.zero_grad(set_to_none=True)
    out = theirs.model(batch.tokens, batch.doc_ids, None, return_hidden=True)
    from ced.model.looped_ced import lm_head as ref_head

    logits = ref_head(out.hidden_aux, theirs.model.head_weight()).float()
    lse = logits.logsumexp(-1)
    ce = lse - logits.gather(-1, batch.targets[..., None])[..., 0]
    valid = batch.target_valid.float()
    ((valid * (ce + cfg.loss.z_loss * lse ** 2)).sum() / n).backward()
    torch.nn.utils.clip_grad_norm_(theirs.model.parameters(), cfg.optim.grad_clip)
    ref_opt.step()
    sd, rsd = mine.model.state_dict(), theirs.model.state_dict()
    worst = max((sd[k] - rsd[k]).abs().max().item() for k in rsd)
    assert worst < 2e-6, worst
    # and back: this trainer's file into the reference's trainer
    path = mine.save_checkpoint()
    back = RefTrainer(ref_cfg, str(tmp_path / "ref2"))
    back.load_state_dict(torch.load(path, weights_only=False), check_data=False)
    assert back.step == mine.step
    bsd = back.model.state_dict()
    assert all(torch.equal(bsd[k], sd[k]) for k in sd)
    st = back.optimizer.state_dict()["state"]
    assert len(st) > 0 and all(float(v["step"]) == 3.0 for v in st.values())
    back.train_step()          # the loaded optimizer steps (every key torch's AdamW reads is in the file's groups)


@pytest.mark.parametrize("injection,extra", [("none", {}), ("mix", {"recur_mix_init": 0.8}), ("parcae", {}),
                                               ("parcae", {"recur_inject_b": "diag", "recur_state_init": "prelude", "recur_prelude_norm": False}), ("depth_mix", {})])
def test_looped_middle_equals_the_reference(reference, injection, extra):
    """The looped middle (loop.recur_layers) under every injection: state-dict keys and starts, logits and parameter
    gradients at several pass counts, and the cache of a chunked read."""
    cfg = C.tiny_control_config()
    cfg.encoder.n_layers = 8
    cfg.loop.recur_layers, cfg.loop.injection, cfg.loop.t_eval, cfg.loop.t_max = (2, 6), injection, 2, 3
    cfg.loop.t_choices, cfg.loop.t_probs = [1, 2, 3], [0.25, 0.5, 0.25]
    for k, v in extra.items():
        setattr(cfg.loop, k, v)
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40)
    for T in (1, 2, 3):
        a, b = mine(tok, doc, T=T).logits, theirs(tok, doc, T=T).logits
        assert (a - b).abs().max() < 1e-10, T
        ga = torch.autograd.grad(a.logsumexp(-1).sum(), list(mine.parameters()), allow_unused=True)
        gb = torch.autograd.grad(b.logsumexp(-1).sum(), list(theirs.parameters()), allow_unused=True)
        for x, y in zip(ga, gb):
            assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9)
    assert torch.equal(mine(tok, doc).logits, mine(tok, doc, T=2).logits)                      # the default is loop.t_eval
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc, T=3).logits
        out = mine.prefill(tok[:, :17], doc[:, :17], T=3)
        ref_out = theirs.prefill(tok[:, :17], doc[:, :17], T=3)
        parts = [out.logits]
        for lo, hi in ((17, 18), (18, 40)):
            out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], None, out.cache)
            ref_out = theirs.extend(tok[:, lo:hi], doc[:, lo:hi], None, ref_out.cache)
            parts.append(out.logits)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10
        assert (torch.cat(parts, 1) - full).abs().max() < 1e-9 and len(out.cache.encoder) == 2 + 3 * 4 + 2 and out.cache.T == 3
        with pytest.raises(ValueError, match="keeps its pass count"):
            mine.extend(tok[:, :2], doc[:, :2], None, out.cache, T=2)


def test_qmix_static_pair_equals_the_reference(reference):
    """qmix's static top-2 query mix (gdn_qmix_select_step): the buffer in the state dict, the recorded weight sums, the
    choice, and logits / gradients / cached reads before and after it."""
    from ced.model import gdn_arms as ref_arms

    from gdn_hybrid_architecture_ideas_b200.models import qmix_select

    cfg = C.tiny_full_config()
    cfg.encoder.gdn_qmix_select_step = 2
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd)
    keeps = [k for k in sd if k.endswith("qmix_keep")]
    assert len(keeps) == 3 and all(sd[k].tolist() == [-1, -1] for k in keeps)        # the GDN layers of the third block: 3 sources
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40)

    def same():
        a, b = mine(tok, doc).logits, theirs(tok, doc).logits
        assert (a - b).abs().max() < 1e-10
        ga = torch.autograd.grad(a.logsumexp(-1).sum(), list(mine.parameters()), allow_unused=True)
        gb = torch.autograd.grad(b.logsumexp(-1).sum(), list(theirs.parameters()), allow_unused=True)
        for x, y in zip(ga, gb):
            assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9)
        return a

    before = same()
    assert qmix_select.pending(mine.encoder) and ref_arms.qmix_pending(theirs.encoder)
    mine.encoder.qmix_record, theirs.encoder.qmix_record = {}, {}
    mine(tok, doc), theirs(tok, doc)
    rec, ref_rec = mine.encoder.qmix_record, theirs.encoder.qmix_record
    mine.encoder.qmix_record = theirs.encoder.qmix_record = None
    assert sorted(rec) == sorted(ref_rec) and len(rec) == 6          # every layer with a query mix of its own (blocks 2 and 3)
    for i in rec:
        assert rec[i][1] == ref_rec[i][1] == 80 and (rec[i][0] - ref_rec[i][0]).abs().max() < 1e-9
        assert abs(float(rec[i][0].sum()) - 80) < 1e-9
    chosen, ref_chosen = qmix_select.select_pairs(mine.encoder, rec), ref_arms.select_qmix_pairs(theirs.encoder, ref_rec)
    assert list(chosen) == list(ref_chosen) == [8, 9, 10]
    assert all(chosen[i]["pair"] == ref_chosen[i]["pair"] for i in chosen)
    assert not qmix_select.pending(mine.encoder) and qmix_select.select_pairs(mine.encoder, rec) == {}
    after = same()
    assert (after - before).abs().max() > 1e-6                         # the third source no longer reaches the query rows
    log = qmix_select.weights_metrics(mine.encoder, rec)
    assert log["chosen"][-3:] == [chosen[i]["pair"] for i in chosen] and log["chosen"][:3] == [None] * 3 and log["n_sources"] == [2] * 3 + [3] * 3
    # the state dict carries the choice: a new model reads the pair form
    torch.manual_seed(0)
    again = build_model(cfg).double()
    assert not again.encoder.layers[8].gdn_arms.qmix_static
    again.load_state_dict(mine.state_dict())
    assert again.encoder.layers[8].gdn_arms.qmix_static and again.encoder.layers[8].gdn_arms.chosen_sources() == chosen[8]["pair"]
    assert torch.equal(again(tok, doc).logits, after)
    bad = mine.state_dict()
    bad[keeps[0]] = torch.tensor([1, 1])
    with pytest.raises(ValueError, match="ascending"):
        again.load_state_dict(bad)
    # after the choice the recorded weights are the pair's, zero on the third source
    mine.encoder.qmix_record = {}
    mine(tok, doc)
    rec2, mine.encoder.qmix_record = mine.encoder.qmix_record, None
    left_out = ({0, 1, 2} - set(chosen[9]["pair"])).pop()
    assert float(rec2[9][0][left_out]) == 0 and abs(float(rec2[9][0].sum()) - 80) < 1e-9
    mine.eval(), theirs.eval()
    with torch.no_grad():
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17]), theirs.prefill(tok[:, :17], doc[:, :17])
        out, ref_out = mine.extend(tok[:, 17:], doc[:, 17:], None, out.cache), theirs.extend(tok[:, 17:], doc[:, 17:], None, ref_out.cache)
        assert (out.logits - ref_out.logits).abs().max() < 1e-10 and (out.logits - after[:, 17:]).abs().max() < 1e-9
    for key, value, match in (("gdn_write_variant", "none", "qmix"), ("gdn_qmix_select_step", -1, "0 \\(off\\)"), ("gdn_qmix_select_step", True, "0 \\(off\\)")):
        wrong = C.tiny_full_config()
        wrong.encoder.gdn_qmix_select_step = 2
        setattr(wrong.encoder, key, value)
        with pytest.raises(ValueError, match=match):
            build_model(wrong)


@pytest.mark.parametrize("base,keys", [
    ("control", {"gdn_ccr_spacing": 8}),
    ("control", {"gdn_ccr_spacing": 8, "gdn.kernel": "chunked", "gdn.chunk_size": 16}),
    ("control", {"gdn_ccr_spacing": 4, "gdn_ccr_target": "lowest", "gdn_ccr_translator": "key_head", "gdn_ccr_gate_init": 0.09}),
    ("control", {"gdn_ccr_spacing": 8, "gdn_ccr_target": "group_first", "gdn_ccr_gate_init": 0.09, "gdn_ccr_gate_floor": 0.05}),
    ("full", {"gdn_ccr_spacing": 8, "gdn_write_variant": "none"}),
    ("full", {"gdn_ccr_spacing": 8, "gdn_write_variant": "none", "gdn_ccr_target": "group_first", "gdn_ccr_translator": "key_head"})])
def test_checkpoint_cross_read_equals_the_reference(reference, base, keys):
    """The checkpoint cross-read (gdn_ccr_spacing) under its three targets, with and without the translator, alone and with the
    write mix: state-dict keys and starts, logits, gradients (the gates' among them, nonzero), chunked cached reads whose
    cuts fall inside and across checkpoint spans, and activation_checkpoint 'layer'."""
    cfg = C.tiny_full_config() if base == "full" else C.tiny_control_config()
    for k, v in keys.items():
        C.apply_override(cfg, f"encoder.{k}={v}")
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd)
    gates = [k for k in sd if k.endswith("ccr_gate")]
    assert gates and all(float(sd[k].min()) == float(sd[k].max()) and abs(float(sd[k][0]) - cfg.encoder.gdn_ccr_gate_init) < 1e-7 for k in gates)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40)            # documents of 5 to 24 tokens: checkpoints at 8 and 16 (or 4 .. 20) are read

    def grads(model, logits):
        return torch.autograd.grad(logits.logsumexp(-1).sum(), list(model.parameters()), allow_unused=True)

    a, b = mine(tok, doc).logits, theirs(tok, doc).logits
    assert (a - b).abs().max() < 1e-10
    ga, gb = grads(mine, a), grads(theirs, b)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9), n
        if n.endswith("ccr_gate") or n.endswith("ccr_translator_delta"):
            assert x.abs().max() > 1e-8, n
    mine.encoder.activation_checkpoint = "layer"
    gc = grads(mine, mine(tok, doc).logits)
    assert all((x is None and y is None) or (x - y).abs().max() < 1e-12 for x, y in zip(ga, gc))
    mine.encoder.activation_checkpoint = "block"
    with pytest.raises(ValueError, match="activation_checkpoint"):
        mine(tok, doc)
    mine.encoder.activation_checkpoint = "none"
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc).logits
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17]), theirs.prefill(tok[:, :17], doc[:, :17])
        parts = [out.logits]
        for lo, hi in ((17, 18), (18, 29), (29, 40)):
            out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], None, out.cache)
            ref_out = theirs.extend(tok[:, lo:hi], doc[:, lo:hi], None, ref_out.cache)
            parts.append(out.logits)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10
        assert (torch.cat(parts, 1) - full).abs().max() < 1e-9


def test_checkpoint_cross_read_records_and_refusals():
    """The record's slots against a loop over positions; one state per pick, not per position; what the arm is refused with."""
    from gdn_hybrid_architecture_ideas_b200.models import ccr

    g = torch.Generator().manual_seed(0)
    B, L, C_ = 3, 37, 5
    start = torch.randint(0, 9, (B,), generator=g)            # the first document began before the call
    cuts = [sorted(torch.randint(1, L, (2,), generator=g).tolist()) for _ in range(B)]
    pos = torch.stack([torch.tensor([(start[b] + t if t < cuts[b][0] else t - cuts[b][0] if t < cuts[b][1] else t - cuts[b][1]) for t in range(L)]) for b in range(B)]).long()
    picks, slot, nxt = ccr.picks_and_slots(pos, C_)
    assert picks.shape == (B, L // C_ + 1)
    for b in range(B):
        taken = [t for t in range(L) if (int(pos[b, t]) + 1) % C_ == 0]
        assert picks[b].tolist() == taken + [L] * (picks.shape[1] - len(taken))
        for t in range(L + 1):
            p = int(pos[b, t]) if t < L else int(pos[b, -1]) + 1
            c = C_ * (p // C_)
            j = t - (p - c) - 1
            want = 0 if c == 0 else 1 if j < 0 else 2 + taken.index(j)
            assert (int(slot[b, t]) if t < L else int(nxt[b])) == want, (b, t)
    cfg = C.tiny_control_config()
    cfg.encoder.gdn_ccr_spacing = 8
    model = build_model(cfg)
    tok, doc = random_rows(2, 40)
    layer = model.encoder.layers[0]
    seen = {}
    layer.mixer.register_forward_hook(lambda m, a, out: seen.update(rec=out[1].ccr))
    caches = model.prefill(tok, doc).cache.encoder
    assert seen["rec"].states.shape[:2] == (2, 40 // 8 + 1 + 2) and all(getattr(c, "ccr", None) is None for c in caches)
    assert caches[0].ckpt is not None and caches[-1].ckpt is None          # a writer carries its checkpoint; the last GDN layer writes none
    for key, value, match in (("encoder.gdn_ccr_target", "nearest", "one of"), ("encoder.gdn_ccr_spacing", -1, "positive spacing"),
                              ("encoder.layer_scalars", "skip", "layer_scalars"), ("encoder.gdn_ccr_gate_floor", 0.2, "above"),
                              ("loop.recur_layers", "[1, 3]", "one pass"), ("encoder.attn_res", "block", "attn_res")):
        bad = C.tiny_control_config()
        bad.encoder.gdn_ccr_spacing = 8
        C.apply_override(bad, f"{key}={value}")
        with pytest.raises(ValueError, match=match):
            build_model(bad)
    off = C.tiny_control_config()
    off.encoder.gdn_ccr_gate_init = 0.1
    with pytest.raises(ValueError, match="CCR on"):
        build_model(off)


def test_delta_product_placement_is_resolved_and_refused_by_name():
    """The placement keys of Gated DeltaProduct: which heads of which GDN layer carry, the tensors a split layer holds, and the
    values refused by name."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_dprod

    cfg = C.tiny_control_config()                       # 8 GDN layers of 2 key / 4 value heads
    d = cfg.encoder.gdn.dprod
    d.n_h, d.layers, d.heads, d.heads_by_layer = 2, (1, 2, 5), 2, {2: (2, 3), 5: (0, 1, 2, 3)}
    assert cfg.encoder.dprod_carry() == [(), (0, 1), (2, 3), (), (), (0, 1, 2, 3), (), ()]
    built = cfg.encoder.gdn_layer_configs()
    assert [c.dprod.n_h for c, _ in built] == [1, 2, 2, 1, 1, 2, 1, 1] and [h for _, h in built] == [None, (0, 1), (2, 3), None, None, None, None, None]
    assert all(c.dprod.layers == () and c.dprod.heads == 0 and c.dprod.heads_by_layer == {} for c, _ in built)
    model = build_model(cfg)
    mixers = [layer.mixer for layer in model.encoder.layers if layer.kind == "gdn"]
    assert [type(m.dprod).__name__ for m in mixers] == ["NoneType", "PartialSteps", "PartialSteps", "NoneType", "NoneType", "DeltaProductSteps", "NoneType", "NoneType"]
    g = cfg.encoder.gdn
    assert mixers[1].dprod.in_proj_kv.weight.shape[0] == g.k_head_dim + 2 * g.v_head_dim and mixers[1].dprod.in_proj_b.weight.shape[0] == 2
    assert mixers[2].dprod.split.v["carry"] == (2, 3) and mixers[2].dprod.split.k["plain"] == (0,)
    assert sum(p.numel() for p in mixers[5].dprod.parameters()) == gdn_dprod.params_per_layer(cfg.d_model, g)
    t = torch.arange(24.0).reshape(2, 6, 2)
    cut = gdn_dprod.HeadSplit(3, 6, (0, 1, 4, 5))
    assert cut.v["plain"] == (2, 3) and cut.k == {"carry": (0, 2), "plain": (1,)}
    assert torch.equal(cut.pick(t, "carry", 1)[:, :, 0], t[:, [0, 1, 4, 5], 0]) and torch.equal(cut.join(cut.pick(t, "carry", 1), cut.pick(t, "plain", 1), 1), t)
    for key, value, match in (("layers", "[2, 1]", "ascending"), ("layers", "[9]", "ordinals"), ("heads", 3, "multiple"), ("heads", 6, "at most"),
                              ("heads_by_layer", "{0: [1, 2]}", "cut"), ("heads_by_layer", "{0: [3, 2]}", "ascending"),
                              ("heads_by_layer", "{9: [0, 1]}", "ordinals of layers"), ("beta_max", 1, "carry only some")):
        bad = C.tiny_control_config()
        bad.encoder.gdn.dprod.n_h, bad.encoder.gdn.dprod.heads = 2, 2
        C.apply_override(bad, f"encoder.gdn.dprod.{key}={value}")
        with pytest.raises(ValueError, match=match):
            build_model(bad)
    off = C.tiny_control_config()
    off.encoder.gdn.dprod.heads = 2
    with pytest.raises(ValueError, match="n_h 1"):
        build_model(off)


def test_delta_product_derived_second_step_tensors_and_refusals():
    """The second step made from the first: the tensors each key adds, their optimizer group, the size of the low-rank
    correction at the start, the rotation, the previous key across a cached cut, and the values refused by name."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_dprod_derived as D
    from gdn_hybrid_architecture_ideas_b200.train import optim

    def cfg_of(key, **kw):
        cfg = C.tiny_control_config()
        d = cfg.encoder.gdn.dprod
        d.n_h, d.key, d.value, d.conv = 2, key, "v1", False
        for k, v in kw.items():
            setattr(d, k, v)
        return cfg

    cfg = cfg_of("lowrank", rank=4)
    model = build_model(cfg)
    steps = model.encoder.layers[0].mixer.dprod
    g = cfg.encoder.gdn
    assert sum(p.numel() for p in steps.parameters()) == D.params_per_layer(cfg.d_model, g)
    x = torch.randn(4, 64, cfg.d_model)
    k1 = torch.nn.functional.normalize(torch.randn(4, 64, g.n_k_heads, g.k_head_dim), dim=-1)
    k2 = steps.second_key(x, k1, torch.zeros(4, 64, dtype=torch.bool), None)
    cos = float((k1 * k2).sum(-1).mean())
    assert 0.5 < cos < 0.9 and abs(float(k2.norm(dim=-1).mean()) - 1) < 1e-3          # a second address of k1's size, not k1 itself
    groups = optim.param_groups(model, C.OptimConfig(name="muon"))
    muon = [n for grp in groups if grp["kind"] == "muon" for n in grp["names"]]
    assert not any(".dprod." in n for n in muon)
    rot = build_model(cfg_of("rot")).encoder.layers[0].mixer.dprod.rot.double()
    assert (rot @ rot.T - torch.eye(rot.shape[0], dtype=torch.double)).abs().max() < 1e-6 and abs(float(torch.linalg.det(rot)) - 1) < 1e-5
    prev = build_model(cfg_of("prev")).double().eval()
    tok, doc = random_rows(2, 40)
    with torch.no_grad():
        out = prev.prefill(tok[:, :17], doc[:, :17])
        assert out.cache.encoder[0].k_prev.shape == (2, g.n_k_heads, g.k_head_dim)
        out.cache.encoder[0].k_prev = None
        with pytest.raises(ValueError, match="previous key"):
            prev.extend(tok[:, 17:], doc[:, 17:], None, out.cache)
    for key, kw, match in (("lowrank", {"rank": 99}, "rank"), ("prev", {"rank": 4}, "rank"), ("rot", {"perm": "random"}, "perm"), ("perm", {"value": "proj"}, "value"),
                           ("perm", {"conv": True}, "conv"), ("perm", {"n_h": 3}, "n_h 2"), ("perm", {"beta_max": 1}, "beta_max"), ("perm", {"heads": 2}, "every head"),
                           ("twist", {}, "one of"), ("proj", {}, "not built together")):
        with pytest.raises(ValueError, match=match):
            build_model(cfg_of(key, **kw))
    off = C.tiny_control_config()
    off.encoder.gdn.dprod.key = "rot"
    with pytest.raises(ValueError, match="n_h 1"):
        build_model(off)


def test_delta_product_sparse_second_step_layout_and_refusals():
    """The second step on a subset of the tokens: the row layout's maps, the group sums across documents and calls, the tensors
    each form holds, and the values refused by name."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_dprod_sparse as SP

    rows, last, n_c = SP.row_maps(10, 4, 1)                # tokens 1, 5, 9 carry
    assert n_c == 3 and rows == [0, 1, 10, 2, 3, 4, 5, 11, 6, 7, 8, 9, 12] and last == [0, 2, 3, 4, 5, 7, 8, 9, 10, 12]
    assert SP.carry_flags(10, 4, 2) == [i in (1, 5, 9) for i in range(10)] and SP.first_carry(2, 4) == 1
    u = torch.arange(20.0).reshape(1, 10, 2)
    doc = torch.tensor([[0, 0, 0, 0, 1, 1, 1, 1, 1, 1]])
    sums, counts = SP.group_sums(u, doc, 4, 1, (torch.tensor([[100.0, 200.0]]), torch.tensor([2.0]), torch.tensor([1.0])))
    assert counts.tolist() == [[4.0, 2.0, 4.0]]            # head group: tokens 0, 1 and the two carried; second: tokens 4, 5 of document 1 only
    assert sums[0, 0].tolist() == [102.0, 204.0] and sums[0, 1].tolist() == [18.0, 20.0]
    acc, cnt = SP.tail_sums(u[:, :9], doc[:, :9], 4, 1)
    assert cnt.tolist() == [3.0] and acc[0].tolist() == [12.0 + 14 + 16, 13.0 + 15 + 17]

    def cfg_of(**kw):
        cfg = C.tiny_control_config()
        d = cfg.encoder.gdn.dprod
        d.n_h, d.conv = 2, False
        for k, v in kw.items():
            setattr(d, k, v)
        return cfg

    g = C.tiny_control_config().encoder.gdn
    for kw in ({"stride": 4}, {"stride": 8, "summary": "kvmean"}):
        model = build_model(cfg_of(**kw))
        steps = model.encoder.layers[0].mixer.dprod
        assert sum(p.numel() for p in steps.parameters()) == SP.params_per_layer(model.cfg.d_model, cfg_of(**kw).encoder.gdn)
        assert not hasattr(steps, "conv_weight")
    tok, doc2 = random_rows(2, 40)
    summed = build_model(cfg_of(stride=8, summary="xmean")).double().eval()
    with torch.no_grad():
        out = summed.prefill(tok[:, :17], doc2[:, :17])
        assert out.cache.encoder[0].acc.shape == (2, summed.cfg.d_model) and out.cache.encoder[0].cnt.shape == (2,)
        out.cache.encoder[0].acc = None
        with pytest.raises(ValueError, match="running sums"):
            summed.extend(tok[:, 17:], doc2[:, 17:], None, out.cache)
    for kw, match in (({"stride": 4, "conv": True}, "conv"), ({"stride": 0}, "stride"), ({"summary": "max"}, "one of"), ({"stride": 4, "n_h": 3}, "n_h 2"),
                      ({"stride": 4, "heads": 2}, "placement|every head"), ({"stride": 4, "key": "rot", "value": "v1"}, "not built together"),
                      ({"stride": 4, "beta_init": 0.9}, "beta_init"), ({"first_beta": "some"}, "one of"), ({"sparse_path": "slow"}, "sparse_path")):
        with pytest.raises(ValueError, match=match):
            build_model(cfg_of(**kw))
    off = C.tiny_control_config()
    off.encoder.gdn.dprod.stride = 4
    with pytest.raises(ValueError, match="n_h 1"):
        build_model(off)


@pytest.mark.parametrize("keys", [{}, {"encoder.gdn.kernel": "chunked", "encoder.gdn.chunk_size": 16, "loop.loop_embedding": False, "loop.pass2_layers": 10},
                                  {"encoder.attention.rope_max_distance": 12, "encoder.attention.temperature": "ssmax", "encoder.attention.temperature_ref_len": 64}])
def test_gated_second_pass_equals_the_reference(reference, keys):
    """The read-only second pass through the top layers (loop.pass2_gate 'scalar'): the two new tensors first and last in
    the state dict, logits and gradients at T = 1 and T = 2 (pass 1's keys, values and states trained through pass 2), cached
    reads where a mask marks the positions whose logits are read, slots by capacity, activation_checkpoint 'layer'."""
    cfg = C.tiny_control_config()
    cfg.loop.pass2_gate, cfg.loop.pass2_layers, cfg.loop.t_max, cfg.loop.t_eval, cfg.loop.t_choices, cfg.loop.t_probs = "scalar", 6, 2, 2, [2], [1.0]
    for k, v in keys.items():
        C.apply_override(cfg, f"{k}={v}")
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd)
    names = ["loop_embedding_pass2"] * bool(cfg.loop.loop_embedding) + ["hyper_connections.pass2_gate"]
    assert mine.pass2_parameter_names() == theirs.pass2_parameter_names() == names and (list(sd)[0] == names[0] or not cfg.loop.loop_embedding)
    tok, doc = random_rows(2, 40)
    assert torch.equal(mine(tok, doc, T=2).logits, mine(tok, doc, T=1).logits)            # alpha = 0: the single-pass model exactly
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())

    def grads(model, logits):
        return torch.autograd.grad(logits.logsumexp(-1).sum(), list(model.parameters()), allow_unused=True)

    for T in (1, 2):
        a, b = mine(tok, doc, T=T).logits, theirs(tok, doc, T=T).logits
        assert (a - b).abs().max() < 1e-10
        ga, gb = grads(mine, a), grads(theirs, b)
        for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
            assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9), (T, n)
    assert torch.equal(mine(tok, doc).logits, mine(tok, doc, T=2).logits) and not torch.equal(mine(tok, doc).logits, mine(tok, doc, T=1).logits)
    mine.encoder.activation_checkpoint = "layer"
    gc = grads(mine, mine(tok, doc, T=2).logits)
    assert all((x is None and y is None) or (x - y).abs().max() < 1e-12 for x, y in zip(ga, gc))
    mine.encoder.activation_checkpoint = "none"
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc).logits
        one = mine(tok, doc, T=1).logits
        mask = torch.zeros(2, 40, dtype=torch.bool)
        mask[:, 30:], mask[0, 5] = True, True
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17], mask[:, :17]), theirs.prefill(tok[:, :17], doc[:, :17], mask[:, :17])
        parts, kept = [out.logits], [out.kept]
        assert (out.logits - ref_out.logits).abs().max() < 1e-10 and torch.equal(out.kept, ref_out.kept)
        for lo, hi in ((17, 18), (18, 33), (33, 40)):
            out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], mask[:, lo:hi], out.cache)
            ref_out = theirs.extend(tok[:, lo:hi], doc[:, lo:hi], mask[:, lo:hi], ref_out.cache)
            parts.append(out.logits), kept.append(out.kept)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10 and torch.equal(out.kept, ref_out.kept) and torch.equal(out.n_dropped, ref_out.n_dropped)
            assert all(getattr(c, "pass1", None) is None for c in out.cache.encoder)                 # the cache is pass 1's
        got, k = torch.cat(parts, 1), torch.cat(kept, 1)
        assert torch.equal(k, mask) and (got - full)[k].abs().max() < 1e-9 and (got - one)[~k].abs().max() < 1e-9
        a, b = mine(tok, doc, pass2_mask=mask, pass2_capacity=3), theirs(tok, doc, pass2_mask=mask, pass2_capacity=3)
        assert (a.logits - b.logits).abs().max() < 1e-10 and torch.equal(a.kept, b.kept) and torch.equal(a.n_dropped, b.n_dropped)
        assert a.kept.sum(1).tolist() == [3, 3] and a.n_dropped.tolist() == [8, 7]
        assert torch.equal(mine(tok, doc, pass2_mask=mask, pass2_capacity=0).logits, one)


def test_gated_second_pass_is_refused_by_name_where_it_is_not_built():
    def cfg_of(**kw):
        cfg = C.tiny_control_config()
        cfg.loop.pass2_gate, cfg.loop.pass2_layers, cfg.loop.t_max, cfg.loop.t_eval = "scalar", 4, 2, 2
        for k, v in kw.items():
            C.apply_override(cfg, f"{k}={v}")
        return cfg

    for kw, match in (({"loop.pass2_layers": 0}, "pass2_layers"), ({"loop.pass2_layers": 99}, "pass2_layers"), ({"loop.t_max": 3}, "t_max"),
                      ({"loop.t_eval": 3}, "t_eval"), ({"loop.pass2_gate": "hc"}, "hc"), ({"encoder.layer_scalars": "skip"}, "layer_scalars"),
                      ({"encoder.canon_kernel": 4}, "canon_kernel"), ({"loop.recur_layers": "[2, 6]"}, "recur_layers"),
                      ({"encoder.gdn.dprod.n_h": 2}, "dprod"), ({"loop.segment_passes": "{a: 2}"}, "segment_passes")):
        with pytest.raises(ValueError, match=match):
            build_model(cfg_of(**{k: v for k, v in kw.items()}))
    full = C.tiny_full_config()
    full.loop.pass2_gate, full.loop.pass2_layers, full.loop.t_max, full.loop.t_eval = "scalar", 4, 2, 2
    with pytest.raises(ValueError, match="attn_res"):
        build_model(full)
    plain = C.tiny_control_config()
    plain.loop.pass2_layers = 3
    with pytest.raises(ValueError, match="without loop.pass2_gate"):
        build_model(plain)
    model = build_model(C.tiny_control_config())
    tok, doc = random_rows(1, 8)
    with pytest.raises(ValueError, match="gated second pass"):
        model(tok, doc, pass2_mask=torch.ones(1, 8, dtype=torch.bool))


@pytest.mark.parametrize("base,keys", [("control", {}), ("control", {"qk_norm": True, "init": "reference"}),
                                       ("control", {"qk_norm": True, "temperature": "ssmax", "sink_count": True}), ("full", {"qk_norm": True}),
                                       ("control", {"window": 7}), ("full", {"pointer_input": "mix", "qk_norm": True, "temperature": "ssmax"}),
                                       ("full", {"pointer_input": "mix", "qk_norm": True, "n_heads": 3, "init": "reference"}), ("full", {"pointer_input": "mix", "qk_norm": True, "n_heads": 2, "temperature": "ssmax"}),
                                       ("full", {"pointer_input": "mix", "qk_norm": True, "n_heads": 3, "combine": "or"}), ("full", {"pointer_input": "mix", "qk_norm": True, "combine": "or"}),
                                       ("full", {"pointer_input": "shared", "qk_norm": True, "shared_head": 3, "init": "reference"}),
                                       ("full", {"pointer_input": "shared", "qk_norm": True, "shared_ssmax": True, "sink_count": True})])
def test_copy_paste_head_equals_the_reference(reference, base, keys):
    """The Copy-Paste head in its base form: the head's tensors last in the state dict with equal starts, the mixture's log p over V
    (it sums to one and equals the training cross entropy at the target), the blockwise terms against the reference's and an
    all-at-once statement, the loss's gradients through trunk and head, and cached generation with the copy cache."""
    from ced.model import cp_head as RCP

    from gdn_hybrid_architecture_ideas_b200.models import cp_head as CP

    cfg = C.tiny_full_config() if base == "full" else C.tiny_control_config()
    cfg.cp_head.enabled, cfg.cp_head.d_c, cfg.cp_head.query_chunk, cfg.encoder.gdn_write_variant = True, 8, 16, "none"
    for k, v in keys.items():
        setattr(cfg.cp_head, k, v)
    if keys.get("n_heads", 1) > 1 or keys.get("combine") == "or" or keys.get("pointer_input") == "shared":
        cfg.encoder.gdn_write_mix = "none"
    if keys.get("pointer_input") == "shared":
        cfg.encoder.nope_global_layers = (2,)            # the last global layer has no rotary part
        cfg.cp_head.d_c = type(cfg.cp_head)().d_c        # the pointer's width is the shared head's: the key stays at its default
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd) and list(sd)[-1].startswith("cp_head.")
    plain = C.tiny_full_config() if base == "full" else C.tiny_control_config()
    plain.encoder.gdn_write_variant, plain.encoder.gdn_write_mix = "none", cfg.encoder.gdn_write_mix
    torch.manual_seed(0)
    trunk = build_model(plain).double().state_dict()
    assert all(torch.equal(trunk[k], sd[k]) for k in trunk)                    # the base model starts as the model without the key
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40, vocab=12)                                     # a small alphabet: most targets occur in the context
    tgt = torch.roll(tok, -1, 1)
    a, b = mine(tok, doc).logits, theirs(tok, doc).logits
    assert (a - b).abs().max() < 1e-10 and (a.exp().sum(-1) - 1).abs().max() < 1e-9
    oa, ob = mine(tok, doc, return_hidden=True), theirs(tok, doc, return_hidden=True)
    ha, hb, pa, pb = oa.hidden_aux, ob.hidden_aux, oa.cp_pointer, ob.cp_pointer
    assert (pa is None) == (keys.get("pointer_input") not in ("mix", "shared"))
    ta, tb = CP.terms(mine.cp_head, ha, tok, tgt, doc, pointer=pa), RCP.cp_terms(theirs.cp_head, hb, tok, tgt, doc, pointer=pb)
    tn = ta if keys.get("combine") == "or" else CP.terms_naive(mine.cp_head, ha, tok, tgt, doc, pointer=pa)
    for x, y, z in zip(ta, tb, tn):
        fin = torch.isfinite(y)
        assert torch.equal(torch.isfinite(x), fin) and torch.equal(torch.isfinite(z), fin) and (x - y)[fin].abs().max() < 1e-10 and (x - z)[fin].abs().max() < 1e-9
    assert 0 < int((~torch.isfinite(ta[2])).sum()) < tgt.numel()                # some targets have no match in their context, most have one
    w, z = torch.ones_like(tgt, dtype=torch.double), torch.full(tgt.shape, 1e-4, dtype=torch.double)
    loss, ce, lam = CP.mixture_loss(mine, ha, tgt, tok, doc, w, z, chunk=16, pointer=pa)
    ce_r, lse_r = RCP.head_token_ce(theirs, hb, tgt, tok, doc, pointer=pb)
    assert (ce - ce_r).abs().max() < 1e-10 and (-a.gather(-1, tgt[..., None]).squeeze(-1) - ce).abs().max() < 1e-9 and 0 < float(lam.min()) and float(lam.max()) < 1
    ga = torch.autograd.grad(loss, list(mine.parameters()), allow_unused=True)
    gb = torch.autograd.grad((w * ce_r + z * lse_r * lse_r).sum(), list(theirs.parameters()), allow_unused=True)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None or ((x - y).abs().max() < 1e-9 and torch.isfinite(x).all())), n
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc).logits
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17]), theirs.prefill(tok[:, :17], doc[:, :17])
        parts = [out.logits]
        for lo, hi in ((17, 18), (18, 40)):
            out, ref_out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], None, out.cache), theirs.extend(tok[:, lo:hi], doc[:, lo:hi], None, ref_out.cache)
            parts.append(out.logits)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10
        assert (torch.cat(parts, 1) - full).abs().max() < 1e-9 and out.cache.copy.keys.k.shape[:2] == (2, 40)
        oe = mine(tok, doc, return_hidden=True)
        ce_eval, _ = CP.head_token_ce(mine, oe.hidden_aux, tgt, tok, doc, pointer=oe.cp_pointer)
        assert (ce_eval + full.gather(-1, tgt[..., None]).squeeze(-1)).abs().max() < 1e-9
        with pytest.raises(ValueError, match="Copy-Paste head"):
            mine.head_weight()
        mine.cfg.cp_head.score = "lm"
        lm = mine(tok, doc).logits
        assert (lm - torch.nn.functional.linear(mine(tok, doc, return_hidden=True).hidden_aux, mine.lm_head_weight())).abs().max() < 1e-12


def test_copy_paste_head_is_refused_by_name_where_it_is_not_built():
    for key, value, match in (("cp_head.pointer_input", "mix", "block_entry"), ("cp_head.pointer_input", "shared", "shared"), ("cp_head.shared_head", 2, "shared_head"), ("cp_head.n_heads", 2, "n_heads"), ("cp_head.combine", "or", "combine"), ("cp_head.combine", "xor", "combine"),
                              ("cp_head.trunk_copy", "all", "trunk_copy"), ("cp_head.train_mode", "addon", "train_mode"), ("cp_head.window", -1, "window"), ("cp_head.kernel", "fused", "kernel"),
                              ("cp_head.init", "zeros", "init"), ("cp_head.d_c", 0, "d_c"), ("loop.recur_layers", "[2, 6]", "one pass"),
                              ("encoder.gdn_ccr_spacing", 8, "gdn_ccr_spacing"), ("encoder.attn_res", "ldm", "attn_res")):
        cfg = C.tiny_control_config()
        cfg.cp_head.enabled = True
        C.apply_override(cfg, f"{key}={value}")
        with pytest.raises(ValueError, match=match):
            build_model(cfg)


@pytest.mark.parametrize("arm", ["base", "lanes", "depth", "untied", "routed", "per_layer", "scaled"])
def test_looped_encoder_decoder_equals_the_reference(reference, arm):
    """arch looped_ced: equal starts under equal seeds, the logits at every position (decoder head at the kept slots, aux
    head elsewhere), the drafts, the two-head loss's gradients, prefill + cached extension, at T = 1 .. 3 and every loop
    boundary arm; rows with more decoder positions than slots drop the later ones."""
    from ced.model.control import build_model as ref_build  # noqa: F401

    cfg = C.tiny_looped_config()
    lp, dec = cfg.loop, cfg.decoder
    if arm == "lanes":
        lp.hyper_connections, lp.injection, lp.hc_streams = "static", "none", 3
    if arm == "depth":
        lp.depth_attention, lp.depth_attention_head_dim = "layer", 8
    if arm == "untied":
        dec.untie_mixers, dec.n_layers, dec.memory_attn_interval = "all", 3, 3
    if arm == "routed":
        dec.ffn_experts, dec.ffn_top_k, dec.router_z_weight = 4, 2, 0.01
    if arm == "per_layer":
        dec.n_layers, dec.memory_attn_interval, dec.memory_kv_per_layer, cfg.tie_embeddings = 2, 1, True, False
    if arm == "scaled":
        cfg.residual_scale.mode, cfg.residual_scale.lam = "inverse_loops", 1.5
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd)
    if arm == "base":
        for change, match in ((lambda c: setattr(c.decoder.attention, "rope_max_distance", 6), "rope_max_distance"), (lambda c: setattr(c.loop, "injection", "mix"), "injection"),
                              (lambda c: setattr(c.decoder, "memory_attn_interval", 5), "memory-attention"), (lambda c: setattr(c.encoder, "attn_res", "block_entry"), "attn_res"),
                              (lambda c: setattr(c.loop, "t_eval", 4), "t_eval"), (lambda c: setattr(c.decoder, "untie_mixers", "some"), "untie_mixers")):
            bad = C.tiny_looped_config()
            change(bad)
            with pytest.raises(ValueError, match=match):
                build_model(bad)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40)
    dm = torch.rand(2, 40, generator=g) < 0.3
    dm[1, 5:30] = True                                           # more decoder positions than the row's 16 slots: the later ones are dropped
    tgt = torch.roll(tok, -1, 1)
    for T in (1, 2, 3):
        a, b = mine(tok, doc, dm, T=T, return_drafts=True), theirs(tok, doc, dm, T=T, return_drafts=True)
        assert torch.equal(a.kept, b.kept) and torch.equal(a.n_dropped, b.n_dropped) and int(a.n_dropped[1]) > 0 and torch.equal(a.slot_index, b.slot_index)
        assert (a.logits - b.logits).abs().max() < 1e-10, T
        for x, y in zip(a.draft_logits, b.draft_logits):
            assert (x - y)[a.slot_valid].abs().max() < 1e-10
    from gdn_hybrid_architecture_ideas_b200.models.looped_decoder import two_head_loss

    a, b = mine(tok, doc, dm, T=3, return_hidden=True, return_drafts=True), theirs(tok, doc, dm, T=3, return_hidden=True, return_drafts=True)
    valid = torch.ones_like(dm)
    loss, sums = two_head_loss(mine, a, tgt, valid, n_valid=80.0, n_dec=float(a.kept.sum()), n_aux=float((~a.kept).sum()), z_loss=1e-4, aux_weight=0.5, draft_weight=0.3)
    W = theirs.head_weight()
    ce = lambda h, t: torch.nn.functional.cross_entropy(h @ W.t(), t, reduction="none")                  # noqa: E731
    lse = lambda h: torch.logsumexp(h @ W.t(), -1)                                                          # noqa: E731
    from ced.model.capacity import gather_slots

    t_slots = gather_slots(tgt, b.slot_index, fill=0)
    flat = lambda h: h.reshape(-1, h.shape[-1])                                                              # noqa: E731
    ce_d = (ce(flat(b.hidden_dec), t_slots.reshape(-1)) + 1e-4 * lse(flat(b.hidden_dec)) ** 2).reshape(t_slots.shape)
    ce_a = (ce(flat(b.hidden_aux), tgt.reshape(-1)) + 1e-4 * lse(flat(b.hidden_aux)) ** 2).reshape(tgt.shape)
    ref_loss = ((ce_d * b.slot_valid).sum() + 0.5 * (ce_a * ~b.kept).sum()) / 80.0
    for h in b.hidden_drafts:
        ref_loss = ref_loss + 0.3 * (ce(flat(h), t_slots.reshape(-1)).reshape(t_slots.shape) * b.slot_valid).sum() / float(b.kept.sum())
    if b.aux_loss is not None:
        ref_loss = ref_loss + b.aux_loss
    assert abs(float(loss) - float(ref_loss)) < 1e-10
    ga = torch.autograd.grad(loss, list(mine.parameters()), allow_unused=True)
    gb = torch.autograd.grad(ref_loss, list(theirs.parameters()), allow_unused=True)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9), n
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc, dm, T=2, capacity=40).logits
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17], dm[:, :17], T=2), theirs.prefill(tok[:, :17], doc[:, :17], dm[:, :17], T=2)
        parts = [out.logits]
        for lo, hi in ((17, 18), (18, 40)):
            out, ref_out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], dm[:, lo:hi], out.cache), theirs.extend(tok[:, lo:hi], doc[:, lo:hi], dm[:, lo:hi], ref_out.cache)
            parts.append(out.logits)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10
        assert (torch.cat(parts, 1) - full).abs().max() < 1e-9
        prompt, pdoc, pmask = tok[:, :12], doc[:, :12] * 0, torch.ones(2, 12, dtype=torch.bool)
        mine_tokens, mine_logits = mine.generate(prompt, pdoc, pmask, 5, T=2)
        ref_tokens, ref_logits = theirs.generate(prompt, pdoc, pmask, 5, T=2)
        assert torch.equal(mine_tokens, ref_tokens) and (mine_logits - ref_logits).abs().max() < 1e-10


def test_copy_paste_pointer_trained_on_its_auxiliary_loss_equals_the_reference(reference):
    """cp_head.train_mode aux: no <copy> row and the other tensors the mixture head's of the same seed; the pointer's inputs are
    formed in training mode only; L_aux and its gradients (the pointer's tensors alone learn from it); in eval mode the model
    is the model without the head (logits, cached generation)."""
    from ced.model import cp_aux as RAUX
    from ced.model import cp_head as RCP

    from gdn_hybrid_architecture_ideas_b200.models import cp_head as CP

    cfg = C.tiny_full_config()
    cfg.encoder.gdn_write_variant, cfg.encoder.gdn_write_mix = "none", "none"
    cfg.cp_head.enabled, cfg.cp_head.d_c, cfg.cp_head.query_chunk, cfg.cp_head.pointer_input, cfg.cp_head.qk_norm = True, 8, 16, "mix", True
    gated, _ = _pair(reference, cfg)
    cfg.cp_head.train_mode, cfg.cp_head.aux_weight = "aux", 0.5
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd) and "cp_head.w_copy" not in sd
    assert all(torch.equal(sd[k], v) for k, v in gated.state_dict().items() if k != "cp_head.w_copy")
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40, vocab=12)
    tgt = torch.roll(tok, -1, 1)
    oa, ob = mine(tok, doc, return_hidden=True), theirs(tok, doc, return_hidden=True)
    la, sink_a = CP.aux_terms(CP.terms(mine.cp_head, oa.hidden_aux, tok, tgt, doc, pointer=oa.cp_pointer))
    lb, sink_b = RAUX.aux_ce(*RCP.cp_terms(theirs.cp_head, ob.hidden_aux, tok, tgt, doc, pointer=ob.cp_pointer))
    assert torch.equal(sink_a, sink_b) and 0 < int(sink_a.sum()) < sink_a.numel() and (la - lb).abs().max() < 1e-10
    ga = torch.autograd.grad(la.sum(), list(mine.parameters()), allow_unused=True)
    gb = torch.autograd.grad(lb.sum(), list(theirs.parameters()), allow_unused=True)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None or ((x - y).abs().max() < 1e-9 and torch.isfinite(x).all())), n
    assert all(x is not None for (n, _), x in zip(mine.named_parameters(), ga) if n.startswith("cp_head."))
    with pytest.raises(ValueError, match="no <copy> row"):
        mine.cp_head.copy_logit(oa.hidden_aux)
    mine.eval(), theirs.eval()
    with torch.no_grad():
        out = mine(tok, doc, return_hidden=True)
        assert out.cp_pointer is None
        full, ref_full = mine(tok, doc).logits, theirs(tok, doc).logits
        assert (full - ref_full).abs().max() < 1e-10 and (full - torch.nn.functional.linear(out.hidden_aux, mine.head_weight())).abs().max() < 1e-12
        a = mine.prefill(tok[:, :20], doc[:, :20])
        b = mine.extend(tok[:, 20:], doc[:, 20:], None, a.cache)
        assert a.cache.copy is None and (torch.cat([a.logits, b.logits], 1) - full).abs().max() < 1e-9
    for key, value, match in (("aux_weight", 0.0, "aux_weight"), ("pointer_input", "final", "pointer_input"), ("force_lambda_zero", True, "force_lambda_zero"), ("train_mode", "addon", "train_mode")):
        bad = copy.deepcopy(cfg)
        setattr(bad.cp_head, key, value)
        with pytest.raises(ValueError, match=match):
            build_model(bad)


def test_add_on_copy_paste_head_equals_the_reference(reference):
    """cp_head.train_mode addon: the mixture head's tensors; evaluation reads the mixture; in training mode the pointer's inputs
    carry no gradient into the stack, and the head's own term, the mixture's CE with p_LM's numbers and h detached, equals
    the reference's and sends its gradient to the head's tensors alone."""
    from ced.model import cp_aux as RAUX
    from ced.model import cp_head as RCP

    from gdn_hybrid_architecture_ideas_b200.models import cp_head as CP

    cfg = C.tiny_full_config()
    cfg.encoder.gdn_write_variant = "none"
    cfg.cp_head.enabled, cfg.cp_head.d_c, cfg.cp_head.query_chunk, cfg.cp_head.pointer_input, cfg.cp_head.qk_norm = True, 8, 16, "mix", True
    gated, _ = _pair(reference, cfg)
    cfg.cp_head.train_mode = "addon"
    mine, theirs = _pair(reference, cfg)
    sd, rsd = mine.state_dict(), theirs.state_dict()
    assert list(sd) == list(rsd) and all(torch.equal(sd[k], rsd[k]) for k in sd) and all(torch.equal(sd[k], v) for k, v in gated.state_dict().items())
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40, vocab=12)
    tgt = torch.roll(tok, -1, 1)
    w = torch.full(tgt.shape, 1.0 / tgt.numel(), dtype=torch.double)
    oa, ob = mine(tok, doc, return_hidden=True), theirs(tok, doc, return_hidden=True)
    assert not oa.cp_pointer.q.requires_grad or all(x is None for x in torch.autograd.grad(oa.cp_pointer.q.sum(), [p for n, p in mine.named_parameters() if not n.startswith("cp_head.")], allow_unused=True))
    loss, ce_mix, lam = CP.addon_loss(mine, oa.hidden_aux, tgt, tok, doc, w, pointer=oa.cp_pointer)
    hb = ob.hidden_aux.detach()
    W = theirs.lm_head_weight().detach()
    logits = hb @ W.t()
    lse_r = torch.logsumexp(logits, -1)
    log_lm = logits.gather(-1, tgt[..., None]).squeeze(-1) - lse_r
    ls, l1s, lp = RCP.cp_terms(theirs.cp_head, hb, tok, tgt, doc, pointer=ob.cp_pointer)
    ce_r = -RAUX.addon_log_prob(lse_r, log_lm, theirs.cp_head.copy_logit(hb), ls, l1s, lp)
    assert (ce_mix - ce_r).abs().max() < 1e-10 and abs(float(loss) - float((ce_r * w).sum())) < 1e-12 and 0 < float(lam.min()) and float(lam.max()) < 1
    ga = torch.autograd.grad(loss, list(mine.parameters()), allow_unused=True)
    gb = torch.autograd.grad((ce_r * w).sum(), list(theirs.parameters()), allow_unused=True)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None) == (not n.startswith("cp_head.")), n
        assert x is None or (x - y).abs().max() < 1e-9, n
    mine.eval(), theirs.eval()
    with torch.no_grad():
        a, b = mine(tok, doc).logits, theirs(tok, doc).logits
        assert (a - b).abs().max() < 1e-10 and (a.exp().sum(-1) - 1).abs().max() < 1e-9
    for key, value in (("pointer_input", "final"), ("temperature", "ssmax"), ("aux_weight", 0.5)):
        bad = copy.deepcopy(cfg)
        setattr(bad.cp_head, key, value)
        with pytest.raises(ValueError, match="addon|aux_weight"):
            build_model(bad)
