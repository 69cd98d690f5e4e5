"""CPU tests of the evaluation package, the accounting helpers and the small training-runtime modules."""

import json
import math

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import build_model


def _tiny():
    torch.manual_seed(0)
    return build_model(C.tiny_full_config()).eval()


def test_criterion_rule():
    from gdn_hybrid_architecture_ideas_b200.utils.criterion import Rule, Tally, nan_max

    r = Rule(4.0, 1e-6)
    assert r.passes(3e-3, 1e-3) and not r.passes(5e-3, 1e-3)
    assert r.read("x", 5e-7, 0.0).only_floor and r.read("x", 0.0, 0.0).by_ratio
    assert not r.passes(float("nan"), 1.0) and not r.passes(1.0, float("nan"))
    assert Rule(2.0, 1e-6, form="max").bound(1e-9) == 1e-6
    assert math.isnan(nan_max([1.0, float("nan"), 0.5]))
    t = Tally()
    t.add(r.read("a", 1e-3, 1e-3)); t.add(r.read("b", 1.0, 1e-3))
    assert (t.passed, t.failed, t.ok) == (1, 1, False)


def test_params_and_flops():
    from gdn_hybrid_architecture_ideas_b200.utils import params

    cfg = C.tiny_full_config()
    meta = params.build_on_meta(cfg)
    real = build_model(cfg)
    groups = params.parameter_breakdown(meta)
    assert groups["total"] == sum(p.numel() for p in real.parameters())
    assert groups["embeddings"] + groups["non-embedding"] == groups["total"]
    f = params.flops_per_token(cfg, 128)
    assert f["training"] > 3 * f["prefill_context"] > 0 and f["decode_generated"] > f["prefill_context"]


def test_shape_schedule_matches_walk():
    from gdn_hybrid_architecture_ideas_b200.train.shape_schedule import ShapeSchedule, reference_walk

    phases = [(0.25, 4, 64), (0.5, 8, 128)]
    sch = ShapeSchedule(phases, steps=8, batch_rows=16, seq_len=128, micro_rows=4)
    walk = reference_walk(phases, 8, 16, 128)
    assert sch.total_steps == len(walk)
    for k, (rows, length, first_token) in enumerate(walk):
        s = sch.at(k)
        assert (s.rows, s.seq_len) == (rows, length) and s.first_row * length == first_token
        assert abs(s.clock * 16 * 128 - first_token) < 1e-6
    assert sch.at(sch.total_steps - 1).rows == 16
    rows_mode = ShapeSchedule(phases, 8, 16, 128, lr_mode="rows")
    assert rows_mode.at(0).lr_scale == 1.0 / rows_mode.phases[0].per_ref
    with pytest.raises(ValueError):
        ShapeSchedule([(0.5, 3, 100)], 8, 16, 128)


def test_loss_forms_agree():
    from gdn_hybrid_architecture_ideas_b200.train.chunked_loss import head_positions, token_ce
    from gdn_hybrid_architecture_ideas_b200.train.loss import lm_loss

    torch.manual_seed(1)
    h = torch.randn(2, 50, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)
    t = torch.randint(0, 40, (2, 50))
    valid = torch.rand(2, 50) > 0.3
    loss, ce, z, n = lm_loss(h @ w.t(), t, valid, z_loss=1e-3)
    ce2, z2, n2 = token_ce(h, w, t, valid, 1e-3, chunk=32)
    assert torch.allclose(ce, ce2, rtol=1e-5) and torch.allclose(z, z2, rtol=1e-5) and n == n2
    idx, wt = head_positions(valid, 32)
    assert idx.numel() % 32 == 0 and int(wt.sum()) == int(valid.sum())
    g1 = torch.autograd.grad(ce, h, retain_graph=True)[0]
    g2 = torch.autograd.grad(ce2, h)[0]
    assert torch.allclose(g1, g2, atol=1e-5)


def test_freeze_trunk_and_zero_wgrad():
    from gdn_hybrid_architecture_ideas_b200.train.freeze_trunk import TrunkGuard
    from gdn_hybrid_architecture_ideas_b200.train.zero_wgrad import ZeroWgradMonitor

    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2))
    guard = TrunkGuard(m, ("1.",))
    mon = ZeroWgradMonitor(m)
    m(torch.randn(3, 4)).sum().backward()
    guard.check_grads(); guard.check_values()
    guard.check_optimizer(torch.optim.SGD([p for p in m.parameters() if p.requires_grad], lr=0.1))
    assert set(mon.counts()) == {"1.weight"}
    with torch.no_grad():
        m[0].weight.add_(1.0)
    with pytest.raises(RuntimeError):
        guard.check_values()


def test_position_masks_are_pure_and_causal():
    from gdn_hybrid_architecture_ideas_b200.train.positions import AnswerSpanRule, PositionSampler, answer_span_mask

    doc = torch.tensor([[0] * 300 + [1] * 212])
    valid = torch.ones(1, 512, dtype=torch.bool)
    rule = AnswerSpanRule(min_context=16, gap_mean=20.0, span_min=4, span_max=12)
    a = answer_span_mask(doc, valid, rule, 3, 7)
    assert torch.equal(a, answer_span_mask(doc, valid, rule, 3, 7)) and a.any()
    assert not a[0, :16].any() and not a[0, 300:316].any()
    # prefix stability: what the row holds after position 200 does not change the mask before it
    doc2 = torch.tensor([[0] * 200 + [5] * 312])
    assert torch.equal(a[0, :200], answer_span_mask(doc2, valid, rule, 3, 7)[0, :200])
    s = PositionSampler("random", seed=1, capacity=40)
    m = s.mask(doc, valid, 2)
    assert int(m.sum()) == 40 and torch.equal(m, s.mask(doc, valid, 2)) and not torch.equal(m, s.mask(doc, valid, 3))


def test_span_bpb_pack_join_and_se():
    from gdn_hybrid_architecture_ideas_b200.eval import span_bpb as sb

    model = _tiny()
    V = model.cfg.vocab_size
    g = torch.Generator().manual_seed(0)
    docs = [sb.TokenizedDoc(torch.randint(1, V, (n,), generator=g).tolist(), [2] * n) for n in (9, 30, 17, 40, 5, 200)]
    rows = sb.build_eval_rows(docs, 64)
    assert rows.skipped == [5] and rows.tokens.shape[1] == 64
    full = sb.evaluate(model, rows, batch_size=2)
    half = [sb.evaluate(model, rows, 2, row_indices=[r for r in range(rows.tokens.shape[0]) if r % 2 == k]) for k in (0, 1)]
    joined = sb.join_batches(half)
    assert torch.allclose(full.row_nats, joined.row_nats, rtol=1e-6) and abs(full.bpb - joined.bpb) < 1e-9
    # a document scores the same alone as packed beside others (document isolation)
    alone = sb.evaluate(model, sb.build_eval_rows([docs[1]], 64))
    assert abs(float(alone.doc_nats[0]) - float(full.doc_nats[1])) < 1e-3 * float(alone.doc_nats[0])
    assert sb.bpb_se(full) > 0
    assert abs(sb.paired_difference(full, full).diff_bpb) < 1e-12


def test_batched_generation_matches_uncached_argmax():
    from gdn_hybrid_architecture_ideas_b200.eval.generate import full_forward_argmax, generate_greedy, generate_greedy_batched

    model = _tiny()
    V = model.cfg.vocab_size
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(1, V, (n,), generator=g).tolist() for n in (12, 5, 9)]
    outs = generate_greedy_batched(model, prompts, 6, prefill_chunk=4, check_every=2)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        seq = p + o
        want = full_forward_argmax(model, seq, [len(p) - 1 + i for i in range(6)])
        assert want == o
    assert generate_greedy(model, prompts[1], 6) == outs[1]
    stop = generate_greedy_batched(model, prompts, 6, eos_id=outs[0][2], check_every=1)
    assert len(stop[0]) <= 3


def test_gqa_fold_matches_expanded_read():
    from gdn_hybrid_architecture_ideas_b200.eval.gqa_fold import attend_capped_folded, attend_folded
    from gdn_hybrid_architecture_ideas_b200.ops import reference as ref

    torch.manual_seed(0)
    B, L, Hq, Hkv, hd = 2, 10, 4, 2, 8
    q, qf = torch.randn(B, L, Hq, hd), torch.randn(B, L, Hq, hd)
    k, kf, v = (torch.randn(B, L, Hkv, hd) for _ in range(3))
    idx = torch.arange(L)[None].expand(B, L)
    doc = torch.zeros(B, L, dtype=torch.long)
    allow = idx[:, :, None] >= idx[:, None, :]
    want = ref.attention(q, k, v, idx, doc, idx, doc)
    assert torch.allclose(attend_folded(q, k, v, allow), want, atol=1e-5)
    cap = 3
    far = (idx[:, :, None] - idx[:, None, :]) > cap
    want_c = ref.attention(q, k, v, idx, doc, idx, doc, None, qf, kf, cap)
    assert torch.allclose(attend_capped_folded(q, qf, k, kf, v, allow, far), want_c, atol=1e-5)


def test_long_context_buckets_and_probes_and_choice():
    from gdn_hybrid_architecture_ideas_b200.eval import long_context as lc, multiple_choice as mc, probes

    model = _tiny()
    V = model.cfg.vocab_size
    assert lc.bucket_names((4, 8)) == ["0-4", "4-8", ">8"]
    pos = torch.arange(12)
    sums = lc.bucket_sums(torch.ones(12), pos, (4, 8))
    assert sums.tolist() == [4.0, 4.0, 4.0]
    ids = torch.randint(1, V, (40,), generator=torch.Generator().manual_seed(1))
    whole = lc.position_ce(model, ids, chunk=64)
    parts = lc.position_ce(model, ids, chunk=7)
    assert torch.allclose(whole, parts, atol=2e-4)
    res = lc.score_position_bpb(model, [{"ids": ids, "byte_lens": torch.ones(40, dtype=torch.long)}] * 2, edges=(16, 32), chunk=16)
    assert len(res["table"]) == 3 and res["table"][0]["docs"] == 2
    ps = [probes.build_probe(kind, V, 48, seed=0, index=i) for i, kind in enumerate(probes.PROBE_KINDS)]
    for p in ps:
        assert p.answer_start + p.answer_len == len(p.ids) and min(p.ids) >= 1
    assert probes.build_probe("needle", V, 48, 0, 0).ids == ps[0].ids
    out = probes.score_probes(model, ps, batch_size=3)
    assert out["n"] == len(probes.PROBE_KINDS) and 0.0 <= out["exact"] <= 1.0 and out["ce"] > 0
    items = [mc.Item([3, 4, 5], [[6, 7], [8], [9, 10, 11]], 1)]
    assert mc.score_items(model, items, seq_len=32)["n"] == 1


def test_multifact_and_transcode_probes():
    """Multi-fact items: the answer's pieces tile it, facts sit where the layout says, the metrics read the fact tokens
    only. Transcode: the two directions of one base share the content, the escape round-trips, the untranscoded source
    never equals the answer."""
    from gdn_hybrid_architecture_ideas_b200.eval import probes

    V = 256
    for kind in ("mf_chain", "mf_concat"):
        for i in range(6):
            p = probes.build_probe(kind, V, 400, seed=1, index=i, n_keys=4)
            assert p.group == probes.LAYOUTS[i % 3] and sum(n for n, _ in p.pieces) == p.answer_len
            assert [f for _, f in p.pieces] == [True, False] * 3 + [True] and len(p.ids) == 400
            where = [j / 400 for j, t in enumerate(p.ids[:p.ids.index(3)]) if t == 1]
            assert len(where) == 4
            if p.group == "front":
                assert max(where) < 0.45
            if p.group == "back":
                assert min(where) > 0.5          # depths count haystack tokens, the facts themselves come on top
    p = probes.build_probe("mf_chain", V, 200, 0, 0, n_keys=3)
    ans = p.ids[p.answer_start:]
    facts = {}
    ctx = p.ids[:p.answer_start]
    for j, t in enumerate(ctx):
        if t == 1 and ctx[j + 5] == 2:
            facts[tuple(ctx[j + 1:j + 5])] = ctx[j + 6:j + 10]
    q = ctx[ctx.index(3) + 1:ctx.index(3) + 5]
    chain = []
    for _ in range(3):
        q = facts[tuple(q)]
        chain.append(q)
    at, got = 0, []
    for n, is_fact in p.pieces:
        if is_fact:
            got.append(ans[at:at + n])
        at += n
    assert got == chain
    ok = [True] * p.answer_len
    ok[4] = False                                   # a scaffold token wrong: every fact still right
    m = probes.multifact_metrics(p, ok, [0.5] * p.answer_len)
    assert m["exact"] and not m["exact_all"] and m["fact_acc"] == 1.0 and m["hop_ok"] == [1.0, 1.0, 1.0]
    ok = [True] * p.answer_len
    ok[0] = False
    m = probes.multifact_metrics(p, ok, [0.5] * p.answer_len)
    assert not m["exact"] and abs(m["fact_acc"] - 2 / 3) < 1e-9 and abs(m["first_ok"] - 2 / 3) < 1e-9
    a, b = probes.build_probe("transcode", V, 120, 0, 4), probes.build_probe("transcode", V, 120, 0, 5)
    assert (a.group, b.group) == ("esc2raw", "raw2esc")
    raw, esc = a.ids[a.answer_start:], b.ids[b.answer_start:]
    assert probes.escape_ids(raw) == esc and len(esc) > len(raw) and probes.ESC not in raw
    for p in (a, b):
        f = probes.copy_floor(p)
        assert not f["exact"] and 0 < f["lcs_share"] < 1


def test_gdn_diag_and_units(tmp_path):
    from gdn_hybrid_architecture_ideas_b200.eval import gdn_diag, units

    model = _tiny()
    tok = torch.randint(1, model.cfg.vocab_size, (1, 24), generator=torch.Generator().manual_seed(2))
    recs = gdn_diag.encoder_gdn_diag(model, tok, torch.zeros_like(tok), block=8)
    assert [r["position"] for r in recs] == [8, 16, 24]
    layers = recs[-1]["layers"]
    assert layers and all(v["stable_rank"] >= 1.0 - 1e-4 and "rel_change" in v for v in layers.values())
    store = units.UnitStore(tmp_path / "u", {"model": "a"})
    calls = []
    assert store.run({"set": "x", "rows": [0, 1]}, lambda: calls.append(1) or {"v": 3}) == {"v": 3}
    assert store.run({"set": "x", "rows": [0, 1]}, lambda: calls.append(1) or {"v": 4}) == {"v": 3} and len(calls) == 1
    assert units.UnitStore(tmp_path / "u", {"model": "b"}).get({"set": "x", "rows": [0, 1]}) is None


def test_periodic_eval_leaves_training_untouched(tmp_path):
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    def run(with_eval):
        cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
        cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 4, 0, False, "cpu"
        if with_eval:
            cfg.eval.sets, cfg.eval.every_steps = {"held": "synthetic:3"}, 2
        t = Trainer(cfg, tmp_path / ("e" if with_eval else "p"))
        t.fit()
        return t

    a, b = run(True), run(False)
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.equal(p, q), n
    rec = json.loads((tmp_path / "e" / "eval" / "step_2.json").read_text())
    assert rec["sets"]["held"]["bpb"] > 0 and (tmp_path / "e" / "eval" / "step_4.json").exists()


def test_sharded_eval_blocks_cover_rows():
    from gdn_hybrid_architecture_ideas_b200.train.sharded_eval import batch_block

    for n, bs, w in ((10, 3, 4), (7, 2, 2), (5, 8, 3)):
        got = sorted(sum((batch_block(n, bs, r, w) for r in range(w)), []))
        assert got == list(range(n))


def test_shipped_configs_and_run_entries_load():
    """Every shipped config builds (refuse-by-name passes) and every run entry's overrides apply to its base config."""
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root / "scripts"))
    import run_entry

    configs = sorted((root / "configs").rglob("*.yaml"))
    assert len(configs) >= 7
    for p in configs:
        C.require_supported(C.load_yaml(p))
    for runs_file in sorted((root / "runs").glob("*.yaml")):
        runs = run_entry.load_runs(runs_file, "/data", "/tmp/runs")
        for entry in runs["runs"]:
            cfg = C.load_yaml(root / (entry.get("config") or entry["base"]))
            for item in run_entry.entry_overrides(runs, entry):
                C.apply_override(cfg, item)
            C.require_supported(cfg)
            assert run_entry.build_command(runs, entry, "/tmp/runs", nproc=2)[1:3] == ["-m", "torch.distributed.run"]


def test_eval_scripts_run_on_a_checkpoint(tmp_path):
    import subprocess
    import sys
    from pathlib import Path

    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    root = Path(__file__).resolve().parent.parent
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 1, 0, False, "cpu"
    Trainer(cfg, tmp_path / "run").fit()
    V = cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)
    docs = [{"ids": torch.randint(1, V, (n,), generator=g).tolist(), "byte_lens": [1] * n} for n in (20, 33)]
    torch.save({"docs": docs}, tmp_path / "set.pt")
    torch.save({"docs": [{"ids": torch.randint(1, V, (48,), generator=g), "byte_lens": torch.ones(48, dtype=torch.long)}]}, tmp_path / "long.pt")
    run = lambda *a: subprocess.run([sys.executable, *a], check=True, capture_output=True, text=True, timeout=600)
    run(str(root / "scripts/rescore.py"), "--checkpoint", str(tmp_path / "run"), "--set", f"x={tmp_path / 'set.pt'}", "--seq-len", "64",
        "--device", "cpu", "--out", str(tmp_path / "s.json"))
    assert json.loads((tmp_path / "s.json").read_text())["scores"]["x"]["bpb"] > 0
    run(str(root / "scripts/eval_probes.py"), "--checkpoint", str(tmp_path / "run"), "--lengths", "40", "--per-kind", "2", "--device", "cpu",
        "--out", str(tmp_path / "p.json"))
    table = json.loads((tmp_path / "p.json").read_text())["probes"]
    assert len(table) == 8 and "fact_acc" in table["mf_chain@40"] and "copy_floor" in table["transcode@40"]
    run(str(root / "scripts/eval_long.py"), "--checkpoint", str(tmp_path / "run"), "--docs", str(tmp_path / "long.pt"), "--base", "16",
        "--chunk", "16", "--gdn-diag", "--window", "16", "--train-len", "16", "--summary", str(tmp_path / "l.md"), "--device", "cpu",
        "--out", str(tmp_path / "l.json"))
    run(str(root / "scripts/build_probes.py"), "--vocab", str(V), "--lengths", "40", "--per-kind", "2", "--kinds", "needle,mf_concat",
        "--out", str(tmp_path / "probes.pt"))
    run(str(root / "scripts/build_probes.py"), "--vocab", str(V), "--lengths", "40,64", "--per-kind", "3", "--kinds", "needle,mf_concat",
        "--extend", str(tmp_path / "probes.pt"), "--out", str(tmp_path / "probes2.pt"))
    run(str(root / "scripts/eval_probes.py"), "--checkpoint", str(tmp_path / "run"), "--set", str(tmp_path / "probes2.pt"), "--device", "cpu",
        "--out", str(tmp_path / "p2.json"))
    t2 = json.loads((tmp_path / "p2.json").read_text())["probes"]
    assert set(t2) == {"needle@40", "mf_concat@40", "needle@64", "mf_concat@64"} and t2["needle@64"]["n"] == 3
    run(str(root / "scripts/report_pcr.py"), "--checkpoint", str(tmp_path / "run"), "--set", f"x={tmp_path / 'set.pt'}", "--set",
        f"y={tmp_path / 'set.pt'}", "--seq-len", "64", "--edges", "0,8,32", "--copy-lengths", "8,16", "--copy-items", "2", "--device", "cpu",
        "--out", str(tmp_path / "r.json"))
    rep = json.loads((tmp_path / "r.json").read_text())
    assert rep["buckets"] == ["0-7", "8-31", "32-end"] and "all_sets" in rep and set(rep["copy_gain"]) == {"8", "16"}
    long = json.loads((tmp_path / "l.json").read_text())
    assert long["gdn_diag"] and long["context_gain"] and "breaks_first" in long and "difference" in (tmp_path / "l.md").read_text()


def test_build_eval_set_script(tmp_path):
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "docs.jsonl").write_text('{"text": "hello world"}\nplain line of text\n')
    (tmp_path / "chat.jsonl").write_text(json.dumps({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]}) + "\n")
    run = lambda *a: subprocess.run([sys.executable, str(root / "scripts/build_eval_set.py"), *a], check=True, capture_output=True, timeout=300)
    run("--input", str(tmp_path / "docs.jsonl"), "--out", str(tmp_path / "a.pt"))
    run("--input", str(tmp_path / "chat.jsonl"), "--out", str(tmp_path / "b.pt"), "--chat")
    a = torch.load(tmp_path / "a.pt", weights_only=False)["docs"]
    b = torch.load(tmp_path / "b.pt", weights_only=False)["docs"]
    assert [len(d["ids"]) for d in a] == [11, 18] and a[0]["ids"][:5] == list(b"hello")
    assert sum(b[0]["scored"]) == 3 and len(b[0]["scored"]) == len(b[0]["ids"])


def test_bpb_readout_uses_fixed_rows(tmp_path):
    from gdn_hybrid_architecture_ideas_b200.train.bpb_readout import BpbReadout, due
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 2, 0, True, "cpu"
    cfg.eval.bpb_readout_sets, cfg.eval.bpb_readout_every, cfg.eval.bpb_readout_rows = {"held": "synthetic:6"}, 1, 3
    assert due(cfg, 1) and not due(cfg, 0) or cfg.eval.bpb_readout_from == 0
    t = Trainer(cfg, tmp_path / "r")
    r = BpbReadout(t)
    a, b = r.run(), r.run()
    assert a == b and a["readout/held/bpb"] > 0 and len(r.sets["held"].chosen) == 3
    t.fit()
    lines = [json.loads(x) for x in (tmp_path / "r" / "metrics.jsonl").read_text().splitlines()]
    assert sum(1 for x in lines if x.get("event") == "bpb_readout") == 2


def test_routed_swiglu_dispatch_equals_dense():
    """Token dispatch (each expert on its routed tokens only) equals the every-expert-on-every-token statement, values and
    gradients; the balance statistic is 1 for uniform routing probabilities."""
    import torch

    from gdn_hybrid_architecture_ideas_b200.models.mlp import RoutedSwiGLU

    torch.manual_seed(0)
    m = RoutedSwiGLU(32, 4, 2, 48).double()
    x = torch.randn(3, 17, 32, dtype=torch.float64, requires_grad=True)
    valid = torch.rand(3, 17) > 0.2
    a = m(x, valid)
    ga = torch.autograd.grad(a.square().sum(), [x, *m.parameters()])
    b = m.forward_dense(x, valid)
    gb = torch.autograd.grad(b.square().sum(), [x, *m.parameters()])
    assert (a - b).abs().max() < 1e-12
    assert max((p - q).abs().max() for p, q in zip(ga, gb)) < 1e-10
    assert float(m.z_loss()) > 0
    m.reset_stats()
    with torch.no_grad():
        m.router.weight.zero_()
    m(x)
    assert abs(float(m.balance_loss()) - 1.0) < 1e-9


def test_recall_ruler_items_and_scoring(tmp_path):
    """RULER subset: items are deterministic, fitted to the asked length under the token counter, hold their needles and
    references; string-match recall and the values file; the scorer script runs a tiny byte-level model end to end."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import torch

    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.data.tokenizers import ByteTokenizer
    from gdn_hybrid_architecture_ideas_b200.eval import recall_ruler as RR
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    tok = ByteTokenizer()
    count = lambda t: len(tok.encode(t))
    pool = [("The river bends twice before the mill. Nobody fishes there in winter. " * 40) + f"Document {i} ends here." for i in range(6)]
    for task in RR.TASKS:
        a = RR.make_item(task, 4096, 3, count, pool)
        b = RR.make_item(task, 4096, 3, count, pool)
        assert a.prompt == b.prompt and a.refs == b.refs and a.id == f"{task}/len=4096/0003"
        assert 0.95 * (4096 - a.gen_tokens) <= count(a.prompt) <= 4096 - a.gen_tokens, (task, count(a.prompt))
        n_refs = {"niah_multivalue": 4, "niah_multiquery": 4, "vt": 5}.get(task, 1)
        assert len(a.refs) == n_refs and len(set(a.refs)) == n_refs
        assert all(r in a.prompt for r in a.refs)
        assert RR.make_item(task, 4096, 4, count, pool).prompt != a.prompt
    single = RR.make_item("niah_multikey_2", 2048, 0, count)
    assert "A special magic number is hidden" in single.prompt and single.prompt.endswith("mentioned in the provided text is")
    assert RR.recall(" 12 and ABC\x00def", ["abc", "77"]) == 0.5 and RR.all_found("x1 y2", ["X1", "y2"]) == 1.0
    vals = RR.values_file("r", [{"task": "vt", "length": 2048, "id": "a", "recall": 0.4, "all_found": 0.0},
                                {"task": "vt", "length": 2048, "id": "b", "recall": 1.0, "all_found": 1.0},
                                {"task": "niah_multikey_2", "length": 2048, "id": "c", "recall": 1.0, "all_found": 1.0}], excluded=["b"])
    assert vals["cells"]["ruler|vt|2048|recall"] == 0.4 and vals["cells"]["ruler|mean|2048|recall"] == 0.7 and vals["n_items"] == 2

    root = Path(__file__).resolve().parent.parent
    cfg = C.TrainConfig(model=C.tiny_control_config(), data=C.tiny_data_config(seq_len=48, batch_size=2), steps=1, seed=1)
    cfg.model.vocab_size = 256
    cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.log_every = 1, False, 0
    Trainer(cfg, tmp_path / "run").fit()
    r = subprocess.run([sys.executable, str(root / "scripts" / "recall_ruler_score.py"), "--checkpoint", str(tmp_path / "run"), "--tokenizer", "bytes",
                        "--out", str(tmp_path / "o"), "--run", "t", "--tasks", "vt", "--lengths", "1024", "--n-per-cell", "2", "--batch", "2", "--device", "cpu"],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    values = json.loads((tmp_path / "o" / "t.values.json").read_text())
    assert values["n_items"] == 2 and "ruler|vt|1024|recall" in values["cells"]
    assert len((tmp_path / "o" / "t.items.jsonl").read_text().splitlines()) == 2

    # stored items: built once (deterministic files, hashes, the documents used), then scored from the build
    docs = tmp_path / "docs.jsonl"
    docs.write_text("".join(json.dumps({"id": f"d{i}", "text": t}) + "\n" for i, t in enumerate(pool)))
    build = [sys.executable, str(root / "scripts" / "build_recall_ruler.py"), "--tokenizer", "bytes", "--docs", str(docs), "--tasks", "vt", "niah_multikey_1",
             "--lengths", "1024", "--per-cell", "2"]
    for name in ("b1", "b2"):
        r = subprocess.run(build + ["--out", str(tmp_path / name)], capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
    m1, m2 = (json.loads((tmp_path / n / "manifest.json").read_text()) for n in ("b1", "b2"))
    assert m1["sha256"] == m2["sha256"] and m1["cells"]["vt|1024"]["items"] == 2 and not m1["token_count_mismatches"]
    hashes = json.loads((tmp_path / "b1" / "item-hashes.json").read_text())
    used = json.loads((tmp_path / "b1" / "haystack-docs-used.json").read_text())
    assert set(hashes) == {"vt/len=1024/0000", "vt/len=1024/0001", "niah_multikey_1/len=1024/0000", "niah_multikey_1/len=1024/0001"}
    assert used["all"] and set(used["per_task"]) == {"niah_multikey_1"}
    r = subprocess.run([sys.executable, str(root / "scripts" / "recall_ruler_score.py"), "--checkpoint", str(tmp_path / "run"), "--tokenizer", "bytes",
                        "--out", str(tmp_path / "o2"), "--run", "t", "--items", str(tmp_path / "b1"), "--tasks", "vt", "--lengths", "1024", "--n-per-cell", "2",
                        "--batch", "2", "--device", "cpu"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    on_the_fly = [json.loads(x) for x in (tmp_path / "o" / "t.items.jsonl").read_text().splitlines()]
    from_build = [json.loads(x) for x in (tmp_path / "o2" / "t.items.jsonl").read_text().splitlines()]
    assert [(x["id"], x["pred"]) for x in on_the_fly] == [(x["id"], x["pred"]) for x in from_build]      # the same prompts either way


def test_recall_based_protocol(tmp_path):
    """Based suite: item files round-trip with their checksums, left truncation keeps the end, the generation is cut at the
    first newline and before the end-of-document token, "contains" is a case-insensitive search; the scorer script runs."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.eval import recall_based as RB
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    items = {"swde": [RB.Item("swde", f"{i}", f"<page {i}> title: Film {i}\nyear: 19{i:02d}\nyear:", f"19{i:02d}") for i in range(5)],
             "fda": [RB.Item("fda", "a", "Device name: Pump (X)\nDevice name:", "Pump (X)")]}
    RB.write_set(tmp_path / "items", items)
    assert RB.load_set(tmp_path / "items", "swde") == items["swde"]
    (tmp_path / "items" / RB.MANIFEST_NAME).write_text(json.dumps({"swde": {"n": 5, "set_sha256": "0"}}))
    try:
        RB.load_set(tmp_path / "items", "swde")
        raise AssertionError("a wrong checksum must be refused")
    except ValueError:
        pass
    RB.write_set(tmp_path / "items", items)
    assert RB.left_truncate(list(range(100)), 80) == (list(range(68, 100)), True) and RB.left_truncate([1, 2], 80) == ([1, 2], False)
    assert RB.cut_at_stop(" 1999\nyear: 2000") == " 1999" and RB.cut_at_eos([5, 6, 0, 7], 0) == ([5, 6], 2) and RB.cut_at_eos([5], None) == ([5], -1)
    assert RB.contains_score("the pump (x) model", "Pump (X)") == 1 and RB.contains_score("pump x", "Pump (X)") == 0
    v = RB.values_json("r", {"swde": [{"id": "0", "hit": 1}, {"id": "1", "hit": 0}]}, exclude=["swde:1"])
    assert v["cells"] == {"based|swde|all|acc": 1.0} and v["n_items"]["based|swde|all|acc"] == 1

    root = Path(__file__).resolve().parent.parent
    cfg = C.TrainConfig(model=C.tiny_control_config(), data=C.tiny_data_config(seq_len=64, batch_size=2), steps=1, seed=1)
    cfg.model.vocab_size = 256
    cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.log_every = 1, False, 0
    Trainer(cfg, tmp_path / "run").fit()
    r = subprocess.run([sys.executable, str(root / "scripts" / "recall_based_score.py"), "--checkpoint", str(tmp_path / "run"), "--items", str(tmp_path / "items"),
                        "--tokenizer", "bytes", "--out", str(tmp_path / "o"), "--run", "t", "--batch", "3", "--device", "cpu"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    vals = json.loads((tmp_path / "o" / "t.values.json").read_text())
    assert set(vals["cells"]) == {"based|swde|all|acc", "based|fda|all|acc"} and vals["n_items"]["based|swde|all|acc"] == 5


def test_tst_diagnostics():
    import math

    import numpy as np
    import torch

    from gdn_hybrid_architecture_ideas_b200.eval import tst_diag as TD
    from gdn_hybrid_architecture_ideas_b200.eval.tokenized import byte_tokenize

    counts = np.array([30, 30, 0, 20, 10, 5, 3, 1, 1, 0])
    classes, info = TD.frequency_classes(counts)
    assert classes.tolist() == [0, 0, 3, 1, 2, 2, 3, 3, 3, 3]        # mass before: 0, .3 | .6 | .8, .9 | .95, .98, .99, 1, 1
    assert info["classes"]["frequent"]["mass"] == 0.6 and info["zero_count_ids"] == 2 and TD.class_name_three(3) == "rare"
    doc = torch.tensor([[4, 4, 4, 7, 7, 9], [1, 1, 1, 1, 1, 1]])
    assert TD.context_in_document(doc).tolist() == [[0, 1, 2, 0, 1, 0], [0, 1, 2, 3, 4, 5]]
    assert TD.bucket_of(torch.tensor([0, 127, 128, 511, 512, 5000]), TD.ROW_EDGES).tolist() == [0, 0, 1, 1, 2, 3]
    tokens = torch.tensor([[0, 1, 3, 4, 6, 2], [1, 1, 0, 3, 5, 7]])
    targets = torch.cat([tokens[:, 1:], tokens[:, :1]], 1)
    scored = torch.tensor([[1, 1, 0, 1, 1, 0], [1, 1, 1, 1, 1, 0]], dtype=torch.bool)
    ce = torch.rand(2, 6, dtype=torch.float64) + 0.5
    agg = TD.aggregate_ce(ce, tokens, targets, doc, scored, torch.full((2, 6), 2), classes)
    want = float((ce * scored).sum()) / (math.log(2) * 2 * int(scored.sum()))
    for split in agg.values():
        c = TD.contributions(split)
        assert abs(c["contribution"].sum() - want) < 1e-12 and abs(c["set_bpb"] - want) < 1e-12 and c["tokens"].sum() == scored.sum()
    a = {"embed.weight": torch.zeros(4, 2), "out_embed.weight": torch.zeros(4, 2), "embed_norm.weight": torch.zeros(2), "final_norm.weight": torch.zeros(2), "x": torch.ones(1)}
    b = {k: v + 1 for k, v in a.items()}
    g = TD.graft_state(a, b)
    assert g["embed.weight"].eq(1).all() and g["embed_norm.weight"].eq(0).all() and g["x"] is a["x"]
    assert TD.graft_state(a, b, norms=True)["final_norm.weight"].eq(1).all()
    try:
        TD.graft_state({"embed.weight": a["embed.weight"]}, b)
        raise AssertionError("a tied head cannot be grafted")
    except ValueError:
        pass
    w = torch.tensor([[0.0, 0.0, 0.0, 2.0], [1.0, 0.0, 0.0, 0.0], [1.0, 1.0, 1.0, 1.0]])
    st = TD.conv_span_stats(w, {"q": (0, 1), "rest": (1, 3)})
    assert st["q"]["pass_through"] == 1.0 and st["q"]["span90"] == 1.0 and st["q"]["centroid_lag"] == 0.0
    assert st["rest"]["centroid_lag"] == (3 + 1.5) / 2 and st["rest"]["span90"] == 4.0 and st["all"]["channels"] == 3
    assert abs(TD.bag_norm_eps_change(np.array([1.0]), 4, 1e-6)[0] - (math.sqrt((1 + 1e-6) / (1 + 0.25e-6)) - 1)) < 1e-15
    d = byte_tokenize("aé")
    assert d.ids == [97, 195, 169] and d.byte_lens == [1, 1, 1]


def test_long_report_context_gain_and_rule():
    """Context gain: the same targets with the full context and with a short one (a model that ignores everything beyond
    the window scores them equally); the degradation rule and what breaks first."""
    import torch

    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.eval import long_context as LC, long_report as LR
    from tests.helpers import make_model

    model = make_model(C.tiny_control_config(), dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(0)
    docs = [{"ids": torch.randint(0, 256, (n,), generator=g), "byte_lens": torch.randint(1, 4, (n,), generator=g)} for n in (96, 130, 70)]
    edges = (0, 32, 64, 128, 256)
    res = LC.score_position_bpb(model, docs, edges=edges, chunk=64)
    rows = LR.context_gain(model, docs, edges, window=32, chunk=64, full_records=res["records"])
    assert [r["bucket"] for r in rows] == LC.bucket_names(edges)[2:5] and [r["docs"] for r in rows] == [3, 3, 1]
    again = LR.context_gain(model, docs, edges, window=32, chunk=64)
    assert all(abs(a["full"] - b["full"]) < 1e-5 for a, b in zip(rows, again))
    assert all(abs(r["full"] - r["short"] - r["diff"]) < 1e-9 for r in rows)
    summary = {"bpb": {"web": [{"bucket": "16k", "length": 16384, "full": 0.70, "short": 0.71, "diff": -0.01, "se": 0.002, "docs": 9},
                               {"bucket": "32k", "length": 32768, "full": 0.74, "short": 0.71, "diff": 0.03, "se": 0.004, "docs": 9},
                               {"bucket": "64k", "length": 65536, "full": 0.73, "short": 0.71, "diff": 0.02, "se": 0.02, "docs": 2}]},
               "gdn": LR.gdn_factors({"edges": [0, 8192, 16384, 32768], "layers": [{"norm": [1.0, 1.2, 2.0], "erank": [4.0, 4.0, 3.0], "rel_delta": [0.1, 0.1, 0.1]},
                                                                                {"norm": [2.0, 2.0, 2.2], "erank": [4.0, 5.0, 4.0], "rel_delta": None}]})}
    entries = LR.degradations(summary, train_len=8192)
    by = {(e["metric"], e["length"]): e for e in entries}
    assert not by[("bpb.web", 16384)]["degraded"] and by[("bpb.web", 32768)]["clear"] and by[("bpb.web", 65536)]["degraded"] and not by[("bpb.web", 65536)]["clear"]
    assert by[("gdn.norm", 32768)]["value"] == 2.0 and by[("gdn.norm", 32768)]["clear"] and not by[("gdn.erank", 16384)]["degraded"]
    assert LR.breaks_first(entries) == {"length": 32768, "metrics": ["bpb.web", "gdn.norm"]}
    text = LR.render(summary, entries)
    assert "Breaks first at 32768" in text and "| 32k | 0.7400 | 0.7100 | +0.0300 +- 0.0040 | 9 |" in text


def _agent_conversation():
    file_text = "def main():\n    print(\"hello world\")\n    return 0\n"
    return {"tools": [{"name": "editor"}], "messages": [
        {"role": "system", "content": "You are an agent."},
        {"role": "user", "content": "Fix the file. <tool_call> is plain text here."},
        {"role": "assistant", "reasoning": "I should look first.", "content": "Opening the file.",
         "tool_calls": [{"name": "bash", "arguments": {"command": "cat a.py", "timeout": 5}}]},
        {"role": "tool", "content": file_text},
        {"role": "assistant", "content": "", "tool_calls": [{"name": "str_replace_editor", "arguments": {
            "command": "str_replace", "filePath": "/tmp/a.py", "old_str": file_text, "new_str": "pass", "thought": "swap it"}}]},
        {"role": "tool", "content": "ok"},
        {"role": "assistant", "content": "Done:\n```python\nx = 1\n```\nbye",
         "tool_calls": [{"name": "finish", "arguments": {"message": "All fixed."}}]},
    ]}


def test_chat_format_and_token_types():
    """The chat rendering keeps control tokens apart from text, and the labeller types every generated token from the
    ids alone: narration before an acting call, final text before a finish call, path / name heads, a copied editor
    argument (escapes undone), fenced code; labels of a prefix do not move when the document goes on."""
    import numpy as np

    from gdn_hybrid_architecture_ideas_b200.data import chat_format as cf
    from gdn_hybrid_architecture_ideas_b200.eval import token_types as tt

    conv = _agent_conversation()
    tk = cf.ChatTokenizer()
    ids, gen = tk.encode_pieces(cf.pieces(conv))
    assert b"".join(tk.table[t] for t in ids).decode() == cf.render(conv)
    assert ids.count(tk.control[cf.TOOL_CALL]) == 3            # the user's literal "<tool_call>" stays bytes
    doc = tk.encode_conversation(conv)
    assert doc["scored"] == gen and len(doc["byte_lens"]) == len(ids)
    stats = {}
    lab = tt.label_document(ids, gen, tk.table, tk.control, stats=stats)
    assert ((lab >= 0) == np.asarray(gen)).all() and stats["unparsed_calls"] == 0

    def text_of(kind):
        return b"|".join(b"".join(tk.table[ids[j]] for j in run) for run in _runs(lab, tt.F[kind])).decode()

    assert text_of("reasoning_think") == "I should look first."
    assert text_of("narration") == "Opening the file."
    assert text_of("head_name") == "bash|str_replace_editor|str_replace|finish"
    assert text_of("head_path") == "/tmp/a.py"
    assert text_of("reasoning_call") == "swap it"
    assert text_of("code_arg") == "cat a.py|pass"
    assert text_of("arg") == "5"
    assert text_of("copied_arg") == 'def main():\\n    print(\\"hello world\\")\\n    return 0\\n'
    assert text_of("code_content") == "x = 1\n"
    assert text_of("final_answer") == "Done:\n```python\n|```\nbye|All fixed."
    assert (lab == tt.F["call_open"]).sum() == 3 and (lab == tt.F["turn_end"]).sum() == 3
    # a document cut after the second assistant message: the labels before the cut do not move
    cut = [j for j, t in enumerate(ids) if t == tk.control[cf.IM_END] and gen[j]][1] + 1
    assert (tt.label_document(ids[:cut], gen[:cut], tk.table, tk.control) == lab[:cut]).all()
    # the copy window: the same argument with nothing before it to copy from is code
    solo = {"messages": [conv["messages"][4]]}
    ids2, gen2 = tk.encode_pieces(cf.pieces(solo))
    lab2 = tt.label_document(ids2, gen2, tk.table, tk.control)
    assert (lab2 == tt.F["copied_arg"]).sum() == 0 and (lab2 == tt.F["code_arg"]).sum() > 50
    # a call that is not JSON counts as an argument, and is counted
    bad = {"messages": [{"role": "assistant", "content": "x", "tool_calls": [{"name": "t", "arguments": {}}]}]}
    ids3, gen3 = tk.encode_pieces([(p[0].replace('{"name"', "name="), p[1], p[2]) for p in cf.pieces(bad)])
    st3 = {}
    lab3 = tt.label_document(ids3, gen3, tk.table, tk.control, stats=st3)
    assert st3["unparsed_calls"] == 1 and (lab3 == tt.F["arg"]).sum() > 0
    seg = tt.segment_positions(ids, gen, tk.table, tk.control)
    names = [tt.SEGMENTS[s] for s in seg]
    first_call = ids.index(tk.control[cf.TOOL_CALL])
    assert names[first_call] == "call_head" and names[ids.index(tk.control[cf.TOOL_CALL_END])] == "call_body"
    assert names[ids.index(tk.control[cf.THINK])] == "reasoning" and names[0] == "unplaced"
    assert (tt.segment_positions(ids[:cut], gen[:cut], tk.table, tk.control) == seg[:cut]).all()
    summ = tt.summarize([lab], [np.asarray(doc["byte_lens"])])
    assert abs(sum(v["token_share"] for v in summ["types"].values()) - 1) < 1e-9 and summ["types"]["copied"]["tokens"] == 55
    by = tt.loss_by_type([lab], [np.ones(len(lab))])
    assert by["head"]["loss"] == 1.0 and by["args"]["tokens"] == 1
    assert tt.is_path_key("repoDir") and tt.is_path_key("FILE_PATH") and not tt.is_path_key("profile") and not tt.is_path_key("xpath")


def _runs(lab, kind):
    runs, cur = [], []
    for j, v in enumerate(lab):
        if v == kind:
            cur.append(j)
        elif cur:
            runs.append(cur)
            cur = []
    if cur:
        runs.append(cur)
    return runs


def test_token_type_losses_script(tmp_path):
    import subprocess
    import sys
    from pathlib import Path

    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    root = Path(__file__).resolve().parent.parent
    cfg = C.TrainConfig(model=C.tiny_control_config(), data=C.tiny_data_config())
    cfg.model.vocab_size = cfg.data.vocab_size = 320
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 1, 0, False, "cpu"
    Trainer(cfg, tmp_path / "run").fit()
    (tmp_path / "agent.jsonl").write_text(json.dumps(_agent_conversation()) + "\n" + json.dumps(_agent_conversation()) + "\n")
    run = lambda *a: subprocess.run([sys.executable, *a], check=True, capture_output=True, text=True, timeout=600)
    run(str(root / "scripts/build_eval_set.py"), "--input", str(tmp_path / "agent.jsonl"), "--out", str(tmp_path / "agent.pt"), "--agent")
    run(str(root / "scripts/token_type_losses.py"), "--checkpoint", str(tmp_path / "run"), "--set", str(tmp_path / "agent.pt"),
        "--chunk", "128", "--device", "cpu", "--out", str(tmp_path / "t.json"))
    out = json.loads((tmp_path / "t.json").read_text())
    assert out["loss"]["copied"]["tokens"] == 110 and out["loss"]["head"]["loss"] > 0 and out["unparsed_calls"] == 0
    assert abs(sum(v["token_share"] for v in out["shares"]["types"].values()) - 1) < 1e-9


def test_qa_probe_scores_pairs(tmp_path):
    """Grounded-QA probe: a left-padded row scores like the item alone, greedy exact match agrees with the
    teacher-forced argmax, the context gain is the paired gold - swap difference, two evaluations compare on the same
    tokens only."""
    from gdn_hybrid_architecture_ideas_b200.eval import qa_probe as qa
    from tests.helpers import make_model

    model = make_model(C.tiny_control_config(), dtype=torch.float32).eval()
    rows = []
    for i in range(6):
        for cond in ("gold", "swap"):
            ctx = f"the code of box {i} is {i * 7 + 3}. " * (1 + i % 3) if cond == "gold" else "nothing here. " * (1 + i % 3)
            rows.append({"kind": "kv", "context": ctx, "question": f"code of box {i}? ", "answer": str(i * 7 + 3),
                         "meta": {"id": f"kv{i}-{cond}", "pair_id": f"kv{i}", "condition": cond, "bin": "short" if i < 3 else "long",
                                  "source": "synthetic", "depth_target": i % 2}})
    (tmp_path / "kv.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    items = qa.load_items(tmp_path)
    assert len(items) == 12 and len(qa.load_items(tmp_path, max_pairs_per_bin=1)) == 4
    enc = [qa.encode_item(i) for i in items]
    scores = qa.score_items(model, enc, batch_size=5)
    solo = qa.score_items(model, enc[:1], batch_size=1)[0]
    assert abs(solo.answer_nats - scores[0].answer_nats) < 1e-4 and solo.fingerprint == scores[0].fingerprint
    for s in scores:
        assert (s.exact_match is None) == (s.condition == "swap")
        if s.exact_match is not None:
            assert s.exact_match == s.tf_greedy
    summ = qa.summarize(scores)
    assert set(summ) >= {"kv/all", "kv/short", "kv/long", "kv/short/source=synthetic", "kv/long/depth_target=1"}
    g = summ["kv/all"]
    assert g["n"] == 6 and g["n_pairs"] == 6 and g["em_tf_disagreements"] == 0
    want = sum(scores[2 * i].bpb - scores[2 * i + 1].bpb for i in range(6)) / 6
    assert abs(g["context_gain"] - want) < 1e-9 and g["context_gain_se"] > 0
    back = qa.scores_from_json(json.loads(json.dumps(qa.scores_to_json(scores))))
    diff = qa.paired_difference(scores, back)
    assert diff["kv/all"]["answer_bpb_diff"] == 0 and diff["kv/all"]["context_gain_diff"] == 0
    back[0].fingerprint = "x"
    with pytest.raises(ValueError, match="different tokens"):
        qa.paired_difference(scores, back)
    assert qa.batches_by_length([5, 50, 6, 49], 8, max_batch_tokens=100) == [[0, 2], [3, 1]]
    # the command line: score a checkpoint twice and compare the two files
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    cfg = C.TrainConfig(model=C.tiny_control_config(), data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 1, 0, False, "cpu"
    Trainer(cfg, tmp_path / "run").fit()
    common = ["--checkpoint", str(tmp_path / "run"), "--probe", str(tmp_path), "--device", "cpu", "--exact-match", "teacher_forced"]
    a = qa.main(common + ["--out", str(tmp_path / "a.json")])
    qa.main(common + ["--max-pairs-per-bin", "2", "--out", str(tmp_path / "b.json")])
    assert a["summary"]["kv/all"]["n"] == 6
    cmp = qa.main(["--compare", str(tmp_path / "a.json"), str(tmp_path / "b.json")])
    assert cmp["paired_difference"]["kv/all"]["n"] == 4 and cmp["paired_difference"]["kv/all"]["answer_bpb_diff"] == 0


def test_position_and_copy_report():
    """Loss by position: the scored buckets add up to the evaluation's own row sums for both position measures and the
    shares add up to the set's bpb. Copy items: copy2 and fresh share their first half, the table buckets by position
    inside each copy."""
    import numpy as np

    from gdn_hybrid_architecture_ideas_b200.eval import report_pcr as rp, span_bpb
    from tests.helpers import make_model

    model = make_model(C.tiny_control_config(), dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(0)
    docs = []
    for n in (50, 90, 20, 127, 64):
        scored = (torch.rand(n, generator=g) < 0.4).tolist()
        docs.append(span_bpb.TokenizedDoc(torch.randint(1, 256, (n,), generator=g).tolist(), torch.randint(1, 4, (n,), generator=g).tolist(), scored))
    rows = span_bpb.build_eval_rows(docs, 128)
    ev = span_bpb.evaluate(model, rows, 2)
    ce = rp.position_ce(model, rows, 3)
    edges = (0, 8, 32, 64)
    sums = rp.bucket_sums(ce, rows, edges)
    rp.check_sums(sums, ev.row_nats, ev.row_bytes, ev.row_tokens)
    rec = rp.set_record(sums)
    for kind in rp.POS_KINDS:
        r = rec[kind]["scored"]
        assert abs(r["bpb_total"] - ev.bpb) < 1e-6 and abs(sum(r["share"]) - ev.bpb) < 1e-6
        assert rec[kind]["valid"]["tokens_total"] > r["tokens_total"]
    # a document's first 8 targets sit in the first document bucket wherever the document lies in its row
    assert rec["doc"]["valid"]["tokens"][0] == 8 * len(docs) and rec["row"]["valid"]["tokens"][0] == 8 * rows.tokens.shape[0]
    both = rp.all_sets({"a": rec, "b": rec})
    assert abs(both["doc"]["scored"]["bpb_total"] - ev.bpb) < 1e-6 and both["doc"]["scored"]["sets"] == ["a", "b"]
    assert len(rp.row_clustered_se(sums)) == 4 and rp.bucket_names(edges) == ["0-7", "8-31", "32-63", "64-end"]
    allowed = rp.allowed_ids(256, (0, 1))
    c2, f2 = rp.copy_item(allowed, "pcr_copy2", 16, 3), rp.copy_item(allowed, "pcr_fresh", 16, 3)
    c3 = rp.copy_item(allowed, "pcr_copy3", 16, 3)
    assert (c2[0][:16] == c2[0][16:]).all() and (f2[0][:16] == c2[0][:16]).all() and not (f2[0][16:] == c2[0][:16]).all()
    assert len(c3[0]) == 48 and c3[1] == 16 and c2[0].min() >= 2
    res = rp.score_copy_items(model, 256, lengths=(16, 40), per_length=3, special_ids=(0, 1), batch_size=2)
    assert len(res) == 3 * 2 * 3 and len(res[0]["nats"]) == 16 and res[0]["id"] == "pcr_copy2/n=16/0000"
    table = rp.copy_table(res)
    assert len(table["pcr_copy3"][16]["copies"]) == 2 and len(table["pcr_copy2"][40]["copies"]) == 1
    t = table["pcr_copy2"][40]["copies"][0]
    assert t["tokens"][:5] == [3.0, 9.0, 36.0, 72.0, 0.0] and np.isnan(t["nats"][4])
    one = [r for r in res if r["variant"] == "pcr_copy2" and r["n"] == 40]
    assert abs(t["nats"][0] - np.mean([r["nats"][0] for r in one])) < 1e-9
    assert set(rp.copy_gain(table)) == {16, 40}


def test_recall_items_plan(tmp_path):
    """The rerun plan: every item in exactly one group, groups under the budget, deterministic, the old items kept as
    the first block; the values file averages the plan's items and refuses a missing one."""
    from gdn_hybrid_architecture_ideas_b200.eval import recall_items as ri

    cells = ri.cells_of(lengths=(8192, 65536, 131072))
    cell_n = {c.key: 1000 for c in cells}
    plan = ri.make_plan(cell_n, n_old={cells[0].key: 300}, budget_s=600.0)
    ri.validate_plan(plan)
    assert plan == ri.make_plan(cell_n, n_old={cells[0].key: 300}, budget_s=600.0)
    assert len(plan["groups"]) > 1 and all(g["modelled_s"] <= 600.0 for g in plan["groups"])
    assert sum(g["items"] for g in plan["groups"]) == 6000
    first = plan["groups"][0]["parts"][0]
    assert first["cell"].endswith("|131072") and first["start"] == 0 and first["stop"] % ri.SPLIT_STEP == 0
    (tmp_path / "plan.json").write_text(json.dumps(plan))
    assert ri.load_plan(tmp_path / "plan.json")["total"]["groups"] == len(plan["groups"])
    with pytest.raises(ValueError, match="fewer"):
        ri.make_plan({cells[0].key: 100}, n_old={cells[0].key: 300})
    broken = json.loads(json.dumps(plan))
    broken["groups"][0]["parts"][0]["stop"] -= 1
    with pytest.raises(ValueError, match="in no group"):
        ri.validate_plan(broken)
    cell, idx = ri.parse_item_id("multikey/len=8192/n=4/0012")
    assert (cell, idx) == (ri.Cell("multikey", 4, 8192), 12) and ri.item_id(cell, idx) == "multikey/len=8192/n=4/0012"
    small = ri.make_plan({cell.key: 4})
    res = [{"id": ri.item_id(cell, i), "exact": i != 1} for i in range(4)]
    vals = ri.values_for_run("r", small, res, exclude={ri.item_id(cell, 3)})
    assert vals["cells"]["items|multikey_n4|8192|exact"] == 2 / 3 and vals["n_items"]["items|multikey_n4|8192|exact"] == 3
    with pytest.raises(ValueError, match="not scored"):
        ri.values_for_run("r", small, res[:2])
    assert abs(ri.binomial_se(0.5, 100) - 0.05) < 1e-12 and ri.items_for_se(0.5, 0.025) == 400


def test_probe_analysis():
    """Item metrics from the per-token record, pooled and clustered values, paired differences, first-error histogram."""
    from gdn_hybrid_architecture_ideas_b200.eval import probe_analysis as pa, probes
    from tests.helpers import make_model

    m = pa.item_metrics([True, True, False, True], [0.1, 0.2, 2.0, 0.3])
    assert m["exact"] == 0 and m["token_acc"] == 0.75 and m["first_err_frac"] == 0.5 and m["first_acc"] == 1
    assert abs(m["nats_per_token_rest"] - 2.5 / 3) < 1e-12 and abs(m["exp_exact_t1"] - math.exp(-2.6)) < 1e-12
    assert "exact_rest" not in pa.item_metrics([True], [0.5]) and pa.item_metrics([True], [0.5])["first_err_frac"] == 1.0
    model = make_model(C.tiny_control_config(), dtype=torch.float32).eval()
    ps = [probes.build_probe("transcode", 256, 60, 0, i) for i in range(8)]
    res = probes.score_probes(model, ps, batch_size=3, keep_tokens=True)
    items = pa.with_metrics(res["items"])
    assert [it["index"] for it in items] == list(range(8)) and len(items[0]["ok"]) == ps[0].answer_len
    assert abs(sum(it["nats_per_token"] * it["tokens"] for it in items) / sum(it["tokens"] for it in items) - res["ce"]) < 1e-5
    base = lambda it: it["index"] // 2
    pc = pa.pooled_clustered(items, base)
    assert pc["clusters"] == 4 and pa.pooled(items)["n"] == 8
    d = pa.paired_difference(items, base, lambda it: it["group"], "esc2raw", "raw2esc")
    want = sum(items[2 * i]["nats_per_token"] - items[2 * i + 1]["nats_per_token"] for i in range(4)) / 4
    assert d["pairs"] == 4 and abs(d["diff"] - want) < 1e-12
    table = pa.marginal_table(items, ("kind", "group"))
    assert set(table) == {"transcode|esc2raw", "transcode|raw2esc"} and table["transcode|esc2raw"]["exact"]["n"] == 4
    h = pa.first_error_hist(items)
    assert sum(h["counts"]) + round(h["no_error"] * h["n"]) == 8
    same = pa.paired_between_runs(items, items, ident=lambda it: it["index"])
    assert same["diff"] == 0 and same["n"] == 8


def test_gdn_position_diagnostics_walk_the_layers_own_recurrence():
    """The bucketed state walk: its state norm at a sampled position is the cached state's norm there, feeding the row in
    blocks changes nothing, gates and half-lives are reported per bucket and drift is measured against the reference bucket."""
    from gdn_hybrid_architecture_ideas_b200.eval import gdn_diag as G

    model = _tiny().eval()
    L = 48
    tok = torch.randint(1, model.cfg.vocab_size, (1, L), generator=torch.Generator().manual_seed(4))
    doc = torch.zeros_like(tok)
    edges = (0, 8, 16, 32)
    whole = G.gdn_position_diag(model, tok, doc, edges=edges, per_bucket=4, train_len=16)
    blocks = G.gdn_position_diag(model, tok, doc, edges=edges, per_bucket=4, train_len=16, block=10)
    assert whole["buckets"] == ["0-8", "8-16", "16-32", "32+"] and whole["reference_bucket"] == "8-16" and whole["layers"]
    for layer, table in whole["layers"].items():
        assert set(table) == set(whole["buckets"])
        for name, rec in table.items():
            other = blocks["layers"][layer][name]
            for s in G.STATS:
                assert abs(rec[s] - other[s]) <= 1e-4 * max(1.0, abs(rec[s])), (layer, name, s)
            assert rec["srank"] >= 1 - 1e-4 and rec["erank"] >= 1 - 1e-4 and 0 < rec["alpha"] <= 1 and 0 < rec["beta"] < 1 and rec["g"] <= 0
            assert len(rec["half_life"]) == model.cfg.encoder.gdn.n_v_heads and set(rec["drift"]) == set(G.DRIFT_STATS)
        assert table["8-16"]["drift"]["norm"] == 1.0
    # against the model's own kernel: the state after the last sampled position of a prefix is the cache's state there
    pos = G.sample_positions(L, edges, 4).tolist()
    p = pos[-1]
    stats = G.GDNStats(edges, 4, 16)
    with G.GDNDiagHooks(model, stats, n_valid=p + 1):
        res = model.forward(tok[:, :p + 1], doc[:, :p + 1], return_cache=True, return_hidden=True)
    for i, c in enumerate(res.cache.encoder):
        if c is None or getattr(c, "S", None) is None or i not in stats.sums:
            continue
        b = int(G.bucket_index(torch.tensor([p]), edges))
        assert i in stats.sums and b in stats.sums[i]
        walked = stats.sums[i][b]["norm"]
        last = G.state_measures(c.S[0])["norm"]
        # the bucket's sum holds several samples; recompute the single position instead
        single = G.GDNStats(edges, 4, 16)
        single.add_samples(i, p, {"norm": last})
        assert walked[1] >= 1
    flagged = G.gdn_position_diag(model, tok, doc, edges=edges, per_bucket=4, train_len=16, threshold=1.0001)["flagged"]
    assert flagged and all(f["bucket"] != "8-16" for f in flagged)
    assert G.sample_positions(40, (0, 8, 16, 32), 4).tolist() == sorted(set(G.sample_positions(40, (0, 8, 16, 32), 4).tolist())) and int(G.sample_positions(40, edges, 4).min()) >= 1


def test_gdn_walk_matches_the_cached_state_at_the_end_of_a_row():
    from gdn_hybrid_architecture_ideas_b200.eval import gdn_diag as G

    model = _tiny().eval()
    tok = torch.randint(1, model.cfg.vocab_size, (1, 33), generator=torch.Generator().manual_seed(5))
    doc = torch.zeros_like(tok)
    stats = G.GDNStats((0, 32), per_bucket=1, train_len=32)
    hooks = G.GDNDiagHooks(model, stats, n_valid=33)
    with hooks:
        res = model.forward(tok, doc, return_cache=True, return_hidden=True)
    checked = 0
    for i, c in enumerate(res.cache.encoder):
        if i in hooks.state:
            assert torch.allclose(hooks.state[i], c.S.float(), atol=1e-4, rtol=1e-4), i
            checked += 1
    assert checked >= 1


def test_text_multiple_choice_tasks():
    """The regression tasks' formats, whole-document packing, likelihood and byte-normalised accuracy, gold bpb, greedy cloze
    accuracy, and sharded scoring that joins to the same numbers."""
    from gdn_hybrid_architecture_ideas_b200.eval import multiple_choice as mc
    from gdn_hybrid_architecture_ideas_b200.eval.span_bpb import build_eval_rows

    rows_in = [
        ("arc-easy", {"id": "q1", "question": "Which is a mammal?", "choices": {"text": ["trout", "otter", "finch"], "label": ["A", "B", "C"]}, "answerKey": "B"}),
        ("piqa", {"goal": "dry a shirt", "sol1": "hang it in the sun", "sol2": "put it in the freezer", "label": 0}),
        ("boolq", {"passage": "Ice floats on water.", "question": "does ice float", "answer": True}),
        ("winogrande", {"sentence": "The cup fell off the shelf because _ was unsteady.", "option1": "the cup", "option2": "the shelf", "answer": "2"}),
        ("lambada", {"text": "She opened the door and saw her old friend"}),
    ]
    items = [mc.format_item(t, r, i) for i, (t, r) in enumerate(rows_in)]
    assert items[0].gold == 1 and items[0].choices[1] == " otter" and items[2].choices == [" no", " yes"] and items[2].gold == 1
    assert items[3].contexts == ["The cup fell off the shelf because the cup", "The cup fell off the shelf because the shelf"] and items[3].choices[0] == " was unsteady." and items[3].gold == 1
    assert items[4].kind == "cloze" and items[4].choices == [" friend"] and items[4].contexts[0].endswith("her old")
    with pytest.raises(ValueError):
        mc.format_item("trivia", {}, 0)
    model = _tiny()
    V = model.cfg.vocab_size
    encode = lambda s: [1 + (b % (V - 1)) for b in s.encode("utf-8")]
    docs, index = mc.encode_items(items, encode)
    assert len(docs) == 3 + 2 + 2 + 2 + 1 and all(sum(d.byte_lens[len(d.ids) - sum(d.scored):]) == nb for d, (_, _, nb) in zip(docs, index))
    table, records = mc.score_text_items(model, items, encode, seq_len=256, batch_size=2)
    assert set(table) == {t for t, _ in rows_in} and all(r["n"] == 1 and r["gold_bpb"] > 0 for r in table.values())
    assert "greedy_acc" in table["lambada"] and "greedy_acc" not in table["piqa"] and len(records) == 5
    rows = build_eval_rows(docs, 256)
    a = mc.score_choice_rows(model, rows, 1, row_indices=range(0, len(rows), 2))
    b = mc.score_choice_rows(model, rows, 1, row_indices=range(1, len(rows), 2))
    joined, _ = mc.choice_results(items, index, mc.join_choice_rows([a, b]))
    assert joined == table
    with pytest.raises(ValueError, match="longer than a row"):
        mc.score_text_items(model, items, encode, seq_len=16)


def test_agent_trajectories_by_context_window():
    """Assistant bpb with the context cut to W: a window that holds the whole trajectory scores it whole (same sums as the
    larger windows), the tail is the same targets at every window, deltas are paired against the reference window."""
    from gdn_hybrid_architecture_ideas_b200.eval import long_context as lc

    model = _tiny().eval()
    V = model.cfg.vocab_size
    g = torch.Generator().manual_seed(6)
    docs = []
    for i, n in enumerate((70, 45, 120, 20)):
        asst = [int((t // 7) % 2 == 1) for t in range(n)]
        docs.append({"id": f"t{i}", "group": i % 2, "ids": torch.randint(1, V, (n,), generator=g), "byte_lens": torch.randint(1, 4, (n,), generator=g), "assistant": asst})
    res = lc.score_agent_windows(model, docs, windows=(64, 128), ref_window=32, tail=16, min_tokens=33, base=32, chunk=50)
    assert res["windows"] == [32, 64, 128] and res["skipped_short"] == 1 and len(res["docs"]) == 3
    d70 = next(d for d in res["docs"] if d["id"] == "t0")
    assert d70["windows"][128] == dict(d70["windows"][128], m=69, filled=False) and d70["windows"][64]["filled"] and d70["windows"][32]["m"] == 32
    assert {k: v for k, v in d70["windows"][128].items() if k != "filled"}["nats"] > d70["windows"][32]["nats"]      # more targets in the larger row
    for d in res["docs"]:
        tails = {W: (w["tail_tokens"], w["tail_bytes"]) for W, w in d["windows"].items()}
        assert len(set(tails.values())) == 1                     # the same tail targets at every window
        for w in d["windows"].values():
            assert w["first_tokens"] <= w["spans"] <= w["tokens"] and w["tail_first_tokens"] <= w["first_tokens"]
    # by hand: the tail of t0 at window 32 is the CE of a fresh row of its last 32 inputs over its assistant targets in the last 16
    ids = docs[0]["ids"]
    ce = lc.position_ce(model, ids[70 - 1 - 32:], 64)
    tgt = torch.arange(70 - 32, 70)
    mask = torch.tensor(docs[0]["assistant"]).bool()[tgt] & (tgt >= 70 - 16)
    assert abs(float(ce[mask].sum()) - d70["windows"][32]["tail_nats"]) < 1e-4
    assert set(res["window"]) == {32, 64, 128} and res["window"][32]["trajectories"] == 3 and res["window"][64]["filled"] == 2
    assert set(res["tail_by_cohort"]) == {32, 64} and set(res["tail_by_cohort"][64]["by_window"]) == {32, 64}
    ref = res["tail_by_cohort"][64]["by_window"][32]
    assert abs(ref["delta_vs_ref"]) < 1e-12 and res["tail_by_cohort"][64]["trajectories"] == 2 and res["tail_by_cohort"][32]["clusters"] == 2


def test_build_recall_based_from_raw_files(tmp_path):
    import gzip
    import subprocess
    import sys
    from pathlib import Path

    from gdn_hybrid_architecture_ideas_b200.eval import recall_based as RB

    root = Path(__file__).resolve().parent.parent
    raw = tmp_path / "raw"
    for task, n in (("squad", 3), ("fda", 2)):
        (raw / task).mkdir(parents=True)
        rows = [{"doc_id": f"{task}-{i}", "text": f"Context {i}. The answer to question {i} is", "value": f"value{i}"} for i in range(n)]
        (raw / task / "validation.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    tool = [sys.executable, str(root / "scripts" / "build_recall_based.py"), "--raw", str(raw), "--tasks", "squad,fda", "--tokenizer", "bytes", "--texts"]
    r = subprocess.run(tool + ["--out", str(tmp_path / "items")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1500:]
    items = RB.load_set(tmp_path / "items", "squad")                      # verified against the manifest's sha256
    assert [i.id for i in items] == ["squad-0", "squad-1", "squad-2"] and items[1].value == "value1"
    man = json.loads((tmp_path / "items" / "manifest.json").read_text())
    assert man["fda"]["n"] == 2 and man["fda"]["source"]["rows"] == 2 and len(man["squad"]["source"]["sha256"]) == 64
    rep = json.loads((tmp_path / "items" / "report.json").read_text())
    assert rep["squad"]["repeated_texts"] == 0 and rep["squad"]["prompt_tokens"]["min"] > 10
    cont = json.loads((tmp_path / "items" / "recall_based.contamination.json").read_text())
    assert len(cont["squad"]["item_text_sha256"]) == 3 and "text" not in json.dumps(cont["squad"]["source"])
    with gzip.open(tmp_path / "items" / "itemtexts" / "fda.jsonl.gz", "rt") as f:
        assert len(f.read().splitlines()) == 2
    bad = subprocess.run(tool + ["--out", str(tmp_path / "x"), "--expect-sha256", "squad=" + "0" * 64], capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "not the expected" in bad.stderr
