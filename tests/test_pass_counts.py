"""Pass counts by segment: the position labelling against the reference's, generated flags from the stream, the scheduler's
counts, the scheduled passes of the model against the reference, and a training step."""

import copy

import numpy as np
import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.data import chat_format as CF
from gdn_hybrid_architecture_ideas_b200.models import build_model, pass_counts as PC
from tests.helpers import random_rows

CONV = {"tools": [{"name": "run"}], "messages": [
    {"role": "system", "content": "sys"}, {"role": "user", "content": "do it"},
    {"role": "assistant", "reasoning": "think hard", "content": "I will run.",
     "tool_calls": [{"name": "run", "arguments": {"cmd": "ls -la"}}, {"name": "view", "arguments": {"path": "a/b.py"}}]},
    {"role": "tool", "content": "file1\nfile2"}, {"role": "assistant", "content": "Done: two files."},
    {"role": "user", "content": "thanks"}, {"role": "assistant", "content": "", "tool_calls": [{"name": "finish", "arguments": {}}]}]}


def encoded():
    chat = CF.ChatTokenizer()
    ids, gen = chat.encode_pieces(CF.pieces(CONV))
    return chat, np.array(ids), np.array(gen)


def test_position_segments_follow_the_message_structure():
    chat, ids, gen = encoded()
    seg = PC.position_segments(ids, gen, chat.table, chat.control)
    text = lambda sel: b"".join(chat.table[i] for i in ids[1:][sel[:-1]]).decode()          # noqa: E731  the NEXT tokens of the selected positions
    assert "think hard" in text(seg == PC.REASONING) and "</think>" in text(seg == PC.REASONING) and "I will run." in text(seg == PC.CONTENT)
    assert text(seg == PC.CALL_HEAD).count('"name": "') == 3 and "ls -la" in text(seg == PC.CALL_BODY) and "ls -la" not in text(seg == PC.CALL_HEAD)
    assert (seg[:-1][~gen[1:]] == PC.OTHER).all() and (seg[:-1][gen[1:]] != PC.OTHER).all() and seg[-1] == PC.OTHER
    assert np.array_equal(PC.stream_flags(ids, chat.table, chat.control), gen)
    # prefix-only: replacing the tokens after t changes nothing before or at t (given the flag of t + 1)
    for t in (40, 120, 200):
        other = ids.copy()
        other[t + 2:] = chat.table.index(b"x")
        assert np.array_equal(PC.position_segments(other, gen, chat.table, chat.control)[:t + 1], seg[:t + 1])
    cut = len(ids) // 2                          # a piece that opens inside a message: its first run cannot be placed
    assert gen[cut] and PC.position_segments(ids[cut:], gen[cut:], chat.table, chat.control)[0] == PC.OTHER
    assert not PC.stream_flags(ids[cut:], chat.table, chat.control)[:5].any()


def test_position_segments_equal_the_reference(reference):
    from ced.eval import token_types as RT

    chat, ids, gen = encoded()
    ref_ids = np.array([RT.ID[chat.table[i].decode()] if i >= 256 else RT.N_SPECIAL + i for i in ids])
    table = RT.TokenTable([s.encode() for s in RT.cf.SPECIAL_TOKENS] + [bytes([b]) for b in range(256)])
    to_mine = {RT.SEG["reasoning"]: PC.REASONING, RT.SEG["content"]: PC.CONTENT, RT.SEG["call_head"]: PC.CALL_HEAD, RT.SEG["call_body"]: PC.CALL_BODY,
               RT.SEG["unplaced"]: PC.OTHER, -1: PC.OTHER}
    for lo in (0, len(ids) // 2, len(ids) // 3):
        want = np.array([to_mine[int(s)] for s in RT.segment_positions(ref_ids[lo:], gen[lo:], table)])
        assert np.array_equal(PC.position_segments(ids[lo:], gen[lo:], chat.table, chat.control), want)


def test_schedule_and_scheduler_counts():
    lp = C.LoopConfig()
    assert PC.schedule_of(lp) is None
    lp.t_max, lp.segment_passes = 2, {"reasoning": 3, "other": 1}
    sched = PC.schedule_of(lp)
    assert sched.counts == {"reasoning": 3, "call_head": 2, "content": 2, "call_body": 2, "other": 1} and PC.built_passes(lp) == 3
    for bad, match in (({"thinking": 2}, "unknown segment"), ({"reasoning": 4}, "1, 2 or 3"), ([2], "a map")):
        lp.segment_passes = bad
        with pytest.raises(ValueError, match=match):
            PC.schedule_of(lp)
    lp.segment_passes, lp.unscored_passes = None, 2
    with pytest.raises(ValueError, match="unscored_passes"):
        PC.schedule_of(lp)
    chat, ids, gen = encoded()
    sch = PC.PassScheduler.from_tokenizer(sched, "bytes")
    row = torch.tensor(np.concatenate([ids, ids[:50]]))[None]
    doc = torch.cat([torch.zeros(len(ids), dtype=torch.long), torch.ones(50, dtype=torch.long)])[None]
    counts = sch.counts(row, doc)
    seg = PC.position_segments(ids, gen, chat.table, chat.control)
    assert counts.shape == row.shape and torch.equal(counts[0, :len(ids)], torch.from_numpy(sched.table()[seg]))
    assert torch.equal(counts[0, len(ids):], counts[0, :50]) or int(counts[0, len(ids) + 49]) == 1          # the second document is labelled on its own
    assert set(counts.unique().tolist()) == {1, 2, 3}
    un = PC.PassScheduler(PC.PassSchedule(sched.counts, 1, 2), chat.table, chat.control)
    scored = torch.zeros_like(row, dtype=torch.bool)
    scored[0, 100:140] = True
    masked = un.counts(row, doc, scored=scored)
    assert torch.equal(masked[0, 100:140], counts[0, 100:140]) and int(masked[0, :100].max()) == 1


@pytest.mark.parametrize("segments,unscored", [({"reasoning": 3, "content": 2, "call_head": 1, "call_body": 2, "other": 1}, None), ({"reasoning": 2, "other": 1}, None), (None, 1)])
def test_scheduled_passes_equal_the_reference(reference, segments, unscored):
    import ced.config as RC
    from ced.model.control import build_model as ref_build

    cfg = C.tiny_control_config()
    lp = cfg.loop
    lp.pass2_gate, lp.pass2_layers, lp.t_max, lp.t_eval, lp.t_choices, lp.t_probs, lp.segment_passes, lp.unscored_passes = "scalar", 6, 2, 2, [2], [1.0], segments, unscored
    torch.manual_seed(0)
    mine = build_model(cfg).double()
    torch.manual_seed(0)
    theirs = ref_build(RC.from_dict(RC.ModelConfig, C.to_dict(cfg))).double()
    assert list(mine.state_dict()) == list(theirs.state_dict()) and mine.n_passes == (3 if segments and 3 in segments.values() else 2)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    mine.load_state_dict(theirs.state_dict())
    tok, doc = random_rows(2, 40)
    counts = torch.randint(1, mine.n_passes + 1, (2, 40), generator=g)
    a, b = mine(tok, doc, pass_counts=counts), theirs(tok, doc, pass_counts=counts)
    assert (a.logits - b.logits).abs().max() < 1e-10 and torch.equal(a.kept, b.kept) and torch.equal(a.kept, counts >= 2)
    ga = torch.autograd.grad(a.logits.logsumexp(-1).sum(), list(mine.parameters()), allow_unused=True)
    gb = torch.autograd.grad(b.logits.logsumexp(-1).sum(), list(theirs.parameters()), allow_unused=True)
    for (n, _), x, y in zip(mine.named_parameters(), ga, gb):
        assert (x is None) == (y is None) and (x is None or (x - y).abs().max() < 1e-9), n
    ones = mine(tok, doc, pass_counts=torch.ones_like(counts)).logits
    assert torch.equal(ones, mine(tok, doc, T=1).logits)                                    # every position at one pass: pass 1 alone
    mine.eval(), theirs.eval()
    with torch.no_grad():
        full = mine(tok, doc, pass_counts=counts).logits
        out, ref_out = mine.prefill(tok[:, :17], doc[:, :17], pass_counts=counts[:, :17]), theirs.prefill(tok[:, :17], doc[:, :17], pass_counts=counts[:, :17])
        parts = [out.logits]
        for lo, hi in ((17, 18), (18, 40)):
            out = mine.extend(tok[:, lo:hi], doc[:, lo:hi], None, out.cache, pass_counts=counts[:, lo:hi])
            ref_out = theirs.extend(tok[:, lo:hi], doc[:, lo:hi], None, ref_out.cache, pass_counts=counts[:, lo:hi])
            parts.append(out.logits)
            assert (out.logits - ref_out.logits).abs().max() < 1e-10
        assert (torch.cat(parts, 1) - full).abs().max() < 1e-9
        mask = torch.zeros(2, 40, dtype=torch.bool)
        mask[:, 25:] = True
        a, b = mine(tok, doc, pass_counts=counts, pass2_mask=mask), theirs(tok, doc, pass_counts=counts, pass2_mask=mask)
        assert (a.logits - b.logits)[mask].abs().max() < 1e-10 and torch.equal(a.kept, b.kept) and not a.kept[:, :25].any()
        with pytest.raises(ValueError, match="pass_counts"):
            mine.extend(tok[:, :2], doc[:, :2], None, out.cache)
        with pytest.raises(ValueError, match="pass2_capacity"):
            mine(tok, doc, pass_counts=counts, pass2_mask=mask, pass2_capacity=3)
        with pytest.raises(ValueError, match="integers from 1"):
            mine(tok, doc, pass_counts=counts + 3)


def test_a_scheduled_model_trains_on_chat_tokens_with_its_own_counts(tmp_path):
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    cfg = C.TrainConfig(model=C.tiny_control_config(), data=C.tiny_data_config(seq_len=48, batch_size=4), steps=4, seed=3)
    cfg.model.vocab_size = 272
    lp = cfg.model.loop
    lp.pass2_gate, lp.pass2_layers, lp.t_max, lp.t_eval, lp.t_choices, lp.t_probs = "scalar", 4, 2, 2, [2], [1.0]
    lp.segment_passes, lp.unscored_passes, lp.segment_tokenizer = {"reasoning": 3, "other": 1}, 1, "bytes"
    cfg.log_every, cfg.metrics_jsonl = 1, False
    t = Trainer(copy.deepcopy(cfg), None)
    names = [n for g in t.optimizer.groups for n in g["names"]] if hasattr(t.optimizer, "groups") else []
    assert t.model.n_passes == 3 and "hyper_connections.pass3_gate" in dict(t.model.named_parameters())
    m = t.train_step()
    assert m["T"] == 2 and abs(sum(m["pass_counts"].values()) - 1) < 1e-6 and m["pass_counts"]["1"] == 1.0         # random tokens hold no assistant header: every position is "other"
    chat = CF.ChatTokenizer()
    ids, _ = chat.encode_pieces(CF.pieces(CONV))
    row = torch.tensor(ids[:200])[None]
    out = t.model(row, torch.zeros_like(row))
    assert set(t.model.last_counts.unique().tolist()) == {1, 2, 3} and torch.equal(out.kept.cpu(), t.model.last_counts >= 2)
    off = copy.deepcopy(cfg)
    off.model.loop.pass2_gate, off.model.loop.pass2_layers = "none", 0
    with pytest.raises(ValueError, match="this model has none"):
        Trainer(off, None)
