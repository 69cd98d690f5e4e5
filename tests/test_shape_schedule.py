"""Batch-shape schedule: the closed form equals the slow walk, a scheduled run reads the unscheduled run's tokens in the
same order, trains its extra optimizer steps with the LR read at the token clock, and resumes bit for bit."""

import copy

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.data import make_data
from gdn_hybrid_architecture_ideas_b200.data.synthetic import short_rows
from gdn_hybrid_architecture_ideas_b200.train.shape_schedule import ShapeSchedule, reference_walk
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer


def test_closed_form_equals_the_walk():
    phases = [[0.25, 2, 16], [0.5, 4, 16], [0.75, 4, 32]]
    sched = ShapeSchedule(phases, 8, 4, 32)
    walk = reference_walk(phases, 8, 4, 32)
    assert sched.total_steps == len(walk)
    for k, (rows, length, first_token) in enumerate(walk):
        sh = sched.at(k)
        assert (sh.rows, sh.seq_len, sh.first_row * sh.seq_len) == (rows, length, first_token)
        assert sh.clock == pytest.approx(first_token / (4 * 32))


def test_short_rows_cut_the_base_rows_in_order():
    dcfg = C.tiny_data_config(seq_len=32, batch_size=4)
    data = make_data(dcfg, 256)
    base = data.rows(3, 2)
    cut = short_rows(data, 3 * 4, 8, 8, 32)
    seq = torch.cat([base.tokens, base.targets[:, -1:]], 1)
    for i in range(8):
        r, j = i // 4, i % 4
        assert torch.equal(cut.tokens[i], seq[r, j * 8:j * 8 + 8]) and torch.equal(cut.targets[i], seq[r, j * 8 + 1:j * 8 + 9])
    assert torch.equal(short_rows(data, 5, 3, 32, 32).tokens, data.rows(5, 3).tokens)


def _cfg(**kw):
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config(seq_len=32, batch_size=4), steps=4, seed=3)
    cfg.optim.warmup_steps, cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.head_impl, cfg.log_every, cfg.device = 2, 0, False, "fused", 0, "cpu"
    cfg.shape_schedule = [[0.5, 2, 16]]
    for k, v in kw.items():
        C.apply_override(cfg, f"{k}={v}")
    return cfg


def test_scheduled_run_trains_and_resumes(tmp_path):
    cfg = _cfg()
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    assert a.total_steps == 2 * 4 + 2          # two reference steps as 4 optimizer steps each (2 x 16 of 4 x 32 tokens), then two plain steps
    shapes = []
    for _ in range(a.total_steps):
        b = a.batch_at(a.step)
        shapes.append(tuple(b.tokens.shape))
        a.train_step()
    assert shapes == [(2, 16)] * 8 + [(4, 32)] * 2
    # the LR is the unscheduled schedule read at the tokens seen
    plain = Trainer(_cfg(shape_schedule=[]), None)
    assert a.lr_at(8) == plain.lr_at(2) and a.lr_at(0) == plain.lr_at(0)
    assert plain.lr_at(0) < a.lr_at(2) < plain.lr_at(1)          # half a reference step into the warm-up
    rows_mode = Trainer(_cfg(shape_lr="rows"), None)
    assert rows_mode.lr_at(1) == pytest.approx(plain.lr_at(0) / 4)
    # a stop inside the first phase resumes into the same run
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=3)
    b.save_checkpoint()
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    wa, wc = a.model.state_dict(), c.model.state_dict()
    assert all(torch.equal(wa[k], wc[k]) for k in wa)


def test_refused_combinations():
    with pytest.raises(ValueError, match="shape_schedule"):
        Trainer(_cfg(**{"tst.schedule": [[0, 2], [2, 1]]}), None)
    with pytest.raises(ValueError, match="divide"):
        Trainer(_cfg(shape_schedule=[[0.5, 3, 16]]), None)
