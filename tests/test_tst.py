"""Token-superposition training: a bag size of 1 is plain training bit for bit, every base row of the data is read
exactly once and in order across the switches, a stop on either side of a switch resumes into the uninterrupted run,
the switch's options act as documented, and two data-parallel ranks equal one process."""

import copy
import math

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.data import make_data
from gdn_hybrid_architecture_ideas_b200.train import tst
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer


def _cfg(schedule, **kw):
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config(seq_len=24, batch_size=4), steps=6, seed=3)
    cfg.optim.warmup_steps, cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.head_impl, cfg.log_every, cfg.device = 2, 0, True, "fused", 0, "cpu"
    cfg.tst.schedule = schedule
    for k, v in kw.items():
        C.apply_override(cfg, f"{k}={v}")
    return cfg


def _weights(t):
    return {k: v.clone() for k, v in t.model.state_dict().items()}


def test_bag_size_one_is_plain_training_bit_for_bit():
    a = Trainer(_cfg([]), None)
    b = Trainer(_cfg([[0, 1]]), None)
    for _ in range(3):
        la, lb = a.train_step()["loss"], b.train_step()["loss"]
        assert la == lb
    wa, wb = _weights(a), _weights(b)
    assert all(torch.equal(wa[k], wb[k]) for k in wa)


@pytest.mark.parametrize("kind", ["synthetic", "uniform"])
def test_every_base_row_is_read_once_in_order(kind):
    dcfg = C.tiny_data_config(seq_len=16, batch_size=3)
    dcfg.kind = kind
    data = make_data(dcfg, 256)
    cfg_t = C.TSTConfig(schedule=[[0, 3], [2, 2], [4, 1]])
    plan = tst.TSTPlan(cfg_t, data, 256, 3, seed=1)
    L, at = 16, 0
    for step in range(6):
        s = plan.s_at(step)
        assert plan.schedule.rows_before(step, 3) == at
        b = plan.batch_at(step, 0, 3)
        for r in range(3):
            rows = data.rows(at + r * s, s)
            seq = torch.cat([rows.tokens, rows.targets[:, -1:]], 1).reshape(-1)        # the s base rows, whole
            if s == 1:
                assert torch.equal(b.tokens[r], rows.tokens[0]) and torch.equal(b.targets[r], rows.targets[0])
                continue
            got = torch.cat([b.tokens[r].reshape(-1), b.multi_targets[r, -1]])          # every input, then the last target bag
            assert torch.equal(got, seq)
            assert torch.equal(b.multi_targets[r, :-1], b.tokens[r, 1:])                # a position's targets are the next bag
        at += 3 * s
    # a data-parallel rank's rows are the single process's rows of the same index
    whole, part = plan.batch_at(1, 0, 3), plan.batch_at(1, 1, 2)
    assert torch.equal(whole.tokens[1:], part.tokens) and torch.equal(whole.multi_valid[1:], part.multi_valid)


def test_bag_documents_and_validity():
    dcfg = C.tiny_data_config(seq_len=16, batch_size=2)
    data = make_data(dcfg, 256)
    row = tst.bag_row(data, 5, 3)
    seq, docs = tst._row_block(data, 5, 3)
    shift = torch.cat([torch.zeros(1, dtype=torch.long), (docs[:-1, -1] + 1).cumsum(0)])
    flat_doc = (docs + shift[:, None]).reshape(-1)
    assert bool((flat_doc[1:] >= flat_doc[:-1]).all())                                  # documents never decrease along a bag row
    for j in range(16):
        assert row["doc_ids"][j] == flat_doc[3 * j + 2]                                 # a position's document: its last input token's
        for i in range(3):
            assert bool(row["multi_valid"][j, i]) == bool(flat_doc[3 * (j + 1) + i] == flat_doc[3 * j + 2])


@pytest.mark.parametrize("stop", [2, 3, 4])
def test_stop_around_the_switch_resumes_into_the_same_run(tmp_path, stop):
    cfg = _cfg([[0, 2], [3, 1]], **{"tst.gdn_conv_reinit": True, "tst.rewarm_steps": 2, "tst.bag_lr_power": 0.5})
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=stop)
    b.save_checkpoint()
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == stop
    c.fit()
    wa, wc = _weights(a), _weights(c)
    assert all(torch.equal(wa[k], wc[k]) for k in wa)
    assert '"tst_switch"' in (tmp_path / "a" / "metrics.jsonl").read_text()


def test_switch_options():
    cfg = _cfg([[0, 4], [2, 2], [4, 1]], **{"tst.gdn_decay_rescale": True, "tst.gdn_conv_reinit": True, "tst.rewarm_steps": 3, "tst.bag_lr_power": 1.0})
    t = Trainer(cfg, None)
    layers = tst.gdn_layers(t.model)
    a0 = layers[0].A_log.detach().clone()
    assert t.tst.lr_factor(0) == 4.0 and t.tst.lr_factor(2) == 2.0
    assert [t.tst.lr_factor(k) for k in (4, 5, 6, 7)] == [pytest.approx(1 / 3), pytest.approx(2 / 3), pytest.approx(1.0), None]
    for _ in range(2):
        t.train_step()
    drift = layers[0].A_log.detach().clone() - a0                        # two updates moved A_log a little
    m = t.train_step()                                                   # step 2: switch 4 -> 2
    assert m["tst_switch"]["s_from"] == 4 and m["tst_switch"]["s_to"] == 2 and "gdn_conv_reinit" not in m["tst_switch"]
    assert m["tst_switch"]["gdn_decay_rescaled"] == len(layers)
    assert torch.allclose(layers[0].A_log.detach() - a0 - drift, torch.full_like(a0, math.log(0.5)), atol=5e-2)
    t.train_step()
    w_before = layers[0].conv_weight.detach().clone()
    want = tst.conv_reinit_draws(t.model, cfg.seed, 4)[0]
    assert not torch.equal(w_before, want)
    assert t.optimizer.steps == 2                                        # moments restarted at the first switch
    m = t.train_step()                                                   # step 4: switch 2 -> 1, taps drawn again, then one update on them
    assert m["tst_switch"]["gdn_conv_reinit"] == len(layers) and t.optimizer.steps == 1
    assert (layers[0].conv_weight.detach() - want).abs().max() < 1e-2 and not torch.equal(layers[0].conv_weight.detach(), w_before)


def test_refusals():
    for key, value, match in (("tst.output_only", True, "output_only"), ("tst.aux_multi_hot", 3, "aux_multi_hot"), ("tst.bag_input", "sum_sqrt", "bag_input")):
        with pytest.raises(ValueError, match=match):
            Trainer(_cfg([[0, 2], [2, 1]], **{key: value}), None)
    with pytest.raises(ValueError, match="one of them"):
        Trainer(_cfg([[0, 2], [2, 1]], **{"tst.gdn_decay_rescale": True, "tst.gdn_resolution_gates": "E"}), None)
    with pytest.raises(ValueError, match="moments"):
        Trainer(_cfg([[0, 2], [2, 1]], **{"tst.keep_optimizer_state": True, "tst.gdn_conv_reinit": True}), None)
