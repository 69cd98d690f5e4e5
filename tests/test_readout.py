"""The exact-match readout inside training: fixed sample, records, no effect on training, resumed runs, failures."""

import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.train import readout as R
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def probe_file(tmp_path_factory):
    out = tmp_path_factory.mktemp("probes") / "probes.pt"
    vocab = C.tiny_full_config().vocab_size
    r = subprocess.run([sys.executable, str(ROOT / "scripts/build_probes.py"), "--vocab", str(vocab), "--lengths", "48", "--kinds", "needle,copy,mf_chain",
                        "--per-kind", "3", "--out", str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return out


def train_cfg(probe_file, every):
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 4, 0, True, "cpu"
    cfg.eval.readout_every, cfg.eval.readout_sets, cfg.eval.readout_batch_tokens = every, [[str(probe_file), "*", 2]], 128
    return cfg


def records(run_dir, event):
    return [json.loads(x) for x in (Path(run_dir) / "metrics.jsonl").read_text().splitlines() if json.loads(x).get("event") == event]


def test_readout_records_and_leaves_training_alone(tmp_path, probe_file):
    on = Trainer(train_cfg(probe_file, 2), tmp_path / "on")
    on.fit()
    off_cfg = train_cfg(probe_file, 0)
    off = Trainer(off_cfg, tmp_path / "off")
    off.fit()
    for (k, a), (_, b) in zip(on.model.state_dict().items(), off.model.state_dict().items()):
        assert torch.equal(a, b), k                              # bit for bit the same training
    recs = records(tmp_path / "on", "readout")
    assert [r["step"] for r in recs] == [2, 4] and not records(tmp_path / "off", "readout")
    r = recs[0]
    label = f"{probe_file.parent.name}/{probe_file.stem}"
    assert r["items"] == 6 and set(r["rows"]) == {f"{label}/needle@48", f"{label}/copy@48", f"{label}/mf_chain@48"} and r["sample"] == recs[1]["sample"]
    assert all(v["n"] == 2 and 0.0 <= v["exact"] <= 1.0 and v["logp"] < 0 for v in r["rows"].values())
    assert abs(r["exact"] - sum(v["exact"] for v in r["rows"].values()) / 3) < 1e-6
    # the first items of each cell, in file order: what the offline scorer scores first
    blob = torch.load(probe_file, weights_only=False)
    first_needles = [p["ids"] for p in blob["probes"] if p["kind"] == "needle"][:2]
    assert [p.ids for row in on._probe_readout.rows if row["row"].endswith("needle@48") for p in row["probes"]] == first_needles


def test_a_resumed_run_scores_no_step_twice(tmp_path, probe_file):
    cfg = train_cfg(probe_file, 2)
    cfg.ckpt_every_steps = 2
    a = Trainer(copy.deepcopy(cfg), tmp_path / "run")
    a.fit(until_step=2) if "until_step" in Trainer.fit.__code__.co_varnames else a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "run")
    assert b.resume_from_checkpoint()
    b.fit()
    steps = [r["step"] for r in records(tmp_path / "run", "readout")]
    assert sorted(steps) == sorted(set(steps)) and 4 in steps and 2 in steps


def test_bad_samples_stop_the_run_before_it_trains_and_scoring_errors_do_not(tmp_path, probe_file):
    cfg = train_cfg(probe_file, 2)
    cfg.eval.readout_sets = [[str(tmp_path / "missing.pt"), "*", 2]]
    with pytest.raises(FileNotFoundError):
        Trainer(cfg, tmp_path / "x")
    cfg.eval.readout_sets = [[str(probe_file), "*", 50]]
    with pytest.raises(ValueError, match="fewer than 50"):
        Trainer(cfg, tmp_path / "x")
    cfg.eval.readout_sets = [[str(probe_file), ["needle"]]]
    with pytest.raises(ValueError, match="items per cell"):
        Trainer(cfg, tmp_path / "x")
    cfg.eval.readout_sets, cfg.eval.readout_every = [], 2
    with pytest.raises(ValueError, match="nothing to score"):
        Trainer(cfg, tmp_path / "x")
    t = Trainer(train_cfg(probe_file, 1), tmp_path / "y")
    t._probe_readout.rows[0]["probes"][0].ids.append(10 ** 9)          # an id outside the vocabulary: scoring raises
    t.fit()
    assert t.step == 4 and len(records(tmp_path / "y", "readout_failed")) == 1 and not records(tmp_path / "y", "readout")


def test_cells_can_be_chosen_by_name_and_batches_respect_the_token_budget(probe_file):
    rows = R.load_sample(R.parse_sets([[str(probe_file), ["copy"], 3]]), 10 ** 6)
    assert [r["row"] for r in rows] == [f"{probe_file.parent.name}/{probe_file.stem}/copy@48"] and len(rows[0]["probes"]) == 3
    with pytest.raises(ValueError, match="larger vocabulary|vocabulary of"):
        R.load_sample(R.parse_sets([[str(probe_file), "*", 1]]), 4)
    items = rows[0]["probes"]
    longest = max(len(p.ids) for p in items)
    assert [len(b) for b in R.batches_by_tokens(items, 2 * longest)] == [2, 1] and [len(b) for b in R.batches_by_tokens(items, 1)] == [1, 1, 1]
    assert R.readout_due(train_cfg(probe_file, 3), 3) and R.readout_due(train_cfg(probe_file, 3), 4) and not R.readout_due(train_cfg(probe_file, 3), 2)


def test_a_model_with_a_second_pass_is_scored_at_one_pass_and_at_two(tmp_path, probe_file):
    """The readout of a gated second pass: both pass counts on the same items, gaps paired by item, a record at the switch
    step; before the gate leaves zero the two pass counts are one function (gap 0); the numbers are the scorer's own."""
    from gdn_hybrid_architecture_ideas_b200.eval import probes

    cfg = train_cfg(probe_file, 4)
    cfg.model = C.tiny_control_config()
    lp = cfg.model.loop
    lp.pass2_gate, lp.pass2_layers, lp.t_max, lp.t_eval, lp.t_choices, lp.t_probs = "scalar", 4, 2, 2, [2], [1.0]
    cfg.steps, cfg.loop_switch_step, cfg.optim.pass2_lr_scale, cfg.activation_checkpoint = 8, 2, 50.0, "layer"
    t = Trainer(cfg, tmp_path / "g")
    t.fit()
    recs = records(tmp_path / "g", "readout")
    assert [r["step"] for r in recs] == [2, 4, 8] and all(r["passes"] == [1, 2] for r in recs)
    at_switch, last = recs[0], recs[-1]
    assert at_switch["gap"] == {"mean": 0.0, "se": 0.0} and at_switch["gap_logp"] == {"mean": 0.0, "se": 0.0} and at_switch["logp"]["1"] == at_switch["logp"]["2"]
    assert last["gap_logp"]["mean"] != 0.0 and last["gap_logp"]["se"] > 0 and set(last["exact"]) == {"1", "2"}
    row = next(iter(t._probe_readout.rows))
    t.model.eval()
    by_pass = [probes.score_probes(t.model, row["probes"], batch_size=len(row["probes"]), passes=p) for p in (1, 2)]
    got = last["rows"][row["row"]]
    diffs = [-(b["ce"]) + a["ce"] for a, b in zip(by_pass[0]["items"], by_pass[1]["items"])]
    assert abs(got["gap_logp"]["mean"] - sum(diffs) / len(diffs)) < 1e-5 and got["exact"] == [round(s["exact"], 6) for s in by_pass]
    assert abs(last["gap"]["mean"] - sum(v["gap"]["mean"] for v in last["rows"].values()) / len(last["rows"])) < 1e-6
    assert R.paired_gap([1.0, 0.0, 1.0], [0.0, 0.0, 1.0]) == {"mean": 0.333333, "se": 0.333333} and R.paired_gap([2.0], [1.0]) == {"mean": 1.0, "se": 0.0}
    assert R.pooled_gap([{"mean": 0.2, "se": 0.3}, {"mean": 0.4, "se": 0.4}]) == {"mean": 0.3, "se": 0.25}
