"""Host-side guards that need no GPU: the benchmark's reference arm assembles its result line from a stub trainer (a
name error in its tail cannot reach a GPU run), the trainer raises when the kernel status word is set, and a
tensor-parallel Trainer started from its seed holds different slices on different ranks and checkpoints the full model."""

import copy
import importlib.util
import os
import subprocess
import sys
import types
from pathlib import Path

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200 import ops
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt
from gdn_hybrid_architecture_ideas_b200.train.trainer import KernelStatus, Trainer

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Event:
    def __init__(self, enable_timing=True):
        pass

    def record(self):
        pass

    def elapsed_time(self, other):
        return 80.0


def test_reference_arm_assembles_its_line(monkeypatch, tmp_path):
    """run_reference from import to return, with the reference package, the device and the clock sampler stubbed."""
    bench = _bench()
    pkg = tmp_path / "baseline" / "_ref" / "ced"
    (pkg / "train").mkdir(parents=True)
    (pkg / "__init__.py").write_text("")
    (pkg / "config.py").write_text("class TrainConfig: pass\ndef from_dict(cls, d):\n    return d\n")
    (pkg / "train" / "__init__.py").write_text("")
    (pkg / "train" / "data_parallel.py").write_text("def from_environment():\n    return None\n")
    (pkg / "train" / "trainer.py").write_text(
        "class Trainer:\n    def __init__(self, cfg, run_dir, dp=None):\n        self.cfg = cfg\n"
        "    def train_step(self):\n        return {'loss': 1.0}\n")
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    for name in [m for m in sys.modules if m == "ced" or m.startswith("ced.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    monkeypatch.setattr(bench, "ClockSampler", lambda enabled: types.SimpleNamespace(stop=lambda n: {"sm_mhz": 1.0, "sm_max_mhz": 1.0, "reasons": []}))
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    args = types.SimpleNamespace(rows=16, seq_len=4096, steps=4, warmup=1, gpus=1)
    monkeypatch.setattr(sys, "path", list(sys.path))          # the arm puts its package directory in front: undone with the test
    out = bench.run_reference(args)
    for name in [m for m in sys.modules if m == "ced" or m.startswith("ced.")]:
        del sys.modules[name]          # the stub package must not outlive the test (a monkeypatched deletion would be undone)
    assert out.get("impl") == "reference" and "unavailable" not in out, out
    assert out["config"]["global_batch"] == 16 and out["ms_per_step"] == 20.0
    assert out["value"] == pytest.approx(16 * 4096 / 0.020) and out["e2e"]["value"] == out["value"]


def _tiny(**kw):
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config(seq_len=48, batch_size=4), steps=4, seed=3)
    cfg.optim.warmup_steps, cfg.metrics_jsonl, cfg.head_impl, cfg.log_every, cfg.device = 2, True, "fused", 0, "cpu"
    for k, v in kw.items():
        C.apply_override(cfg, f"{k}={v}")
    return cfg


def test_status_word_stops_the_trainer(tmp_path):
    t = Trainer(_tiny(), tmp_path / "r")
    t.train_step()
    ops.status_word("cpu").fill_(401)
    try:
        with pytest.raises(KernelStatus, match="401"):
            t.train_step()
    finally:
        ops.clear_status("cpu")
    assert '"kernel_status"' in (tmp_path / "r" / "metrics.jsonl").read_text()
    t.train_step()      # the word was cleared by the raise: the next step runs


WORKER = """
import sys, os
sys.path.insert(0, {root!r})
import torch
from gdn_hybrid_architecture_ideas_b200 import config as C, ops
from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer, KernelStatus
dp = data_parallel.from_environment()
cfg = C.load_yaml(sys.argv[1])
t = Trainer(cfg, sys.argv[2], dp)
mode = sys.argv[3]
if mode == "status":
    t.train_step()
    if dp.rank == 1:
        ops.status_word("cpu").fill_(402)
    try:
        t.train_step()
        print("NO RAISE", flush=True)
    except KernelStatus as e:
        print(f"rank {{dp.rank}} raised: {{e}}", flush=True)
elif mode == "zero2":
    for _ in range(2):
        t.train_step()
    print(f"rank {{dp.rank}} early {{t.zero.early}} buckets {{len(t.zero.buckets)}}", flush=True)
else:
    # shards drawn from the full model's seed differ across ranks
    w = dict(t.model.named_parameters())
    name = next(n for n in w if n.endswith("w_gate.weight"))
    got = dp.gather_host(w[name].detach().clone())
    assert not torch.equal(got[0], got[1]), "tensor-parallel ranks hold the same slice"
    t.fit()
dp.barrier()
dp.close()
"""


def _run_worker(tmp_path, cfg, mode, port):
    C.save_yaml(cfg, tmp_path / "c.yaml")
    script = tmp_path / "w.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(script), str(tmp_path / "c.yaml"), str(tmp_path / "run"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env={**os.environ, "GHB_DP_BACKEND": "gloo", "OMP_NUM_THREADS": "2", "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stderr[-3000:]
    return r.stdout


def test_one_ranks_status_stops_every_rank(tmp_path):
    out = _run_worker(tmp_path, _tiny(), "status", 29811)
    assert "rank 0 raised" in out and "rank 1 raised" in out and "NO RAISE" not in out, out


def test_zero2_buckets_leave_during_the_backward(tmp_path):
    """Stage 2 reduces each block's matrices from a hook inside the backward (only the last micro-batch's): 3 blocks,
    2 steps -> 6 early reductions per rank; the equality with one process is tests/test_training.py's."""
    out = _run_worker(tmp_path, _tiny(optimizer_sharding="zero2", micro_batch_size=1), "zero2", 29815)
    assert "rank 0 early 6 buckets 4" in out and "rank 1 early 6 buckets 4" in out, out


def _tp_config():
    cfg = _tiny(steps=3)
    m = cfg.model
    m.d_model, m.ffn_hidden = 64, 64
    g, a = m.encoder.gdn, m.encoder.attention
    g.n_k_heads = g.n_v_heads = 2
    a.n_q_heads, a.n_kv_heads = 4, 2
    cfg.head_impl, cfg.tensor_parallel, cfg.ckpt_every_steps = "chunked", 2, 0
    cfg.data.batch_size, cfg.micro_batch_size = 2, None
    return cfg


def test_tensor_parallel_trainer_from_seed_checkpoints_the_full_model(tmp_path):
    cfg = _tp_config()
    _run_worker(tmp_path, cfg, "tp", 29813)
    state = ckpt.load(ckpt.latest_path(tmp_path / "run"))
    # the file holds the full model: it loads into an unsharded model of cfg.model and into a 1-process Trainer with its moments
    one = copy.deepcopy(cfg)
    one.tensor_parallel = 1
    t = Trainer(one, None)
    t.load_state_dict(state, check_config=False)
    assert t.step == 3
    full = {k: v.shape for k, v in t.model.state_dict().items()}
    assert {k: v.shape for k, v in state["model"].items()} == full
    st = state["optimizer"]
    for index, name in enumerate(st["names"]):
        if index in st["state"]:
            assert tuple(st["state"][index]["exp_avg"].shape) == tuple(full[name]), name
    # the sharded run started from the full model's seeded draw: its first-step loss is the unsharded run's
    ref = Trainer(copy.deepcopy(one), None)
    first = ref.train_step()["loss"]
    import json
    lines = [json.loads(x) for x in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines()]
    got = next(x for x in lines if x.get("step") == 0 and "loss" in x)["loss"]
    assert abs(got - first) < 1e-4 * max(1.0, abs(first)), (got, first)


def test_monitors_and_best_effort_wandb(tmp_path, capsys):
    """A logging step carries the gradient norm per parameter family (their squares add up to the clipped norm's), the
    depth-mix readers' state and, when asked, the stream RMS per layer; an unusable W&B sink warns and the run goes on."""
    import json

    cfg = _tiny(steps=2, log_every=1, log_stream_rms_every=1)
    cfg.wandb.mode = "offline"
    cfg.ckpt_every_steps = 0
    t = Trainer(cfg, tmp_path / "r")
    t.fit()
    lines = [json.loads(x) for x in (tmp_path / "r" / "metrics.jsonl").read_text().splitlines()]
    step0 = next(x for x in lines if x.get("step") == 0 and "loss" in x)
    fam = {k: v for k, v in step0.items() if k.startswith("grad_norm/")}
    assert set(fam) >= {"grad_norm/embed", "grad_norm/gdn", "grad_norm/attention", "grad_norm/mlp", "grad_norm/depth_mix"}
    assert sum(v * v for v in fam.values()) ** 0.5 == pytest.approx(step0["grad_norm"], rel=1e-4)
    assert len(step0["stream_rms"]) == len(t.model.encoder.layers) and len(step0["depth_readers"]["readers"]) > 0
    assert t.step == 2          # the run finished whether or not the W&B package exists here


def test_cuda_graphs_step_is_refused_by_name():
    cfg = _tiny()
    cfg.cuda_graphs = "step"
    with pytest.raises(ValueError, match="cuda_graphs"):
        Trainer(cfg, None)
