"""A training step runs no op whose output shape depends on tensor values (what a CUDA-graph capture and a static-buffer
engine rely on), and resuming through the command line in a new process is the uninterrupted run."""

import copy
import subprocess
import sys
from pathlib import Path

import pytest
import torch
from torch.utils._python_dispatch import TorchDispatchMode

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

ROOT = Path(__file__).resolve().parent.parent
DYNAMIC = ("nonzero", "masked_select", "unique", "unique_consecutive", "unique_dim", "_unique2", "repeat_interleave.Tensor", "bincount", "_local_scalar_dense",
           "index.Tensor_bool")


class OpRecorder(TorchDispatchMode):
    """Every dispatched op with its output shapes; ops whose result size (or a host-side value) depends on data are flagged."""

    def __init__(self):
        super().__init__()
        self.ops, self.flagged = [], []

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        name = func.__name__ if hasattr(func, "__name__") else str(func)
        full = str(func).replace("aten.", "")
        shapes = tuple(tuple(o.shape) for o in (out if isinstance(out, (tuple, list)) else [out]) if isinstance(o, torch.Tensor))
        self.ops.append((full, shapes))
        bool_index = "index.Tensor" in full and any(isinstance(i, torch.Tensor) and i.dtype in (torch.bool, torch.uint8)
                                                      for i in (args[1] if len(args) > 1 and isinstance(args[1], (list, tuple)) else []))
        if any(d in full for d in DYNAMIC) or bool_index:
            self.flagged.append(full)
        return out


def batch(vocab, rows, length, seed, doc_every):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(1, vocab, (rows, length + 1), generator=g)
    docs = (torch.arange(length + 1) // doc_every)[None, :].expand(rows, -1).contiguous()
    return tokens[:, :-1], tokens[:, 1:], docs[:, :-1], docs[:, 1:] == docs[:, :-1]


@pytest.mark.parametrize("preset", ["control", "full"])
def test_forward_and_backward_run_no_data_dependent_shapes(preset):
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.train.loss import lm_loss

    cfg = C.tiny_control_config() if preset == "control" else C.tiny_full_config()
    torch.manual_seed(0)
    model = build_model(cfg).train()
    traces = []
    for seed, doc_every in ((0, 48), (1, 7), (2, 19)):           # one document per row, many short ones, a few
        x, y, d, valid = batch(cfg.vocab_size, 2, 47, seed, doc_every)
        model.zero_grad(set_to_none=True)
        with OpRecorder() as rec:
            out = model(x, d)
            loss = lm_loss(out.logits, y, valid)[0] if isinstance(lm_loss(out.logits, y, valid), tuple) else lm_loss(out.logits, y, valid)
            loss.backward()
        assert len(rec.ops) > 100
        assert rec.flagged == [], f"data-dependent shapes in the step: {sorted(set(rec.flagged))}"
        traces.append(rec.ops)
    assert traces[0] == traces[1] == traces[2]                    # the same ops with the same shapes whatever the document layout


def test_resume_in_a_new_process_matches_the_uninterrupted_run(tmp_path):
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device, cfg.ckpt_every_steps = 6, 1, True, "cpu", 100
    C.save_yaml(cfg, tmp_path / "cfg.yaml")

    def cli(run_dir, *extra):
        return subprocess.run([sys.executable, str(ROOT / "scripts" / "train.py"), "--config", str(tmp_path / "cfg.yaml"), "--run-dir", str(run_dir), "--threads", "1", *extra],
                              check=True, capture_output=True, text=True, timeout=900)

    cli(tmp_path / "straight")
    cli(tmp_path / "resumed", "--until-step", "3")
    assert ckpt.load(ckpt.latest_path(tmp_path / "resumed"))["step"] == 3
    out = cli(tmp_path / "resumed")
    assert "resum" in (out.stdout + out.stderr).lower()
    a, b = (ckpt.load(ckpt.latest_path(tmp_path / n)) for n in ("straight", "resumed"))
    assert a["step"] == b["step"] == 6
    for k in a["model"]:
        assert torch.equal(a["model"][k], b["model"][k]), k
    flat = lambda o: [o] if isinstance(o, torch.Tensor) else [t for v in (o.values() if isinstance(o, dict) else o if isinstance(o, (list, tuple)) else []) for t in flat(v)]
    for x, y in zip(flat(a["optimizer"]), flat(b["optimizer"])):
        assert torch.equal(x, y)
