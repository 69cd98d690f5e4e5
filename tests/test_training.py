"""Trainer behaviour on CPU: resume is bit-exact, micro-batching matches, data-parallel gloo ranks equal one process
(replicated, ZeRO-1, ZeRO-2), SIGTERM saves and leaves, a non-finite loss marks the run, a changed config is refused."""

import copy
import json
import math
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch
import yaml

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt
from gdn_hybrid_architecture_ideas_b200.train.trainer import Diverged, Trainer

ROOT = Path(__file__).resolve().parent.parent


def tiny_train_config(**kw) -> C.TrainConfig:
    cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config(seq_len=48, batch_size=4), steps=6, seed=3)
    cfg.optim.warmup_steps, cfg.ckpt_every_steps, cfg.metrics_jsonl, cfg.head_impl, cfg.log_every = 2, 3, True, "fused", 0
    for k, v in kw.items():
        C.apply_override(cfg, f"{k}={v}")
    return cfg


def weights(t: Trainer):
    return {k: v.clone() for k, v in t.model.state_dict().items()}


def test_resume_is_bit_exact(tmp_path):
    cfg = tiny_train_config()
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(3)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    wa, wc = weights(a), weights(c)
    assert all(torch.equal(wa[k], wc[k]) for k in wa)
    assert (tmp_path / "b" / "checkpoints" / "latest").read_text() == "step_00000006.pt"
    lines = [json.loads(x) for x in (tmp_path / "a" / "metrics.jsonl").read_text().splitlines()]
    assert lines[0]["event"] == "start" and lines[-1]["step"] == 5


def test_fused_head_equals_chunked_head():
    g = {}
    for impl in ("fused", "chunked"):
        t = Trainer(tiny_train_config(head_impl=impl), None)
        t.train_step()
        g[impl] = t.flat.grads.clone()
    assert torch.allclose(g["fused"], g["chunked"], atol=1e-6, rtol=1e-4)


def test_microbatch_gradients_match():
    full = Trainer(tiny_train_config(), None)
    half = Trainer(tiny_train_config(micro_batch_size=2), None)
    full.train_step(), half.train_step()
    assert torch.allclose(full.flat.grads, half.flat.grads, atol=2e-6, rtol=1e-4)


def test_changed_config_is_refused(tmp_path):
    a = Trainer(tiny_train_config(), tmp_path)
    a.fit(3)
    other = tiny_train_config()
    other.model.ffn_hidden = 128
    b = Trainer(other, tmp_path)
    with pytest.raises(ValueError, match="different config"):
        b.load_state_dict(ckpt.load(ckpt.latest_path(tmp_path)))


def test_non_finite_loss_marks_the_run(tmp_path):
    t = Trainer(tiny_train_config(), tmp_path)
    with torch.no_grad():
        t.model.final_norm.weight.fill_(float("nan"))
    with pytest.raises(Diverged):
        t.fit()
    assert (tmp_path / "diverged.json").exists()
    with pytest.raises(Diverged):
        Trainer(tiny_train_config(), tmp_path).fit()


def test_async_checkpoint_equals_sync(tmp_path):
    a = Trainer(tiny_train_config(), tmp_path / "s")
    a.fit()
    b = Trainer(tiny_train_config(ckpt_async=True), tmp_path / "a")
    b.fit()
    sa = ckpt.load(ckpt.latest_path(tmp_path / "s"))
    sb = ckpt.load(ckpt.latest_path(tmp_path / "a"))
    assert all(torch.equal(sa["model"][k], sb["model"][k]) for k in sa["model"])
    assert sa["step"] == sb["step"] == 6


def _write_config(path: Path, cfg: C.TrainConfig) -> Path:
    C.save_yaml(cfg, path)
    return path


def _run_cli(args, nproc=1, port=29541, env=None, **popen):
    cmd = [sys.executable]
    if nproc > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += [str(ROOT / "scripts" / "train.py")] + args
    e = {**os.environ, "GHB_DP_BACKEND": "gloo", "OMP_NUM_THREADS": "2", **(env or {})}
    return subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600, **popen)


@pytest.mark.parametrize("sharding,optim", [("replicated", "adamw"), ("zero1", "adamw"), ("zero2", "adamw"), ("zero1", "muon")])
def test_two_gloo_ranks_equal_one_process(tmp_path, sharding, optim):
    cfg = tiny_train_config(micro_batch_size=2, steps=4)
    cfg.optim.name = optim
    cfg.device = "cpu"
    path = _write_config(tmp_path / "c.yaml", cfg)
    one = _run_cli(["--config", str(path), "--run-dir", str(tmp_path / "one")])
    assert one.returncode == 0, one.stderr[-2000:]
    two = _run_cli(["--config", str(path), "--run-dir", str(tmp_path / "two"), "--set", f"optimizer_sharding={sharding}"],
                   nproc=2, port=29541 + hash((sharding, optim)) % 200)
    assert two.returncode == 0, two.stderr[-2000:]
    a = ckpt.load(ckpt.latest_path(tmp_path / "one"))
    b = ckpt.load(ckpt.latest_path(tmp_path / "two"))
    worst = max((a["model"][k] - b["model"][k]).abs().max().item() for k in a["model"])
    assert worst < (1e-6 if optim == "adamw" else 2e-3), worst
    if sharding != "replicated":   # the sharded run's optimizer state loads into one process (world size change)
        t = Trainer(copy.deepcopy(cfg), None)
        t.load_state_dict(b, check_config=False)
        assert t.step == 4


def test_sigterm_saves_and_resumes(tmp_path):
    cfg = tiny_train_config(steps=4000)
    cfg.ckpt_every_steps, cfg.device = 0, "cpu"
    cfg.ckpt_every_minutes = 0.0
    path = _write_config(tmp_path / "c.yaml", cfg)
    cmd = [sys.executable, str(ROOT / "scripts" / "train.py"), "--config", str(path), "--run-dir", str(tmp_path / "r")]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    deadline = time.time() + 120
    while time.time() < deadline and not (tmp_path / "r" / "metrics.jsonl").exists():
        time.sleep(0.2)
    time.sleep(1.0)
    p.send_signal(signal.SIGTERM)
    p.wait(timeout=120)
    latest = ckpt.latest_path(tmp_path / "r")
    assert latest is not None, p.stderr.read().decode()[-2000:]
    step = ckpt.load(latest)["step"]
    assert 0 < step < 4000
    t = Trainer(copy.deepcopy(cfg), tmp_path / "r")
    assert t.resume_from_checkpoint() and t.step == step


@pytest.mark.parametrize("mode", ["layer", "block", "host"])
def test_activation_memory_modes_give_the_same_gradients(mode):
    """Recomputing layers or blocks, or parking saved activations in the host pool, changes no gradient."""
    from gdn_hybrid_architecture_ideas_b200.models import act_checkpoint, build_model

    cfg = C.tiny_full_config()
    torch.manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (2, 24))
    doc = torch.zeros_like(tok)
    grads = {}
    for m in ("none", mode):
        torch.manual_seed(1)
        model = build_model(cfg)
        model.encoder.activation_checkpoint = m
        if m == "host":
            model.encoder.host_pool = act_checkpoint.HostPool(torch.device("cpu"), min_bytes=0)
        model(tok, doc).logits.float().square().mean().backward()
        grads[m] = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
        if m == "host":
            st = model.encoder.host_pool.stats
            assert st["packed"] > 0 and 0 < st["unpacked"] <= st["packed"] and st["allocated"] <= st["packed"]
            del model
            import gc
            gc.collect()
    assert grads["none"].keys() == grads[mode].keys()
    for k in grads["none"]:
        assert torch.allclose(grads["none"][k], grads[mode][k], atol=1e-6, rtol=1e-5), k


def test_data_prefetch_trains_on_the_same_batches(tmp_path):
    """Building step N + 1's batch on a background thread changes nothing about the run."""
    def run(prefetch):
        cfg = C.TrainConfig(model=C.tiny_full_config(), data=C.tiny_data_config())
        cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device, cfg.data_prefetch = 3, 0, False, "cpu", prefetch
        t = Trainer(cfg, None)
        return [t.train_step()["loss"] for _ in range(3)]

    assert run(False) == run(True)


def test_experimental_arms_train(tmp_path):
    """Residual scalars (span form: stored values projected back into [-3, 3] after each step, no weight decay), Canon
    layers and the doubled write-strength range train through the public trainer."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    cfg = tiny_train_config()
    cfg.model = C.tiny_control_config()
    cfg.model.encoder.layer_scalars = "skip_x0_span"
    cfg.model.encoder.gdn.negeig.beta_max = 2
    t = Trainer(copy.deepcopy(cfg), tmp_path / "s")
    groups = optim.param_groups(t.model, cfg.optim)
    plain = [g for g in groups if g["weight_decay"] == 0.0][0]["names"]
    assert "encoder.skip_gain" in plain and "encoder.x0_gain" in plain
    with torch.no_grad():
        t.model.encoder.skip_gain.fill_(7.0)
    t.train_step()
    assert float(t.model.encoder.skip_gain.abs().max()) <= 3.0
    assert t.model.encoder.x0_gain[0] == 0 and t.model.encoder.x0_gain[1:].abs().sum() > 0     # b_0 is never read
    cfg2 = tiny_train_config()
    cfg2.model = C.tiny_control_config()
    cfg2.model.encoder.canon_kernel, cfg2.model.encoder.canon_init = 4, "uniform"
    t2 = Trainer(copy.deepcopy(cfg2), tmp_path / "c")
    before = {n: p.detach().clone() for n, p in t2.model.named_parameters() if n.endswith("canon.conv_weight")}
    assert before and all(v.abs().max() > 0 for v in before.values())
    l0 = t2.train_step()["loss"]
    for _ in range(3):
        l1 = t2.train_step()["loss"]
    assert l1 < l0
    assert all(not torch.equal(before[n], p) for n, p in t2.model.named_parameters() if n in before)


def test_asentmax_attention_trains(tmp_path):
    """alpha = 1.5 entmax attention with its learned query scale: the two heads sit in the undecayed AdamW group (Muon
    never takes them), start from their own generator and train."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    cfg = tiny_train_config()
    cfg.model = C.tiny_control_config()
    a = cfg.model.encoder.attention
    a.normalizer, a.temperature, a.rope_max_distance = "asentmax", "fixed", None
    cfg.optim.name = "muon"
    t = Trainer(copy.deepcopy(cfg), tmp_path / "e")
    heads = [n for n, _ in t.model.named_parameters() if ".beta_proj." in n or ".gamma_proj." in n]
    assert heads
    for g in optim.param_groups(t.model, cfg.optim):
        if set(heads) & set(g["names"]):
            assert g["weight_decay"] == 0.0 and g.get("kind", "adamw") == "adamw", g
    before = {n: p.detach().clone() for n, p in t.model.named_parameters() if n in heads}
    l0 = t.train_step()["loss"]
    for _ in range(3):
        l1 = t.train_step()["loss"]
    assert l1 < l0
    assert all(not torch.equal(before[n], p) for n, p in t.model.named_parameters() if n in before)
    bad = tiny_train_config()
    bad.model = C.tiny_control_config()
    bad.model.encoder.attention.normalizer = "asentmax"
    bad.model.encoder.attention.temperature = "learned"
    with pytest.raises(ValueError, match="asentmax"):
        Trainer(bad, tmp_path / "b")


def test_kda_channel_decay(tmp_path):
    """Per-channel decay: the chunked form equals the token loop (float64, documents and a carried state), a uniform decay
    is the scalar rule, the cached path equals the full forward, the floored channels' decay never falls below
    1 - 1/H, the gate's matrices train in AdamW's decayed group and its dt_bias in the undecayed one."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_kda
    from gdn_hybrid_architecture_ideas_b200.ops import reference as R
    from gdn_hybrid_architecture_ideas_b200.train import optim
    from tests.helpers import make_model

    g = torch.Generator().manual_seed(0)
    B, L, H, dk, dv = 2, 70, 2, 8, 4
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, v = rn(B, L, H, dk), torch.nn.functional.normalize(rn(B, L, H, dk), dim=-1), rn(B, L, H, dv)
    gl, beta = -torch.rand(B, L, H, dk, generator=g, dtype=torch.float64) * 4, torch.rand(B, L, H, generator=g, dtype=torch.float64)
    starts = torch.zeros(B, L, dtype=torch.bool)
    starts[0, 33], starts[1, 16], starts[1, 17] = True, True, True
    S0 = rn(B, H, dk, dv)
    o1, S1 = R.kda_recurrence(q, k, v, gl, beta, starts, S0)
    o2, S2 = R.kda_chunked(q, k, v, gl, beta, starts, S0, 16)
    assert (o1 - o2).abs().max() < 1e-11 and (S1 - S2).abs().max() < 1e-11
    same = gl[..., :1].expand_as(gl)
    o3, S3 = R.delta_rule_recurrence(q, k, v, same[..., 0], beta, starts, S0)
    o4, S4 = R.kda_recurrence(q, k, v, same, beta, starts, S0)
    assert torch.equal(o3, o4) or (o3 - o4).abs().max() < 1e-13
    cfg = C.tiny_control_config()
    kk = cfg.encoder.gdn.kda
    kk.decay, kk.floor_channels, kk.floor_min, kk.floor_max = "channel", 4, 8.0, 64.0
    model = make_model(cfg, dtype=torch.float64).eval()
    tok, doc = torch.randint(0, 256, (2, 40), generator=g), torch.zeros(2, 40, dtype=torch.long)
    doc[1, 13:] = 1
    full = model(tok, doc).logits
    cfg2 = copy.deepcopy(cfg)
    cfg2.encoder.gdn.kernel, cfg2.encoder.gdn.chunk_size = "chunked", 16
    chunked = make_model(cfg2, dtype=torch.float64).eval()
    chunked.load_state_dict(model.state_dict())
    assert (chunked(tok, doc).logits - full).abs().max() < 1e-9
    out = chunked.prefill(tok[:, :30], doc[:, :30])
    cache, parts = out.cache, [out.logits]
    for i in range(30, 40):
        out = chunked.extend(tok[:, i:i + 1], doc[:, i:i + 1], None, cache)
        cache = out.cache
        parts.append(out.logits)
    assert (torch.cat(parts, 1) - full).abs().max() < 1e-9
    layer = next(m for m in model.modules() if getattr(m, "kda", None) is not None)
    assert not hasattr(layer, "in_proj_a") and "floor_log" not in layer.kda.state_dict()
    gg, _ = gdn_kda.gates(layer, torch.randn(3, 5, cfg.d_model, generator=g, dtype=torch.float64) * 50)
    bound = 1 - 1 / torch.tensor(layer.kda.horizons, dtype=torch.float64)
    assert (torch.exp(gg[..., :4]) >= bound - 1e-12).all() and (gg <= 0).all()
    tc = tiny_train_config()
    tc.model = cfg
    tc.optim.name = "muon"
    t = Trainer(copy.deepcopy(tc), tmp_path / "k")
    for grp in optim.param_groups(t.model, tc.optim):
        names = grp["names"]
        if any(n.endswith(".kda.f_up.weight") for n in names):
            assert grp.get("kind", "adamw") == "adamw" and grp["weight_decay"] > 0
        if any(n.endswith(".kda.dt_bias") for n in names):
            assert grp["weight_decay"] == 0.0
    l0 = t.train_step()["loss"]
    for _ in range(3):
        l1 = t.train_step()["loss"]
    assert l1 < l0
    bad = C.tiny_full_config()
    bad.encoder.gdn.kda.decay = "channel"
    m = make_model(bad, dtype=torch.float32)
    with pytest.raises(ValueError, match="write / query mixes"):
        m(tok, doc)


def test_erase_direction(tmp_path):
    """The erase direction: the 2T interleave into the chunked rule equals the token loop on both decays, gamma = 0 is
    the base rule, the inward clamp passes only gradients that move the scale back toward [0, 1], the scale leaves weight
    decay under zero_gate_decay none, and the layer trains."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_erase
    from gdn_hybrid_architecture_ideas_b200.ops import reference as R
    from gdn_hybrid_architecture_ideas_b200.train import optim
    from tests.helpers import make_model

    g = torch.Generator().manual_seed(0)
    B, L, H, dk, dv = 2, 45, 2, 8, 4
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    unit = lambda t: torch.nn.functional.normalize(t, dim=-1)
    q, k, e, v = rn(B, L, H, dk), unit(rn(B, L, H, dk)), unit(rn(B, L, H, dk)), rn(B, L, H, dv)
    beta, gamma = (torch.rand(B, L, H, generator=g, dtype=torch.float64) for _ in range(2))
    starts = torch.zeros(B, L, dtype=torch.bool)
    starts[0, 20], starts[1, 7], starts[1, 8] = True, True, True
    S0 = rn(B, H, dk, dv)
    for gl in (-torch.rand(B, L, H, generator=g, dtype=torch.float64), -torch.rand(B, L, H, dk, generator=g, dtype=torch.float64) * 3):
        o1, S1 = gdn_erase.rule(q, k, v, gl, beta, e, gamma, starts, S0, "recurrence", 16)
        o2, S2 = gdn_erase.rule(q, k, v, gl, beta, e, gamma, starts, S0, "chunked", 16)
        assert (o1 - o2).abs().max() < 1e-10 and (S1 - S2).abs().max() < 1e-10
        base = R.kda_recurrence if gl.dim() == 4 else R.delta_rule_recurrence
        o3, _ = base(q, k, v, gl, beta, starts, S0)
        o4, _ = gdn_erase.rule(q, k, v, gl, beta, e, torch.zeros_like(gamma), starts, S0, "chunked", 16)
        assert (o3 - o4).abs().max() < 1e-10 and (o3 - o1).abs().max() > 1e-3
    s = torch.tensor([-0.5, -0.5, 0.0, 0.5, 1.0, 1.5, 1.5], requires_grad=True)
    up = torch.tensor([1.0, -1.0, 1.0, 1.0, -1.0, 1.0, -1.0])
    (gdn_erase.inward_clamp(s) * up).sum().backward()
    assert s.grad.tolist() == [0.0, -1.0, 1.0, 1.0, -1.0, 1.0, 0.0]
    assert gdn_erase.inward_clamp(s).tolist() == [0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 1.0]
    tc = tiny_train_config()
    tc.model = C.tiny_control_config()
    tc.model.encoder.gdn.erase.mode, tc.model.encoder.gdn.erase.rank = "eda", 4
    tc.model.encoder.gdn.kernel, tc.model.encoder.gdn.chunk_size = "chunked", 16
    tc.optim.zero_gate_decay = "none"
    t = Trainer(copy.deepcopy(tc), tmp_path / "e")
    scales = [n for n, _ in t.model.named_parameters() if n.endswith(".erase.scale")]
    assert scales and all(float(p.abs().max()) == 0 for n, p in t.model.named_parameters() if n in scales)
    for grp in optim.param_groups(t.model, tc.optim):
        if set(scales) & set(grp["names"]):
            assert grp["weight_decay"] == 0.0
        if any(n.endswith(".erase.e_up.weight") for n in grp["names"]):
            assert grp.get("kind", "adamw") == "adamw" and grp["weight_decay"] > 0
    l0 = t.train_step()["loss"]
    for _ in range(3):
        l1 = t.train_step()["loss"]
    assert l1 < l0 and any(float(p.abs().max()) > 0 for n, p in t.model.named_parameters() if n in scales)
    plain = C.tiny_control_config()
    torch.manual_seed(5)
    a = make_model(plain, dtype=torch.float32, seed=5, perturbed=False)
    b = make_model(tc.model, dtype=torch.float32, seed=5, perturbed=False)
    sa, sb = a.state_dict(), b.state_dict()
    assert all(torch.equal(sa[n], sb[n]) for n in sa)          # the base tensors start as in the base model of the same seed
    bad = C.tiny_full_config()
    bad.encoder.gdn.erase.mode = "eda"
    with pytest.raises(ValueError, match="gdn_write_mix"):
        make_model(bad, dtype=torch.float32)


def test_gated_deltaproduct(tmp_path):
    """n_h steps a token: the n_h T interleave into the chunked rule equals the token-and-step loop, one step is the
    plain rule, the extra key / value projection goes to Muon and the extra beta projection and conv to AdamW, the
    base tensors start as in the base model, and the layer trains on the chunked path."""
    from gdn_hybrid_architecture_ideas_b200.models import gdn_dprod
    from gdn_hybrid_architecture_ideas_b200.ops import reference as R
    from gdn_hybrid_architecture_ideas_b200.train import optim
    from tests.helpers import make_model

    g = torch.Generator().manual_seed(0)
    B, L, H, dk, dv, n_h = 2, 37, 2, 8, 4, 3
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, v = rn(B, L, H, dk), torch.nn.functional.normalize(rn(B, L, n_h, H, dk), dim=-1), rn(B, L, n_h, H, dv)
    gl, beta = -torch.rand(B, L, H, generator=g, dtype=torch.float64), 2 * torch.rand(B, L, n_h, H, generator=g, dtype=torch.float64)
    starts = torch.zeros(B, L, dtype=torch.bool)
    starts[0, 20], starts[1, 7], starts[1, 8] = True, True, True
    S0 = rn(B, H, dk, dv)
    o1, S1 = gdn_dprod.dprod_recurrence(q, k, v, gl, beta, starts, S0)
    qi, ki, vi, gi, bi, si = gdn_dprod.interleave(q, k, v, gl, beta, starts)
    oi, S2 = R.chunked_delta_rule(qi, ki, vi, gi, bi, si, S0, 16)
    assert (gdn_dprod.last_substep(oi, n_h) - o1).abs().max() < 1e-10 and (S1 - S2).abs().max() < 1e-10
    o3, S3 = gdn_dprod.dprod_recurrence(q, k[:, :, :1], v[:, :, :1], gl, beta[:, :, :1], starts, S0)
    o4, S4 = R.delta_rule_recurrence(q, k[:, :, 0], v[:, :, 0], gl, beta[:, :, 0], starts, S0)
    assert (o3 - o4).abs().max() < 1e-13
    tc = tiny_train_config()
    tc.model = C.tiny_control_config()
    tc.model.encoder.gdn.dprod.n_h = 2
    tc.model.encoder.gdn.kernel, tc.model.encoder.gdn.chunk_size = "chunked", 16
    tc.optim.name = "muon"
    t = Trainer(copy.deepcopy(tc), tmp_path / "d")
    for grp in optim.param_groups(t.model, tc.optim):
        kind = grp.get("kind", "adamw")
        for n in grp["names"]:
            if n.endswith(".dprod.in_proj_kv.weight"):
                assert kind == "muon"
            if n.endswith((".dprod.in_proj_b.weight", ".dprod.conv_weight")):
                assert kind == "adamw"
    l0 = t.train_step()["loss"]
    for _ in range(3):
        l1 = t.train_step()["loss"]
    assert l1 < l0
    a = make_model(C.tiny_control_config(), dtype=torch.float32, seed=5, perturbed=False).state_dict()
    b = make_model(tc.model, dtype=torch.float32, seed=5, perturbed=False).state_dict()
    assert all(torch.equal(a[n], b[n]) for n in a) and len(b) > len(a)
    layer = next(m for m in t.model.modules() if getattr(m, "dprod", None) is not None)
    assert sum(p.numel() for p in layer.dprod.parameters()) == gdn_dprod.params_per_layer(tc.model.d_model, tc.model.encoder.gdn)
    for key, value in (("key", "lowrank"), ("heads", 1), ("route", "one-readout")):
        bad = C.tiny_control_config()
        bad.encoder.gdn.dprod.n_h = 2
        setattr(bad.encoder.gdn.dprod, key, value)
        with pytest.raises(ValueError, match=key):
            make_model(bad, dtype=torch.float32)
    bad = C.tiny_control_config()
    bad.encoder.gdn.dprod.n_h, bad.encoder.gdn.negeig.beta_max = 2, 2
    with pytest.raises(ValueError, match="negeig"):
        make_model(bad, dtype=torch.float32)


def test_linear_depth_memory(tmp_path):
    """attn_res "ldm": the write is lam (I - w k k^T) M + w k v^T, the added tensors count as the shapes say and start
    without moving any base tensor, every gate starts at 1, the address networks train in AdamW, and the model trains."""
    from gdn_hybrid_architecture_ideas_b200.models import ldm
    from gdn_hybrid_architecture_ideas_b200.train import optim
    from tests.helpers import make_model

    base = C.tiny_control_config()
    cfg = C.tiny_control_config()
    cfg.encoder.attn_res, cfg.encoder.ldm_groups, cfg.encoder.ldm_key_dim, cfg.encoder.ldm_hidden = "ldm", 4, 4, 6
    a = make_model(base, dtype=torch.float64, seed=3, perturbed=False)
    b = make_model(cfg, dtype=torch.float64, seed=3, perturbed=False)
    sa, sb = a.state_dict(), b.state_dict()
    assert all(torch.equal(sa[n], sb[n]) for n in sa)
    added = sum(p.numel() for n, p in b.named_parameters() if ".attn_res." in n)
    assert added == ldm.parameter_count(cfg.d_model, cfg.encoder.n_layers, 4, 4, 6)
    w = b.encoder.layers[1].attn_res.mixer_write
    with torch.no_grad():
        w.net.gate.bias.fill_(0.3)
    g = torch.Generator().manual_seed(0)
    x, v = torch.randn(2, 5, cfg.d_model, generator=g, dtype=torch.float64), torch.randn(2, 5, cfg.d_model, generator=g, dtype=torch.float64)
    M = torch.randn(2, 5, 4, 4, cfg.d_model // 4, generator=g, dtype=torch.float64)
    k, val, wgt = w._observation(x, v)                         # unit key per group, the value per group, the write weight
    assert torch.allclose((k * k).sum(-1), torch.ones_like(wgt)) and torch.equal(val, v.unflatten(-1, (4, -1)))
    lam = torch.sigmoid(w.lam_logit.detach().double())
    want = lam[:, None, None] * (M - wgt[..., None, None] * k[..., None] * (M * k[..., None]).sum(-2, keepdim=True)) \
        + wgt[..., None, None] * k[..., None] * v.unflatten(-1, (4, -1))[..., None, :]
    assert (w.write(M, x, v) - want).abs().max() < 1e-12
    assert (ldm.memory_read(want, k) - (want * k[..., None]).sum(-2)).abs().max() < 1e-12
    assert abs(float(lam[0]) - 0.99) < 1e-6 and torch.allclose(wgt, torch.full_like(wgt, 2 * torch.sigmoid(torch.tensor(0.3, dtype=torch.float64))))
    tc = tiny_train_config()
    tc.model = cfg
    tc.optim.name = "muon"
    t = Trainer(copy.deepcopy(tc), tmp_path / "l")
    for grp in optim.param_groups(t.model, tc.optim):
        if any(".attn_res." in n for n in grp["names"]):
            assert grp.get("kind", "adamw") == "adamw"
    before = {n: p.detach().clone() for n, p in t.model.named_parameters() if ".attn_res." in n}
    losses = [t.train_step()["loss"] for _ in range(4)]
    assert all(math.isfinite(v) for v in losses)
    moved = [n for n, p in t.model.named_parameters() if ".attn_res." in n and not torch.equal(p.detach(), before[n])]
    assert len(moved) > 0.8 * len(before), (len(moved), len(before))          # the memory's tensors take part in training
    bad = C.tiny_full_config()
    bad.encoder.attn_res = "ldm"
    with pytest.raises(ValueError):
        make_model(bad, dtype=torch.float32)
    graphs = copy.deepcopy(tc)
    graphs.cuda_graphs = "microbatch"
    with pytest.raises(ValueError, match="tensor ops"):
        Trainer(graphs, tmp_path / "g")


def test_train_mtp_script(tmp_path):
    """The drafter-head script: loads a trained trunk, freezes it, trains the head, saves the head's tensors only."""
    cfg = tiny_train_config()
    cfg.model = C.tiny_control_config()
    t = Trainer(copy.deepcopy(cfg), tmp_path / "run")
    t.fit()
    trunk = weights(t)
    out = tmp_path / "head.pt"
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "train_mtp.py"), "--checkpoint", str(tmp_path / "run"), "--steps", "12", "--lr", "3e-3",
                        "--device", "cpu", "--log-every", "11", "--out", str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert lines[-1]["loss"] < lines[0]["loss"]
    saved = torch.load(out, weights_only=False)
    assert saved["trunk_step"] == 6 and all(k.startswith("mtp.") for k in saved["head"]) and "mtp.eh_proj.weight" in saved["head"]
    with pytest.raises(ValueError, match="mtp"):
        bad = copy.deepcopy(cfg)
        bad.model.mtp.enabled = True
        Trainer(bad, tmp_path / "bad")


def test_gdn_mup_groups_and_init(tmp_path):
    """optim.gdn_mup: the GDN gate projections get base_width / fan_in times the learning rate in a group of their own,
    A_log / dt_bias a group without decay, nothing else moves; the gates start scaled by sqrt(base_width / fan_in)."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    cfg = tiny_train_config()
    plain = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    cfg.optim.gdn_mup, cfg.optim.gdn_mup_base_width = True, 16
    t = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    d = cfg.model.d_model
    groups = optim.param_groups(t.model, cfg.optim)
    base = optim.param_groups(plain.model, copy.deepcopy(plain.cfg.optim))
    gate = [g for g in groups if any(n.endswith("in_proj_a.weight") for n in g["names"])]
    assert len(gate) == 1 and gate[0]["lr_scale"] == 16 / d and gate[0]["weight_decay"] == cfg.optim.weight_decay
    assert all(n.endswith(("in_proj_a.weight", "in_proj_b.weight")) for n in gate[0]["names"])
    scal = [g for g in groups if any(n.endswith(".A_log") for n in g["names"])]
    assert len(scal) == 1 and scal[0]["weight_decay"] == 0.0 and all(n.endswith((".A_log", ".dt_bias")) for n in scal[0]["names"])
    assert sorted(n for g in groups for n in g["names"]) == sorted(n for g in base for n in g["names"])
    pa, pb = dict(plain.model.named_parameters()), dict(t.model.named_parameters())
    for n in pa:
        want = pa[n] * (16 / d) ** 0.5 if n.endswith(("in_proj_a.weight", "in_proj_b.weight")) else pa[n]
        assert torch.allclose(pb[n], want), n
    l0 = t.train_step()["loss"]
    for _ in range(4):
        l1 = t.train_step()["loss"]
    assert l1 < l0


@pytest.mark.parametrize("head", ["fused", "chunked"])
def test_fixed_cross_entropy_trains(tmp_path, head):
    """loss.ce_form "fixed" through the trainer: the first loss equals the standard form's (the two differ only where a row
    has collapsed), training proceeds."""
    cfg = tiny_train_config()
    cfg.head_impl = head
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    cfg.loss.ce_form = "fixed"
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    la, lb = a.train_step()["loss"], b.train_step()["loss"]
    assert abs(la - lb) < 1e-5 * abs(la)
    for _ in range(4):
        l1 = b.train_step()["loss"]
    assert l1 < lb


@pytest.mark.parametrize("arm", ["block", "token"])
def test_block_attn_res_trains(tmp_path, arm):
    """attn_res "block" (a depth read before every sublayer) and token-dependent block-entry queries through the trainer."""
    cfg = tiny_train_config()
    if arm == "block":
        cfg.model.encoder.attn_res = "block"
    else:
        cfg.model.encoder.attn_res_query, cfg.model.encoder.attn_res_heads = "token", 2
    cfg.model.encoder.gdn_write_mix, cfg.model.encoder.gdn_write_variant = "none", "none"
    t = Trainer(copy.deepcopy(cfg), tmp_path / "r")
    l0 = t.train_step()["loss"]
    for _ in range(4):
        l1 = t.train_step()["loss"]
    assert l1 < l0
    want = "attn_res.pre_mlp.query" if arm == "block" else "attn_res.entry.net.head.weight"
    assert any(n.endswith(want) for n, _ in t.model.named_parameters())


def _entry_config(run_entry, runs, entry, root):
    cmd = run_entry.build_command(runs, entry, "/runs", check_eval=False)
    cfg = C.load_yaml(cmd[cmd.index("--config") + 1])
    for i, x in enumerate(cmd):
        if x == "--set":
            C.apply_override(cfg, cmd[i + 1])
    C.require_supported(cfg)
    return cfg


def test_every_run_entry_builds():
    """Every entry of the shipped runs files resolves through run_entry (common patch, nested patch, flat set list), passes the
    refusal tables and builds (meta device; each distinct model once)."""
    import importlib.util
    import json
    from pathlib import Path

    from gdn_hybrid_architecture_ideas_b200.models import build_model

    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("run_entry", root / "scripts" / "run_entry.py")
    run_entry = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run_entry)
    seen, built = 0, set()
    for path in sorted((root / "runs").glob("*.yaml")):
        runs = run_entry.load_runs(path, "/data", "/runs")
        for entry in runs["runs"]:
            cfg = _entry_config(run_entry, runs, entry, root)
            key = json.dumps(C.to_dict(cfg.model), sort_keys=True, default=str)
            if key not in built:
                built.add(key)
                with torch.device("meta"):
                    model = build_model(cfg.model)
                assert sum(p.numel() for p in model.parameters()) > 0, entry["name"]
            seen += 1
    assert seen >= 140 and len(built) >= 25
    # the flat form and the nested form of one entry resolve to the same config
    flat = {"runs": [{"name": "x", "config": "configs/v2/control-a-60m.yaml", "seed": 1,
                      "set": ["model.encoder.attn_res=block_entry", "model.encoder.n_layers=24", "steps=7", "tst.schedule=[[0,4],[3,1]]"]}]}
    nested = {"common": {"steps": 7}, "runs": [{"name": "x", "base": "configs/v2/control-a-60m.yaml", "seed": 1,
                                                "patch": {"model": {"encoder": {"attn_res": "block_entry", "n_layers": 24}}, "tst": {"schedule": [[0, 4], [3, 1]]}}}]}
    a = _entry_config(run_entry, flat, flat["runs"][0], root)
    b = _entry_config(run_entry, nested, nested["runs"][0], root)
    assert C.to_dict(a) == C.to_dict(b)
    with pytest.raises(KeyError, match="no_such_key"):
        run_entry.flatten_patch({"model": {"no_such_key": 1}})


def test_published_runs_files_load_as_they_are():
    """The reference's own runs files (flat `set` lists over its base configs' names) resolve, pass the refusal tables and name
    the same configs as the nested files shipped here."""
    import importlib.util
    from pathlib import Path

    from tests.helpers import REFERENCE

    theirs = Path(REFERENCE) / "runs"
    if not theirs.is_dir():
        pytest.skip("no reference checkout")
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("run_entry", root / "scripts" / "run_entry.py")
    run_entry = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run_entry)
    n = 0
    for path in sorted(theirs.glob("*.yaml")):
        pub = run_entry.load_runs(path, "/data", "/runs")
        own = run_entry.load_runs(root / "runs" / path.name, "/data", "/runs")
        assert [e["name"] for e in pub["runs"]] == [e["name"] for e in own["runs"]], path.name
        for e_pub, e_own in zip(pub["runs"], own["runs"]):
            assert C.to_dict(_entry_config(run_entry, pub, e_pub, root)) == C.to_dict(_entry_config(run_entry, own, e_own, root)), e_pub["name"]
            n += 1
    assert n >= 140


def test_branch_and_stage_continue_another_run(tmp_path):
    """`resume_from`: a new run that continues another run's kept checkpoint is the uninterrupted longer run bit for bit;
    a changed config is refused unless `stage: continue` frees the field; the LR schedules must agree on the source's updates."""
    src = tiny_train_config(steps=4)
    src.optim.decay_fraction = 0.0
    a = Trainer(copy.deepcopy(src), tmp_path / "a")
    a.fit()
    kept = ckpt.latest_path(tmp_path / "a")
    whole = tiny_train_config(steps=8)
    whole.optim.decay_fraction = 0.0
    w = Trainer(copy.deepcopy(whole), tmp_path / "w")
    w.fit()
    branch = copy.deepcopy(whole)
    branch.resume_from = str(kept)
    b = Trainer(branch, tmp_path / "b")
    b.continue_from(kept)
    assert b.step == 4 and b.resume_info["path"] == str(kept)
    b.fit()
    assert all(torch.equal(x, y) for x, y in zip(weights(w).values(), weights(b).values()))
    other = copy.deepcopy(branch)
    other.optim.weight_decay = 0.3
    with pytest.raises(ValueError, match="optim.weight_decay"):
        Trainer(other, tmp_path / "c").continue_from(kept)
    stage = copy.deepcopy(branch)
    stage.optim.decay_fraction = 0.25          # the decay of the longer run starts after the source's last update: same LR on updates 0..3
    with pytest.raises(ValueError, match="optim.decay_fraction"):
        Trainer(copy.deepcopy(stage), tmp_path / "d").continue_from(kept)
    stage.stage = "continue"
    s = Trainer(stage, tmp_path / "e")
    s.continue_from(kept)
    assert s.step == 4 and s.resume_info["stage"] == "continue"
    s.fit()
    late = copy.deepcopy(stage)
    late.optim.decay_fraction = 0.9            # would have decayed during the source's updates: refused
    with pytest.raises(ValueError, match="schedules must agree"):
        Trainer(late, tmp_path / "f").continue_from(kept)


@pytest.mark.parametrize("injection", ["mix", "parcae", "depth_mix"])
def test_looped_middle_trains_with_a_pass_count_per_step(tmp_path, injection):
    """A looped middle through the trainer: one T per step from t_choices (a pure function of seed and step, so a resumed run
    draws the same), recorded in the metrics; its own tensors train without weight decay on the injection; refusals by key."""
    from gdn_hybrid_architecture_ideas_b200.models.recur import pass_count_for_step
    from gdn_hybrid_architecture_ideas_b200.train.optim import param_groups

    cfg = tiny_train_config(steps=6)
    cfg.model = C.tiny_control_config()
    cfg.model.encoder.n_layers = 8
    lp = cfg.model.loop
    lp.recur_layers, lp.injection, lp.t_eval, lp.t_choices, lp.t_probs = (2, 6), injection, 2, [1, 2, 3], [0.3, 0.4, 0.3]
    cfg.metrics_jsonl, cfg.ckpt_every_steps = True, 3
    t = Trainer(copy.deepcopy(cfg), tmp_path / "r")
    start = {k: v.clone() for k, v in t.model.state_dict().items() if "recur" in k}
    ms = [t.train_step() for _ in range(6)]
    want = [pass_count_for_step(lp, cfg.seed, s) for s in range(6)]
    assert [m["T"] for m in ms] == want and len(set(want)) > 1 and all(math.isfinite(m["loss"]) for m in ms)
    moved = [k for k, v in t.model.state_dict().items() if "recur" in k and not torch.equal(v, start[k])]
    assert moved, "the injection's tensors did not train"
    groups = param_groups(t.model, cfg.optim)
    names = {n: g["weight_decay"] for g in groups for n in g.get("names", [])}
    for n, wd in names.items():
        if n.endswith(("injection.B", ".recur_mix", "injection.A_log", "injection.dt_bias")):
            assert wd == 0.0, n
    # a resumed run continues with the same pass counts and ends in the same state
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=3)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    for (k, x), (_, y) in zip(a.model.state_dict().items(), c.model.state_dict().items()):
        assert torch.equal(x, y), k
    bad = copy.deepcopy(cfg)
    bad.cuda_graphs = "microbatch"
    with pytest.raises(ValueError, match="cuda_graphs"):
        Trainer(bad, None)
    bad = copy.deepcopy(cfg)
    bad.model.encoder.attn_res = "block_entry"
    with pytest.raises(ValueError, match="attn_res"):
        Trainer(bad, None)
    bad = copy.deepcopy(cfg)
    bad.model.loop.recur_layers = ()
    if injection != "parcae":
        with pytest.raises(ValueError, match="looped middle"):
            Trainer(bad, None)


def test_looped_middle_with_a_pass_count_per_row(tmp_path):
    """`t_sampling: sequence`: every step's rows hold the same multiset of pass counts, dealt by (seed, step); the forwards are
    formed from rows of equal count (`micro_batch_by_t` rows at a time) and the accumulated gradient is the gradient of the
    sum of the rows' losses, each row at its own count; the metrics carry the rows' counts; a resume ends in the same state."""
    from gdn_hybrid_architecture_ideas_b200.models.recur import micro_plan, row_pass_counts, rows_by_count

    cfg = tiny_train_config(steps=4)
    cfg.model = C.tiny_control_config()
    cfg.model.encoder.n_layers, cfg.dtype = 8, "float64"
    cfg.data.batch_size = 4
    lp = cfg.model.loop
    lp.recur_layers, lp.injection, lp.t_eval, lp.t_choices, lp.t_probs, lp.t_sampling = (2, 6), "mix", 2, [1, 3], [0.5, 0.5], "sequence"
    cfg.micro_batch_by_t, cfg.ckpt_every_steps, cfg.optim.grad_clip = [2, 2, 1], 2, 0.0
    held = rows_by_count(lp, 4)
    assert held == [1, 1, 3, 3]
    deals = [row_pass_counts(held, cfg.seed, s) for s in range(8)]
    assert all(sorted(d) == held for d in deals) and len({tuple(d) for d in deals}) > 1 and deals[3] == row_pass_counts(held, cfg.seed, 3)
    assert micro_plan([3, 1, 3, 1], lambda t: {1: 2, 3: 1}[t]) == [([1, 3], 1), ([0], 3), ([2], 3)]
    t = Trainer(copy.deepcopy(cfg), tmp_path / "r")
    assert t.micro_rows(1) == 2 and t.micro_rows(3) == 1 and t.micro_rows(7) == 1 and len(t.row_plan(0)) == 3
    batch = t.batch_at(0).to(t.device)
    n = int(batch.target_valid.sum())
    t.device_step(copy.deepcopy(batch), n)
    got = t.flat.grads.clone()
    u = Trainer(copy.deepcopy(cfg), tmp_path / "u")
    counts = u.row_passes(0)
    u.flat.grads.zero_()
    for row, passes in enumerate(counts):                                   # every row on its own, at its own pass count
        from gdn_hybrid_architecture_ideas_b200.train.trainer import _slice

        u.pass_count = passes
        u._micro_loss(_slice(batch, row, row + 1), n)[0].backward()
    assert (got - u.flat.grads).abs().max() < 2e-6 * float(got.abs().max()) and float(got.abs().max()) > 0      # float32 gradient buffers
    m = t.train_step()
    assert m["T_rows"] == t.row_passes(1) and m["T"] == 2.0
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=2)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 2
    c.fit()
    for (k, x), (_, y) in zip(a.model.state_dict().items(), c.model.state_dict().items()):
        assert torch.equal(x, y), k
    for change, match in ((lambda c: setattr(c.model.loop, "t_probs", [0.3, 0.7]), "whole numbers"), (lambda c: setattr(c.model.loop, "injection", "depth_mix"), "depth_mix"),
                          (lambda c: setattr(c, "micro_batch_by_t", [0]), "micro_batch_by_t"), (lambda c: setattr(c.model.loop, "t_sampling", "row"), "t_sampling")):
        bad = copy.deepcopy(cfg)
        change(bad)
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    bad = copy.deepcopy(cfg)
    bad.model.loop.recur_layers, bad.model.loop.injection, bad.model.loop.t_sampling, bad.model.loop.t_eval = (), "none", "step", 1
    with pytest.raises(ValueError, match="micro_batch_by_t"):
        Trainer(bad, None)


def test_head_precision_bf16_rounds_the_operands_of_the_three_products(reference):
    """`head_precision: bf16` on the PyTorch path: logits, dh and dW are exact products of operands rounded once to bfloat16,
    accumulated in the compute dtype; equal to the reference's statement in float64; both heads agree; fp32 is untouched."""
    from ced.train import head_precision as RH

    from gdn_hybrid_architecture_ideas_b200.train import head_precision as HP
    from gdn_hybrid_architecture_ideas_b200.train.fused_head import chunked_ce, fused_linear_ce

    g = torch.Generator().manual_seed(0)
    h = torch.randn(3, 7, 16, generator=g, dtype=torch.float64, requires_grad=True)
    W = torch.randn(40, 16, generator=g, dtype=torch.float64, requires_grad=True)
    mine = HP.head_linear(h, W, "bf16")
    theirs = RH.head_linear(h.detach().clone().requires_grad_(), W.detach().clone().requires_grad_(), "bf16")
    assert torch.equal(mine, theirs) and not torch.equal(mine, torch.nn.functional.linear(h, W))
    up = torch.randn(mine.shape, generator=g, dtype=torch.float64)
    gh, gW = torch.autograd.grad(mine, (h, W), up)
    r = lambda x: x.to(torch.bfloat16).to(torch.float64)
    assert torch.equal(gh, r(up) @ r(W)) and torch.equal(gW, r(up).reshape(-1, 40).t() @ r(h).reshape(-1, 16))
    assert torch.equal(HP.head_linear(h, W, "fp32"), torch.nn.functional.linear(h, W))
    with pytest.raises(ValueError, match="head_precision"):
        HP.head_linear(h, W, "fp8")
    targets = torch.randint(0, 40, (3, 7), generator=g)
    a, b = torch.full((3, 7), 0.1, dtype=torch.float64), torch.full((3, 7), 1e-4, dtype=torch.float64)
    out = {}
    for prec in HP.PRECISIONS:
        for name, fn in (("fused", lambda: fused_linear_ce(h, W, targets, a, b, 8, precision=prec)[0]), ("chunked", lambda: chunked_ce(h, W, targets, a, b, 8, precision=prec)[0])):
            loss = fn()
            out[(prec, name)] = (loss.detach(), *torch.autograd.grad(loss, (h, W)))
    for prec in HP.PRECISIONS:
        for x, y in zip(out[(prec, "fused")], out[(prec, "chunked")]):
            assert torch.allclose(x, y, atol=1e-12, rtol=1e-10), prec
    assert not torch.allclose(out[("bf16", "fused")][0], out[("fp32", "fused")][0], atol=1e-9)
    cfg = tiny_train_config(steps=2)
    cfg.head_precision = "bf16"
    t = Trainer(cfg, None)
    assert math.isfinite(t.train_step()["loss"])


def test_qmix_static_pair_is_chosen_at_its_step_and_survives_a_resume(tmp_path):
    """model.encoder.gdn_qmix_select_step S: before step S the full query mix; the step-S record names each layer's pair;
    the pair sits in the checkpoint, a resume trains on in the pair form bit for bit; refused with what it is not built with."""
    cfg = tiny_train_config()
    cfg.model.encoder.gdn_qmix_select_step, cfg.log_stream_rms_every, cfg.micro_batch_size = 2, 2, 2
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    arms = [a.model.encoder.layers[i].gdn_arms for i in (8, 9, 10)]
    m0 = a.train_step()
    m1 = a.train_step()         # the stream log's cadence counts finished steps: the records of step indices 1 and 3 carry it
    assert "qmix_selection" not in m0 and "qmix_selection" not in m1 and all(x.chosen_sources() is None for x in arms)
    assert m1["qmix_weights"]["chosen"] == [None] * 6 and all(abs(sum(w) - 1) < 1e-6 for w in m1["qmix_weights"]["weights"])
    m2 = a.train_step()
    sel = m2["qmix_selection"]
    assert sel["step"] == 2 and sel["layers"] == [8, 9, 10] and sel["tokens"] == 2 * 48
    assert [x.chosen_sources() for x in arms] == sel["pair"] and all(len(p) == 2 and p[0] < p[1] for p in sel["pair"])
    for w, p in zip(sel["weights"], sel["pair"]):       # the two largest token-means, ties to the lower source
        assert sorted(sorted(range(3), key=lambda s: (-w[s], s))[:2]) == p
    m3 = a.train_step()
    assert "qmix_selection" not in m3 and m3["qmix_weights"]["chosen"][-3:] == sel["pair"]
    for w, p in zip(m3["qmix_weights"]["weights"][-3:], sel["pair"]):
        assert w[({0, 1, 2} - set(p)).pop()] == 0 and abs(sum(w) - 1) < 1e-6
    a.fit()
    assert "qmix_selection" not in a.last_metrics
    first = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    first.fit(3)                                           # stops after the choice, with a checkpoint
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert not any(x.qmix_static for x in (b.model.encoder.layers[i].gdn_arms for i in (8, 9, 10)))
    assert b.resume_from_checkpoint() and b.step == 3
    assert [b.model.encoder.layers[i].gdn_arms.chosen_sources() for i in (8, 9, 10)] == sel["pair"]
    assert all(b.model.encoder.layers[i].gdn_arms.qmix_static for i in (8, 9, 10))
    b.fit()
    wa, wb = weights(a), weights(b)
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    for key, value, match in (("activation_checkpoint", "block", "activation_checkpoint"), ("cuda_graphs", "microbatch", "cuda_graphs")):
        bad = copy.deepcopy(cfg)
        setattr(bad, key, value)
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)


def test_checkpoint_cross_read_trains_with_its_gate_floor(tmp_path):
    """model.encoder.gdn_ccr_spacing through the trainer: gates and translators in their optimizer groups, the floor held
    after every step, the log's summary, a bit-exact resume, and the refusals."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    cfg = tiny_train_config()
    cfg.model = C.tiny_control_config()
    e = cfg.model.encoder
    e.gdn_ccr_spacing, e.gdn_ccr_target, e.gdn_ccr_translator, e.gdn_ccr_gate_init, e.gdn_ccr_gate_floor = 8, "group_first", "key_head", 0.09, 0.09
    cfg.optim.zero_gate_decay, cfg.optim.ccr_translator_decay, cfg.log_every, cfg.activation_checkpoint = "none", "identity", 2, "layer"
    t = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    groups = optim.param_groups(t.model, cfg.optim)
    last = groups[-1]
    assert all(n.endswith("ccr_translator_delta") for n in last["names"]) and last["weight_decay"] == cfg.optim.weight_decay
    plain = [g for g in groups if g["weight_decay"] == 0.0][0]["names"]
    gates = [n for n, _ in t.model.named_parameters() if n.endswith("ccr_gate")]
    assert gates and all(n in plain for n in gates)
    l0 = t.train_step()["loss"]
    t.fit()
    assert t.last_metrics["loss"] < l0
    named = dict(t.model.named_parameters())
    assert all(float(named[n].min()) >= 0.09 - 1e-7 for n in gates)
    assert any(float(named[n].max()) > 0.09 + 1e-6 for n in gates) and any(float(named[n].min()) <= 0.09 + 1e-7 for n in gates)
    assert any(float(named[n].abs().max()) > 0 for n in last["names"])
    lines = [json.loads(x) for x in (tmp_path / "a" / "metrics.jsonl").read_text().splitlines()]
    logged = [x["ccr"] for x in lines if "ccr" in x]
    assert logged and len(logged[0]["ccr_gate"]) == len(gates) == len(logged[0]["ccr_translator_dev"])
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(3)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    wa, wc = weights(t), weights(c)
    assert all(torch.equal(wa[k], wc[k]) for k in wa)
    for key, value, match in (("activation_checkpoint", "host", "activation_checkpoint"), ("optim.zero_gate_decay", "decay", "zero_gate_decay"),
                              ("cuda_graphs", "microbatch", "cuda_graphs")):
        bad = copy.deepcopy(cfg)
        C.apply_override(bad, f"{key}={value}")
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    off = tiny_train_config()
    off.optim.ccr_translator_decay = "identity"
    with pytest.raises(ValueError, match="this model has none"):
        Trainer(off, None)


def test_gated_second_pass_switches_on_at_its_step(tmp_path):
    """loop.pass2_gate 'scalar' through the trainer: T = 1 before loop_switch_step and 2 from it on, the gate leaves 0 only
    then, pass 2's tensors in AdamW groups of their own at pass2_lr_scale, a bit-exact resume across the switch, refusals."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    cfg = tiny_train_config()
    cfg.model = C.tiny_control_config()
    lp = cfg.model.loop
    lp.pass2_gate, lp.pass2_layers, lp.t_max, lp.t_eval, lp.t_choices, lp.t_probs = "scalar", 4, 2, 2, [2], [1.0]
    cfg.loop_switch_step, cfg.optim.pass2_lr_scale, cfg.log_every, cfg.activation_checkpoint, cfg.optim.name = 3, 4.0, 1, "layer", "muon"
    t = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    groups = optim.param_groups(t.model, cfg.optim)
    own = [g for g in groups if any(n in ("loop_embedding_pass2", "hyper_connections.pass2_gate") for n in g["names"])]
    assert [g["names"] for g in own] == [["loop_embedding_pass2"], ["hyper_connections.pass2_gate"]]
    assert all(g["kind"] == "adamw" and g["lr_scale"] == cfg.optim.adamw_lr_scale * 4.0 for g in own) and own[0]["weight_decay"] > 0 and own[1]["weight_decay"] == 0
    rows = [t.train_step() for _ in range(3)]
    assert [r["T"] for r in rows] == [1, 1, 1] and all(r["pass2_alpha"] == 0.0 for r in rows) and "loop_usage" not in rows[-1]
    assert float(t.model.loop_embedding_pass2.abs().max()) == 0
    rows += [t.train_step() for _ in range(3)]
    assert [r["T"] for r in rows[3:]] == [2, 2, 2] and rows[3]["pass2_alpha"] != 0.0 and rows[5]["loop_usage"] > 0
    assert float(t.model.loop_embedding_pass2.abs().max()) > 0 and math.isfinite(rows[-1]["loop_usage"])
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(3)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    wa, wc = weights(t), weights(c)
    assert all(torch.equal(wa[k], wc[k]) for k in wa)
    for key, value, match in (("activation_checkpoint", "block", "activation_checkpoint"), ("cuda_graphs", "microbatch", "cuda_graphs"),
                              ("model.loop.t_choices", "[1, 2]", "t_choices"), ("loop_switch_step", 99, "loop_switch_step")):
        bad = copy.deepcopy(cfg)
        C.apply_override(bad, f"{key}={value}")
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    plain = tiny_train_config()
    plain.loop_switch_step = 2
    with pytest.raises(ValueError, match="this model has none"):
        Trainer(plain, None)
    plain = tiny_train_config()
    plain.optim.pass2_lr_scale = 2.0
    with pytest.raises(ValueError, match="this model has none"):
        Trainer(plain, None)


def test_copy_paste_head_trains_and_then_alone_on_a_frozen_trunk(tmp_path):
    """model.cp_head through the trainer: the mixture's loss on the chunked head, the head's tensors on AdamW, a bit-exact resume;
    then freeze_trunk: a head added to a finished trunk (init_from) trains alone, the trunk's bytes stay the source's, the
    checkpoint carries the trunk's hash, a changed trunk is refused at the save and at a resume, and the refusals by name."""
    from gdn_hybrid_architecture_ideas_b200.train import optim

    base = tiny_train_config(head_impl="chunked")
    base.model = C.tiny_control_config()
    base.log_every = 2
    trunk = Trainer(copy.deepcopy(base), tmp_path / "trunk")
    trunk.fit()
    source = ckpt.latest_path(tmp_path / "trunk")
    cfg = copy.deepcopy(base)
    cfg.model.cp_head.enabled, cfg.model.cp_head.d_c, cfg.model.cp_head.qk_norm, cfg.optim.name = True, 8, True, "muon"
    joint = Trainer(copy.deepcopy(cfg), tmp_path / "joint")
    groups = optim.param_groups(joint.model, cfg.optim)
    assert not any(n.startswith("cp_head.") for g in groups if g["kind"] == "muon" for n in g["names"])
    plain = [n for g in groups if g["weight_decay"] == 0.0 for n in g["names"]]
    assert "cp_head.w_copy" in plain and "cp_head.qk_gain" in plain and "cp_head.w_q" not in plain
    l0 = joint.train_step()["loss"]
    joint.fit()
    assert math.isfinite(joint.last_metrics["loss"]) and joint.last_metrics["loss"] < l0 + 0.5          # (random tokens: a handful of steps only has to stay sane)
    lines = [json.loads(x) for x in (tmp_path / "joint" / "metrics.jsonl").read_text().splitlines()]
    assert any(0 < x.get("cp_lambda", 0) < 1 for x in lines)
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(3)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 3
    c.fit()
    assert all(torch.equal(x, y) for x, y in zip(weights(joint).values(), weights(c).values()))
    # the head alone on the finished trunk
    frozen = copy.deepcopy(cfg)
    frozen.freeze_trunk, frozen.init_from, frozen.optim.name = True, str(source), "adamw"
    f = Trainer(copy.deepcopy(frozen), tmp_path / "frozen")
    src = ckpt.load(source)["model"]
    assert f.init_info["grown"] == sorted(n for n in f.model.state_dict() if n.startswith("cp_head.")) and len(f.init_info["trunk_sha256"]) == 64
    head0 = {n: p.detach().clone() for n, p in f.model.named_parameters() if n.startswith("cp_head.")}
    f.fit()
    now = f.model.state_dict()
    assert all(torch.equal(now[k], src[k]) for k in src) and any(not torch.equal(now[n], v) for n, v in head0.items())
    assert all(not p.requires_grad for n, p in f.model.named_parameters() if not n.startswith("cp_head."))
    saved = ckpt.load(ckpt.latest_path(tmp_path / "frozen"))
    assert saved["freeze_trunk"]["trunk_sha256"] == f.init_info["trunk_sha256"] and saved["freeze_trunk"]["tensors"] == len(src)
    r = Trainer(copy.deepcopy(frozen), tmp_path / "frozen")
    assert r.resume_from_checkpoint() and r.step == frozen.steps
    saved["model"]["embed.weight"] = saved["model"]["embed.weight"] + 1
    with pytest.raises(ValueError, match="does not hash"):
        Trainer(copy.deepcopy(frozen), None).load_state_dict(saved)
    with torch.no_grad():
        f.model.embed.weight.add_(1.0)
    with pytest.raises(RuntimeError, match="changed"):
        f.save_checkpoint()
    for change, match in ((lambda t: setattr(t, "init_from", None), "init_from"), (lambda t: setattr(t.model.cp_head, "enabled", False), "cp_head"),
                          (lambda t: setattr(t, "activation_checkpoint", "layer"), "activation_checkpoint")):
        bad = copy.deepcopy(frozen)
        change(bad)
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    fused = copy.deepcopy(cfg)
    fused.head_impl = "fused"
    with pytest.raises(ValueError, match="head_impl"):
        Trainer(fused, None)


def test_injection_matrix_under_muon_and_the_scalars_own_learning_rate():
    """optim.recur_b puts the looped middle's dense injection matrix on Muon (with the run's decay, or in a last group without);
    optim.layer_scalar_a_lr_scale gives the residual scalars' a a group of its own; both are refused where they name nothing."""
    from gdn_hybrid_architecture_ideas_b200.models import build_model
    from gdn_hybrid_architecture_ideas_b200.train import optim

    mc = C.tiny_control_config()
    mc.encoder.n_layers = 8
    mc.loop.recur_layers, mc.loop.injection, mc.loop.t_eval, mc.loop.t_max, mc.loop.t_choices, mc.loop.t_probs = (2, 6), "parcae", 2, 2, [2], [1.0]
    model = build_model(mc)
    o = C.OptimConfig(name="muon")
    B = "encoder.recur_injection.B"
    base = optim.param_groups(model, o)
    assert B in [n for g in base if g["kind"] == "adamw" and g["weight_decay"] == 0 for n in g["names"]]
    o.recur_b = "muon"
    g1 = optim.param_groups(model, o)
    assert B in g1[0]["names"] and g1[0]["kind"] == "muon" and g1[0]["weight_decay"] == o.weight_decay and len(g1) == len(base)
    o.recur_b = "muon_no_decay"
    g2 = optim.param_groups(model, o)
    assert g2[-1] == {"kind": "muon", "names": [B], "params": g2[-1]["params"], "weight_decay": 0.0, "lr_scale": 1.0} and B not in [n for g in g2[:-1] for n in g["names"]]
    assert sum(len(g["names"]) for g in g2) == sum(len(g["names"]) for g in base)
    cfg = tiny_train_config()
    cfg.model, cfg.optim.name, cfg.optim.recur_b = mc, "muon", "muon"
    t = Trainer(copy.deepcopy(cfg), None)
    before = dict(t.model.named_parameters())[B].detach().clone()
    t.train_step()
    assert not torch.equal(before, dict(t.model.named_parameters())[B])
    for change, match in ((lambda c: setattr(c.optim, "name", "adamw"), "read under optim.name 'muon'"), (lambda c: setattr(c.optim, "recur_b", "sgd"), "one of"),
                          (lambda c: setattr(c.model.loop, "recur_inject_b", "diag"), "this model has none")):
        bad = copy.deepcopy(cfg)
        change(bad)
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    sc = C.tiny_control_config()
    sc.encoder.layer_scalars = "skip_x0"
    o2 = C.OptimConfig(name="muon", layer_scalar_a_lr_scale=0.01)
    groups = optim.param_groups(build_model(sc), o2)
    assert groups[-1]["names"] == ["encoder.skip_gain"] and groups[-1]["weight_decay"] == 0 and abs(groups[-1]["lr_scale"] - 0.01 * o2.adamw_lr_scale) < 1e-12
    assert "encoder.x0_gain" in [n for g in groups[:-1] for n in g["names"]]
    with pytest.raises(ValueError, match="this model has none"):
        optim.param_groups(build_model(C.tiny_control_config()), o2)
    with pytest.raises(ValueError, match="finite number above 0"):
        optim.param_groups(build_model(sc), C.OptimConfig(layer_scalar_a_lr_scale=0.0))


def test_keys_that_nothing_reads_are_refused_off_their_defaults():
    """A key of a part this framework does not build loads and round-trips, and is refused by name when it is set: it would
    change nothing. Every key of the config is either read by the code, in a refusal table, or on that list."""
    import dataclasses
    import re
    import subprocess

    cfg = tiny_train_config()
    assert C.unsupported_options(cfg) == []
    for key, value in (("model.loop.hc_streams", 4), ("loss.aux_weight", 0.25), ("model.decoder.ffn_experts", 8), ("optim.normuon_beta2", 0.9), ("stage_shape", "[4, 4096]")):
        bad = copy.deepcopy(cfg)
        C.apply_override(bad, f"{key}={value}")
        assert any(x.startswith(key + "=") and "read by nothing" in x for x in C.unsupported_options(bad)), key
        with pytest.raises(ValueError, match="read by nothing"):
            Trainer(bad, None)
    root = Path(__file__).resolve().parent.parent
    files = subprocess.run(["git", "ls-files", "gdn_hybrid_architecture_ideas_b200/*.py", "scripts/*.py", "bench.py"], capture_output=True, text=True, cwd=root).stdout.split()
    src = "".join((root / f).read_text() for f in files if not f.endswith("gdn_hybrid_architecture_ideas_b200/config.py"))
    cfg_src = (root / "gdn_hybrid_architecture_ideas_b200" / "config.py").read_text()
    tables = cfg_src[cfg_src.index("_BUILT = {"):]

    def leaves(cls, prefix=""):
        for f in dataclasses.fields(cls):
            t = f.default_factory() if f.default_factory is not dataclasses.MISSING else None
            if dataclasses.is_dataclass(t):
                yield from leaves(type(t), prefix + f.name + ".")
            else:
                yield prefix + f.name, f.name

    orphans = [full for full, leaf in leaves(C.TrainConfig) if not re.search(r"\b" + re.escape(leaf) + r"\b", src) and leaf not in tables
               and not full.startswith("optim.ours.")]
    assert orphans == [], orphans


def test_looped_encoder_decoder_trains_through_the_trainer(tmp_path):
    """arch looped_ced: decoder positions in spans from the data (exactly the row's capacity, from a generator of their own),
    a pass count per step, the two heads' loss and metrics, loop-boundary tensors on AdamW without decay, a bit-exact resume;
    the accumulated gradient does not depend on the micro-batch size; refusals by key."""
    from gdn_hybrid_architecture_ideas_b200.models.recur import pass_count_for_step
    from gdn_hybrid_architecture_ideas_b200.train.optim import param_groups

    cfg = tiny_train_config(steps=4)
    cfg.model = C.tiny_looped_config()
    cfg.model.loop.hyper_connections, cfg.model.loop.draft_loss_weight = "static", 0.2
    cfg.loss.aux_weight, cfg.ckpt_every_steps, cfg.dtype = 0.5, 2, "float64"
    t = Trainer(copy.deepcopy(cfg), tmp_path / "r")
    assert t.capacity == 16 and t.data.capacity == 16
    b0 = t.batch_at(0)
    assert b0.dec_mask.shape == b0.tokens.shape and b0.dec_mask.sum(1).tolist() == [16] * cfg.data.batch_size
    assert torch.equal(b0.dec_mask, t.batch_at(0).dec_mask) and not torch.equal(b0.dec_mask, t.batch_at(1).dec_mask)
    groups = param_groups(t.model, cfg.optim)
    kind = {n: (g["kind"], g["weight_decay"]) for g in groups for n in g["names"]}
    assert kind["injection.B"] == ("adamw", 0.0) and kind["hyper_connections.mix_weights"] == ("adamw", 0.0) and kind["loop_embedding"][0] == "adamw"
    ms = [t.train_step() for _ in range(4)]
    assert [m["T"] for m in ms] == [pass_count_for_step(cfg.model.loop, cfg.seed, s) for s in range(4)]
    assert all(math.isfinite(m["loss"]) and m["ce_dec"] > 0 and m["ce_aux"] > 0 and m["dropped"] == 0 for m in ms)
    assert any("ce_draft_loop1" in m for m in ms) and ms[-1]["loss"] < ms[0]["loss"] + 0.5
    whole, halves = Trainer(copy.deepcopy(cfg), tmp_path / "w"), copy.deepcopy(cfg)
    halves.micro_batch_size = cfg.data.batch_size // 2
    halves = Trainer(halves, tmp_path / "h")
    for tr in (whole, halves):
        tr.train_step()
    assert (whole.flat.grads - halves.flat.grads).abs().max() < 2e-6 * float(whole.flat.grads.abs().max())
    a = Trainer(copy.deepcopy(cfg), tmp_path / "a")
    a.fit()
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=2)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 2
    c.fit()
    for (k, x), (_, y) in zip(a.model.state_dict().items(), c.model.state_dict().items()):
        assert torch.equal(x, y), k
    for change, match in ((lambda c: setattr(c, "cuda_graphs", "microbatch"), "cuda_graphs"), (lambda c: setattr(c.data, "kind", "uniform"), "data.kind"),
                          (lambda c: setattr(c, "freeze_trunk", True), "freeze_trunk|looped_ced")):
        bad = copy.deepcopy(cfg)
        change(bad)
        with pytest.raises(ValueError, match=match):
            Trainer(bad, None)
    plain = tiny_train_config(steps=2)
    plain.loss.aux_weight = 0.5
    with pytest.raises(ValueError, match="aux_weight"):
        Trainer(plain, None)


def test_copy_paste_pointer_trains_on_its_auxiliary_loss_beside_the_plain_loss(tmp_path):
    """cp_head.train_mode aux through the trainer: the loss is p_LM's plus aux_weight x the pointer's own; the trunk's gradient
    from p_LM's term is the plain model's; the pointer's tensors move; metrics cp_aux / cp_aux_sink; a bit-exact resume."""
    cfg = tiny_train_config(steps=4)
    cfg.model = C.tiny_full_config()
    cfg.model.encoder.gdn_write_variant, cfg.model.encoder.gdn_write_mix = "none", "none"
    plain = copy.deepcopy(cfg)
    h = cfg.model.cp_head
    h.enabled, h.d_c, h.qk_norm, h.pointer_input, h.train_mode, h.aux_weight = True, 8, True, "mix", "aux", 0.5
    cfg.head_impl, plain.head_impl, cfg.ckpt_every_steps = "chunked", "chunked", 2
    t, base = Trainer(copy.deepcopy(cfg), tmp_path / "a"), Trainer(plain, tmp_path / "p")
    assert "cp_head.w_copy" not in t.model.state_dict() and "cp_head.mix.read_q.query" in t.model.state_dict()
    start = {n: p.detach().clone() for n, p in t.model.named_parameters() if n.startswith("cp_head.")}
    m, mb = t.train_step(), base.train_step()
    assert m["cp_aux"] > 0 and 0 <= m["cp_aux_sink"] <= 1 and m["loss"] > mb["loss"] and abs(m["ce_dec"] - mb["ce_dec"]) < 1e-5
    assert abs(m["loss"] - mb["loss"] - 0.5 * m["cp_aux"]) < 1e-4
    for _ in range(3):
        t.train_step()
    moved = [n for n, p in t.model.named_parameters() if n.startswith("cp_head.") and not torch.equal(p, start[n])]
    assert {"cp_head.w_q", "cp_head.w_k", "cp_head.k_sink"} <= set(moved)
    b = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    b.fit(until_step=2)
    c = Trainer(copy.deepcopy(cfg), tmp_path / "b")
    assert c.resume_from_checkpoint() and c.step == 2
    c.fit()
    for (k, x), (_, y) in zip(t.model.state_dict().items(), c.model.state_dict().items()):
        assert torch.equal(x, y), k


def test_add_on_copy_paste_head_leaves_the_trunk_training_as_the_plain_model(tmp_path):
    """cp_head.train_mode addon through the trainer: the trunk's and the LM head's updates are those of the model without the
    head (their loss is p_LM's and their clip their own), while the head trains on the mixture's term under a clip of its own;
    metrics ce_mix / cp_lambda / cp_grad_norm; data parallelism is refused."""
    cfg = tiny_train_config(steps=3)
    cfg.model = C.tiny_full_config()
    cfg.model.encoder.gdn_write_variant = "none"
    cfg.head_impl, cfg.log_every, cfg.optim.grad_clip = "chunked", 1, 0.05          # a clip that binds: the two norms must stay apart
    plain = copy.deepcopy(cfg)
    h = cfg.model.cp_head
    h.enabled, h.d_c, h.qk_norm, h.pointer_input, h.train_mode = True, 8, True, "mix", "addon"
    t, base = Trainer(copy.deepcopy(cfg), tmp_path / "a"), Trainer(plain, tmp_path / "p")
    head0 = {n: p.detach().clone() for n, p in t.model.named_parameters() if n.startswith("cp_head.")}
    for _ in range(3):
        m, mb = t.train_step(), base.train_step()
        assert abs(m["grad_norm"] - mb["grad_norm"]) < 1e-4 * mb["grad_norm"] and abs(m["ce_dec"] - mb["ce_dec"]) < 1e-5
        assert m["ce_mix"] > 0 and m["cp_grad_norm"] > 0 and 0 < m["cp_lambda"] < 1 and m["loss"] > mb["loss"]
    ours, theirs = t.model.state_dict(), base.model.state_dict()
    worst = max(float((ours[k] - v).abs().max()) for k, v in theirs.items())
    assert worst < 1e-6, worst
    assert all(not torch.equal(p, head0[n]) for n, p in t.model.named_parameters() if n in ("cp_head.w_q", "cp_head.w_copy", "cp_head.k_sink"))


def test_copy_paste_pointer_on_a_shared_attention_head_trains(tmp_path):
    """cp_head.pointer_input shared through the trainer: no W_Q / W_K, the head and the trunk train; refused with activation checkpointing."""
    cfg = tiny_train_config(steps=2)
    cfg.model = C.tiny_full_config()
    cfg.model.encoder.gdn_write_variant, cfg.model.encoder.gdn_write_mix, cfg.model.encoder.nope_global_layers = "none", "none", (2,)
    h = cfg.model.cp_head
    h.enabled, h.qk_norm, h.pointer_input, h.shared_head, cfg.head_impl, cfg.log_every = True, True, "shared", 1, "chunked", 1
    t = Trainer(copy.deepcopy(cfg), tmp_path / "s")
    names = [n for n, _ in t.model.named_parameters() if n.startswith("cp_head.")]
    assert names == ["cp_head.k_sink", "cp_head.w_copy", "cp_head.qk_gain"] and t.model.cp_head.k_sink.shape[0] == cfg.model.encoder.attention.head_dim
    start = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    ms = [t.train_step() for _ in range(2)]
    assert all(math.isfinite(m["loss"]) and 0 < m["cp_lambda"] < 1 for m in ms)
    assert all(not torch.equal(p, start[n]) for n, p in t.model.named_parameters() if n in ("cp_head.k_sink", "cp_head.w_copy", "encoder.layers.11.mixer.q_proj.weight"))
    bad = copy.deepcopy(cfg)
    bad.activation_checkpoint = "layer"
    with pytest.raises(ValueError, match="activation_checkpoint"):
        Trainer(bad, None)
