"""The host pool's lanes: the emulated side stream shows the ordering mistakes of asynchronous copies on a CPU."""

import gc

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import act_checkpoint as A
from gdn_hybrid_architecture_ideas_b200.models import build_model


def test_a_copy_runs_only_when_waited_for_and_its_target_is_poisoned_until_then():
    lane = A.EmuLane()
    src, dst = torch.arange(6.0), torch.zeros(6)
    ticket = lane.copy(dst, src)
    lane.record(src)
    assert torch.isnan(dst).all()                    # a reader that forgot its wait
    lane.compute_waits(ticket)
    assert torch.equal(dst, src) and lane.done == ticket


def test_a_source_freed_before_its_copy_ran_is_reported_unless_it_was_recorded():
    lane = A.EmuLane()
    dst = torch.zeros(4)
    src = torch.ones(4)
    ticket = lane.copy(dst, src)
    del src
    gc.collect()
    with pytest.raises(A.LaneOrderError, match="not recorded"):
        lane.host_waits(ticket)
    src = torch.ones(4)
    ticket = lane.copy(dst, src)
    lane.record(src)
    del src
    gc.collect()
    lane.host_waits(ticket)
    assert torch.equal(dst, torch.ones(4))


def test_the_poison_of_a_returned_buffer_cannot_pass_a_copy_that_reads_it():
    pool = A.HostPool(torch.device("cpu"), overlap=True, min_bytes=0)
    t = torch.arange(8.0)
    h = pool.pack(t)
    out = pool._start_back(h) or h.back
    ticket = h.back_ticket
    h.back = None
    del h                                            # the buffer goes back (its NaN fill is queued BEHIND the copy back)
    gc.collect()
    assert torch.isnan(out).all()
    pool.lane.compute_waits(ticket)
    assert torch.equal(out, t)
    pool.drain()
    (buf,) = pool.free[((8,), torch.float32)]
    assert torch.isnan(buf).all()


def _grads(mode, pool=None):
    cfg = C.tiny_full_config()
    torch.manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (2, 24))
    torch.manual_seed(1)
    model = build_model(cfg)
    model.encoder.activation_checkpoint = mode
    if pool is not None:
        model.encoder.host_pool = pool
    model(tok, torch.zeros_like(tok)).logits.float().square().mean().backward()
    return {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}


def test_overlapped_parking_gives_the_same_gradients_and_prefetches():
    want = _grads("none")
    pool = A.HostPool(torch.device("cpu"), overlap=True, min_bytes=0)
    got = _grads("host_overlap", pool)
    assert want.keys() == got.keys()
    for k in want:
        assert torch.equal(want[k], got[k]), k
    st = pool.stats
    assert st["packed"] > 0 and st["prefetched"] > 0 and st["prefetch_hits"] > 0
    assert st["prefetch_hits"] <= st["prefetched"]
    gc.collect()
    pool.drain()
    assert st["allocated"] <= st["packed"]
    assert all(torch.isnan(b).all() for bufs in pool.free.values() for b in bufs if b.is_floating_point())


def test_a_backward_that_skips_its_wait_reads_poison():
    """The emulation's point: dropping the compute's wait for a copy back shows as NaN gradients, not as a pass."""
    pool = A.HostPool(torch.device("cpu"), overlap=True, min_bytes=0)
    pool.lane.compute_waits = lambda ticket: None
    got = _grads("host_overlap", pool)
    assert any(torch.isnan(g).any() for g in got.values())


def test_the_lead_bounds_the_copies_in_flight():
    pool = A.HostPool(torch.device("cpu"), overlap=True, lead=2, min_bytes=0)
    keep = [torch.full((4,), float(i)) for i in range(5)]
    handles = [pool.pack(t) for t in keep]
    assert len(pool.in_flight) == 2 and pool.lane.done == 3      # the three oldest were waited for
    assert torch.equal(handles[0].buf, keep[0]) and torch.isnan(handles[4].buf).all()
    assert torch.equal(pool.unpack(handles[4]), keep[4])


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["host", "host_overlap"])
def test_parked_activations_train_the_same_on_the_device(mode):
    """On a GPU the copies run on a CUDA stream (pinned buffers, events): the losses are those of keeping everything, up to
    the summation order of the sliced weight-gradient GEMMs (floating-point reductions, not fixed from run to run)."""
    from gdn_hybrid_architecture_ideas_b200.ops import native
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    def run(m):
        model = C.hybrid_model_config("60m", full=True)
        model.encoder.n_layers, model.encoder.nope_global_layers, model.vocab_size = 4, (0,), 4096
        cfg = C.TrainConfig(model=model, data=C.DataConfig(kind="synthetic", seq_len=1024, batch_size=2, seed=5), steps=100, seed=7)
        cfg.autocast, cfg.head_impl, cfg.metrics_jsonl, cfg.log_every = "bfloat16", "fused", False, 0
        cfg.optim.warmup_steps, cfg.optim.lr, cfg.activation_checkpoint = 1, 1e-4, m
        t = Trainer(cfg, None, None)
        losses = [t.train_step()["loss"] for _ in range(3)]
        native.check_status()
        return losses, t

    want, _ = run("none")
    got, t = run(mode)
    pool = t.model.encoder.host_pool
    assert pool is not None and pool.stats["packed"] > 0 and pool.stats["unpacked"] > 0
    if mode == "host_overlap":
        assert pool.stats["prefetched"] > 0
    assert got[0] == want[0] and max(abs(a - b) for a, b in zip(got, want)) < 1e-3, (got, want)


def test_views_into_a_larger_storage_are_handed_back_untouched():
    """Two neighbouring slices of one buffer, saved for a backward that addresses them as a single block, come back as the
    same views: the pool parks only tensors that own their whole storage."""
    pool = A.HostPool(torch.device("cpu"), min_bytes=0)
    flat = torch.arange(24.0)
    a, b = flat[:8].view(2, 4), flat[8:24].view(4, 4)
    ha, hb, hc = pool.pack(a), pool.pack(b), pool.pack(torch.ones(3))
    assert pool.unpack(ha) is a and pool.unpack(hb) is b and pool.stats["kept"] == 2 and pool.stats["packed"] == 1
    joined = torch.as_strided(pool.unpack(ha), (6, 4), (4, 1))
    assert torch.equal(joined, flat.view(6, 4))
    assert torch.equal(pool.unpack(hc), torch.ones(3))
