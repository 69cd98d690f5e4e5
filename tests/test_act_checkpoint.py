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
