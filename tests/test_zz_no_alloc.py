"""The allocation-free C entry point of decode attention (`ghb_decode_attention_noalloc`, csrc/noalloc.h).

Some callers of this library cannot allocate device memory when they need attention over a static cache: a serving
loop whose device memory is fully planned at start-up, a plug-in that only receives raw pointers from a host runtime,
a latency path where an allocator call is not allowed. For them the library keeps the kernel's split-softmax scratch
in a fixed device array of its own. This test calls that entry through its exported C symbol (ctypes, raw pointers,
no torch allocation inside the call) twice in a row, with different inputs, and checks each result against the regular
entry that takes caller-provided scratch. It also checks that a size beyond the built-in scratch is refused with a
message. The file sorts last so every other test has run before it when a run stops at the first failure.
"""

import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

SO = Path(__file__).resolve().parent.parent / "gdn_hybrid_architecture_ideas_b200" / "_native.so"


def _inputs(seed, B, T, Hq, Hkv, rot, cap):
    g = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda", 0)
    q = torch.randn(B, Hq, 64, generator=g).to(dev)
    k = torch.randn(B, T, Hkv, 64, generator=g).to(dev, torch.bfloat16)
    v = torch.randn(B, T, Hkv, 64, generator=g).to(dev, torch.bfloat16)
    lens = torch.randint(T // 2, T + 1, (B,), generator=g).to(dev, torch.int32)
    n_ang = cap + 1
    inv = 1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    ang = torch.arange(n_ang, dtype=torch.float64)[:, None] * inv
    return q, k, v, lens, ang.cos().float().to(dev).contiguous(), ang.sin().float().to(dev).contiguous()


def test_no_alloc_entry_matches_regular_entry_twice():
    from gdn_hybrid_architecture_ideas_b200.ops import native

    ext = native.ext()
    lib = ctypes.CDLL(str(SO))
    fn = lib.ghb_decode_attention_noalloc
    fn.restype = ctypes.c_int
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, ctypes.c_char_p, I]
    B, T, Hq, Hkv, rot, cap, splits = 3, 700, 8, 2, 16, 200, 5
    stream = torch.cuda.current_stream().cuda_stream
    for seed in (11, 12):      # two calls in a row share the library's scratch: the second must not see the first's leftovers
        q, k, v, lens, cos_t, sin_t = _inputs(seed, B, T, Hq, Hkv, rot, cap)
        want = torch.empty(B, Hq, 64, dtype=torch.bfloat16, device=q.device)
        part_o = torch.zeros(B * Hq * splits * 64, device=q.device)
        part_ml = torch.zeros(B * Hq * splits * 2, device=q.device)
        ext.decode_attention(q, k, v, lens, None, cos_t, sin_t, want, part_o, part_ml, rot, cap, splits, 0.125)
        got = torch.empty_like(want)
        err = ctypes.create_string_buffer(256)
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(), None, cos_t.data_ptr(), sin_t.data_ptr(), got.data_ptr(),
                B, T, Hq, Hkv, rot, cap, cap + 1, splits, 0.125, stream, err, 256)
        assert rc == 0, err.value
        torch.cuda.synchronize()
        assert torch.equal(got, want), (got.float() - want.float()).abs().max()      # the same kernels on the same inputs: bit for bit
    # a request larger than the built-in scratch is refused with a message and launches nothing
    err = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(), None, cos_t.data_ptr(), sin_t.data_ptr(), got.data_ptr(),
            B, T, Hq, Hkv, rot, cap, cap + 1, 1 << 20, 0.125, stream, err, 256)
    assert rc == 1 and b"exceeds the built-in scratch" in err.value
    # a rotary width without angle tables is refused before anything is launched
    err = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(), None, None, None, got.data_ptr(),
            B, T, Hq, Hkv, rot, cap, 0, splits, 0.125, stream, err, 256)
    assert rc == 1 and b"cos/sin tables" in err.value
