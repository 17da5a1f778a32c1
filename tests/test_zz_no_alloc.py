"""The no-allocation decode attention entry point, called through its exported C symbol.

Some callers of the attention kernel cannot obtain device memory where they make the call (a
loop that must not stall in the allocator, a host framework that owns all memory, a process
whose budget was handed out at start-up), so `sb_attention_decode_static` keeps its scratch in
a fixed array inside the library.  This test calls it twice in a row on steps that need
several splits and compares each result with the ordinary entry point's, which is given
scratch by the caller (bit for bit: the same kernel), and with the plain float32 attention
kernel; a refused oversize step in between must leave it usable.  This file is named to be collected last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(hq, hkv, hd, lengths, seed):
    """A filled cache and a one-token-per-sequence step over it (queries at the last position)."""
    from sonicboom_b200.cache import Cache, KVNeed
    from sonicboom_b200.engine.step import StepEntry, StepPlan
    g = torch.Generator().manual_seed(seed)
    cache = Cache([KVNeed(hkv, hd, 0)], [None], 64 * 64, torch.bfloat16, DEV)
    slots = []
    for n in lengths:
        s = cache.open()
        cache.reserve(s, n)
        cache.advance(s, n - 1)                  # the step brings the n-th token
        slots.append(s)
    storage = cache.groups[0].entry_storage(0)
    storage.copy_(torch.randn(storage.shape, generator=g).to(torch.bfloat16))
    plan = StepPlan(cache, [StepEntry(s, [0], []) for s in slots], DEV)
    q = torch.randn(len(lengths), hq, hd, generator=g).to(torch.bfloat16).to(DEV)
    return cache, plan, storage, q


@pytest.mark.parametrize("hq,hkv,hd", [(14, 2, 64), (28, 4, 128)])
def test_static_scratch_entry_point_matches_the_ordinary_one(hq, hkv, hd):
    from sonicboom_b200 import ops
    lib = ops.attention_lib(hd)
    fn = lib.sb_attention_decode_static                      # the exported C symbol
    assert lib.sb_attention_static_scratch_bytes() == 8 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def ptr(t):
        return ctypes.c_void_p(t.data_ptr())

    def call(plan, storage, q, out, n_rows=None, max_len=None):
        g = plan.groups[0]
        return fn(ptr(q), ptr(out), n_rows or q.shape[0], plan.n_seqs, plan.max_new, ptr(plan.seq_row0),
                  ptr(plan.seq_pos0), ptr(g.page_off), ptr(g.page_ids), g.page_size, ptr(storage), hq,
                  hkv, hd, 0, ctypes.c_float(hd ** -0.5), max_len or plan.max_len, stream)

    def check(lengths, seed, what):
        cache, plan, storage, q = _setup(hq, hkv, hd, lengths, seed)
        want = torch.empty(len(lengths), hq * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention(q, want, plan, 0, storage, hq, hkv, hd, 0, hd ** -0.5, kernel="mma")   # the same kernel
        plain = torch.empty_like(want)                       # and another one: float32 arithmetic
        ops.attention(q, plain, plan, 0, storage, hq, hkv, hd, 0, hd ** -0.5, kernel="plain")
        got = torch.full_like(want, float("nan"))
        rc = call(plan, storage, q, got)
        assert rc == 0, lib.sb_last_error().decode()
        torch.cuda.synchronize()
        assert plan.max_len > 256                            # several splits: scratch is in use
        assert torch.equal(got, want), (what, float((got.float() - want.float()).abs().max()))
        err = float((got.float() - plain.float()).abs().max() / plain.float().abs().max())
        assert err < 2e-2, (what, err)
        return plan, storage, q, got

    check([700, 300, 1025, 64], 1, "first call")
    plan, storage, q, got = check([2000, 257], 2, "second call")

    # a step beyond the built-in array is refused before anything runs, with both numbers in
    # the message (the bounds on rows and sequence length alone decide this)
    rc = call(plan, storage, q, got, n_rows=4096, max_len=16000)
    msg = lib.sb_last_error().decode()
    assert rc != 0 and "8388608" in msg and "scratch" in msg, msg
    # the refusal left the array and its counters usable
    check([900, 513, 70], 3, "after the refused call")
