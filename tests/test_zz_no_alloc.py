"""The allocation-free send-counter entry point against the regular one.

Some users of this library cannot allocate device memory where they call it: inside the packet
loop a cudaMalloc would stall every stream of the GPU, and a program that receives packets straight
into device buffers of its own never creates a bnk_batch.  bnk_assign_counters_noalloc serves them
from a scratch area built into the library.  This test hands the same packets to it and to
bnk_seal_submit(BNK_F_ASSIGN_COUNTERS) and wants identical counters, twice in a row (the second,
smaller call runs over the first call's leftovers in the shared scratch).  The device buffers the
caller "owns" come from torch here, which stands in for such a caller's own memory.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _regular(ctx, slots):
    """Counters from the existing entry point: a seal submit that assigns them."""
    from bnk_b200.device import F_ASSIGN_COUNTERS

    n = len(slots)
    b = ctx.batch(n, n * 64)
    b.off[:n] = (np.arange(n, dtype=np.uint64) * 64).astype(np.uint32)
    b.len[:n] = 16
    b.slot[:n] = slots
    b.counter[:n] = 0xDEAD
    b.seal(n, F_ASSIGN_COUNTERS)
    out = np.array(b.counter[:n])
    b.close()
    return out


def _no_alloc(ctx, slots, torch):
    from bnk_b200 import _lib

    n = len(slots)
    d_slot = torch.from_numpy(slots.view(np.int32).copy()).cuda()
    d_ctr = torch.full((n,), 0xDEAD, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    rc = _lib.lib().bnk_assign_counters_noalloc(ctx._h, None, C.c_void_p(d_slot.data_ptr()), n,
                                                C.c_void_p(d_ctr.data_ptr()))
    _lib.check(rc, ctx._h)
    ctx.synchronize()
    torch.cuda.synchronize()
    return d_ctr.cpu().numpy().view(np.uint64)


def test_no_alloc_counters_match_seal_submit(gpu_lib):
    torch = pytest.importorskip("torch")
    from bnk_b200 import Context, _lib

    n_peers = 70_000  # two radix digits
    rng = np.random.default_rng(99)
    keys = np.zeros((n_peers, 32), np.uint8)
    ridx = np.zeros(n_peers, np.uint32)
    a = Context(max_keypairs=n_peers, flow_capacity=0)
    b = Context(max_keypairs=n_peers, flow_capacity=0)
    try:
        for c in (a, b):
            c.set_keypairs(0, keys, keys, ridx)
            c.set_send_counter(7, _lib.REJECT_AFTER_MESSAGES - 2)  # saturates inside the first call
            c.set_send_counter(69_999, 1 << 33)
        hot = np.array([7, 69_999, 0, 65_536], np.uint32)
        calls = []
        for n in (_lib.NOALLOC_MAX_PKTS, 3_001):
            s = np.where(rng.random(n) < 0.4, rng.choice(hot, n), rng.integers(0, n_peers, n)).astype(np.uint32)
            s[5] = n_peers + 1  # not a keypair: left untouched by both paths
            calls.append(s)
        for s in calls:
            want = _regular(a, s)
            got = _no_alloc(b, s, torch)
            real = s < n_peers
            assert np.array_equal(got[real], want[real])
            assert got[5] == 0xDEAD
        for slot in (7, 69_999, 0, 65_536, 123):
            assert a.send_counter(slot) == b.send_counter(slot)
        assert b.send_counter(7) == _lib.REJECT_AFTER_MESSAGES
        # beyond the built-in scratch: refused, with a message that says why
        big = torch.zeros(_lib.NOALLOC_MAX_PKTS + 1, dtype=torch.int32, device="cuda")
        out = torch.zeros(_lib.NOALLOC_MAX_PKTS + 1, dtype=torch.int64, device="cuda")
        rc = _lib.lib().bnk_assign_counters_noalloc(b._h, None, C.c_void_p(big.data_ptr()), _lib.NOALLOC_MAX_PKTS + 1,
                                                    C.c_void_p(out.data_ptr()))
        assert rc == _lib.EINVAL
        assert b"BNK_NOALLOC_MAX_PKTS" in _lib.lib().bnk_last_error_string(b._h)
    finally:
        a.close()
        b.close()
