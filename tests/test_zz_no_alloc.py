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


def _counter_rule(slots, base, n_peers, limit):
    """The rule itself, in numpy: packets of one slot get the slot's send counter plus their rank among the
    slot's packets of the batch, saturating at the limit; the slot's counter moves past them."""
    out = np.full(len(slots), 0xDEAD, np.uint64)
    seen = {}
    for i, s in enumerate(slots.tolist()):
        if s >= n_peers:
            continue
        k = seen.get(s, 0)
        out[i] = min(base[s] + k, limit)
        seen[s] = k + 1
    for s, k in seen.items():
        base[s] = min(base[s] + k, limit)
    return out


@pytest.mark.parametrize("n", [1, 128, 256, 257, 1024, 1025, 16384])
def test_no_alloc_counters_follow_the_counter_rule(gpu_lib, n):
    """Every size class of the grouping behind the entry point (one thread per packet up to 256, one CTA up to
    1024, several kernels beyond), checked against the counter rule computed on the host, for two calls queued
    back to back on a stream of the caller's with no synchronisation in between: the second call runs over
    what the first left in the shared scratch and starts from the counters the first one moved."""
    torch = pytest.importorskip("torch")
    from bnk_b200 import Context, _lib

    n_peers = 600  # two radix digits
    limit = _lib.REJECT_AFTER_MESSAGES
    rng = np.random.default_rng(1000 + n)
    zeros = np.zeros((n_peers, 32), np.uint8)
    c = Context(max_keypairs=n_peers, flow_capacity=0)
    try:
        c.set_keypairs(0, zeros, zeros, np.zeros(n_peers, np.uint32))
        base = {s: 0 for s in range(n_peers)}
        base[3] = limit - 1       # saturates
        base[599] = 1 << 40
        for s in (3, 599):
            c.set_send_counter(s, base[s])
        second_n = max(1, n // 3)
        calls = []
        for m in (n, second_n):
            s = np.where(rng.random(m) < 0.5, rng.choice(np.array([3, 599, 0], np.uint32), m),
                         rng.integers(0, n_peers, m)).astype(np.uint32)
            if m > 2:
                s[m // 2] = n_peers + 7  # not a keypair: its counter entry stays untouched
            calls.append(s)
        stream = torch.cuda.Stream()
        d_slots = [torch.from_numpy(s.view(np.int32).copy()).cuda() for s in calls]
        d_ctrs = [torch.full((len(s),), 0xDEAD, dtype=torch.int64, device="cuda") for s in calls]
        torch.cuda.synchronize()
        for d_slot, d_ctr in zip(d_slots, d_ctrs):  # no synchronisation between the two calls
            rc = _lib.lib().bnk_assign_counters_noalloc(c._h, C.c_void_p(stream.cuda_stream), C.c_void_p(d_slot.data_ptr()),
                                                        d_slot.numel(), C.c_void_p(d_ctr.data_ptr()))
            _lib.check(rc, c._h)
        stream.synchronize()
        for s, d_ctr in zip(calls, d_ctrs):
            want = _counter_rule(s, base, n_peers, limit)
            got = d_ctr.cpu().numpy().view(np.uint64)
            assert np.array_equal(got, want), np.flatnonzero(got != want)[:8]
        for slot in (0, 3, 599, 17):
            assert c.send_counter(slot) == base[slot]
        # nothing to do is not an error
        assert _lib.lib().bnk_assign_counters_noalloc(c._h, C.c_void_p(stream.cuda_stream), C.c_void_p(d_slots[0].data_ptr()),
                                                      0, C.c_void_p(d_ctrs[0].data_ptr())) == 0
    finally:
        c.close()
