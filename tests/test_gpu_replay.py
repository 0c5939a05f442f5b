"""Send counters and the anti-replay window on the GPU against the sequential CPU walk."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _sealed_ring(oracle, keys, slots, counters, sizes, rng):
    msgs = [oracle.wg_seal(keys[s].tobytes(), 1, int(c), rng.integers(0, 256, int(l), dtype=np.uint8).tobytes(), 0)
            for s, c, l in zip(slots, counters, sizes)]
    lengths = np.array([len(m) for m in msgs], np.uint32)
    off = H.layout_packed(lengths, slack=16)
    return msgs, lengths, off


# 256 blocks: too large for the walk in shared memory; 1500 packets: the walk without the gather pass
@pytest.mark.parametrize("blocks,n", [(32, 3000), (128, 3000), (256, 3000), (128, 1500)])
def test_replay_verdicts_follow_arrival_order(gpu_lib, oracle, blocks, n):
    """Many peers, heavy reordering, duplicates, stale counters, forged packets in between, across
    several batches so the window state carries over."""
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY

    rng = np.random.default_rng(blocks)
    n_peers = 37
    window = (blocks - 1) * 64
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, replay_ring_blocks=blocks, mtu=0, flow_capacity=0)
    state = {}
    try:
        c.set_keypairs(0, keys, keys, np.ones(n_peers, np.uint32))
        top = rng.integers(1 << 20, 1 << 40, n_peers).astype(np.int64)
        for batch_no in range(4):
            slots = rng.integers(0, n_peers, n).astype(np.uint32)
            if batch_no == 1:
                slots[:] = 5  # one peer owns the whole batch: a long sequential walk
            counters = np.zeros(n, np.uint64)
            for i in range(n):
                s = int(slots[i])
                r = rng.random()
                if r < 0.55:
                    top[s] += int(rng.integers(1, 4))
                    cval = top[s]
                elif r < 0.80:
                    cval = top[s] - int(rng.integers(0, 80))
                elif r < 0.90:
                    cval = top[s] - int(rng.integers(window - 70, window + 70))
                elif r < 0.95:
                    top[s] += int(rng.integers(window // 2, 3 * window))
                    cval = top[s]
                else:
                    cval = top[s] - int(rng.integers(0, 3))
                counters[i] = max(int(cval), 0)
            sizes = rng.choice([0, 16, 64], n)
            msgs, lengths, off = _sealed_ring(oracle, keys, slots, counters, sizes, rng)
            forged = rng.random(n) < 0.03
            b = c.batch(n, H.ring_bytes_for(off, lengths))
            H.fill_payloads(b.ring, off, msgs, headroom=0)
            for i in np.flatnonzero(forged):
                b.ring[int(off[i]) + int(lengths[i]) - 1] ^= 0x40
            b.off[:n], b.len[:n], b.slot[:n] = off, lengths, slots
            _, st, ctr, _ = H.oracle_open(oracle, keys, b.ring, off, lengths, slots)
            want, state = H.oracle_replay(oracle, blocks, slots, ctr, st, state)
            b.open(n, F_REPLAY)
            got = np.array(b.status[:n])
            b.close()
            assert np.array_equal(got, want), f"batch {batch_no}: {np.flatnonzero(got != want)[:8]}"
            assert (want == oracle.REPLAY).sum() > 50 and (want == oracle.AUTH_FAIL).sum() > 20
        for s, r in state.items():
            last, ring = c.replay_export(s)
            assert last == r.last and np.array_equal(ring, r.ring()), s
    finally:
        c.close()


@pytest.mark.parametrize("blocks", [32, 128])
def test_replay_dominant_peer_large_batch(gpu_lib, oracle, blocks):
    """One peer owns most of a 120,000-packet batch (the scan form of the window): reordering inside the
    window, repeats of earlier counters far apart in the batch, stale counters at the window's edge, and
    jumps of several rings; two batches so the second starts from the state the first left."""
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY

    rng = np.random.default_rng(1000 + blocks)
    n_peers, n, size = 41, 120_000, 16
    window = (blocks - 1) * 64
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    stride = 16 + size + 16
    off = (np.arange(n, dtype=np.uint64) * stride).astype(np.uint32)
    lengths = np.full(n, size, np.uint32)
    c = Context(max_keypairs=n_peers, replay_ring_blocks=blocks, mtu=0, flow_capacity=0)
    state = {}
    top = rng.integers(1 << 20, 1 << 40, n_peers).astype(np.uint64)
    try:
        c.set_keypairs(0, keys, keys, np.ones(n_peers, np.uint32))
        b = c.batch(n, n * stride + 64)
        for batch_no in range(2):
            slots = np.where(rng.random(n) < 0.7, 0, rng.integers(1, n_peers, n)).astype(np.uint32)
            counters = np.zeros(n, np.uint64)
            for s in range(n_peers):
                idx = np.flatnonzero(slots == s)
                m = len(idx)
                kind = rng.random(m)
                step = np.where(kind < 0.90, rng.integers(1, 3, m), 0)
                step = np.where(kind > 0.995, rng.integers(window // 2, 3 * window + 200, m), step)
                tops = top[s] + np.cumsum(step).astype(np.uint64)
                back = np.zeros(m, np.int64)
                r2 = rng.random(m)
                back = np.where(r2 < 0.25, rng.integers(0, 100, m), back)                       # reordered / repeated
                back = np.where(r2 < 0.04, rng.integers(window - 70, window + 70, m), back)     # the window's edge
                back = np.where(r2 < 0.01, rng.integers(0, 6000, m), back)                      # far repeats
                counters[idx] = tops - np.minimum(back.astype(np.uint64), tops)
                if m:
                    top[s] = tops[-1]
            ring = np.zeros(n * stride + 64, np.uint8)
            body = rng.integers(0, 256, (n, size), dtype=np.uint8)
            ring[: n * stride].reshape(n, stride)[:, 16:16 + size] = body
            st, out_len = oracle.wg_seal_batch(keys, np.ones(n_peers, np.uint32), 0, ring, off, lengths, slots, counters)
            assert (st == oracle.OK).all()
            forged = np.flatnonzero(rng.random(n) < 0.01)
            ring[off[forged].astype(np.int64) + 20] ^= 1
            b.ring[: len(ring)] = ring
            b.off[:n], b.len[:n], b.slot[:n] = off, out_len, slots
            _, ost, ctr, _ = H.oracle_open(oracle, keys, ring, off, out_len, slots)
            want, state = H.oracle_replay(oracle, blocks, slots, ctr, ost, state)
            b.open(n, F_REPLAY)
            got = np.array(b.status[:n])
            assert np.array_equal(got, want), f"batch {batch_no}: {np.flatnonzero(got != want)[:8]}"
            assert (want == oracle.REPLAY).sum() > 5000 and (want == oracle.AUTH_FAIL).sum() > 500
            assert (want == oracle.OK).sum() > n // 2
        b.close()
        for s, r in state.items():
            last, ring_words = c.replay_export(s)
            assert last == r.last and np.array_equal(ring_words, r.ring()), s
    finally:
        c.close()


def test_replay_burst_of_copies(gpu_lib, oracle):
    """A captured packet sent over and over: 60 distinct counters of one peer, each repeated about 300 times in
    shuffled order among other peers' traffic.  Only first occurrences may pass."""
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY

    rng = np.random.default_rng(4242)
    n_peers, n, size, blocks = 7, 20_000, 16, 128
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    stride = 16 + size + 16
    off = (np.arange(n, dtype=np.uint64) * stride).astype(np.uint32)
    slots = np.where(rng.random(n) < 0.9, 3, rng.integers(0, n_peers, n)).astype(np.uint32)
    counters = (1000 + rng.integers(0, 60, n)).astype(np.uint64)              # the copies
    others = slots != 3
    counters[others] = 5000 + np.arange(int(others.sum()), dtype=np.uint64)  # ordinary traffic of the rest
    ring = np.zeros(n * stride + 64, np.uint8)
    ring[: n * stride].reshape(n, stride)[:, 16:16 + size] = rng.integers(0, 256, (n, size), dtype=np.uint8)
    st, out_len = oracle.wg_seal_batch(keys, np.ones(n_peers, np.uint32), 0, ring, off, np.full(n, size, np.uint32), slots, counters)
    assert (st == oracle.OK).all()
    c = Context(max_keypairs=n_peers, replay_ring_blocks=blocks, mtu=0, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.ones(n_peers, np.uint32))
        b = c.batch(n, n * stride + 64)
        b.ring[: len(ring)] = ring
        b.off[:n], b.len[:n], b.slot[:n] = off, out_len, slots
        _, ost, ctr, _ = H.oracle_open(oracle, keys, ring, off, out_len, slots)
        want, state = H.oracle_replay(oracle, blocks, slots, ctr, ost)
        b.open(n, F_REPLAY)
        got = np.array(b.status[:n])
        b.close()
        assert np.array_equal(got, want), np.flatnonzero(got != want)[:8]
        assert (want[slots == 3] == oracle.OK).sum() == 60
        for s_, r in state.items():
            last, ring_words = c.replay_export(s_)
            assert last == r.last and np.array_equal(ring_words, r.ring()), s_
    finally:
        c.close()


def test_replay_limit_and_state_import(gpu_lib, oracle):
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY, PKT_KEEPALIVE, PKT_REPLAY

    key = np.arange(32, dtype=np.uint8).reshape(1, 32)
    lim = oracle.REJECT_AFTER_MESSAGES
    c = Context(max_keypairs=2, replay_ring_blocks=32, mtu=0, flow_capacity=0)
    try:
        c.set_keypairs(0, np.repeat(key, 2, 0), np.repeat(key, 2, 0), np.ones(2, np.uint32))
        r = oracle.Replay(32)
        for v in (lim - 5000, lim - 4000):
            r.validate(v)
        c.replay_import(1, r.last, r.ring())
        counters = [lim - 4000, lim - 3999, lim - 1, lim, 2**64 - 1, lim - 1, lim - 2]
        msgs = [oracle.wg_seal(key[0].tobytes(), 1, ctr, b"", 0) if ctr < lim else
                # counters at or past the limit cannot be sealed by a conforming sender: build them by hand
                _forge_keepalive(oracle, key[0].tobytes(), ctr) for ctr in counters]
        n = len(msgs)
        lengths = np.array([len(m) for m in msgs], np.uint32)
        off = H.layout_packed(lengths, slack=16)
        b = c.batch(n, H.ring_bytes_for(off, lengths))
        H.fill_payloads(b.ring, off, msgs, headroom=0)
        b.off[:n], b.len[:n], b.slot[:n] = off, lengths, 1
        b.open(n, F_REPLAY)
        want = [PKT_KEEPALIVE if r.validate(ctr) else PKT_REPLAY for ctr in counters]
        assert list(b.status[:n]) == want
        assert want == [PKT_REPLAY, PKT_KEEPALIVE, PKT_KEEPALIVE, PKT_REPLAY, PKT_REPLAY, PKT_REPLAY, PKT_KEEPALIVE]
        b.close()
    finally:
        c.close()


def _forge_keepalive(oracle, key, counter):
    nonce = bytes(4) + counter.to_bytes(8, "little")
    return (4).to_bytes(4, "little") + (1).to_bytes(4, "little") + counter.to_bytes(8, "little") + oracle.aead_seal(key, nonce, b"")


def test_send_counters_assigned_in_batch_order(gpu_lib, oracle):
    """Packets of one peer get consecutive nonces in batch order; the counter saturates at the limit."""
    from bnk_b200 import Context
    from bnk_b200.device import F_ASSIGN_COUNTERS, PKT_COUNTER_EXHAUSTED, PKT_OK

    rng = np.random.default_rng(5)
    n_peers, n = 70000, 20000  # more than 2^16 slots: the grouping sort needs a second digit pass
    lim = oracle.REJECT_AFTER_MESSAGES
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.arange(n_peers, dtype=np.uint32))
        hot = np.array([0, 1, 65535, 65536, 69999, 777], np.uint32)
        slots = np.where(rng.random(n) < 0.5, rng.choice(hot, n), rng.integers(0, n_peers, n)).astype(np.uint32)
        slots[100] = n_peers + 5  # no such keypair
        c.set_send_counter(777, lim - 3)
        c.set_send_counter(65536, 1 << 40)
        nxt = {777: lim - 3, 65536: 1 << 40}
        want = np.zeros(n, np.uint64)
        for i in range(n):
            s = int(slots[i])
            if s >= n_peers:
                continue
            v = nxt.get(s, 0)
            want[i] = min(v, lim)
            nxt[s] = min(v + 1, lim)
        sizes = np.full(n, 64, np.uint32)
        off = H.layout_fixed(n, 112)
        b = c.batch(n, n * 112)
        b.ring[:] = 1
        b.off[:n], b.len[:n], b.slot[:n] = off, sizes, slots
        for rep in range(2):
            b.seal(n, F_ASSIGN_COUNTERS)
            got = np.array(b.counter[:n])
            ok = slots < n_peers
            assert np.array_equal(got[ok], want[ok]), rep
            st = np.array(b.status[:n])
            assert (st[ok & (want < lim)] == PKT_OK).all() and (st[ok & (want >= lim)] == PKT_COUNTER_EXHAUSTED).all()
            for s in (0, 777, 65536, 69999):
                assert c.send_counter(s) == nxt.get(s, 0)
            # sealed bytes use the assigned nonce
            i = int(np.flatnonzero(slots == 65536)[0])
            assert b.message(i) == oracle.wg_seal(keys[65536].tobytes(), 65536, int(want[i]), bytes([1] * 64), 1420)
            # second round continues where the first stopped
            for i in range(n):
                s = int(slots[i])
                if s < n_peers:
                    v = nxt.get(s, 0)
                    want[i] = min(v, lim)
                    nxt[s] = min(v + 1, lim)
            b.ring[:] = 1
        b.close()
    finally:
        c.close()


@pytest.mark.parametrize("n", [1, 2, 31, 33, 128, 255, 256, 257, 1000, 1024, 1025])
def test_send_counters_small_batches(gpu_lib, n):
    """Batches of up to 1024 packets group by keypair in a single launch; the nonces must come out the same way."""
    from bnk_b200 import Context
    from bnk_b200.device import F_ASSIGN_COUNTERS, PKT_OK

    rng = np.random.default_rng(n)
    n_peers = 70000
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        keys = np.zeros((n_peers, 32), np.uint8)
        c.set_keypairs(0, keys, keys, np.zeros(n_peers, np.uint32))
        hot = np.array([3, 65535, 65536, 69999], np.uint32)
        b = c.batch(n, n * 64)
        b.off[:n] = H.layout_fixed(n, 64)
        b.len[:n] = 0
        nxt = {}
        for rep in range(3):
            slots = np.where(rng.random(n) < 0.6, rng.choice(hot, n), rng.integers(0, n_peers, n)).astype(np.uint32)
            want = np.zeros(n, np.uint64)
            for i, s in enumerate(slots):
                want[i] = nxt.get(int(s), 0)
                nxt[int(s)] = int(want[i]) + 1
            b.slot[:n] = slots
            b.seal(n, F_ASSIGN_COUNTERS)
            assert np.array_equal(b.counter[:n], want), rep
            assert (b.status[:n] == PKT_OK).all()
        b.close()
    finally:
        c.close()
