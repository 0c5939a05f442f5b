"""Seal/open parity: the CUDA path (through the C ABI) against the CPU checker, bit-exact."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tpp", "wpp"], autouse=True)
def aead_kernel(request):
    """Every case runs against both seal/open kernels: thread per packet (throughput) and warp per packet (latency)."""
    import os

    os.environ["BNK_AEAD_KERNEL"] = request.param  # read when a context is created
    yield request.param
    os.environ.pop("BNK_AEAD_KERNEL", None)


@pytest.fixture(scope="module")
def ctx(gpu_lib, aead_kernel):
    from bnk_b200 import Context

    c = Context(max_keypairs=300, replay_ring_blocks=128, mtu=1420, flow_capacity=1 << 12)
    yield c
    c.close()


def _run_seal(ctx, O, keys, remote_index, lengths, slots, counters, payloads, off=None, mtu=1420):
    n = len(lengths)
    if off is None:
        off = H.layout_packed(lengths)
    rb = H.ring_bytes_for(off, lengths)
    b = ctx.batch(max(n, 1), rb)
    try:
        b.ring[:] = 0xA5  # stale bytes around the payloads must not leak into the result
        H.fill_payloads(b.ring, off, payloads)
        b.off[:n], b.len[:n], b.slot[:n], b.counter[:n] = off, lengths, slots, counters
        want_ring, want_st, want_len = H.oracle_seal(O, keys, remote_index, mtu, b.ring, off, lengths, slots, counters)
        b.seal(n)
        got_ring, got_st, got_len = np.array(b.ring), np.array(b.status[:n]), np.array(b.out_len[:n])
    finally:
        b.close()
    return (got_ring, got_st, got_len), (want_ring, want_st, want_len), off


def test_config1_seal_then_open(ctx, oracle):
    """128 x 1420 B, one key, counters 0..127, receiver index 1: ciphertext, tags and headers byte for byte."""
    from bnk_b200 import gen

    w = gen.config1()
    ctx.set_keypairs(0, w.keys, w.keys, w.remote_index)
    (g_ring, g_st, g_len), (w_ring, w_st, w_len), off = _run_seal(
        ctx, oracle, w.keys, w.remote_index, w.length, w.peer, w.counter, w.payloads)
    assert np.array_equal(g_st, w_st) and (g_st == 0).all()
    assert np.array_equal(g_len, w_len) and (g_len == 1452).all()
    assert H.spans_equal(g_ring, w_ring, off, g_len) == []
    # open what was sealed: the plaintext comes back and the counters are parsed from the headers
    n = len(off)
    b = ctx.batch(n, len(g_ring))
    b.ring[:] = g_ring
    b.off[:n], b.len[:n], b.slot[:n] = off, g_len, w.peer
    b.open(n)
    assert (b.status[:n] == 0).all()
    assert np.array_equal(b.counter[:n], w.counter)
    assert (b.out_len[:n] == 1420).all()
    for i in range(n):
        assert b.payload(i) == w.payloads[i]
    b.close()


@pytest.mark.parametrize("mtu", [1420, 0, 1280])
def test_seal_edge_lengths(ctx, oracle, mtu):
    """Every length around the 16-byte and 64-byte boundaries, the MTU cap, and beyond the MTU."""
    rng = np.random.default_rng(7)
    lengths = list(range(0, 200)) + [255, 256, 257, 575, 576, 577, 1279, 1280, 1281, 1407, 1408, 1409, 1419, 1420,
                                     1421, 1424, 1500, 2840, 2841, 4000, 9000]
    n = len(lengths)
    keys = rng.integers(0, 256, (8, 32), dtype=np.uint8)
    ridx = rng.integers(0, 2**32, 8, dtype=np.uint64).astype(np.uint32)
    slots = rng.integers(0, 8, n).astype(np.uint32)
    counters = rng.integers(0, 2**63, n, dtype=np.uint64)
    payloads = [rng.integers(0, 256, l, dtype=np.uint8).tobytes() for l in lengths]
    from bnk_b200 import Context

    c = Context(max_keypairs=8, mtu=mtu, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, ridx)
        got, want, off = _run_seal(c, oracle, keys, ridx, np.array(lengths, np.uint32), slots, counters, payloads,
                                   mtu=mtu)
    finally:
        c.close()
    assert np.array_equal(got[1], want[1])
    assert np.array_equal(got[2], want[2])
    assert H.spans_equal(got[0], want[0], off, got[2]) == []


def test_seal_counter_exhausted_and_bad_descriptors(ctx, oracle):
    rng = np.random.default_rng(3)
    keys = rng.integers(0, 256, (4, 32), dtype=np.uint8)
    ridx = np.arange(4, dtype=np.uint32)
    ctx.set_keypairs(0, keys, keys, ridx)
    b = ctx.batch(8, 8 * 256)
    n = 6
    b.off[:n] = [0, 256, 512, 8, 1024, 2000]  # 8: misaligned; 2000: runs past the ring
    b.len[:n] = [64, 64, 64, 64, 64, 64]
    b.slot[:n] = [0, 1, 999, 2, 3, 0]         # 999: no such keypair
    lim = 0xFFFFFFFFFFFFDFFF
    b.counter[:n] = [lim - 1, lim, 0, 0, 2**64 - 1, 0]
    b.ring[:] = 7
    b.seal(n)
    from bnk_b200.device import PKT_BAD_DESC, PKT_COUNTER_EXHAUSTED, PKT_OK

    assert list(b.status[:n]) == [PKT_OK, PKT_COUNTER_EXHAUSTED, PKT_BAD_DESC, PKT_BAD_DESC, PKT_COUNTER_EXHAUSTED,
                                  PKT_BAD_DESC]
    want = oracle.wg_seal(keys[0].tobytes(), 0, lim - 1, bytes([7] * 64), 1420)
    assert b.message(0) == want
    # refused packets are left untouched
    assert (b.ring[256:512] == 7).all() and (b.ring[1024:1280] == 7).all()
    b.close()


def test_open_rejects_forgeries_and_malformed(ctx, oracle):
    """One flipped bit anywhere in header counter, ciphertext or tag must fail; failed packets release no plaintext."""
    rng = np.random.default_rng(11)
    keys = rng.integers(0, 256, (4, 32), dtype=np.uint8)
    ctx.set_keypairs(0, keys, keys, np.arange(4, dtype=np.uint32))
    msgs, slots, expect = [], [], []
    for i, l in enumerate([0, 1, 15, 16, 17, 64, 100, 576, 1420, 33, 48]):
        s = i % 4
        pt = rng.integers(0, 256, l, dtype=np.uint8).tobytes()
        m = bytearray(oracle.wg_seal(keys[s].tobytes(), 5, 1000 + i, pt, 0))
        kind = i % 4
        if kind == 1:
            m[-1 - (i % 16)] ^= 0x01          # tag byte
        elif kind == 2 and len(m) > 32:
            m[16 + (i % (len(m) - 32))] ^= 0x80  # ciphertext byte
        elif kind == 3:
            m[8] ^= 0x01                      # counter in the header -> wrong nonce
        msgs.append(bytes(m))
        slots.append(s)
    msgs.append(b"\x04\x00\x00\x00" + bytes(27))              # 31 bytes: too short
    slots.append(0)
    bad_type = bytearray(oracle.wg_seal(keys[1].tobytes(), 5, 77, b"x" * 32, 0))
    bad_type[0] = 1
    msgs.append(bytes(bad_type))
    slots.append(1)
    wrong_key = oracle.wg_seal(keys[2].tobytes(), 5, 78, b"y" * 40, 0)
    msgs.append(wrong_key)
    slots.append(3)
    n = len(msgs)
    lengths = np.array([len(m) for m in msgs], np.uint32)
    off = H.layout_packed(lengths, slack=16)
    b = ctx.batch(n, H.ring_bytes_for(off, lengths))
    b.ring[:] = 0x3C
    H.fill_payloads(b.ring, off, msgs, headroom=0)
    b.off[:n], b.len[:n], b.slot[:n] = off, lengths, np.array(slots, np.uint32)
    w_ring, w_st, w_ctr, w_len = H.oracle_open(oracle, keys, b.ring, off, lengths, b.slot[:n])
    b.open(n)
    assert np.array_equal(b.status[:n], w_st)
    assert np.array_equal(b.out_len[:n], w_len)
    ok = w_st != oracle.MALFORMED
    assert np.array_equal(b.counter[:n][ok], w_ctr[ok])
    assert H.spans_equal(np.array(b.ring), w_ring, off, np.maximum(lengths, 32) - 32, start=16) == []
    assert set(w_st) >= {oracle.OK, oracle.KEEPALIVE, oracle.AUTH_FAIL, oracle.MALFORMED}
    b.close()


def test_seal_open_round_trip_mixed_sizes_sorted(ctx, oracle):
    """IMIX-like mix with the by-length scheduling order switched on: same bytes as without it."""
    from bnk_b200 import gen
    from bnk_b200.device import F_SORT_BY_LENGTH

    w = gen.config2(n_arrivals=1024, n_peers=64).base
    ctx.set_keypairs(0, w.keys, w.keys, w.remote_index)
    n = len(w.length)
    off = H.layout_packed(w.length)
    b = ctx.batch(n, H.ring_bytes_for(off, w.length))
    H.fill_payloads(b.ring, off, w.payloads)
    b.off[:n], b.len[:n], b.slot[:n], b.counter[:n] = off, w.length, w.peer, w.counter
    want_ring, want_st, want_len = H.oracle_seal(oracle, w.keys, w.remote_index, 1420, b.ring, off, w.length, w.peer,
                                                 w.counter)
    b.seal(n, F_SORT_BY_LENGTH)
    assert np.array_equal(b.out_len[:n], want_len)
    assert H.spans_equal(np.array(b.ring), want_ring, off, want_len) == []
    b.len[:n] = b.out_len[:n]
    b.open(n, F_SORT_BY_LENGTH)
    assert (b.status[:n] == 0).all()
    for i in range(0, n, 17):
        assert b.payload(i)[:len(w.payloads[i])] == w.payloads[i]
    b.close()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_descriptor_fuzz(ctx, oracle, seed):
    """Random descriptors, many of them invalid (misaligned, out of range, absurd lengths, unknown keypairs): valid
    packets come out bit-exact, invalid ones are refused with BAD_DESC / MALFORMED and nothing outside a valid packet's
    own slot changes."""
    from bnk_b200.device import PKT_BAD_DESC, PKT_MALFORMED

    rng = np.random.default_rng(seed)
    keys = rng.integers(0, 256, (300, 32), dtype=np.uint8)
    ridx = rng.integers(0, 2**32, 300, dtype=np.uint64).astype(np.uint32)
    ctx.set_keypairs(0, keys, keys, ridx)
    n, slot_bytes = 400, 4096
    ring_bytes = n * slot_bytes
    b = ctx.batch(n, ring_bytes)
    base = rng.integers(0, 256, ring_bytes, dtype=np.uint8)
    for mode in ("seal", "open"):
        b.ring[:] = base
        off = (np.arange(n, dtype=np.uint64) * slot_bytes).astype(np.uint32)
        length = rng.choice([0, 1, 15, 16, 17, 63, 64, 65, 100, 576, 1420, 1421, 2000, 3000, 4000], n).astype(np.uint32)
        slot = rng.integers(0, 300, n).astype(np.uint32)
        counter = rng.integers(0, 2**62, n, dtype=np.uint64)
        kind = rng.integers(0, 10, n)
        valid = np.ones(n, bool)
        for i in range(n):
            if kind[i] == 0:
                off[i] += int(rng.choice([1, 4, 8, 12]))           # misaligned
                valid[i] = False
            elif kind[i] == 1:
                slot[i] = int(rng.choice([300, 301, 2**31, 2**32 - 1]))  # no such keypair
                valid[i] = False
            elif kind[i] == 2:
                length[i] = int(rng.choice([2**31, 2**32 - 1, ring_bytes, ring_bytes - 8]))  # runs far past the ring
                off[i] = int(rng.integers(0, n)) * slot_bytes
                valid[i] = False
            elif kind[i] == 3 and i == n - 1:
                length[i] = slot_bytes                              # last slot: a seal's header/tag room would pass the ring end
        if mode == "open":
            # put real messages into the valid slots (payload length such that the message is `length` long when possible)
            for i in range(n):
                if valid[i] and length[i] >= 32:
                    pt = rng.integers(0, 256, int(length[i]) - 32, dtype=np.uint8).tobytes()
                    m = oracle.wg_seal(keys[slot[i]].tobytes(), 1, int(counter[i]), pt, 0)
                    if len(m) != length[i]:     # padding made it longer: open the padded message instead
                        length[i] = len(m)
                    o = int(off[i])
                    b.ring[o:o + len(m)] = np.frombuffer(m, np.uint8)
        seal_fits = lambda i: int(off[i]) + 16 + oracle.wg_padded_len(int(length[i]), 1420) + 16 <= ring_bytes  # noqa: E731
        before = np.array(b.ring)
        b.off[:n], b.len[:n], b.slot[:n], b.counter[:n] = off, length, slot, counter
        if mode == "seal":
            b.seal(n)
        else:
            b.open(n)
        after = np.array(b.ring)
        st = np.array(b.status[:n])
        touched = np.zeros(ring_bytes, bool)
        for i in range(n):
            ok_desc = valid[i] and (seal_fits(i) if mode == "seal" else int(off[i]) + int(length[i]) <= ring_bytes)
            if not ok_desc:
                assert st[i] == PKT_BAD_DESC, (mode, i, st[i], off[i], length[i], slot[i])
                continue
            o, l = int(off[i]), int(length[i])
            if mode == "seal":
                want = oracle.wg_seal(keys[slot[i]].tobytes(), int(ridx[slot[i]]), int(counter[i]), before[o + 16:o + 16 + l].tobytes(), 1420)
                assert st[i] == 0 and after[o:o + len(want)].tobytes() == want, (mode, i)
                touched[o:o + len(want)] = True
            else:
                if l < 32:
                    assert st[i] == PKT_MALFORMED
                    continue
                wst, pt, ctr, _ = oracle.wg_open(keys[slot[i]].tobytes(), before[o:o + l].tobytes())
                assert st[i] == wst and b.counter[i] == ctr, (mode, i, st[i], wst)
                assert after[o + 16:o + 16 + len(pt)].tobytes() == pt
                touched[o + 16:o + l - 16] = True
        assert np.array_equal(after[~touched], before[~touched]), "bytes outside valid packets changed"
    b.close()
