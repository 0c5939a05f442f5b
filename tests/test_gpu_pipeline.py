"""Configuration 2 end to end on the GPU: open + replay (+ filter) of an IMIX arrival stream with
reordering, duplicates and damaged tags; statuses and plaintext equal to the CPU checker's."""
import numpy as np
import pytest

from tests import helpers as H
from tests import reference_cases as RC

pytestmark = pytest.mark.gpu


def _arrival_stream(oracle, w):
    b = w.base
    sealed = [oracle.wg_seal(b.keys[int(b.peer[i])].tobytes(), int(b.remote_index[int(b.peer[i])]), int(b.counter[i]),
                             b.payloads[i], 1420) for i in range(len(b.payloads))]
    msgs = [bytearray(sealed[i]) for i in w.arrival]
    for p, k in zip(w.flip_pos, w.flip_byte):
        msgs[int(p)][len(msgs[int(p)]) - 16 + int(k)] ^= 0x01
    slots = b.peer[w.arrival].astype(np.uint32)
    return [bytes(m) for m in msgs], slots


@pytest.mark.parametrize("blocks,sort", [(32, False), (128, True)])
def test_config2_open_replay(gpu_lib, oracle, blocks, sort):
    from bnk_b200 import Context, gen
    from bnk_b200.device import F_REPLAY, F_SORT_BY_LENGTH

    w = gen.config2()
    msgs, slots = _arrival_stream(oracle, w)
    n = len(msgs)
    assert n == 4096
    lengths = np.array([len(m) for m in msgs], np.uint32)
    off = H.layout_packed(lengths, slack=16)
    c = Context(max_keypairs=w.n_peers, replay_ring_blocks=blocks, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, w.base.keys, w.base.keys, w.base.remote_index)
        b = c.batch(n, H.ring_bytes_for(off, lengths))
        H.fill_payloads(b.ring, off, msgs, headroom=0)
        b.off[:n], b.len[:n], b.slot[:n] = off, lengths, slots
        w_ring, st, ctr, w_len = H.oracle_open(oracle, w.base.keys, b.ring, off, lengths, slots)
        want, _ = H.oracle_replay(oracle, blocks, slots, ctr, st)
        b.open(n, F_REPLAY | (F_SORT_BY_LENGTH if sort else 0))
        got = np.array(b.status[:n])
        assert np.array_equal(got, want)
        assert np.array_equal(b.counter[:n], ctr)
        assert np.array_equal(b.out_len[:n], w_len)
        assert H.spans_equal(np.array(b.ring), w_ring, off, lengths - 32, start=16) == []
        n_dup = n - len(w.base.payloads)
        assert (want == oracle.AUTH_FAIL).sum() >= len(set(w.flip_pos.tolist())) > 0
        assert 0 < (want == oracle.REPLAY).sum() <= n_dup
        b.close()
    finally:
        c.close()


def test_open_replay_filter_chain(gpu_lib, oracle):
    """Open -> replay -> CheckInbound in one submit: only authenticated, fresh, permitted packets stay OK."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import F_CHECK_INBOUND, F_REPLAY
    from bnk_b200.filter import CompiledRule, PortRange, flatten_rules

    w = gen.config2(n_arrivals=1024, n_peers=32)
    msgs, slots = _arrival_stream(oracle, w)
    n = len(msgs)
    lengths = np.array([len(m) for m in msgs], np.uint32)
    off = H.layout_packed(lengths, slack=16)
    # peers 0..15 may reach udp/51820; everyone else only as a reply (none here)
    rules = [CompiledRule(srcs=["100.64.1.0/28"], proto="udp", ports=[PortRange(51820, 51820)])]
    c = Context(max_keypairs=32, replay_ring_blocks=128, mtu=1420, flow_capacity=1 << 10)
    try:
        c.set_keypairs(0, w.base.keys, w.base.keys, w.base.remote_index)
        c.acl_set(True, flatten_rules(rules))
        b = c.batch(n, H.ring_bytes_for(off, lengths))
        H.fill_payloads(b.ring, off, msgs, headroom=0)
        b.off[:n], b.len[:n], b.slot[:n] = off, lengths, slots
        w_ring, st, ctr, w_len = H.oracle_open(oracle, w.base.keys, b.ring, off, lengths, slots)
        want, _ = H.oracle_replay(oracle, 128, slots, ctr, st)
        f = oracle.Filter()
        f.set_rules([([(gen.ip4(100, 64, 1, 0), 28)], "udp", [(51820, 51820)])])
        for i in range(n):
            if want[i] == oracle.OK:
                o = int(off[i]) + 16
                if not f.check_inbound(w_ring[o:o + int(w_len[i])].tobytes(), RC.T0):
                    want[i] = oracle.FILTER_DENY
        b.open(n, F_REPLAY | F_CHECK_INBOUND, now_ns=RC.T0)
        assert np.array_equal(np.array(b.status[:n]), want)
        assert (want == oracle.FILTER_DENY).sum() > 100 and (want == oracle.OK).sum() > 100
        b.close()
    finally:
        c.close()


def test_seal_with_note_outbound_then_reply_passes(gpu_lib, oracle):
    """Seal with NOTE_OUTBOUND records the flows of the plaintext packets before they are encrypted."""
    from bnk_b200 import Context
    from bnk_b200.device import F_NOTE_OUTBOUND
    from bnk_b200.filter import Filter

    c = Context(max_keypairs=2, mtu=1420, flow_capacity=1 << 10)
    try:
        key = np.arange(64, dtype=np.uint8).reshape(2, 32)
        c.set_keypairs(0, key, key, np.array([7, 8], np.uint32))
        f = Filter(c, batch_pkts=8)
        f.set_rules([])
        out = [RC.udp(RC.SELF, RC.PEER, 40000, 9999), RC.tcp(RC.SELF, RC.OTHER, 40001, 443)]
        b = c.batch(4, 4 * 128)
        n = b.put_packets(out, stride=128)
        b.slot[:n] = [0, 1]
        b.counter[:n] = [10, 11]
        b.seal(n, F_NOTE_OUTBOUND, now_ns=RC.T0)
        assert b.message(0) == oracle.wg_seal(key[0].tobytes(), 7, 10, out[0], 1420)
        assert c.flows_count() == 2
        assert f.check_inbound(RC.udp(RC.PEER, RC.SELF, 9999, 40000), RC.T0 + RC.SEC)
        assert f.check_inbound(RC.tcp(RC.OTHER, RC.SELF, 443, 40001, False), RC.T0 + RC.SEC)
        assert not f.check_inbound(RC.tcp(RC.OTHER, RC.SELF, 443, 40002, False), RC.T0 + RC.SEC)
        b.close()
    finally:
        c.close()


def test_wait_timeout_and_busy(gpu_lib):
    """bnk_wait with a deadline returns BNK_ETIMEDOUT-or-done without blocking; a second submit before
    the wait is refused with BNK_EBUSY."""
    from bnk_b200 import Context, _lib

    c = Context(max_keypairs=1, mtu=1420, flow_capacity=0)
    try:
        c.set_keypair(0, bytes(range(32)), bytes(range(32)), 1)
        b = c.batch(1 << 14, (1 << 14) * 1472)
        n = 1 << 14
        b.off[:n] = (np.arange(n, dtype=np.uint64) * 1472).astype(np.uint32)
        b.len[:n] = 1420
        b.seal(n, wait=False)
        rc = _lib.lib().bnk_seal_submit(b._h, n, 0, 0)
        assert rc == _lib.EBUSY
        done = b.try_wait(0)
        assert done in (True, False)
        assert b.try_wait(5_000_000_000)
        assert (b.status[:n] == 0).all()
        b.close()
    finally:
        c.close()


def test_wait_runs_out_of_time(gpu_lib):
    """bnk_wait really returns BNK_ETIMEDOUT while work is in flight, the batch stays usable, and a wait
    without limit then delivers the results: several milliseconds of device-resident seals are queued
    back to back and polled at once."""
    from bnk_b200 import Context, _lib
    from bnk_b200.device import F_NO_D2H, F_NO_H2D

    n = 1 << 19
    c = Context(max_keypairs=4, mtu=1420, flow_capacity=0)
    try:
        key = np.arange(32, dtype=np.uint8)
        c.set_keypairs(0, np.repeat(key[None, :], 4, 0), np.repeat(key[None, :], 4, 0), np.arange(4, dtype=np.uint32))
        b = c.batch(n, n * 1472)
        b.off[:n] = (np.arange(n, dtype=np.uint64) * 1472).astype(np.uint32)
        b.len[:n] = 1420
        b.slot[:n] = np.arange(n) % 4
        b.counter[:n] = np.arange(n)
        b.upload(n)
        for _ in range(8):  # ~0.6 ms each on a B200, queued without waiting
            b.seal(n, F_NO_H2D | F_NO_D2H, wait=False)
        assert _lib.lib().bnk_wait(b._h, 0) == _lib.ETIMEDOUT          # one poll: still running
        assert _lib.lib().bnk_wait(b._h, 20_000) == _lib.ETIMEDOUT     # 20 us: still running
        assert _lib.lib().bnk_seal_submit(b._h, n, 0, 0) == _lib.EBUSY  # and the batch knows it
        b.wait()
        assert _lib.lib().bnk_wait(b._h, 0) == 0
        b.download(n)
        assert (b.status[:n] == 0).all() and (b.out_len[:n] == 1452).all()
        assert (b.counter[:n] == np.arange(n)).all()
        b.close()
    finally:
        c.close()


def test_demux_by_receiver_index_and_inner_check(gpu_lib, oracle):
    """Open with the keypair looked up from the header's receiver index, then the post-decrypt checks:
    IPv4 total-length truncation and source-address check, against the CPU checker."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_DEMUX_INDEX, F_INNER_CHECK, F_REPLAY, PKT_BAD_INNER, PKT_KEEPALIVE, PKT_MALFORMED,
                                 PKT_NO_KEYPAIR, PKT_OK)

    rng = np.random.default_rng(21)
    n_peers = 50
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    local_index = rng.choice(2**32, n_peers, replace=False).astype(np.uint64)
    local_index[0] = 0                     # index 0 is a legal index
    peer_ip = gen.ip4(100, 64, 1, 0) + np.arange(n_peers)
    c = Context(max_keypairs=64, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.zeros(n_peers, np.uint32))
        for s in range(n_peers):
            c.index_set(int(local_index[s]), s)
            c.set_allowed_ip(s, int(peer_ip[s]))
        c.index_set(0xDEAD0001, 7)
        c.index_clear(0xDEAD0001)          # removed again: must not resolve
        c.set_allowed_ip(49, 0)            # a peer without an allowed address can deliver nothing
        msgs, want_slot, want = [], [], []
        for i in range(600):
            s = int(rng.integers(0, n_peers))
            kind = i % 10
            size = int(rng.choice([28, 64, 576, 1420]))
            src = int(peer_ip[s])
            total = size
            version, ihl = 4, 5
            if kind == 1:
                src = int(peer_ip[(s + 1) % n_peers])      # spoofed source
            elif kind == 2:
                total = size + 1                            # claims more than was sent
            elif kind == 3:
                total = max(20, size - int(rng.integers(1, 9)))  # shorter than the padded payload: cut
            elif kind == 4:
                total = 19                                  # below an IPv4 header
            elif kind == 5:
                version = 6
            hdr = bytes(gen.ipv4_header(17, src, gen.ip4(100, 64, 0, 1), total, ihl, version))
            pt = hdr + rng.integers(0, 256, size - 20, dtype=np.uint8).tobytes()
            idx = int(local_index[s])
            if kind == 6:
                idx = 0xDEAD0001 if i % 20 == 6 else int(rng.integers(1, 2**32))  # unknown receiver index
            if kind == 7:
                pt = b""                                    # keepalive
            m = oracle.wg_seal(keys[s].tobytes(), idx, 1000 + i, pt, 1420)
            if kind == 8:
                m = m[:24]                                  # truncated datagram
            msgs.append(m)
            known = {int(v): k for k, v in enumerate(local_index)}
            slot = known.get(idx)
            if kind == 8:
                want.append(PKT_MALFORMED)
            elif slot is None:
                want.append(PKT_NO_KEYPAIR)
            elif not pt:
                want.append(PKT_KEEPALIVE)
            else:
                padded = pt + bytes(oracle.wg_padded_len(len(pt), 1420) - len(pt))
                nl = oracle.inner_check(padded, 0 if slot == 49 else int(peer_ip[slot]))
                want.append((PKT_OK, nl) if nl is not None else PKT_BAD_INNER)
            want_slot.append(slot)
        n = len(msgs)
        lengths = np.array([len(m) for m in msgs], np.uint32)
        off = H.layout_packed(lengths, slack=16)
        b = c.batch(n, H.ring_bytes_for(off, lengths))
        H.fill_payloads(b.ring, off, msgs, headroom=0)
        b.off[:n], b.len[:n] = off, lengths
        b.slot[:n] = 0xFFFFFFFF
        b.open(n, F_DEMUX_INDEX | F_REPLAY | F_INNER_CHECK)
        seen = set()
        for i in range(n):
            w = want[i]
            if isinstance(w, tuple):
                assert b.status[i] == PKT_OK and b.out_len[i] == w[1], i
            else:
                assert b.status[i] == w, (i, b.status[i], w)
            if want_slot[i] is not None and w != PKT_MALFORMED:
                assert b.slot[i] == want_slot[i]
            seen.add(int(b.status[i]))
        assert seen == {PKT_OK, PKT_BAD_INNER, PKT_NO_KEYPAIR, PKT_KEEPALIVE, PKT_MALFORMED}
        b.close()
    finally:
        c.close()


def test_receive_classification(gpu_lib, oracle):
    """Bind.classify on the GPU: disco and STUN peel off first, then the source address decides."""
    import ipaddress

    from bnk_b200 import Context, _lib

    rng = np.random.default_rng(33)

    def a16(text):
        ip = ipaddress.ip_address(text)
        return (ipaddress.IPv6Address("::ffff:" + text) if ip.version == 4 else ip).packed

    known = [("203.0.113.5", 51820, 3), ("203.0.113.5", 51821, 4), ("2001:db8::7", 4000, 9), ("198.51.100.200", 1, 0)]
    magic = b"bnk\x00disco\x00"
    stun = bytes([0x01, 0x01, 0x00, 0x00, 0x21, 0x12, 0xA4, 0x42]) + bytes(12)
    wg = b"\x04\x00\x00\x00" + bytes(60)
    cases = []  # (datagram, source text, port)
    for pkt in [magic + bytes(80), magic, magic[:9] + b"\x01" + bytes(20), magic[:9], stun, stun[:19], bytes([0x41]) + stun[1:],
                stun[:4] + b"\x21\x12\xA4\x43" + bytes(12), wg, b"", b"\x04"]:
        for src in [("203.0.113.5", 51820), ("203.0.113.5", 51822), ("2001:db8::7", 4000), ("2001:db8::8", 4000),
                    ("198.51.100.200", 1), ("10.1.1.1", 9)]:
            cases.append((pkt, src[0], src[1]))
    n = len(cases)
    with Context(max_keypairs=16, flow_capacity=0) as c:
        for text, port, peer in known:
            c.addr_set(a16(text), port, peer)
        c.addr_set(a16("10.1.1.1"), 9, 5)
        c.addr_clear(a16("10.1.1.1"), 9)  # a path that was demoted again
        lengths = np.array([len(p) for p, _, _ in cases], np.uint32)
        off = H.layout_packed(lengths, slack=16)
        b = c.batch(n, H.ring_bytes_for(off, lengths))
        H.fill_payloads(b.ring, off, [p for p, _, _ in cases], headroom=0)
        b.off[:n], b.len[:n] = off, lengths
        b.slot[:n] = 0xFFFFFFFF
        for i, (_, text, port) in enumerate(cases):
            b.src_addr[i, :16] = np.frombuffer(a16(text), np.uint8)
            b.src_addr[i, 16], b.src_addr[i, 17] = port >> 8, port & 0xFF
        b.classify(n)
        table = {(a16(t), p): peer for t, p, peer in known}
        seen = set()
        for i, (pkt, text, port) in enumerate(cases):
            shape = oracle.classify_shape(pkt)
            if shape:
                want = shape
            else:
                peer = table.get((a16(text), port))
                want = _lib.CLASS_WIREGUARD if peer is not None else _lib.CLASS_STRANGER
                if peer is not None:
                    assert b.slot[i] == peer
            assert b.status[i] == want, (i, pkt[:12], text, port)
            seen.add(int(b.status[i]))
        assert seen == {_lib.CLASS_WIREGUARD, _lib.CLASS_DISCO, _lib.CLASS_STUN, _lib.CLASS_STRANGER}
        b.close()


def test_config4_full_size_every_byte(gpu_lib, oracle):
    """BASELINE configuration 4 at its stated size, 1,048,576 x 1420 B over 65,536 peers, device resident.
    Every byte of the sealed ring equals what OpenSSL (all host cores) makes of the same plaintext ring, and
    its digest equals the committed one; every opened packet equals its plaintext; counters are the 16
    sequential nonces per peer; sealing and opening the same ring again is refused packet for packet."""
    import hashlib
    import json
    import os

    from bnk_b200 import Context, gen
    from bnk_b200.device import F_ASSIGN_COUNTERS, F_NO_D2H, F_NO_H2D, F_REPLAY, F_USE_OUT_LEN, PKT_OK, PKT_REPLAY

    n, peers, size = 1 << 20, 1 << 16, 1420
    plan = gen.config4(n, peers, size)
    stride = plan.stride
    keys = gen.bulk_keys(plan)
    ridx = np.arange(peers, dtype=np.uint32)
    i = np.arange(n, dtype=np.uint64)
    off = (i * np.uint64(stride)).astype(np.uint32)
    slot = (i % np.uint64(peers)).astype(np.uint32)
    # the checker's side: the same ring regenerated on the host and sealed in place
    want = gen.splitmix_fill(plan.payload_seed, n * stride)
    plain = want.reshape(n, stride)[:, 16:16 + size].copy()
    _, st, ol = oracle.cpu_aead_batch(False, oracle.host_cores(), keys, ridx, size, want, off, np.full(n, size, np.uint32),
                                      slot, i // np.uint64(peers))
    assert (st == 0).all() and (ol == size + 32).all()
    c = Context(max_keypairs=peers, mtu=size, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, ridx)
        b = c.batch(n, n * stride)
        b.off[:] = off
        b.len[:] = size
        b.slot[:] = slot
        b.upload(n)
        b.fill_random(plan.payload_seed)
        dev = F_NO_H2D | F_NO_D2H
        b.seal(n, dev | F_ASSIGN_COUNTERS, wait=False)
        b.wait()
        b.download(n)
        assert (b.status[:n] == PKT_OK).all() and (b.out_len[:n] == size + 32).all()
        assert np.array_equal(b.counter[:n], i // np.uint64(peers))
        got = b.ring[:n * stride]
        if not np.array_equal(got, want):
            bad = np.flatnonzero((got.reshape(n, stride) != want.reshape(n, stride)).any(axis=1))
            raise AssertionError(f"{len(bad)} sealed packets differ from OpenSSL's, first {bad[:8]}")
        golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "aead_golden.json")))["config4_full"]
        digest = hashlib.sha256(np.ascontiguousarray(got.reshape(n, stride)[:, :size + 32])).hexdigest()
        assert digest == golden["sealed_sha256"]
        del want
        b.open(n, dev | F_REPLAY | F_USE_OUT_LEN, wait=False)
        b.wait()
        b.download(n)
        assert (b.status[:n] == PKT_OK).all() and (b.out_len[:n] == size).all()
        opened = b.ring[:n * stride].reshape(n, stride)[:, 16:16 + size]
        if not np.array_equal(opened, plain):
            bad = np.flatnonzero((opened != plain).any(axis=1))
            raise AssertionError(f"{len(bad)} opened packets differ from their plaintext, first {bad[:8]}")
        # the same ciphertext again: every packet is a replay now
        b.seal(n, dev, wait=False)            # same counters as before (host counters were downloaded = the assigned ones)
        b.open(n, dev | F_REPLAY | F_USE_OUT_LEN, wait=False)
        b.wait()
        b.download(n)
        assert (b.status[:n] == PKT_REPLAY).all()
        b.close()
    finally:
        c.close()


def test_imix_full_size_two_batches_in_flight(gpu_lib, oracle):
    """The benchmark's mixed-size leg at its size: 2 x 524,288 packets of 64/576/1420 B (7:4:1) in packed rings,
    two batches in flight on their own streams with the by-length scheduling order, counters handed out on the
    device, replay window on.  At this size the seal/open launches run on the low-priority stream beside the short
    kernels of the other batch and the length classes are laid out longest first; none of that may change a byte:
    every sealed message equals OpenSSL's (all host cores), every opened packet its plaintext, every packet is
    refused when the same messages come again."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_ASSIGN_COUNTERS, F_NO_D2H, F_NO_H2D, F_REPLAY, F_SORT_BY_LENGTH, F_USE_OUT_LEN,
                                 PKT_OK, PKT_REPLAY)

    per, peers_b, nb = 1 << 19, 1 << 15, 2
    g = gen.SplitMix64(gen.seed_for(2) + 31)
    keys = gen.SplitMix64(99).bytes(nb * peers_b * 32).reshape(nb * peers_b, 32)
    ridx = np.arange(nb * peers_b, dtype=np.uint32)
    c = Context(max_keypairs=nb * peers_b, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, ridx)
        bs, plans = [], []
        for j in range(nb):
            sizes = gen.imix_sizes(g, per)
            slot_bytes = ((sizes.astype(np.uint64) + np.uint64(48 + 15)) // np.uint64(16)) * np.uint64(16)
            off = np.concatenate([[0], np.cumsum(slot_bytes)[:-1]]).astype(np.uint32)
            total = int(off[-1]) + int(slot_bytes[-1])
            slot = (j * peers_b + np.arange(per, dtype=np.uint64) % np.uint64(peers_b)).astype(np.uint32)
            b = c.batch(per, total)
            b.off[:], b.len[:], b.slot[:] = off, sizes, slot
            b.upload(per)
            b.fill_random(4242 + j)
            b.download(per)  # the plaintext ring as the device made it
            plain_ring = np.array(b.ring[:total])
            bs.append(b)
            plans.append((sizes, off, slot, total, plain_ring))
        dev = F_NO_H2D | F_NO_D2H
        for b in bs:
            b.seal(per, dev | F_ASSIGN_COUNTERS | F_SORT_BY_LENGTH, wait=False)
        for b in bs:
            b.wait()
        for b, (sizes, off, slot, total, plain_ring) in zip(bs, plans):
            b.download(per)
            want_ctr = np.arange(per, dtype=np.uint64) // np.uint64(peers_b)  # packet i of a batch is the peer's (i div peers)-th
            assert np.array_equal(b.counter[:per], want_ctr)
            want = plain_ring.copy()
            _, st, ol = oracle.cpu_aead_batch(False, oracle.host_cores(), keys, ridx, 1420, want, off, sizes, slot, want_ctr)
            assert (st == 0).all()
            assert (b.status[:per] == PKT_OK).all() and np.array_equal(b.out_len[:per], ol)
            assert H.spans_differ_count(np.asarray(b.ring[:total]), want, off, ol) == 0
        for b in bs:
            b.open(per, dev | F_REPLAY | F_USE_OUT_LEN | F_SORT_BY_LENGTH, wait=False)
        for b in bs:
            b.wait()
        for b, (sizes, off, slot, total, plain_ring) in zip(bs, plans):
            b.download(per)
            assert (b.status[:per] == PKT_OK).all() and np.array_equal(b.out_len[:per], sizes)
            assert H.spans_differ_count(np.asarray(b.ring[:total]), plain_ring, off, sizes, start=16) == 0
        # the same messages again: seal with the counters that came down, open: all replays
        for b in bs:
            b.seal(per, dev | F_SORT_BY_LENGTH, wait=False)
            b.open(per, dev | F_REPLAY | F_USE_OUT_LEN | F_SORT_BY_LENGTH, wait=False)
        for b in bs:
            b.wait()
            b.download(per)
            assert (b.status[:per] == PKT_REPLAY).all()
            b.close()
    finally:
        c.close()
