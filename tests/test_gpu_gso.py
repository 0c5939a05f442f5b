"""Segmentation offload on the GPU against the CPU checker, and configuration 5's pipeline:
split -> note outbound -> counters -> seal on the sender, open -> replay -> inner check -> filter on the receiver."""
import numpy as np
import pytest

from tests import helpers as H
from tests import reference_cases as RC

pytestmark = pytest.mark.gpu


def _plan(supers, meta, stride):
    """Segment descriptors + super descriptors for a list of super-packets.  meta[j] = (hdr, gso, csum_start, csum_off, proto)."""
    from bnk_b200.device import GSO_SUPER_DTYPE

    sup = np.zeros(len(supers), GSO_SUPER_DTYPE)
    seg_len, first = [], 0
    for j, (pkt, (hdr, gso, cs, co, proto)) in enumerate(zip(supers, meta)):
        n = max(0, -(-(len(pkt) - hdr) // gso))
        for k in range(n):
            seg_len.append(hdr + min(gso, len(pkt) - hdr - k * gso))
        sup[j]["first_pkt"], sup[j]["n_pkts"] = first, n
        sup[j]["hdr_len"], sup[j]["gso_size"], sup[j]["csum_start"], sup[j]["csum_offset"], sup[j]["proto"] = hdr, gso, cs, co, proto
        sup[j]["src_len"] = len(pkt)
        first += n
    n_pkts = first
    at = n_pkts * stride
    for j, pkt in enumerate(supers):
        sup[j]["src_off"] = at
        at += (len(pkt) + 15) & ~15
    return sup, np.array(seg_len, np.uint32), n_pkts, at


def _tcp_super(rng, payload_len, ihl=5, tcp_words=5, flags=0x19):
    from bnk_b200 import gen

    iph = bytearray(gen.ipv4_header(6, gen.ip4(100, 64, 0, 1), gen.ip4(100, 64, 0, 2), ihl * 4 + tcp_words * 4 + payload_len, ihl))
    iph[4:6] = int(rng.integers(0, 65536)).to_bytes(2, "big")
    iph[20:] = rng.integers(0, 256, ihl * 4 - 20, dtype=np.uint8).tobytes()
    tcp = bytearray(tcp_words * 4)
    tcp[0:4] = bytes(gen.l4_ports(int(rng.integers(1, 65536)), 443))
    tcp[4:8] = int(rng.integers(0, 2**32)).to_bytes(4, "big")
    tcp[12] = tcp_words << 4
    tcp[13] = flags
    tcp[16:18] = b"\xAB\xCD"  # stale partial checksum: must be overwritten
    tcp[20:] = rng.integers(0, 256, tcp_words * 4 - 20, dtype=np.uint8).tobytes()
    return bytes(iph) + bytes(tcp) + rng.integers(0, 256, payload_len, dtype=np.uint8).tobytes(), ihl * 4, ihl * 4 + tcp_words * 4


def _udp_super(rng, payload_len):
    from bnk_b200 import gen

    iph = bytearray(gen.ipv4_header(17, gen.ip4(100, 64, 0, 1), gen.ip4(100, 64, 0, 2), 28 + payload_len))
    iph[4:6] = (65535).to_bytes(2, "big")  # id wraps
    udp = bytearray(8)
    udp[0:4] = bytes(gen.l4_ports(5000, 6000))
    udp[4:6] = (8 + payload_len).to_bytes(2, "big")
    return bytes(iph) + bytes(udp) + rng.integers(0, 256, payload_len, dtype=np.uint8).tobytes(), 20, 28


def test_split_matches_checker_byte_for_byte(gpu_lib, oracle):
    from bnk_b200 import Context

    rng = np.random.default_rng(8)
    supers, meta = [], []
    for payload_len, gso, kw in [(47 * 1380, 1380, {}), (10 * 1380 + 17, 1380, {}), (5000, 1001, {}), (1380, 1380, {}),
                                 (999, 1380, {"flags": 0x11}), (7777, 537, {"ihl": 6}), (4000, 1000, {"tcp_words": 8}),
                                 (3001, 333, {"ihl": 7, "tcp_words": 10})]:
        pkt, cs, hdr = _tcp_super(rng, payload_len, **kw)
        supers.append(pkt)
        meta.append((hdr, gso, cs, 16, 6))
    for payload_len, gso in [(9 * 1400, 1400), (5001, 1203), (100, 1400)]:
        pkt, cs, hdr = _udp_super(rng, payload_len)
        supers.append(pkt)
        meta.append((hdr, gso, cs, 6, 17))
    stride = 1536
    sup, seg_len, n_pkts, ring_bytes = _plan(supers, meta, stride)
    want = []
    for pkt, (hdr, gso, cs, co, proto) in zip(supers, meta):
        segs = oracle.gso_split(pkt, hdr, gso, cs, co, proto)
        assert segs is not None
        want.extend(segs)
    assert len(want) == n_pkts and [len(s) for s in want] == list(seg_len)
    with Context(max_keypairs=4, mtu=1420, flow_capacity=0) as c:
        key = np.arange(32, dtype=np.uint8).reshape(1, 32)
        c.set_keypairs(0, key, key, np.array([9], np.uint32))
        b = c.batch(n_pkts, ring_bytes + 64)
        b.ring[:] = 0xEE
        for j, pkt in enumerate(supers):
            o = int(sup[j]["src_off"])
            b.ring[o:o + len(pkt)] = np.frombuffer(pkt, np.uint8)
        b.off[:n_pkts] = H.layout_fixed(n_pkts, stride)
        b.len[:n_pkts] = seg_len
        b.slot[:n_pkts] = 0
        b.gso_split(sup, n_pkts)
        b.download(n_pkts)
        for i in range(n_pkts):
            o = int(b.off[i]) + 16
            assert b.ring[o:o + len(want[i])].tobytes() == want[i], f"segment {i}"
        # independent property: every segment carries valid IPv4 and transport checksums
        for i in range(n_pkts):
            s = want[i]
            ihl = (s[0] & 15) * 4
            assert oracle.inet_checksum(s[:ihl]) == 0
            pseudo = s[12:20] + bytes([0, s[9]]) + (len(s) - ihl).to_bytes(2, "big")
            assert oracle.inet_checksum(pseudo + s[ihl:]) == 0
        # a descriptor that disagrees with the split is refused by the seal that follows
        b.len[3] += 1
        b.gso_split(sup, n_pkts)
        from bnk_b200.device import F_NO_H2D, PKT_BAD_DESC, PKT_OK

        b.counter[:n_pkts] = np.arange(n_pkts)
        b.upload(n_pkts)       # counters only matter here; the ring on the device is overwritten by the next split
        b.gso_split(sup, n_pkts)
        b.seal(n_pkts, F_NO_H2D)
        st = np.array(b.status[:n_pkts])
        assert st[3] == PKT_BAD_DESC and (np.delete(st, 3) == PKT_OK).all()
        b.close()


def test_config5_pipeline(gpu_lib, oracle):
    """Reduced configuration 5: 64 super-packets (3008 segments) over Zipf-popular peers, 2,000-rule ACL."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_ASSIGN_COUNTERS, F_CHECK_INBOUND, F_DEMUX_INDEX, F_INNER_CHECK, F_NO_H2D,
                                 F_NOTE_OUTBOUND, F_REPLAY, PKT_FILTER_DENY, PKT_OK)
    from bnk_b200.filter import flatten_rule_arrays

    n_peers = 10_000
    w = gen.config5(n_super=64, n_peers=n_peers)
    meta = [(w.hdr_len, w.mss, w.csum_start, w.csum_offset, 6)] * len(w.supers)
    stride = 1456
    sup, seg_len, n_pkts, ring_bytes = _plan(w.supers, meta, stride)
    assert n_pkts == 64 * 47 and (seg_len == 1420).all()
    seg_peer = np.repeat(w.peer, 47).astype(np.uint32)
    # --- CPU checker: split, counters in batch order per peer, seal ---
    segs = []
    for pkt in w.supers:
        segs.extend(oracle.gso_split(pkt, 40, w.mss, 20, 16, 6))
    nxt, want_msgs = {}, []
    for i, s in enumerate(segs):
        p = int(seg_peer[i])
        ctr = nxt.get(p, 0)
        nxt[p] = ctr + 1
        want_msgs.append(oracle.wg_seal(w.keys[p].tobytes(), 0x1000 + p, ctr, s, 1420))
    # --- sender (this node) ---
    tx = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=1 << 14)
    rx = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=1 << 14)
    try:
        tx.set_keypairs(0, w.keys, w.keys, (0x1000 + np.arange(n_peers)).astype(np.uint32))
        tx.acl_set(True, None)  # enforcing: outbound flows are recorded
        b = tx.batch(n_pkts, ring_bytes + 64)
        for j, pkt in enumerate(w.supers):
            o = int(sup[j]["src_off"])
            b.ring[o:o + len(pkt)] = np.frombuffer(pkt, np.uint8)
        b.off[:n_pkts] = H.layout_fixed(n_pkts, stride)
        b.len[:n_pkts] = seg_len
        b.slot[:n_pkts] = seg_peer
        b.gso_split(sup, n_pkts)
        b.seal(n_pkts, F_NO_H2D | F_NOTE_OUTBOUND | F_ASSIGN_COUNTERS, now_ns=RC.T0)
        assert (b.status[:n_pkts] == PKT_OK).all()
        for i in range(n_pkts):
            assert b.message(i) == want_msgs[i], f"sealed segment {i}"
        assert tx.flows_count() == len({(int(p), s[20:24]) for p, s in zip(seg_peer, segs)})
        # --- receiver: one node that has this sender as its only peer, behind a 2,000-rule ACL ---
        # every peer of the sender is modelled by the same receiving context: receiver index 0x1000+p -> slot p,
        # and slot p accepts inner packets from the sender's address only
        f3 = gen.config3(n_rules=2000, n_nodes=5000, n_out=16, n_in=16, seed=gen.seed_for(5) + 1)
        rules, srcs, ports = f3.rules.copy(), f3.srcs.copy(), f3.ports.copy()
        # let a few tcp rules name the sender so that both verdicts occur
        hit = np.flatnonzero(rules["proto"] == 6)[:3]
        for r in hit:
            srcs["addr"][rules["src_begin"][r]] = w.self_ip
            srcs["bits"][rules["src_begin"][r]] = 32
        rx.set_keypairs(0, w.keys, w.keys, np.zeros(n_peers, np.uint32))
        used = sorted(set(seg_peer.tolist()))
        for p in used:
            rx.index_set(0x1000 + p, p)
            rx.set_allowed_ip(p, w.self_ip)
        rx.acl_set(True, flatten_rule_arrays(rules, srcs, ports))
        fo = oracle.Filter()
        fo.set_rules_arrays(rules.astype(oracle.RULE_DTYPE), srcs.astype(oracle.PREFIX_DTYPE), ports.astype(oracle.PORT_DTYPE))
        want_status = [PKT_OK if fo.check_inbound(s, RC.T0) else PKT_FILTER_DENY for s in segs]
        lengths = np.array([len(m) for m in want_msgs], np.uint32)
        r = rx.batch(n_pkts, n_pkts * stride)
        r.off[:n_pkts] = H.layout_fixed(n_pkts, stride)
        r.len[:n_pkts] = lengths
        H.fill_payloads(r.ring, r.off[:n_pkts], want_msgs, headroom=0)
        r.open(n_pkts, F_DEMUX_INDEX | F_REPLAY | F_INNER_CHECK | F_CHECK_INBOUND, now_ns=RC.T0)
        assert list(r.status[:n_pkts]) == want_status
        assert np.array_equal(r.slot[:n_pkts], seg_peer)
        assert 0 < want_status.count(PKT_OK) < n_pkts
        for i in range(0, n_pkts, 5):
            assert r.payload(i, 1420) == segs[i]
        b.close()
        r.close()
    finally:
        tx.close()
        rx.close()


def test_config5_full_size_every_segment(gpu_lib, oracle):
    """BASELINE configuration 5 at the size the benchmark runs: 2,048 super-packets -> 96,256 segments of 1420 B,
    Zipf(1.1) over 10,000 peers, 2,000-rule ACL.  Sender: every sealed segment equals the CPU checker's split
    sealed by OpenSSL, and the digests equal the committed ones.  Receiver: every status, slot and plaintext."""
    import hashlib
    import json
    import os

    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_ASSIGN_COUNTERS, F_CHECK_INBOUND, F_DEMUX_INDEX, F_INNER_CHECK, F_NO_H2D,
                                 F_NOTE_OUTBOUND, F_REPLAY, F_STATS, PKT_FILTER_DENY, PKT_OK)
    from bnk_b200.filter import flatten_rule_arrays

    n_peers, n_super, stride = 10_000, 2048, 1456
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "aead_golden.json")))["config5_full"]
    w = gen.config5(n_super=n_super, n_peers=n_peers)
    assert hashlib.sha256(b"".join(w.supers)).hexdigest() == golden["supers_sha256"]
    meta = [(w.hdr_len, w.mss, w.csum_start, w.csum_offset, 6)] * n_super
    sup, seg_len, n_pkts, ring_bytes = _plan(w.supers, meta, stride)
    assert n_pkts == golden["segments"] and (seg_len == 1420).all()
    seg_peer = np.repeat(w.peer, 47).astype(np.uint32)
    off = H.layout_fixed(n_pkts, stride)
    # --- CPU checker: split; counters in batch order per peer; sealed by OpenSSL on all cores ---
    segs = []
    for pkt in w.supers:
        segs.extend(oracle.gso_split(pkt, 40, w.mss, 20, 16, 6))
    seg_bytes = np.frombuffer(b"".join(segs), np.uint8).reshape(n_pkts, 1420)
    assert hashlib.sha256(seg_bytes).hexdigest() == golden["segments_sha256"]
    counter = np.zeros(n_pkts, np.uint64)
    nxt = {}
    for k, p in enumerate(seg_peer.tolist()):
        counter[k] = nxt.get(p, 0)
        nxt[p] = int(counter[k]) + 1
    ridx = (0x1000 + np.arange(n_peers)).astype(np.uint32)
    want = np.zeros(n_pkts * stride, np.uint8)
    want.reshape(n_pkts, stride)[:, 16:16 + 1420] = seg_bytes
    _, st, ol = oracle.cpu_aead_batch(False, oracle.host_cores(), w.keys, ridx, 1420, want, off,
                                      np.full(n_pkts, 1420, np.uint32), seg_peer, counter)
    assert (st == 0).all() and (ol == 1452).all()
    want_msgs = want.reshape(n_pkts, stride)[:, :1452]
    assert hashlib.sha256(np.ascontiguousarray(want_msgs)).hexdigest() == golden["sealed_sha256"]
    tx = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=1 << 18)
    rx = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=1 << 14)
    try:
        tx.set_keypairs(0, w.keys, w.keys, ridx)
        tx.acl_set(True, None)
        b = tx.batch(n_pkts, ring_bytes + 64)
        for j, pkt in enumerate(w.supers):
            o = int(sup[j]["src_off"])
            b.ring[o:o + len(pkt)] = np.frombuffer(pkt, np.uint8)
        b.off[:n_pkts] = off
        b.len[:n_pkts] = seg_len
        b.slot[:n_pkts] = seg_peer
        b.gso_split(sup, n_pkts)
        b.seal(n_pkts, F_NO_H2D | F_NOTE_OUTBOUND | F_ASSIGN_COUNTERS | F_STATS, now_ns=RC.T0)
        assert (b.status[:n_pkts] == PKT_OK).all()
        assert b.stats()["by_status"][PKT_OK] == n_pkts and b.stats()["bytes_out"] == 1452 * n_pkts
        assert np.array_equal(b.counter[:n_pkts], counter)
        got_msgs = b.ring[:n_pkts * stride].reshape(n_pkts, stride)[:, :1452]
        if not np.array_equal(got_msgs, want_msgs):
            bad = np.flatnonzero((got_msgs != want_msgs).any(axis=1))
            raise AssertionError(f"{len(bad)} sealed segments differ, first {bad[:8]}")
        assert hashlib.sha256(np.ascontiguousarray(got_msgs)).hexdigest() == golden["sealed_sha256"]
        assert tx.flows_count() == len({(int(p), s[20:24]) for p, s in zip(seg_peer, segs)})
        # --- receiver ---
        f3 = gen.config3(n_rules=2000, n_nodes=5000, n_out=16, n_in=16, seed=gen.seed_for(5) + 1)
        rules, srcs, ports = f3.rules.copy(), f3.srcs.copy(), f3.ports.copy()
        hit = np.flatnonzero(rules["proto"] == 6)[:3]
        for r in hit:
            srcs["addr"][rules["src_begin"][r]] = w.self_ip
            srcs["bits"][rules["src_begin"][r]] = 32
        rx.set_keypairs(0, w.keys, w.keys, np.zeros(n_peers, np.uint32))
        for p in sorted(set(seg_peer.tolist())):
            rx.index_set(0x1000 + p, p)
            rx.set_allowed_ip(p, w.self_ip)
        rx.acl_set(True, flatten_rule_arrays(rules, srcs, ports))
        fo = oracle.Filter()
        fo.set_rules_arrays(rules.astype(oracle.RULE_DTYPE), srcs.astype(oracle.PREFIX_DTYPE), ports.astype(oracle.PORT_DTYPE))
        allow = fo.check_batch_mt(seg_bytes, 1420, np.full(n_pkts, 1420, np.uint32), RC.T0)
        want_status = np.where(allow == 1, PKT_OK, PKT_FILTER_DENY).astype(np.uint8)
        r = rx.batch(n_pkts, n_pkts * stride)
        r.off[:n_pkts] = off
        r.len[:n_pkts] = 1452
        r.ring[:n_pkts * stride] = b.ring[:n_pkts * stride]
        r.open(n_pkts, F_DEMUX_INDEX | F_REPLAY | F_INNER_CHECK | F_CHECK_INBOUND | F_STATS, now_ns=RC.T0)
        assert np.array_equal(r.status[:n_pkts], want_status)
        assert np.array_equal(r.slot[:n_pkts], seg_peer)
        assert 0 < int(allow.sum()) < n_pkts
        assert r.stats()["by_status"][PKT_OK] == int(allow.sum())
        opened = r.ring[:n_pkts * stride].reshape(n_pkts, stride)[:, 16:16 + 1420]
        assert np.array_equal(opened, seg_bytes)  # the filter's verdict does not touch the plaintext
        # the same messages once more: every one is a replay
        r.ring[:n_pkts * stride] = b.ring[:n_pkts * stride]
        r.open(n_pkts, F_DEMUX_INDEX | F_REPLAY | F_INNER_CHECK | F_CHECK_INBOUND, now_ns=RC.T0)
        assert (r.status[:n_pkts] == 2).all()
        b.close()
        r.close()
    finally:
        tx.close()
        rx.close()
