"""Configurations 3 and 5 against the committed digests (tests/golden/make_golden.py): the CPU checker on CPU,
the CUDA path on the GPU.  The sealed messages of configuration 5 were produced by OpenSSL and libsodium."""
import hashlib
import json
import os

import numpy as np
import pytest

from tests import helpers as H
from tests import reference_cases as RC

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "aead_golden.json")
SEC = 1_000_000_000


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def _sha(*arrays):
    return hashlib.sha256(b"".join(np.ascontiguousarray(a).tobytes() for a in arrays)).hexdigest()


def _config3(golden):
    from bnk_b200 import gen

    w = gen.config3(*golden["config3"]["sizes"])
    assert _sha(w.rules, w.srcs, w.ports) == golden["config3"]["tables_sha256"]
    assert _sha(w.outbound, w.outbound_len, w.inbound, w.inbound_len, w.late, w.late_len) == golden["config3"]["headers_sha256"]
    return w


def test_config3_checker_matches_golden(oracle, golden):
    w = _config3(golden)
    f = oracle.Filter()
    f.set_rules_arrays(w.rules.astype(oracle.RULE_DTYPE), w.srcs.astype(oracle.PREFIX_DTYPE), w.ports.astype(oracle.PORT_DTYPE))
    f.note_batch(np.ascontiguousarray(w.outbound), 28, w.outbound_len, w.t0_ns)
    v1 = f.check_batch(np.ascontiguousarray(w.inbound), 28, np.ascontiguousarray(w.inbound_len), w.t0_ns + SEC)
    v2 = f.check_batch(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 600 * SEC)
    v3 = f.check_batch(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 2 * SEC)
    assert _sha(v1.astype(np.uint8), v2.astype(np.uint8), v3.astype(np.uint8)) == golden["config3"]["verdicts_sha256"]
    assert [int(v1.sum()), int(v2.sum()), int(v3.sum())] == golden["config3"]["allowed"]
    assert f.flow_count == golden["config3"]["flows"]


def _config5_segments(oracle, golden):
    from bnk_b200 import gen

    w = gen.config5(n_super=golden["config5"]["n_super"])
    assert hashlib.sha256(b"".join(w.supers)).hexdigest() == golden["config5"]["supers_sha256"]
    assert [int(x) for x in w.peer] == golden["config5"]["peers"]
    segs = []
    for sp in w.supers:
        segs.extend(oracle.gso_split(sp, w.hdr_len, w.mss, w.csum_start, w.csum_offset, 6))
    return w, segs


def test_config5_checker_matches_golden(oracle, golden):
    w, segs = _config5_segments(oracle, golden)
    assert hashlib.sha256(b"".join(segs)).hexdigest() == golden["config5"]["segments_sha256"]
    nxt, msgs = {}, []
    for i, s in enumerate(segs):
        p = int(w.peer[i // 47])
        c = nxt.get(p, 0)
        nxt[p] = c + 1
        msgs.append(oracle.wg_seal(w.keys[p].tobytes(), p + 1, c, s, 1420))
    assert hashlib.sha256(b"".join(msgs)).hexdigest() == golden["config5"]["sealed_sha256"]


@pytest.mark.gpu
def test_config3_gpu_matches_golden(gpu_lib, golden):
    from bnk_b200 import Context, gen
    from bnk_b200.device import PKT_OK
    from bnk_b200.filter import flatten_rule_arrays

    w = _config3(golden)
    c = Context(max_keypairs=4, flow_capacity=1 << 14)
    try:
        c.acl_set(True, flatten_rule_arrays(w.rules, w.srcs, w.ports))
        cap = max(len(w.outbound), len(w.inbound))
        b = c.batch(cap, cap * gen.HDR_STRIDE)

        def load(hdr, lens):
            n = len(lens)
            view = b.ring[: n * gen.HDR_STRIDE].reshape(n, gen.HDR_STRIDE)
            view[:] = 0
            view[:, 16:16 + hdr.shape[1]] = hdr
            b.off[:n] = (np.arange(n, dtype=np.uint64) * gen.HDR_STRIDE).astype(np.uint32)
            b.len[:n] = lens
            return n

        def verdicts(n):
            return (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)

        b.filter_note(load(w.outbound, w.outbound_len), w.t0_ns)
        n = load(w.inbound, w.inbound_len)
        b.filter_check(n, w.t0_ns + SEC)
        v1 = verdicts(n)
        n = load(w.late, w.late_len)
        b.filter_check(n, w.t0_ns + 600 * SEC)
        v2 = verdicts(n)
        b.filter_check(n, w.t0_ns + 2 * SEC)
        v3 = verdicts(n)
        assert _sha(v1, v2, v3) == golden["config3"]["verdicts_sha256"]
        assert c.flows_count() == golden["config3"]["flows"]
        b.close()
    finally:
        c.close()


@pytest.mark.gpu
def test_config5_gpu_matches_golden(gpu_lib, oracle, golden):
    """Split and seal on the GPU; the digest of the messages is the one OpenSSL and libsodium produced."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import F_ASSIGN_COUNTERS, F_NO_H2D, GSO_SUPER_DTYPE, PKT_OK

    w = gen.config5(n_super=golden["config5"]["n_super"])
    n_super, n_seg, stride = len(w.supers), 47, 1456
    n_pkts = n_super * n_seg
    n_peers = len(w.keys)
    sup = np.zeros(n_super, GSO_SUPER_DTYPE)
    at = n_pkts * stride
    for j, sp in enumerate(w.supers):
        sup[j]["first_pkt"], sup[j]["n_pkts"] = j * n_seg, n_seg
        sup[j]["hdr_len"], sup[j]["gso_size"] = w.hdr_len, w.mss
        sup[j]["csum_start"], sup[j]["csum_offset"], sup[j]["proto"] = w.csum_start, w.csum_offset, 6
        sup[j]["src_off"], sup[j]["src_len"] = at, len(sp)
        at += (len(sp) + 15) & ~15
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, w.keys, w.keys, (1 + np.arange(n_peers)).astype(np.uint32))
        b = c.batch(n_pkts, at + 64)
        for j, sp in enumerate(w.supers):
            o = int(sup[j]["src_off"])
            b.ring[o:o + len(sp)] = np.frombuffer(sp, np.uint8)
        b.off[:n_pkts] = H.layout_fixed(n_pkts, stride)
        b.len[:n_pkts] = w.hdr_len + w.mss
        b.slot[:n_pkts] = np.repeat(w.peer, n_seg)
        b.gso_split(sup, n_pkts)
        b.download(n_pkts)
        segs = b"".join(b.payload(i, 1420) for i in range(n_pkts))
        assert hashlib.sha256(segs).hexdigest() == golden["config5"]["segments_sha256"]
        b.seal(n_pkts, F_NO_H2D | F_ASSIGN_COUNTERS)
        assert (b.status[:n_pkts] == PKT_OK).all()
        msgs = b"".join(b.message(i) for i in range(n_pkts))
        assert hashlib.sha256(msgs).hexdigest() == golden["config5"]["sealed_sha256"]
        b.close()
    finally:
        c.close()
