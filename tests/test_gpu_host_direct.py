"""Small batches run on the caller's pinned buffers (no copies); larger ones through the copy engines.  Both
ways must give the same bytes, and a batch that ran without copies must still chain into device-resident calls."""
import os

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _context(direct_bytes, **kw):
    from bnk_b200 import Context

    old = os.environ.get("BNK_HOST_DIRECT_BYTES")
    os.environ["BNK_HOST_DIRECT_BYTES"] = str(direct_bytes)
    try:
        return Context(**kw)
    finally:
        if old is None:
            del os.environ["BNK_HOST_DIRECT_BYTES"]
        else:
            os.environ["BNK_HOST_DIRECT_BYTES"] = old


def _load(b, rng, n, n_peers):
    sizes = rng.choice([0, 1, 40, 576, 1300, 1420], n)
    off = (np.arange(n, dtype=np.uint64) * 1472).astype(np.uint32)
    for i in range(n):
        b.ring[int(off[i]) + 16:int(off[i]) + 16 + int(sizes[i])] = rng.integers(0, 256, int(sizes[i]), dtype=np.uint8)
    b.off[:n], b.len[:n] = off, sizes
    b.slot[:n] = rng.integers(0, n_peers, n)
    return off, sizes


@pytest.mark.parametrize("n", [1, 7, 64, 200, 256, 300])  # 300: beyond the mode's packet limit, copied both times
def test_same_bytes_with_and_without_copies(gpu_lib, oracle, n):
    from bnk_b200.device import F_ASSIGN_COUNTERS, F_REPLAY

    n_peers = 9
    keys = np.random.default_rng(5).integers(0, 256, (n_peers, 32), dtype=np.uint8)
    results = []
    for direct_bytes in (0, 1 << 20):  # never / for everything this test sends
        rng = np.random.default_rng(77 + n)
        c = _context(direct_bytes, max_keypairs=n_peers, mtu=1420, flow_capacity=0)
        try:
            c.set_keypairs(0, keys, keys, np.arange(n_peers, dtype=np.uint32))
            b = c.batch(n, n * 1472)
            _load(b, rng, n, n_peers)
            plain = np.array(b.ring)
            b.seal(n, F_ASSIGN_COUNTERS)
            sealed = (np.array(b.ring), np.array(b.out_len[:n]), np.array(b.counter[:n]), np.array(b.status[:n]))
            # twice through open: the second time every packet is a replay
            b.len[:n] = b.out_len[:n]
            b.open(n, F_REPLAY)
            opened = (np.array(b.ring), np.array(b.out_len[:n]), np.array(b.status[:n]))
            b.ring[:] = sealed[0]
            b.open(n, F_REPLAY)
            again = np.array(b.status[:n])
            b.close()
            results.append((plain, sealed, opened, again))
        finally:
            c.close()
    (plain0, sealed0, opened0, again0), (plain1, sealed1, opened1, again1) = results
    assert np.array_equal(plain0, plain1)
    for x, y in zip(sealed0 + opened0, sealed1 + opened1):
        assert np.array_equal(x, y)
    assert (sealed0[3] == oracle.OK).all()
    assert set(np.unique(opened0[2])) <= {oracle.OK, oracle.KEEPALIVE}
    assert (again0 == oracle.REPLAY).all() and (again1 == oracle.REPLAY).all()
    # and the plaintext came back
    off = (np.arange(n, dtype=np.uint64) * 1472).astype(np.int64)
    rng = np.random.default_rng(77 + n)
    sizes = rng.choice([0, 1, 40, 576, 1300, 1420], n)
    for i in range(n):
        o, l = int(off[i]) + 16, int(sizes[i])
        assert np.array_equal(opened1[0][o:o + l], plain1[o:o + l]), i


def test_device_resident_call_after_a_batch_without_copies(gpu_lib, oracle):
    """seal without copies leaves the device ring behind; a following open that asks for no upload must still
    see the sealed bytes, and a download must not bring stale device bytes over the results."""
    from bnk_b200.device import F_ASSIGN_COUNTERS, F_NO_D2H, F_NO_H2D

    n, n_peers = 48, 5
    rng = np.random.default_rng(9)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = _context(1 << 20, max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.arange(n_peers, dtype=np.uint32))
        b = c.batch(n, n * 1472)
        off, sizes = _load(b, rng, n, n_peers)
        plain = np.array(b.ring)
        b.seal(n, F_ASSIGN_COUNTERS)               # no copies
        sealed = np.array(b.ring)
        assert not np.array_equal(sealed, plain)
        b.download(n)                              # nothing newer on the device
        assert np.array_equal(np.array(b.ring), sealed)
        b.len[:n] = b.out_len[:n]
        b.open(n, F_NO_H2D | F_NO_D2H)             # device-resident call: the library uploads first
        b.download(n)
        assert (np.array(b.status[:n]) != oracle.AUTH_FAIL).all()
        got = np.array(b.ring)
        for i in range(n):
            o, l = int(off[i]) + 16, int(sizes[i])
            assert np.array_equal(got[o:o + l], plain[o:o + l]), i
        b.close()
    finally:
        c.close()


def test_classify_and_gso_after_a_batch_without_copies(gpu_lib, oracle):
    """A submit that ran on the host arrays leaves every device descriptor behind.  classify and the GSO split
    upload only what they read; when the device copies are stale they must bring all descriptor fields along,
    or a device-resident seal after them would read old counters."""
    from bnk_b200.device import F_NO_D2H, F_NO_H2D

    n, n_peers = 32, 3
    rng = np.random.default_rng(21)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = _context(1 << 20, max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.arange(n_peers, dtype=np.uint32))
        for i in range(n_peers):
            c.addr_set(bytes(10) + b"\xff\xff" + bytes([10, 0, 0, 1 + i]), 51820, i)
        b = c.batch(n, n * 1472)
        off, sizes = _load(b, rng, n, n_peers)
        sizes = np.maximum(sizes, 40)
        b.len[:n] = sizes
        b.counter[:n] = 1000 + np.arange(n)
        b.seal(n)                                   # host-direct: device descriptors are now behind
        first = np.array(b.ring)
        # new plaintext and new caller-chosen counters, written to the host arrays only
        for i in range(n):
            b.ring[int(off[i]) + 16:int(off[i]) + 16 + int(sizes[i])] = rng.integers(0, 256, int(sizes[i]), dtype=np.uint8)
        plain = np.array(b.ring)
        b.len[:n] = sizes
        b.counter[:n] = 5000 + np.arange(n)
        peers = rng.integers(0, n_peers, n)
        for i in range(n):
            b.src_addr[i, :] = 0
            b.src_addr[i, 10:12] = 0xFF
            b.src_addr[i, 12:16] = [10, 0, 0, 1 + int(peers[i])]
            b.src_addr[i, 16:18] = [51820 >> 8, 51820 & 255]
        b.classify(n)                               # uploads; must refresh counter/out_len/status too
        assert list(b.slot[:n]) == list(peers)
        b.seal(n, F_NO_H2D | F_NO_D2H)              # caller-supplied counters, read from the device copies
        b.download(n)
        assert (b.status[:n] == 0).all()
        assert (b.counter[:n] == 5000 + np.arange(n)).all()
        # (classify uploads datagrams, ring[off, off+len): the furthest packet's last 16 payload bytes, which lie
        # behind that span, are not part of its upload, so that one packet is left out of the byte comparison)
        for i in range(n - 1):
            o, l = int(off[i]) + 16, int(sizes[i])
            want = oracle.wg_seal(keys[int(peers[i])].tobytes(), int(peers[i]), 5000 + i, plain[o:o + l].tobytes(), 1420)
            assert b.message(i) == want, i
        assert not np.array_equal(np.array(b.ring), first)
        b.close()
    finally:
        c.close()
