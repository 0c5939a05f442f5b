"""The submit queue: upstream-sized caller batches from several threads, packed into GPU batches.  Whatever the
packing, every caller gets its own packets back, byte for byte what the CPU checker makes of them; nonces run
per keypair in submit order and replay verdicts follow arrival order across GPU batches."""
import threading
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("depth,max_pkts", [(1, 256), (2, 1024), (3, 4096)])
def test_queue_round_trip_from_several_threads(gpu_lib, oracle, depth, max_pkts):
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY, PKT_KEEPALIVE, PKT_OK, PKT_REPLAY, Queue

    n_threads, peers_per_thread, rounds, per_call = 6, 5, 12, 128
    n_peers = n_threads * peers_per_thread
    rng = np.random.default_rng(depth)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    errors = []
    try:
        c.set_keypairs(0, keys, keys, (0x300 + np.arange(n_peers)).astype(np.uint32))
        sealq = Queue(c, False, 0, max_pkts=max_pkts, depth=depth)
        openq = Queue(c, True, F_REPLAY, max_pkts=max_pkts, depth=depth)

        def collect(q, pending):
            t = pending.pop(0)
            return q.wait(t[0]), t[1]

        def worker(t):
            try:
                r = np.random.default_rng(100 + t)
                nxt = {}
                sealed_all = []
                pending = []

                def check_sealed(res, meta):
                    (msgs, st, ctr, _), (pkts, slots) = res, meta
                    for k in range(len(pkts)):
                        s = int(slots[k])
                        want_ctr = nxt.get(s, 0)
                        nxt[s] = want_ctr + 1
                        assert st[k] == PKT_OK and ctr[k] == want_ctr, (t, k, st[k], ctr[k], want_ctr)
                        if k % 7 == 0:  # the checker is scalar: a spread sample of the bytes, all of the counters
                            assert msgs[k] == oracle.wg_seal(keys[s].tobytes(), 0x300 + s, want_ctr, pkts[k], 1420)
                    sealed_all.append((msgs, pkts, slots))

                for _ in range(rounds):
                    n = int(r.integers(1, per_call + 1))
                    sizes = r.choice([0, 64, 576, 1420], n)
                    pkts = [r.integers(0, 256, int(s), dtype=np.uint8).tobytes() for s in sizes]
                    slots = (t * peers_per_thread + r.integers(0, peers_per_thread, n)).astype(np.uint32)
                    while True:
                        ticket = sealq.submit(pkts, slots)
                        if ticket is not None:
                            break
                        if pending:   # what this thread holds may be what keeps a GPU batch from being reused
                            check_sealed(*collect(sealq, pending))
                        else:         # the other threads are ahead: let them collect
                            time.sleep(0)
                    pending.append((ticket, (pkts, slots)))
                    if len(pending) >= 3:
                        check_sealed(*collect(sealq, pending))
                while pending:
                    check_sealed(*collect(sealq, pending))
                # receive side: everything once, then everything again (all replays), two tickets in flight
                for second in (False, True):
                    pend = []

                    def check_opened(res, meta):
                        (pts, st, ctr, _), (pkts, slots) = res, meta
                        for k in range(len(pkts)):
                            if second:
                                assert st[k] == PKT_REPLAY and pts[k] == b"", (t, k, st[k])
                            else:
                                assert st[k] == (PKT_OK if len(pkts[k]) else PKT_KEEPALIVE), (t, k, st[k])
                                assert pts[k][:len(pkts[k])] == pkts[k]

                    for msgs, pkts, slots in sealed_all:
                        while True:
                            ticket = openq.submit(msgs, slots)
                            if ticket is not None:
                                break
                            if pend:
                                check_opened(*collect(openq, pend))
                            else:
                                time.sleep(0)
                        pend.append((ticket, (pkts, slots)))
                        if len(pend) >= 2:
                            check_opened(*collect(openq, pend))
                    while pend:
                        check_opened(*collect(openq, pend))
            except BaseException as e:  # noqa: BLE001
                errors.append((t, repr(e)))

        threads = [threading.Thread(target=worker, args=(t,)) for t in range(n_threads)]
        for th in threads:
            th.start()
        for th in threads:
            th.join()
        assert not errors, errors[:3]
        ss, so = sealq.stats(), openq.stats()
        assert ss["caller_batches"] == n_threads * rounds and ss["gpu_batches"] <= ss["caller_batches"]
        assert so["caller_batches"] == 2 * n_threads * rounds
        sealq.close()
        openq.close()
    finally:
        c.close()


def test_queue_refuses_what_it_cannot_take(gpu_lib):
    import ctypes as C

    from bnk_b200 import Context, _lib
    from bnk_b200.device import Queue

    c = Context(max_keypairs=4, mtu=1420, flow_capacity=0)
    try:
        c.set_keypair(0, bytes(32), bytes(range(32)), 1)
        q = Queue(c, False, 0, max_pkts=8, max_packet=100, depth=1)
        with pytest.raises(_lib.BnkError):
            q.submit([b"x"] * 9, np.zeros(9, np.uint32))          # more than a GPU batch holds
        with pytest.raises(_lib.BnkError):
            q.submit([bytes(101)], np.zeros(1, np.uint32))         # longer than max_packet
        t1 = q.submit([b"abc"] * 8, np.zeros(8, np.uint32))
        outs, st, ctr, _ = q.wait(t1)
        assert (st == 0).all() and list(ctr) == list(range(8)) and all(len(o) == 16 + 16 + 16 for o in outs)
        dummy = np.zeros(64, np.uint8)
        assert _lib.lib().bnk_queue_wait(q._h, t1[0], dummy.ctypes.data, dummy.ctypes.data, None, None,
                                         dummy.ctypes.data) == _lib.EINVAL  # a ticket is good for one wait
        # tickets held without being collected: the rotation runs out and submit says so instead of blocking
        held = []
        for _ in range(8):
            t = q.submit([b"abc"] * 8, np.zeros(8, np.uint32))
            if t is None:
                break
            held.append(t)
        assert 1 <= len(held) < 8
        assert _lib.lib().bnk_queue_wait_room(q._h, 1000) == _lib.ETIMEDOUT  # nobody collects: no room appears
        for t in held:
            q.wait(t)
        assert _lib.lib().bnk_queue_wait_room(q._h, 0xFFFFFFFFFFFFFFFF) == 0
        assert q.submit([b"abc"], np.zeros(1, np.uint32)) is not None
        q.close()
    finally:
        c.close()


def test_queue_spans_without_host_copies(gpu_lib, oracle):
    """reserve / commit / wait_span / release: callers write into the GPU batch's pinned ring and read the results in
    place.  Three threads, mixed with a fourth that uses the copying calls on the same queues; every sealed message
    equals the checker's, counters run per keypair in submit order, opened packets equal their plaintext, a second
    delivery is refused, an oversized packet is refused without touching its neighbours."""
    from bnk_b200 import Context
    from bnk_b200.device import F_REPLAY, PKT_BAD_DESC, PKT_KEEPALIVE, PKT_OK, PKT_REPLAY, Queue

    n_threads, peers_per_thread, rounds = 4, 4, 10
    n_peers = n_threads * peers_per_thread
    rng = np.random.default_rng(5)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    errors = []
    try:
        c.set_keypairs(0, keys, keys, (0x500 + np.arange(n_peers)).astype(np.uint32))
        sealq = Queue(c, False, 0, max_pkts=512, depth=2)
        openq = Queue(c, True, F_REPLAY, max_pkts=512, depth=2)

        def take(q, n):
            while True:
                r = q.reserve(n)
                if r is not None:
                    return r
                time.sleep(0)

        def span_worker(t):
            try:
                r = np.random.default_rng(200 + t)
                nxt = {}
                for _ in range(rounds):
                    n = int(r.integers(1, 97))
                    sizes = r.choice([0, 64, 576, 1420], n).astype(np.uint32)
                    pkts = [r.integers(0, 256, int(s), dtype=np.uint8) for s in sizes]
                    slots = (t * peers_per_thread + r.integers(0, peers_per_thread, n)).astype(np.uint32)
                    ticket, v = take(sealq, n)
                    for k in range(n):
                        v["data"][k, 16:16 + int(sizes[k])] = pkts[k]
                    v["len"][:] = sizes
                    v["slot"][:] = slots
                    sealq.commit(ticket)
                    res = sealq.wait_span(ticket)
                    msgs = []
                    for k in range(n):
                        s = int(slots[k])
                        want_ctr = nxt.get(s, 0)
                        nxt[s] = want_ctr + 1
                        assert res["status"][k] == PKT_OK and res["counter"][k] == want_ctr
                        msg = res["data"][k, :int(res["out_len"][k])].tobytes()
                        if k % 5 == 0:
                            assert msg == oracle.wg_seal(keys[s].tobytes(), 0x500 + s, want_ctr, pkts[k].tobytes(), 1420)
                        msgs.append(msg)
                    sealq.release(ticket)
                    for second in (False, True):
                        ticket, v = take(openq, n)
                        for k in range(n):
                            v["data"][k, :len(msgs[k])] = np.frombuffer(msgs[k], np.uint8)
                            v["len"][k] = len(msgs[k])
                        v["slot"][:] = slots
                        openq.commit(ticket)
                        res = openq.wait_span(ticket)
                        for k in range(n):
                            if second:
                                assert res["status"][k] == PKT_REPLAY
                            else:
                                assert res["status"][k] == (PKT_OK if sizes[k] else PKT_KEEPALIVE)
                                assert res["out_len"][k] >= sizes[k]
                                assert np.array_equal(res["data"][k, 16:16 + int(sizes[k])], pkts[k])
                        openq.release(ticket)
            except Exception as e:  # noqa: BLE001
                errors.append((t, repr(e)))

        def copy_worker(t):
            try:
                r = np.random.default_rng(300 + t)
                nxt = {}
                for _ in range(rounds):
                    n = int(r.integers(1, 65))
                    pkts = [r.integers(0, 256, int(s), dtype=np.uint8).tobytes() for s in r.choice([64, 1420], n)]
                    slots = (t * peers_per_thread + r.integers(0, peers_per_thread, n)).astype(np.uint32)
                    while (ticket := sealq.submit(pkts, slots)) is None:
                        time.sleep(0)
                    msgs, st, ctr, _ = sealq.wait(ticket)
                    for k in range(n):
                        s = int(slots[k])
                        want_ctr = nxt.get(s, 0)
                        nxt[s] = want_ctr + 1
                        assert st[k] == PKT_OK and ctr[k] == want_ctr
                    while (ticket := openq.submit(msgs, slots)) is None:
                        time.sleep(0)
                    pts, st, _, _ = openq.wait(ticket)
                    assert all(st[k] == PKT_OK and pts[k][:len(pkts[k])] == pkts[k] for k in range(n))
            except Exception as e:  # noqa: BLE001
                errors.append((t, repr(e)))

        th = [threading.Thread(target=span_worker, args=(t,)) for t in range(3)]
        th.append(threading.Thread(target=copy_worker, args=(3,)))
        for x in th:
            x.start()
        for x in th:
            x.join()
        assert errors == []
        # an oversized length is refused at commit, the packet comes back BAD_DESC, its neighbours are sealed
        ticket, v = take(sealq, 3)
        v["data"][:, 16:16 + 64] = 7
        v["len"][:] = (64, 5000, 64)
        v["slot"][:] = 0
        with pytest.raises(Exception):
            sealq.commit(ticket)
        res = sealq.wait_span(ticket)
        assert list(res["status"]) == [PKT_OK, PKT_BAD_DESC, PKT_OK]
        assert res["counter"][2] == res["counter"][0] + 1
        sealq.release(ticket)
        with pytest.raises(Exception):
            sealq.release(ticket)  # once per ticket
        sealq.close()
        openq.close()
    finally:
        c.close()


def test_queues_carry_the_filter_and_the_index_lookup(gpu_lib, oracle):
    """The two queues as the device's two directions: the seal queue records outbound flows (BNK_F_NOTE_OUTBOUND),
    the open queue finds the keypair from the receiver index in the header, runs the replay window and the inbound
    filter.  With default-deny rules only replies to what went out come back in; the verdicts are the checker's
    (filter.go:121-147, :189-209), whatever GPU batches the callers' packets happened to share."""
    from tests import reference_cases as RC
    from bnk_b200 import Context
    from bnk_b200.device import (F_CHECK_INBOUND, F_DEMUX_INDEX, F_NOTE_OUTBOUND, F_REPLAY, PKT_FILTER_DENY, PKT_OK,
                                 Queue)

    n_peers = 6
    rng = np.random.default_rng(11)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=1 << 12)
    try:
        # loopback: this context is both ends, so a peer's local and remote index are the same number
        c.set_keypairs(0, keys, keys, (0x600 + np.arange(n_peers)).astype(np.uint32))
        for p in range(n_peers):
            c.index_set(0x600 + p, p)
        c.acl_set(True, np.zeros(0, dtype=np.uint8))  # enforce, no allowances: replies only
        out_q = Queue(c, False, F_NOTE_OUTBOUND, max_pkts=256, depth=2)
        plain_q = Queue(c, False, 0, max_pkts=256, depth=2)  # stands for the far ends sealing what they send us
        in_q = Queue(c, True, F_DEMUX_INDEX | F_REPLAY | F_CHECK_INBOUND, max_pkts=256, depth=2)
        f = oracle.Filter()
        f.set_rules([])
        peer_ip = [RC.ip(f"100.64.3.{10 + p}") for p in range(n_peers)]
        errors = []

        def worker(t):
            try:
                r = np.random.default_rng(400 + t)
                slots = np.full(40, t, np.uint32)
                sent = [RC.udp(RC.SELF, peer_ip[t], 30000 + 50 * t + k, 53) for k in range(40)]
                while (tk := out_q.submit(sent, slots, now_ns=RC.T0)) is None:
                    time.sleep(0)
                _, st, _, _ = out_q.wait(tk)
                assert (st == PKT_OK).all()
                # what comes back: replies to every second flow, and as many packets nobody asked for
                back = [RC.udp(peer_ip[t], RC.SELF, 53, 30000 + 50 * t + k) for k in range(0, 40, 2)]
                back += [RC.udp(peer_ip[t], RC.SELF, 53, 45000 + int(r.integers(0, 1000))) for _ in range(20)]
                while (tk := plain_q.submit(back, slots[:40], now_ns=RC.T0)) is None:
                    time.sleep(0)
                msgs, st, _, _ = plain_q.wait(tk)
                assert (st == PKT_OK).all()
                while (tk := in_q.submit(msgs, None, now_ns=RC.T0 + RC.SEC)) is None:
                    time.sleep(0)
                pts, st, _, slot_found = in_q.wait(tk)
                assert (slot_found == t).all()
                return_value.append((t, sent, back, pts, st))
            except Exception as e:  # noqa: BLE001
                errors.append((t, repr(e)))

        return_value = []
        th = [threading.Thread(target=worker, args=(t,)) for t in range(n_peers)]
        for x in th:
            x.start()
        for x in th:
            x.join()
        assert errors == []
        # the checker, sequentially: all outbound first (one clock value), then each inbound packet
        for _, sent, _, _, _ in return_value:
            for pkt in sent:
                f.note_outbound(pkt, RC.T0)
        for t, _, back, pts, st in return_value:
            for k, pkt in enumerate(back):
                want = f.check_inbound(pkt, RC.T0 + RC.SEC)
                assert st[k] == (PKT_OK if want else PKT_FILTER_DENY), (t, k, st[k], want)
                assert (pts[k][:len(pkt)] == pkt) if want else (pts[k] == b"")
            assert (st[:20] == PKT_OK).all() and (st[20:] == PKT_FILTER_DENY).all()
        for q in (out_q, plain_q, in_q):
            q.close()
    finally:
        c.close()
