"""The multi-GPU dispatcher against a single context and against the CPU checker.

On a box with one GPU the dispatcher is given the same device twice: two contexts, two host threads, the same
routing, so the parity of routing, ordering and result gathering is covered; with two or more GPUs visible the
same test also runs over distinct devices."""
import numpy as np
import pytest

from tests import reference_cases as RC

pytestmark = pytest.mark.gpu


def _device_sets(L):
    n = L.bnk_device_count()
    sets = [[0, 0], [0, 0, 0]]
    if n >= 2:
        sets.append(list(range(min(n, 4))))
    return sets


def _traffic(rng, n, n_peers, heavy):
    """Mixed sizes; one heavy peer; a few packets for peers that do not exist or are not set."""
    sizes = rng.choice([0, 1, 64, 576, 1420], n)
    peers = np.where(rng.random(n) < 0.35, heavy, rng.integers(0, n_peers, n)).astype(np.uint32)
    pkts = []
    for i in range(n):
        body = rng.integers(0, 256, int(sizes[i]), dtype=np.uint8).tobytes()
        pkts.append(body)
    return pkts, peers


@pytest.mark.parametrize("which", [0, 1, 2])
def test_dispatcher_equals_checker_and_keeps_peer_order(gpu_lib, oracle, which):
    from bnk_b200.device import F_REPLAY, PKT_BAD_DESC, PKT_KEEPALIVE, PKT_NO_KEYPAIR, PKT_OK, PKT_REPLAY
    from bnk_b200.mgpu import MultiGpu

    sets = _device_sets(gpu_lib)
    if which >= len(sets):
        pytest.skip("needs two GPUs")
    devices = sets[which]
    n_peers, n = 300, 5000
    rng = np.random.default_rng(31 + which)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    heavy = 17
    with MultiGpu(devices, max_peers=n_peers, max_pkts_per_gpu=1024, max_packet=1420, flow_capacity=0) as m:
        # placement by a measured load: the heavy peer and the runner-up must not share a GPU
        load = np.ones(n_peers, np.uint64)
        load[heavy], load[5] = 5000, 3000
        m.place(load)
        assert m.locate(heavy)[0] != m.locate(5)[0]
        unset = {7, 123}
        for p in range(n_peers):
            if p not in unset:
                m.peer_set(p, keys[p].tobytes(), keys[p].tobytes(), remote_index=0x2000 + p, local_index=0x2000 + p)
        with pytest.raises(Exception):
            m.place(load)  # not while peers are set
        pkts, peers = _traffic(rng, n, n_peers, heavy)
        peers[11] = n_peers + 5       # no such peer
        pkts[12] = bytes(1500)        # longer than max_packet
        msgs, status, counter = m.seal(pkts, peers)
        # the counter rule: consecutive per peer in batch order, whatever GPU the peer lives on
        nxt = {}
        for i in range(n):
            p = int(peers[i])
            if p >= n_peers or p in unset:
                assert status[i] == PKT_NO_KEYPAIR and msgs[i] == b"", i
                continue
            if len(pkts[i]) > 1420:
                assert status[i] == PKT_BAD_DESC, i
                continue
            c = nxt.get(p, 0)
            nxt[p] = c + 1
            assert status[i] == PKT_OK and counter[i] == c, (i, p, counter[i], c)
            assert msgs[i] == oracle.wg_seal(keys[p].tobytes(), 0x2000 + p, c, pkts[i], 1420), i
        pk, by, pg = m.loads()   # what was routed: refused descriptors never reach a GPU
        assert pk[heavy] == nxt[heavy] and pk.sum() == sum(nxt.values()) and pg.sum() == sum(nxt.values())
        assert (pg > 0).all()
        # receive side: the same messages, some damaged, some repeated, one with an unknown receiver index
        good = [i for i in range(n) if status[i] == PKT_OK]
        order = [good[k] for k in rng.permutation(len(good))[:3000]]
        inbound = [msgs[i] for i in order]
        for k in range(0, len(inbound), 13):
            dmg = bytearray(inbound[k])
            dmg[-1] ^= 1
            inbound[k] = bytes(dmg)
        for k in range(5, len(inbound), 17):
            inbound[k] = inbound[k - 1]
            order[k] = order[k - 1]
        stranger = bytearray(inbound[3])
        stranger[4:8] = (0x7FFFFFFF).to_bytes(4, "little")
        inbound[3] = bytes(stranger)
        inbound[4] = b"\x04\x00\x00"   # too short to be a message
        pts, st, ctr, who = m.open(inbound, F_REPLAY)
        # checker: per peer in arrival order, authenticated packets walk the replay window
        state = {}
        for k, msg in enumerate(inbound):
            if k == 3:
                assert st[k] == PKT_NO_KEYPAIR
                continue
            if k == 4:
                assert st[k] == oracle.MALFORMED
                continue
            p = int(peers[order[k]])
            want, pt, c, ridx = oracle.wg_open(keys[p].tobytes(), msg)
            if want in (oracle.OK, oracle.KEEPALIVE):
                w = state.setdefault(p, oracle.Replay(128))
                if not w.validate(c):
                    want = oracle.REPLAY
            assert st[k] == want, (k, st[k], want)
            assert who[k] == p
            if want in (PKT_OK, PKT_KEEPALIVE):
                assert pts[k] == pt and ctr[k] == c
            else:
                assert pts[k] == b""
        assert (st == PKT_REPLAY).sum() > 0 and (st == oracle.AUTH_FAIL).sum() > 0
        # a peer that goes away takes its receiver index along
        m.peer_clear(heavy)
        again = [msgs[i] for i in good if peers[i] == heavy][:4]
        _, st2, _, _ = m.open(again, F_REPLAY)
        assert (st2 == PKT_NO_KEYPAIR).all()


def test_dispatcher_runs_the_filter_of_the_peers_gpu(gpu_lib, oracle):
    """NoteOutbound on the way out and CheckInbound on the way in, through the dispatcher: the reply to a flow
    noted on the peer's GPU passes on that GPU; the rule table is the same on every GPU."""
    from bnk_b200.device import F_CHECK_INBOUND, F_INNER_CHECK, F_NOTE_OUTBOUND, F_REPLAY, PKT_FILTER_DENY, PKT_OK
    from bnk_b200.filter import CompiledRule, PortRange, flatten_rules
    from bnk_b200.mgpu import MultiGpu

    n_peers = 16
    rng = np.random.default_rng(8)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    with MultiGpu([0, 0], max_peers=n_peers, max_pkts_per_gpu=64, flow_capacity=1 << 10) as tx, \
            MultiGpu([0, 0], max_peers=n_peers, max_pkts_per_gpu=64, flow_capacity=1 << 10) as rx:
        for p in range(n_peers):
            tx.peer_set(p, keys[p].tobytes(), keys[p].tobytes(), 0x100 + p, 0x100 + p, RC.PEER + p)
            rx.peer_set(p, keys[p].tobytes(), keys[p].tobytes(), 0x100 + p, 0x100 + p, RC.PEER + p)
        rules = flatten_rules([CompiledRule(["100.64.0.0/10"], "tcp", [PortRange(22, 22)])])
        tx.acl_set(True, rules)
        rx.acl_set(True, rules)
        # this node (rx) opens udp flows towards every peer ...
        out = [RC.udp(RC.SELF, RC.PEER + p, 40000 + p, 53) for p in range(n_peers)]
        _, st, _ = rx.seal(out, np.arange(n_peers, dtype=np.uint32), F_NOTE_OUTBOUND, RC.T0)
        assert (st == PKT_OK).all()
        # ... and the peers answer, plus ssh (allowed by rule) and telnet (refused) from each of them
        inner = []
        for p in range(n_peers):
            inner += [RC.udp(RC.PEER + p, RC.SELF, 53, 40000 + p), RC.tcp(RC.PEER + p, RC.SELF, 5555, 22),
                      RC.tcp(RC.PEER + p, RC.SELF, 5555, 23), RC.udp(RC.PEER + p, RC.SELF, 53, 50000 + p)]
        who = np.repeat(np.arange(n_peers, dtype=np.uint32), 4)
        msgs, st, _ = tx.seal(inner, who)
        assert (st == PKT_OK).all()
        # (the inner check cuts the plaintext back to its IPv4 total length: sealing padded it to 16)
        pts, st, _, got_who = rx.open(msgs, F_REPLAY | F_INNER_CHECK | F_CHECK_INBOUND, RC.T0 + RC.SEC)
        assert np.array_equal(got_who, who)
        assert st.reshape(n_peers, 4).tolist() == [[PKT_OK, PKT_OK, PKT_FILTER_DENY, PKT_FILTER_DENY]] * n_peers
        assert pts[0] == inner[0] and pts[1] == inner[1]
