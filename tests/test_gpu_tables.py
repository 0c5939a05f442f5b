"""The context's tables under churn: keypair slots that hold no keys, receiver indices that come and go,
a flow table that sees many times its capacity in distinct flows, rule sets swapped while packets flow,
and the per-batch counters.  Verdicts are compared with the CPU checker throughout."""
import threading

import numpy as np
import pytest

from tests import helpers as H
from tests import reference_cases as RC

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------------------------
# keypair slots without keys
# ---------------------------------------------------------------------------------------------
def test_slot_without_keys_seals_and_opens_nothing(gpu_lib, oracle):
    """A slot that was never set, or was cleared, holds the all-zero key, which everyone knows: a message
    forged under it must not authenticate, and nothing may be sealed under it."""
    from bnk_b200 import Context
    from bnk_b200.device import PKT_NO_KEYPAIR, PKT_OK

    zero = bytes(32)
    key = np.arange(32, dtype=np.uint8)
    payload = bytes(range(64))
    forged = oracle.wg_seal(zero, 0, 5, payload, 1420)
    c = Context(max_keypairs=4, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(1, key[None, :], key[None, :], np.array([9], np.uint32))
        c.set_keypairs(2, key[None, :], key[None, :], np.array([9], np.uint32))
        c.index_set(0x77, 2)
        c.clear_keypair(2)
        b = c.batch(4, 4 * 1472)
        # open: slot 0 never set, slot 2 cleared, slot 1 live (but the message is not under its key)
        for i, slot in enumerate((0, 2, 1)):
            b.off[i], b.len[i], b.slot[i] = i * 1472, len(forged), slot
            b.ring[i * 1472:i * 1472 + len(forged)] = np.frombuffer(forged, np.uint8)
        b.open(3)
        assert list(b.status[:3]) == [PKT_NO_KEYPAIR, PKT_NO_KEYPAIR, oracle.AUTH_FAIL]
        assert list(b.out_len[:3]) == [0, 0, 0]
        # seal: refused for the empty slots, bytes untouched; fine for the live one
        for i, slot in enumerate((0, 2, 1)):
            b.off[i], b.len[i], b.slot[i], b.counter[i] = i * 1472, len(payload), slot, 5
            b.ring[i * 1472:(i + 1) * 1472] = 0
            b.ring[i * 1472 + 16:i * 1472 + 16 + len(payload)] = np.frombuffer(payload, np.uint8)
        b.seal(3)
        assert list(b.status[:3]) == [PKT_NO_KEYPAIR, PKT_NO_KEYPAIR, PKT_OK]
        assert b.ring[16:16 + 64].tobytes() == payload and not b.ring[:16].any()
        assert b.message(2) == oracle.wg_seal(key.tobytes(), 9, 5, payload, 1420)
        # the receiver index that led to the cleared slot leads nowhere now
        from bnk_b200.device import F_DEMUX_INDEX

        msg = bytearray(oracle.wg_seal(key.tobytes(), 0x77, 1, payload, 1420))
        b.off[0], b.len[0] = 0, len(msg)
        b.ring[:len(msg)] = np.frombuffer(bytes(msg), np.uint8)
        b.open(1, F_DEMUX_INDEX)
        assert b.status[0] == PKT_NO_KEYPAIR
        # setting the slot again brings it back
        c.set_keypairs(2, key[None, :], key[None, :], np.array([9], np.uint32))
        c.index_set(0x77, 2)
        b.ring[:len(msg)] = np.frombuffer(bytes(msg), np.uint8)
        b.open(1, F_DEMUX_INDEX)
        assert b.status[0] == PKT_OK and b.slot[0] == 2 and b.payload(0) == payload
        b.close()
    finally:
        c.close()


# ---------------------------------------------------------------------------------------------
# receiver-index and source-address tables: deleted entries are reclaimed
# ---------------------------------------------------------------------------------------------
def test_index_and_address_tables_reclaim_deleted_entries(gpu_lib, oracle):
    """Every handshake brings a new receiver index.  After many times the table's size in distinct indices the
    table still has room, few tombstones, and a lookup of an unknown index still ends in 'no keypair'."""
    from bnk_b200 import Context
    from bnk_b200.device import F_DEMUX_INDEX, PKT_NO_KEYPAIR, PKT_OK

    key = np.arange(32, dtype=np.uint8)
    c = Context(max_keypairs=8, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, np.repeat(key[None, :], 8, 0), np.repeat(key[None, :], 8, 0), np.arange(8, dtype=np.uint32))
        slots = c.table_stats().index_slots
        assert slots == 16
        rng = np.random.default_rng(4)
        live = {}
        for round_ in range(20 * slots):
            idx = int(rng.integers(1, 1 << 32))
            slot = round_ % 8
            if slot in live:
                c.index_clear(live[slot])
            c.index_set(idx, slot)
            live[slot] = idx
            addr = bytes(10) + b"\xff\xff" + bytes([10, 0, (round_ >> 8) & 255, round_ & 255])
            c.addr_set(addr, 4000 + round_ % 100, slot)
            if round_ >= 4:
                r = round_ - 4
                c.addr_clear(bytes(10) + b"\xff\xff" + bytes([10, 0, (r >> 8) & 255, r & 255]), 4000 + r % 100)
        st = c.table_stats()
        assert st.index_live == 8 and st.index_dead < slots // 4
        assert st.addr_live == 4 and st.addr_dead < st.addr_slots // 4
        b = c.batch(16, 16 * 1472)
        payload = bytes(range(40))
        for i in range(8):
            msg = oracle.wg_seal(key.tobytes(), live[i], i, payload, 1420)
            b.off[i], b.len[i] = i * 1472, len(msg)
            b.ring[i * 1472:i * 1472 + len(msg)] = np.frombuffer(msg, np.uint8)
        for i in range(8, 16):  # indices nobody registered
            msg = oracle.wg_seal(key.tobytes(), int(rng.integers(1, 1 << 32)), i, payload, 1420)
            b.off[i], b.len[i] = i * 1472, len(msg)
            b.ring[i * 1472:i * 1472 + len(msg)] = np.frombuffer(msg, np.uint8)
        b.open(16, F_DEMUX_INDEX)
        assert list(b.status[:8]) == [PKT_OK] * 8 and list(b.slot[:8]) == list(range(8))
        assert list(b.status[8:16]) == [PKT_NO_KEYPAIR] * 8
        b.close()
    finally:
        c.close()


# ---------------------------------------------------------------------------------------------
# flow table: ten times its capacity in distinct flows
# ---------------------------------------------------------------------------------------------
def _udp_headers(src, dst, sport, dport):
    from bnk_b200 import gen

    n = len(sport)
    return gen._headers(np.full(n, 17, np.uint64), np.asarray(src, np.uint64), np.asarray(dst, np.uint64),
                        np.asarray(sport, np.uint64), np.asarray(dport, np.uint64))


def _load(b, hdr):
    from bnk_b200 import gen

    n = len(hdr)
    view = b.ring[:n * gen.HDR_STRIDE].reshape(n, gen.HDR_STRIDE)
    view[:, 16:16 + 28] = hdr
    b.off[:n] = (np.arange(n, dtype=np.uint64) * gen.HDR_STRIDE).astype(np.uint32)
    b.len[:n] = 28
    return n


def test_flow_table_survives_ten_times_its_capacity(gpu_lib, oracle):
    """Go's map deletes expired flows (filter.go:144, 202-208) and so never fills up.  Here deleted entries keep
    their slot until the class is compacted; with 10 x flow_capacity distinct flows over advancing time no
    insert may fail, deleted entries must stay bounded, and every verdict must equal the CPU checker's."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import PKT_OK

    cap, per_round = 1 << 14, 1024
    rounds = 10 * cap // per_round
    f = oracle.Filter()
    f.set_rules([])  # enforce, no rule: only replies to noted flows pass
    c = Context(max_keypairs=4, flow_capacity=cap)
    try:
        c.acl_set(True, None)
        b = c.batch(3 * per_round, 3 * per_round * gen.HDR_STRIDE)
        rng = np.random.default_rng(2024)
        prev = None
        worst_dead = 0
        for r in range(rounds):
            now = RC.T0 + r * 40 * RC.SEC  # udp flows live 30 s: last round's flows have run out
            sport = (np.arange(per_round) + r * per_round) % 60000 + 1024
            remote = RC.PEER + (np.arange(per_round) + r * per_round) // 60000
            dport = rng.integers(1, 65535, per_round)
            out = _udp_headers(np.full(per_round, RC.SELF), remote, sport, dport)
            f.note_batch(np.ascontiguousarray(out), 28, np.full(per_round, 28, np.uint32), now)
            n = _load(b, out)
            b.filter_note(n, now)  # raises BNK_EFULL if an insert found no slot
            # replies to this round's flows, to last round's (expired: refused and deleted), and strangers
            parts = [_udp_headers(remote, np.full(per_round, RC.SELF), dport, sport)]
            if prev is not None:
                parts.append(prev)
            parts.append(_udp_headers(rng.integers(1, 1 << 32, per_round), np.full(per_round, RC.SELF),
                                      rng.integers(1, 65535, per_round), rng.integers(1, 65535, per_round)))
            inbound = np.concatenate(parts)
            want = f.check_batch(np.ascontiguousarray(inbound), 28, np.full(len(inbound), 28, np.uint32), now + RC.SEC)
            n = _load(b, inbound)
            b.filter_check(n, now + RC.SEC)
            got = (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)
            assert np.array_equal(got, want), (r, np.flatnonzero(got != want)[:8])
            assert got[:per_round].all() and not got[per_round:].any()
            prev = parts[0]
            if r % 16 == 15:
                st = c.table_stats()
                assert st.flow_live == f.flow_count, r
                assert H.flows_equal(c.flows_export(), f.flows()), r   # the whole table, not only its size
                worst_dead = max(worst_dead, st.flow_dead[1])
                assert st.flow_used[1] <= cap // 2 + 2 * per_round, (r, st.flow_used[1])
        assert worst_dead > 0  # the churn did produce deleted entries, and they were reclaimed
        assert c.table_stats().flow_used[0] == 0
        b.close()
    finally:
        c.close()


# ---------------------------------------------------------------------------------------------
# rule sets swapped while packets flow
# ---------------------------------------------------------------------------------------------
def test_rule_swap_between_submits(gpu_lib, oracle):
    """Filter.SetRules swaps the table between two packets (filter.go:46-51).  One thread keeps swapping two
    rule sets while another keeps submitting batches: every batch must have been judged by one of the two sets
    as a whole, never by a mixture, and no call may fail."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import PKT_OK
    from bnk_b200.filter import flatten_rule_arrays

    wa = gen.config3(300, 2000, 16, 20000, seed=11)
    wb = gen.config3(300, 2000, 16, 16, seed=12)
    tuples = [flatten_rule_arrays(w.rules, w.srcs, w.ports) for w in (wa, wb)]
    want = []
    for w in (wa, wb):
        f = oracle.Filter()
        f.set_rules_arrays(w.rules.astype(oracle.RULE_DTYPE), w.srcs.astype(oracle.PREFIX_DTYPE),
                           w.ports.astype(oracle.PORT_DTYPE))
        want.append(f.check_batch_mt(np.ascontiguousarray(wa.inbound), 28, np.ascontiguousarray(wa.inbound_len), wa.t0_ns))
    assert not np.array_equal(want[0], want[1])
    c = Context(max_keypairs=4, flow_capacity=1 << 10, max_acl_tuples=max(len(t) for t in tuples))
    try:
        c.acl_set(True, tuples[0])
        n = len(wa.inbound_len)
        batches = [c.batch(n, n * gen.HDR_STRIDE) for _ in range(2)]
        for b in batches:
            view = b.ring[:n * gen.HDR_STRIDE].reshape(n, gen.HDR_STRIDE)
            view[:, 16:16 + 28] = wa.inbound
            b.off[:n] = (np.arange(n, dtype=np.uint64) * gen.HDR_STRIDE).astype(np.uint32)
            b.len[:n] = wa.inbound_len
        stop = threading.Event()
        swaps = [0]
        errors = []

        def swapper():
            try:
                while not stop.is_set():
                    swaps[0] += 1
                    c.acl_set(True, tuples[swaps[0] & 1])
            except Exception as e:  # noqa: BLE001
                errors.append(e)

        t = threading.Thread(target=swapper)
        t.start()
        seen = [0, 0]
        try:
            for it in range(300):
                b = batches[it & 1]
                b.wait()
                if it >= 2:
                    got = (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)
                    which = 0 if np.array_equal(got, want[0]) else 1 if np.array_equal(got, want[1]) else -1
                    assert which >= 0, f"batch {it - 2} was judged by a mixture of two rule sets"
                    seen[which] += 1
                b.filter_check(n, wa.t0_ns, wait=False)
        finally:
            stop.set()
            t.join()
            for b in batches:
                b.wait()
        assert not errors, errors
        assert swaps[0] > 10 and seen[0] > 0 and seen[1] > 0, (swaps, seen)
        for b in batches:
            b.close()
    finally:
        c.close()


# ---------------------------------------------------------------------------------------------
# per-batch counters
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 130, 5000])
def test_batch_counters_equal_a_count_of_the_statuses(gpu_lib, oracle, n):
    from bnk_b200 import Context
    from bnk_b200.device import F_ASSIGN_COUNTERS, F_REPLAY, F_STATS, BnkError

    n_peers = 7
    rng = np.random.default_rng(n)
    keys = rng.integers(0, 256, (n_peers, 32), dtype=np.uint8)
    c = Context(max_keypairs=n_peers, mtu=1420, flow_capacity=0)
    try:
        c.set_keypairs(0, keys, keys, np.arange(n_peers, dtype=np.uint32))
        b = c.batch(n, n * 1472)
        sizes = rng.choice([0, 1, 64, 576, 1420], n)
        b.off[:n] = (np.arange(n, dtype=np.uint64) * 1472).astype(np.uint32)
        b.len[:n] = sizes
        b.slot[:n] = rng.integers(0, n_peers + 1, n)  # some descriptors name a slot that does not exist
        b.seal(n, F_ASSIGN_COUNTERS | F_STATS)
        st = b.stats()
        assert st["packets"] == n
        assert st["by_status"] == np.bincount(b.status[:n], minlength=16).tolist()
        assert st["bytes_out"] == int(b.out_len[:n][b.status[:n] == 0].sum())
        # damage a few tags, repeat a few messages, open
        b.len[:n] = b.out_len[:n]
        for i in range(0, n, 9):
            if b.len[i] >= 32:
                b.ring[int(b.off[i]) + int(b.len[i]) - 1] ^= 1
        for i in range(4, n, 11):
            o, p = int(b.off[i]), int(b.off[i - 1])
            b.ring[o:o + 1472] = b.ring[p:p + 1472]
            b.len[i], b.slot[i] = b.len[i - 1], b.slot[i - 1]
        b.open(n, F_REPLAY | F_STATS)
        st = b.stats()
        assert st["by_status"] == np.bincount(b.status[:n], minlength=16).tolist()
        assert st["bytes_out"] == int(b.out_len[:n][b.status[:n] == 0].sum())
        assert sum(st["by_status"]) == n
        if n > 100:
            assert st["by_status"][oracle.AUTH_FAIL] > 0 and st["by_status"][oracle.REPLAY] > 0
        b.open(n)  # a submit without the flag: the counters of the earlier one are not handed out as its own
        with pytest.raises(BnkError):
            b.stats()
        b.close()
    finally:
        c.close()
