"""Shared plumbing for the parity tests: lay a workload out in a batch, run the CPU checker on a copy."""
from __future__ import annotations

import numpy as np

from bnk_b200.device import slot_size


def layout_fixed(n: int, stride: int) -> np.ndarray:
    return (np.arange(n, dtype=np.uint64) * np.uint64(stride)).astype(np.uint32)


def layout_packed(lengths, slack: int = 48) -> np.ndarray:
    """Back-to-back slots, each 16-aligned with room for header, padding and tag."""
    off = np.zeros(len(lengths), np.uint32)
    cur = 0
    for i, l in enumerate(lengths):
        off[i] = cur
        cur += (int(l) + slack + 15) & ~15
    return off


def ring_bytes_for(off, lengths, slack: int = 64) -> int:
    if len(off) == 0:
        return 64
    return int(((np.max(off.astype(np.int64) + np.asarray(lengths, np.int64)) + slack + 15) // 16) * 16)


def fill_payloads(ring: np.ndarray, off, payloads, headroom: int = 16):
    for o, p in zip(off, payloads):
        o = int(o)
        ring[o + headroom:o + headroom + len(p)] = np.frombuffer(bytes(p), np.uint8)


def oracle_seal(O, keys, remote_index, mtu, ring, off, length, slot, counter):
    """Seals a copy of the ring with the CPU checker.  -> (ring, status, out_len)"""
    r = np.array(ring, copy=True)
    st, ol = O.wg_seal_batch(np.ascontiguousarray(keys, np.uint8), np.ascontiguousarray(remote_index, np.uint32), mtu,
                             r, np.ascontiguousarray(off, np.uint32), np.ascontiguousarray(length, np.uint32),
                             np.ascontiguousarray(slot, np.uint32), np.ascontiguousarray(counter, np.uint64))
    return r, st, ol


def oracle_open(O, keys, ring, off, length, slot):
    r = np.array(ring, copy=True)
    st, ctr, ol = O.wg_open_batch(np.ascontiguousarray(keys, np.uint8), r, np.ascontiguousarray(off, np.uint32),
                                  np.ascontiguousarray(length, np.uint32), np.ascontiguousarray(slot, np.uint32))
    return r, st, ctr, ol


def oracle_replay(O, ring_blocks, slots, counters, statuses, state=None):
    """Sequential replay walk per slot in arrival order over authenticated packets.
    state: dict slot -> O.Replay (created on demand).  Returns the new status array."""
    state = {} if state is None else state
    out = np.array(statuses, copy=True)
    for i in range(len(slots)):
        if out[i] not in (O.OK, O.KEEPALIVE):
            continue
        s = int(slots[i])
        if s not in state:
            state[s] = O.Replay(ring_blocks)
        if not state[s].validate(int(counters[i])):
            out[i] = O.REPLAY
    return out, state


def spans_equal(a: np.ndarray, b: np.ndarray, off, lengths, start: int = 0) -> list:
    """Indices of packets whose bytes [off+start, off+start+len) differ."""
    bad = []
    for i, (o, l) in enumerate(zip(off, lengths)):
        o, l = int(o) + start, int(l)
        if not np.array_equal(a[o:o + l], b[o:o + l]):
            bad.append(i)
    return bad


def spans_differ_count(a: np.ndarray, b: np.ndarray, off, lengths, start: int = 0) -> int:
    """Number of differing bytes inside the packets' spans [off+start, off+start+len), for rings too large to walk
    packet by packet in Python (spans must not overlap)."""
    n = min(len(a), len(b))
    edge = np.zeros(n + 1, dtype=np.int8)
    lo = np.asarray(off, dtype=np.int64) + start
    hi = lo + np.asarray(lengths, dtype=np.int64)
    np.add.at(edge, lo, 1)
    np.add.at(edge, hi, -1)
    inside = np.cumsum(edge[:n], dtype=np.int8).astype(bool)
    return int(np.count_nonzero((a[:n] != b[:n]) & inside))


def flows_equal(gpu_flows: np.ndarray, checker_flows: np.ndarray) -> bool:
    """The library's exported flow table against the checker's map: same keys, same expiries (both sorted by key)."""
    if len(gpu_flows) != len(checker_flows):
        return False
    return bool(np.array_equal(gpu_flows["remote_addr"], checker_flows["remote"])
                and np.array_equal(gpu_flows["remote_port"], checker_flows["rport"])
                and np.array_equal(gpu_flows["local_port"], checker_flows["lport"])
                and np.array_equal(gpu_flows["proto"], checker_flows["proto"])
                and np.array_equal(gpu_flows["expiry_unix_ns"], checker_flows["exp"]))


__all__ = [n for n in dir() if not n.startswith("_")] + ["slot_size"]
