"""Python mirror of the reference's packet-filter interface, backed by the GPU tables.

Names and behaviour follow internal/filter/filter.go and internal/acl/acl.go of the
reference (Filter.SetRules / SetAllowAll / CheckInbound / NoteOutbound, WrapTUN and the
tun.Device batch methods), so that tests read like the reference's own.  Every verdict
is computed by the CUDA kernels behind bnk_filter_note_submit / bnk_filter_check_submit;
this module only flattens rules and moves packets into a pinned batch.
"""
from __future__ import annotations

import ipaddress
from dataclasses import dataclass, field
from typing import Iterable, Protocol, Sequence

import numpy as np

from .device import ACL_TUPLE_DTYPE, PKT_OK, Batch, Context

PROTO_NUMBER = {"tcp": 6, "udp": 17, "icmp": 1}
OFFSET = 16  # headroom the WireGuard device keeps in front of every packet (transport header size)


@dataclass
class PortRange:
    """acl.PortRange, internal/acl/acl.go:39-42."""
    first: int
    last: int


@dataclass
class CompiledRule:
    """acl.CompiledRule, internal/acl/acl.go:33-37.  srcs are CIDR strings."""
    srcs: Sequence[str]
    proto: str
    ports: Sequence[PortRange] = field(default_factory=list)


def _prefix(p: str):
    """-> (addr, bits) for an IPv4 prefix, None for anything that can never contain an IPv4 address."""
    try:
        net = ipaddress.ip_network(p, strict=False)
    except ValueError:
        return None
    if net.version != 4:
        return None
    return int(net.network_address), net.prefixlen


def flatten_rules(rules: Iterable[CompiledRule]) -> np.ndarray:
    """Expands rules to the (prefix, proto, port range) allowances the device table holds.

    Mirrors acl.CompiledRule.Match (internal/acl/acl.go:149-172): a rule with no sources never
    matches, a tcp/udp rule with no ports never matches, icmp ignores ports, and a protocol string
    other than tcp/udp/icmp can never equal a parsed packet's protocol.
    """
    out = []
    for r in rules:
        proto = PROTO_NUMBER.get(r.proto)
        if proto is None:
            continue
        srcs = [s for s in (_prefix(p) for p in r.srcs) if s is not None]
        if proto == 1:
            out.extend((a, b, proto, 0, 0) for a, b in srcs)
        else:
            for pr in r.ports:
                if pr.first <= pr.last:
                    out.extend((a, b, proto, pr.first, pr.last) for a, b in srcs)
    t = np.zeros(len(out), ACL_TUPLE_DTYPE)
    for i, (a, b, proto, lo, hi) in enumerate(out):
        t[i] = (a, b, proto, lo, hi, 0)
    return t


def flatten_rule_arrays(rules: np.ndarray, srcs: np.ndarray, ports: np.ndarray) -> np.ndarray:
    """Same expansion for rules held as arrays (gen.RULE_DTYPE / PREFIX_DTYPE / PORT_DTYPE)."""
    rows = []
    for r in rules:
        proto = int(r["proto"])
        if proto not in (1, 6, 17):
            continue
        ss = srcs[int(r["src_begin"]):int(r["src_end"])]
        ss = ss[(ss["bits"] >= 0) & (ss["bits"] <= 32)]
        if proto == 1:
            pp = [(0, 0)]
        else:
            pp = [(int(p["first"]), int(p["last"])) for p in ports[int(r["port_begin"]):int(r["port_end"])]
                  if p["first"] <= p["last"]]
        for lo, hi in pp:
            t = np.zeros(len(ss), ACL_TUPLE_DTYPE)
            t["addr"], t["prefix_len"], t["proto"], t["port_first"], t["port_last"] = ss["addr"], ss["bits"], proto, lo, hi
            rows.append(t)
    return np.concatenate(rows) if rows else np.zeros(0, ACL_TUPLE_DTYPE)


class Filter:
    """filter.Filter (internal/filter/filter.go:33-59) over one GPU context.

    New filters start in allow-all mode; set_rules turns enforcement on (an empty list means
    deny everything but replies to flows this node opened); the flow table survives rule changes.
    """

    def __init__(self, ctx: Context, batch_pkts: int = 256, mtu: int = 2048):
        self.ctx = ctx
        self._stride = (OFFSET + mtu + 15) & ~15
        self._batch = ctx.batch(batch_pkts, batch_pkts * self._stride)
        ctx.acl_set(False, None)

    def set_rules(self, rules: Iterable[CompiledRule]):
        self.ctx.acl_set(True, flatten_rules(rules))

    def set_allow_all(self):
        self.ctx.acl_set(False, None)

    def _load(self, pkts: Sequence[bytes]) -> int:
        b = self._batch
        for i, p in enumerate(pkts):
            p = p or b""
            o = i * self._stride
            b.off[i] = o
            b.len[i] = len(p)
            b.ring[o + OFFSET:o + OFFSET + len(p)] = np.frombuffer(bytes(p), np.uint8)
        return len(pkts)

    def check_inbound_batch(self, pkts: Sequence[bytes], now_ns: int) -> list[bool]:
        out: list[bool] = []
        cap = self._batch.max_pkts
        for s in range(0, len(pkts), cap):
            n = self._load(pkts[s:s + cap])
            self._batch.filter_check(n, now_ns)
            out.extend(bool(v == PKT_OK) for v in self._batch.status[:n])
        return out

    def note_outbound_batch(self, pkts: Sequence[bytes], now_ns: int) -> None:
        cap = self._batch.max_pkts
        for s in range(0, len(pkts), cap):
            n = self._load(pkts[s:s + cap])
            self._batch.filter_note(n, now_ns)

    def check_inbound(self, pkt: bytes, now_ns: int) -> bool:
        """Filter.CheckInbound, filter.go:121-147."""
        return self.check_inbound_batch([pkt], now_ns)[0]

    def note_outbound(self, pkt: bytes, now_ns: int) -> None:
        """Filter.NoteOutbound, filter.go:189-209."""
        self.note_outbound_batch([pkt], now_ns)


class TunDevice(Protocol):
    """The batch methods of wireguard-go's tun.Device that the filter wraps (shape evidenced by
    internal/filter/tun_test.go:19-41).  bufs are bytearrays; packet i is bufs[i][offset:offset+sizes[i]]."""

    def read(self, bufs: list, sizes: list, offset: int) -> int: ...
    def write(self, bufs: list, offset: int) -> int: ...
    def batch_size(self) -> int: ...
    def mtu(self) -> int: ...


class FilteredTUN:
    """filteredTUN, internal/filter/filter.go:151-186: reads feed the flow table, writes are checked.

    `clock` returns unix nanoseconds and is sampled once per batch, as the reference samples
    time.Now() once per Read/Write call."""

    def __init__(self, inner: TunDevice, f: Filter, clock):
        self.inner = inner
        self.f = f
        self.clock = clock

    def read(self, bufs: list, sizes: list, offset: int) -> int:
        n = self.inner.read(bufs, sizes, offset)
        now = self.clock()
        self.f.note_outbound_batch([bytes(bufs[i][offset:offset + sizes[i]]) for i in range(n)], now)
        return n

    def write(self, bufs: list, offset: int) -> int:
        now = self.clock()
        verdicts = self.f.check_inbound_batch([bytes(b[offset:]) for b in bufs], now)
        kept = [b for b, ok in zip(bufs, verdicts) if ok]
        if not kept:
            return len(bufs)  # a filtered drop is not a short write
        self.inner.write(kept, offset)  # an inner error propagates as the exception it raises
        return len(bufs)

    def batch_size(self) -> int:
        return self.inner.batch_size()

    def mtu(self) -> int:
        return self.inner.mtu()


def wrap_tun(inner: TunDevice, f: Filter, clock) -> FilteredTUN:
    """filter.WrapTUN, filter.go:151."""
    return FilteredTUN(inner, f, clock)
