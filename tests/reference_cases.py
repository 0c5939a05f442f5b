"""The reference's own filter and ACL test cases, restated as data-driven scenarios.

Each scenario takes a `make()` callable that returns a fresh filter object with the reference's
interface (set_rules / set_allow_all / check_inbound / note_outbound) so the same cases pin both the
CPU checker and the CUDA path.  Sources: internal/filter/filter_test.go:56-170,
internal/filter/tun_test.go:43-94, internal/acl/acl_test.go:83-114.
"""
from __future__ import annotations

import ipaddress

from bnk_b200 import gen
from bnk_b200.filter import CompiledRule, PortRange

SEC = 1_000_000_000
MIN = 60 * SEC
T0 = 1_700_000_000 * SEC  # filter_test.go:60


def ip(s: str) -> int:
    return int(ipaddress.ip_address(s))


PEER, OTHER, SELF = ip("100.64.0.9"), ip("100.64.0.7"), ip("100.64.0.1")  # filter_test.go:57-59


def tcp(src, dst, sport, dport, syn=True):
    return gen.tcp_packet(src, dst, sport, dport, syn)


def udp(src, dst, sport, dport):
    return gen.udp_packet(src, dst, sport, dport)


def icmp_echo(src, dst, reply):
    return gen.icmp_packet(src, dst, reply)


SSH_ONLY = [CompiledRule(srcs=["100.64.0.9/32"], proto="tcp", ports=[PortRange(22, 22)])]  # filter_test.go:63-71


def ssh_only(make):
    f = make()
    f.set_rules(SSH_ONLY)
    return f


def case_allow_all_mode_passes_everything(make):  # filter_test.go:73-78
    f = make()
    assert f.check_inbound(tcp(PEER, SELF, 5555, 23), T0)


def case_rule_allows_matching_inbound(make):  # :80-85
    f = ssh_only(make)
    assert f.check_inbound(tcp(PEER, SELF, 5555, 22), T0)


def case_default_deny_drops_non_matching(make):  # :87-98
    f = ssh_only(make)
    assert not f.check_inbound(tcp(PEER, SELF, 5555, 23), T0)
    assert not f.check_inbound(tcp(OTHER, SELF, 5555, 22), T0)
    assert not f.check_inbound(udp(PEER, SELF, 53, 22), T0)


def case_return_traffic_allowed_via_flow_table(make):  # :100-115
    f = ssh_only(make)
    f.note_outbound(udp(SELF, PEER, 40000, 9999), T0)
    assert f.check_inbound(udp(PEER, SELF, 9999, 40000), T0 + 2 * SEC)
    assert not f.check_inbound(udp(PEER, SELF, 9999, 40000), T0 + 5 * MIN)
    assert not f.check_inbound(udp(PEER, SELF, 9998, 40000), T0 + SEC)


def case_tcp_return_flow_allowed(make):  # :117-126
    f = ssh_only(make)
    f.note_outbound(tcp(SELF, PEER, 40000, 8080, True), T0)
    assert f.check_inbound(tcp(PEER, SELF, 8080, 40000, False), T0 + SEC)
    assert not f.check_inbound(tcp(PEER, SELF, 8081, 40000, False), T0 + SEC)


def case_icmp_echo_reply_via_flow(make):  # :128-137
    f = ssh_only(make)
    f.note_outbound(icmp_echo(SELF, PEER, False), T0)
    assert f.check_inbound(icmp_echo(PEER, SELF, True), T0 + SEC)
    assert not f.check_inbound(icmp_echo(OTHER, SELF, True), T0 + SEC)


def case_icmp_rule_allows_inbound_ping(make):  # :139-148
    f = make()
    f.set_rules([CompiledRule(srcs=["100.64.0.9/32"], proto="icmp")])
    assert f.check_inbound(icmp_echo(PEER, SELF, False), T0)


def case_malformed_and_non_ipv4_dropped(make):  # :150-162
    f = ssh_only(make)
    assert not f.check_inbound(bytes([0x60, 0x00, 0x00]), T0)
    assert not f.check_inbound(None, T0)
    assert not f.check_inbound(tcp(PEER, SELF, 1, 22)[:22], T0)


def case_set_allow_all_disables_enforcement(make):  # :164-170
    f = ssh_only(make)
    f.set_allow_all()
    assert f.check_inbound(tcp(OTHER, SELF, 5555, 23), T0)


def case_compiled_rule_match(make):  # acl_test.go:83-107: multi-range rule truth table
    f = make()
    f.set_rules([CompiledRule(srcs=["100.64.0.1/32"], proto="tcp", ports=[PortRange(22, 22), PortRange(8000, 9000)])])
    a, b = ip("100.64.0.1"), ip("100.64.0.9")
    assert f.check_inbound(tcp(a, SELF, 1, 22), T0)
    assert f.check_inbound(tcp(a, SELF, 1, 8500), T0)
    assert not f.check_inbound(tcp(a, SELF, 1, 23), T0)
    assert not f.check_inbound(udp(a, SELF, 1, 22), T0)
    assert not f.check_inbound(tcp(b, SELF, 1, 22), T0)


def case_icmp_rule_ignores_ports_with_wide_prefix(make):  # acl_test.go:109-114
    f = make()
    f.set_rules([CompiledRule(srcs=["100.64.0.0/10"], proto="icmp")])
    assert f.check_inbound(icmp_echo(ip("100.64.0.1"), SELF, False), T0)
    assert f.check_inbound(icmp_echo(ip("100.127.255.254"), SELF, False), T0)
    assert not f.check_inbound(icmp_echo(ip("100.128.0.1"), SELF, False), T0)
    assert not f.check_inbound(tcp(ip("100.64.0.1"), SELF, 1, 22), T0)


def case_rule_shapes_that_never_match(make):  # acl.go:154-172: empty srcs, empty ports, odd proto strings
    f = make()
    f.set_rules([CompiledRule(srcs=[], proto="tcp", ports=[PortRange(1, 65535)]),
                 CompiledRule(srcs=["100.64.0.9/32"], proto="tcp", ports=[]),
                 CompiledRule(srcs=["100.64.0.9/32"], proto="TCP", ports=[PortRange(1, 65535)]),
                 CompiledRule(srcs=["fd00::/8", "::ffff:100.64.0.9/128"], proto="udp", ports=[PortRange(1, 65535)])])
    assert not f.check_inbound(tcp(PEER, SELF, 5, 22), T0)
    assert not f.check_inbound(udp(PEER, SELF, 5, 22), T0)
    f.set_rules([CompiledRule(srcs=["0.0.0.0/0"], proto="udp", ports=[PortRange(53, 53)])])
    assert f.check_inbound(udp(ip("8.8.8.8"), SELF, 5, 53), T0)


def case_flow_details(make):  # filter.go:138-146, 189-209 corner behaviour
    f = ssh_only(make)
    # strict expiry: allowed just before the TTL runs out, refused exactly at it (time.Before)
    f.note_outbound(udp(SELF, PEER, 1000, 2000), T0)
    assert f.check_inbound(udp(PEER, SELF, 2000, 1000), T0 + 30 * SEC - 1)   # refreshes to T0+60s-1
    assert f.check_inbound(udp(PEER, SELF, 2000, 1000), T0 + 60 * SEC - 2)
    f.note_outbound(udp(SELF, PEER, 1001, 2000), T0)
    assert not f.check_inbound(udp(PEER, SELF, 2000, 1001), T0 + 30 * SEC)   # exactly at expiry: deleted
    assert not f.check_inbound(udp(PEER, SELF, 2000, 1001), T0 + SEC)        # stays deleted even if time steps back
    # tcp flows live two minutes, flows are per protocol, options (IHL 6) are skipped
    f.note_outbound(tcp(SELF, PEER, 1002, 443), T0)
    assert not f.check_inbound(udp(PEER, SELF, 443, 1002), T0 + SEC)
    assert f.check_inbound(tcp(PEER, SELF, 443, 1002, False), T0 + 119 * SEC)
    opt = bytearray(gen.ipv4_header(6, PEER, SELF, 48, ihl_words=6)) + bytes(gen.l4_ports(443, 1002)) + bytes(16)
    assert f.check_inbound(bytes(opt), T0 + 120 * SEC)
    # rules changing keeps the flows; allow-all mode records nothing
    f.set_rules([])
    assert f.check_inbound(tcp(PEER, SELF, 443, 1002, False), T0 + 121 * SEC)
    f.set_allow_all()
    f.note_outbound(udp(SELF, PEER, 1003, 2000), T0 + 121 * SEC)
    f.set_rules([])
    assert not f.check_inbound(udp(PEER, SELF, 2000, 1003), T0 + 122 * SEC)


ALL_CASES = [v for k, v in sorted(globals().items()) if k.startswith("case_")]


# ---- tun.Device wrapper (tun_test.go) ---------------------------------------------------
class FakeTUN:
    """fakeTUN, internal/filter/tun_test.go:13-41."""

    def __init__(self):
        self.written: list[bytes] = []
        self.pending: list[bytes] = []

    def read(self, bufs, sizes, offset):
        n = 0
        while n < len(bufs) and self.pending:
            pkt = self.pending.pop(0)
            bufs[n][offset:offset + len(pkt)] = pkt
            sizes[n] = len(pkt)
            n += 1
        return n

    def write(self, bufs, offset):
        for b in bufs:
            self.written.append(bytes(b[offset:]))
        return len(bufs)

    def mtu(self):
        return 1280

    def batch_size(self):
        return 4


def tun_case_drops_denied_inbound_writes(make, wrap):  # tun_test.go:43-66
    inner = FakeTUN()
    wrapped = wrap(inner, ssh_only(make), lambda: T0)
    allowed, denied = tcp(PEER, SELF, 5555, 22), tcp(PEER, SELF, 5555, 23)
    pad = lambda p: bytearray(16) + bytearray(p)  # noqa: E731
    assert wrapped.write([pad(allowed), pad(denied)], 16) == 2
    assert inner.written == [allowed]
    # everything denied: still reports the full count and writes nothing
    assert wrapped.write([pad(denied)], 16) == 1
    assert inner.written == [allowed]


def tun_case_read_records_outbound_flows(make, wrap):  # tun_test.go:68-94
    inner = FakeTUN()
    f = make()
    f.set_rules([])
    wrapped = wrap(inner, f, lambda: T0)
    inner.pending.append(udp(SELF, PEER, 40000, 9999))
    bufs, sizes = [bytearray(2048)], [0]
    assert wrapped.read(bufs, sizes, 16) == 1
    pad = lambda p: bytearray(16) + bytearray(p)  # noqa: E731
    reply, unrelated = udp(PEER, SELF, 9999, 40000), udp(PEER, SELF, 9999, 40001)
    wrapped.write([pad(reply), pad(unrelated)], 16)
    assert inner.written == [reply]
