"""Seeded synthetic workloads for the five benchmark/parity configurations.

Everything is drawn from SplitMix64 (one stream per configuration, seed
0xB2000000 + configuration number) so that C, CUDA and Python can regenerate the
same bytes.  The draw order of each generator is part of its contract and is spelled
out in its docstring; changing it invalidates the golden digests under tests/golden.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

_M64 = (1 << 64) - 1
_GAMMA = 0x9E3779B97F4A7C15


def seed_for(config: int) -> int:
    return 0xB2000000 + config


class SplitMix64:
    """Vectorised SplitMix64; `u64(n)` returns the next n outputs of the sequential generator."""

    def __init__(self, seed: int):
        self.state = seed & _M64

    def u64(self, n: int) -> np.ndarray:
        k = np.arange(1, n + 1, dtype=np.uint64)
        with np.errstate(over="ignore"):
            z = np.uint64(self.state) + k * np.uint64(_GAMMA)
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            z = z ^ (z >> np.uint64(31))
        self.state = (self.state + n * _GAMMA) & _M64
        return z

    def bytes(self, n: int) -> np.ndarray:
        """n bytes: the little-endian bytes of ceil(n/8) outputs, truncated."""
        return self.u64((n + 7) // 8).view(np.uint8)[:n].copy()

    def below(self, n: int, bound: int) -> np.ndarray:
        """n integers in [0, bound): output mod bound (the tiny bias is part of the definition)."""
        return (self.u64(n) % np.uint64(bound)).astype(np.uint64)

    def one_below(self, bound: int) -> int:
        return int(self.below(1, bound)[0])


def splitmix_fill(seed: int, nbytes: int, byte_offset: int = 0) -> np.ndarray:
    """Bytes [byte_offset, byte_offset + nbytes) of what the device-side fill (bnk_batch_fill_random) writes for
    the same seed: word k of the ring is output k of SplitMix64(seed)."""
    first = byte_offset // 8
    g = SplitMix64((seed + first * _GAMMA) & _M64)
    lead = byte_offset - first * 8
    return g.bytes(lead + nbytes)[lead:]


# ---------------------------------------------------------------------------------------
# packet builders (same shapes as the helpers in the reference's filter_test.go:13-54)
# ---------------------------------------------------------------------------------------
def ip4(a: int, b: int, c: int, d: int) -> int:
    return (a << 24) | (b << 16) | (c << 8) | d


def ipv4_header(proto: int, src: int, dst: int, total_len: int, ihl_words: int = 5, version: int = 4) -> np.ndarray:
    h = np.zeros(ihl_words * 4, np.uint8)
    h[0] = (version << 4) | ihl_words
    h[2] = (total_len >> 8) & 0xFF
    h[3] = total_len & 0xFF
    h[8] = 64
    h[9] = proto
    h[12:16] = [(src >> 24) & 0xFF, (src >> 16) & 0xFF, (src >> 8) & 0xFF, src & 0xFF]
    h[16:20] = [(dst >> 24) & 0xFF, (dst >> 16) & 0xFF, (dst >> 8) & 0xFF, dst & 0xFF]
    return h


def l4_ports(sport: int, dport: int) -> np.ndarray:
    return np.array([sport >> 8, sport & 0xFF, dport >> 8, dport & 0xFF], np.uint8)


def tcp_packet(src: int, dst: int, sport: int, dport: int, syn: bool = True) -> bytes:
    t = np.zeros(20, np.uint8)
    t[0:4] = l4_ports(sport, dport)
    t[12] = 5 << 4
    t[13] = 0x02 if syn else 0x10
    return bytes(ipv4_header(6, src, dst, 40)) + bytes(t)


def udp_packet(src: int, dst: int, sport: int, dport: int) -> bytes:
    u = np.zeros(8, np.uint8)
    u[0:4] = l4_ports(sport, dport)
    u[5] = 8
    return bytes(ipv4_header(17, src, dst, 28)) + bytes(u)


def icmp_packet(src: int, dst: int, reply: bool) -> bytes:
    u = np.zeros(8, np.uint8)
    u[0] = 0 if reply else 8
    return bytes(ipv4_header(1, src, dst, 28)) + bytes(u)


# ---------------------------------------------------------------------------------------
# configuration 1: one keypair, 128 x 1420 B
# ---------------------------------------------------------------------------------------
@dataclass
class SealWorkload:
    keys: np.ndarray          # [n_peers, 32] uint8
    remote_index: np.ndarray  # [n_peers] uint32
    peer: np.ndarray          # [n] uint32 keypair slot of each packet
    counter: np.ndarray       # [n] uint64
    length: np.ndarray        # [n] uint32
    payloads: list            # n byte strings (plaintext IP packets)
    mtu: int = 1420


def config1(n: int = 128, size: int = 1420) -> SealWorkload:
    """Draw order: 32 key bytes; then for each packet (size - 28) payload bytes."""
    g = SplitMix64(seed_for(1))
    key = g.bytes(32)
    hdr = bytes(ipv4_header(17, ip4(100, 64, 0, 2), ip4(100, 64, 0, 1), size))
    udp = np.zeros(8, np.uint8)
    udp[0:4] = l4_ports(40000, 51820)
    udp[4], udp[5] = ((size - 20) >> 8) & 0xFF, (size - 20) & 0xFF
    pkts = [hdr + bytes(udp) + g.bytes(size - 28).tobytes() for _ in range(n)]
    return SealWorkload(keys=key.reshape(1, 32), remote_index=np.array([1], np.uint32),
                        peer=np.zeros(n, np.uint32), counter=np.arange(n, dtype=np.uint64),
                        length=np.full(n, size, np.uint32), payloads=pkts, mtu=size)


# ---------------------------------------------------------------------------------------
# configuration 2: IMIX open path with reordering, duplicates and damaged tags
# ---------------------------------------------------------------------------------------
IMIX_SIZES = (64, 576, 1420)
IMIX_WEIGHTS = (7, 4, 1)


@dataclass
class OpenWorkload:
    base: SealWorkload            # the distinct packets, in send order
    arrival: np.ndarray           # [n_arrivals] index into base packets, in arrival order
    flip_pos: np.ndarray          # arrival positions whose tag gets one byte XOR 0x01
    flip_byte: np.ndarray         # which of the 16 tag bytes
    n_peers: int = 256


def imix_sizes(g: SplitMix64, n: int) -> np.ndarray:
    w = g.below(n, sum(IMIX_WEIGHTS))
    edges = np.cumsum(IMIX_WEIGHTS)
    return np.asarray(IMIX_SIZES, np.uint32)[np.searchsorted(edges, w, side="right")]


def config2(n_arrivals: int = 4096, n_peers: int = 256, reorder_pct: int = 5, dup_pct: int = 1,
            flip_pct: int = 1, seed: int | None = None) -> OpenWorkload:
    """Draw order: n_peers*32 key bytes; n_peers counter bases; n_dup = n_arrivals*dup_pct/100,
    n_base = n_arrivals - n_dup; n_base sizes (7:4:1 over 64/576/1420); n_base peers; per packet
    (size-28) payload bytes; n_reorder = n_base*reorder_pct/100 draws of (position, distance 1..64)
    applied as swaps in order; n_dup draws of (position, distance 1..64): a copy of the packet at
    `position` is inserted `distance` later; n_flip = n_arrivals*flip_pct/100 draws of (arrival
    position, tag byte 0..15)."""
    g = SplitMix64(seed_for(2) if seed is None else seed)
    keys = g.bytes(n_peers * 32).reshape(n_peers, 32)
    bases = g.below(n_peers, (1 << 40) - (1 << 20)) + np.uint64(1 << 20)
    n_dup = n_arrivals * dup_pct // 100
    n_base = n_arrivals - n_dup
    sizes = imix_sizes(g, n_base)
    peers = g.below(n_base, n_peers).astype(np.uint32)
    counters = np.zeros(n_base, np.uint64)
    nxt = bases.copy()
    for i in range(n_base):
        counters[i] = nxt[peers[i]]
        nxt[peers[i]] += np.uint64(1)
    self_ip, peer_net = ip4(100, 64, 0, 1), ip4(100, 64, 1, 0)
    pkts = []
    for i in range(n_base):
        sz = int(sizes[i])
        hdr = bytes(ipv4_header(17, peer_net + int(peers[i]), self_ip, sz))
        udp = np.zeros(8, np.uint8)
        udp[0:4] = l4_ports(40000 + int(peers[i]), 51820)
        pkts.append(hdr + bytes(udp) + g.bytes(sz - 28).tobytes())
    order = list(range(n_base))
    for _ in range(n_base * reorder_pct // 100):
        p = g.one_below(n_base)
        q = min(n_base - 1, p + 1 + g.one_below(64))
        order[p], order[q] = order[q], order[p]
    for _ in range(n_dup):
        p = g.one_below(len(order))
        q = min(len(order), p + 1 + g.one_below(64))
        order.insert(q, order[p])
    n_flip = n_arrivals * flip_pct // 100
    flip_pos = np.array([g.one_below(len(order)) for _ in range(n_flip)], np.int64)
    flip_byte = np.array([g.one_below(16) for _ in range(n_flip)], np.int64)
    base = SealWorkload(keys=keys, remote_index=np.arange(1, n_peers + 1, dtype=np.uint32), peer=peers,
                        counter=counters, length=sizes.astype(np.uint32), payloads=pkts, mtu=1420)
    return OpenWorkload(base=base, arrival=np.asarray(order, np.int64), flip_pos=flip_pos, flip_byte=flip_byte,
                        n_peers=n_peers)


# ---------------------------------------------------------------------------------------
# configuration 3: ACL filter
# ---------------------------------------------------------------------------------------
RULE_DTYPE = np.dtype([("proto", "u1"), ("src_begin", "<u4"), ("src_end", "<u4"), ("port_begin", "<u4"),
                       ("port_end", "<u4")], align=True)
PREFIX_DTYPE = np.dtype([("addr", "<u4"), ("bits", "<i4")])
PORT_DTYPE = np.dtype([("first", "<u2"), ("last", "<u2")])
HDR_STRIDE = 48  # 16 bytes of headroom + 28-byte header + 4 spare, keeps slots 16-aligned


@dataclass
class FilterWorkload:
    self_ip: int
    nodes: np.ndarray             # [n_nodes] uint32
    rules: np.ndarray             # RULE_DTYPE
    srcs: np.ndarray              # PREFIX_DTYPE
    ports: np.ndarray             # PORT_DTYPE
    t0_ns: int
    outbound: np.ndarray          # [n_out, 28] uint8 headers noted at t0
    outbound_len: np.ndarray
    inbound: np.ndarray           # [n_in, 28] uint8 headers checked at t0 + 1 s
    inbound_len: np.ndarray
    late: np.ndarray              # [n_late, 28] replies checked again at t0 + 10 min
    late_len: np.ndarray
    extra: dict = field(default_factory=dict)


def _headers(proto, src, dst, sport, dport) -> np.ndarray:
    n = len(proto)
    h = np.zeros((n, 28), np.uint8)
    h[:, 0] = 0x45
    h[:, 3] = 28
    h[:, 8] = 64
    h[:, 9] = proto
    for k in range(4):
        h[:, 12 + k] = (src >> np.uint64(24 - 8 * k)) & np.uint64(0xFF)
        h[:, 16 + k] = (dst >> np.uint64(24 - 8 * k)) & np.uint64(0xFF)
    icmp = proto == 1
    h[:, 20] = np.where(icmp, 8, sport >> np.uint64(8))
    h[:, 21] = np.where(icmp, 0, sport & np.uint64(0xFF))
    h[:, 22] = np.where(icmp, 0, dport >> np.uint64(8))
    h[:, 23] = np.where(icmp, 0, dport & np.uint64(0xFF))
    return h


def config3(n_rules: int = 10_000, n_nodes: int = 50_000, n_out: int = 300_000, n_in: int = 1_000_000,
            seed: int | None = None) -> FilterWorkload:
    """Draw order: n_nodes host parts (22 bits, zero replaced by 1); self index; per rule: proto draw
    (6:3:1 tcp/udp/icmp), prefix-rule draw (1 in 100), source count (geometric, p = 1/4, cap 64) or
    prefix length 16..24 + node index, two port draws 1..65535, single-port draw (1 in 10);
    n_out outbound draws (node, proto, sport, dport); n_in inbound class draws (0..99), then the
    per-class draws described in the code, in array order."""
    g = SplitMix64(seed_for(3) if seed is None else seed)
    base = ip4(100, 64, 0, 0)
    host = g.below(n_nodes, 1 << 22)
    host[host == 0] = 1
    nodes = (np.uint64(base) + host).astype(np.uint64)
    self_ip = int(nodes[g.one_below(n_nodes)])
    protos = np.array([6, 17, 1], np.uint8)

    rules = np.zeros(n_rules, RULE_DTYPE)
    srcs, ports = [], []
    pw = g.below(n_rules, 10)
    is_pref = g.below(n_rules, 100) == 0
    geo_u = g.u64(n_rules)
    plen = g.below(n_rules, 9) + np.uint64(16)
    pnode = g.below(n_rules, n_nodes)
    pa = g.below(n_rules, 65535) + np.uint64(1)
    pb = g.below(n_rules, 65535) + np.uint64(1)
    single = g.below(n_rules, 10) == 0
    # geometric source count with mean 4: 1 + floor(log(u) / log(3/4)), capped
    u = (geo_u >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    cnt = np.minimum(64, 1 + np.floor(np.log(np.maximum(u, 1e-300)) / np.log(0.75))).astype(np.int64)
    total_src = int(np.where(is_pref, 1, cnt).sum())
    src_nodes = g.below(total_src, n_nodes)
    cursor = 0
    for i in range(n_rules):
        proto = protos[0] if pw[i] < 6 else (protos[1] if pw[i] < 9 else protos[2])
        rules[i]["proto"] = proto
        rules[i]["src_begin"] = len(srcs)
        if is_pref[i]:
            bits = int(plen[i])
            addr = int(nodes[src_nodes[cursor]]) & (0xFFFFFFFF << (32 - bits)) & 0xFFFFFFFF
            srcs.append((addr, bits))
            cursor += 1
        else:
            for _ in range(int(cnt[i])):
                srcs.append((int(nodes[src_nodes[cursor]]), 32))
                cursor += 1
        rules[i]["src_end"] = len(srcs)
        rules[i]["port_begin"] = len(ports)
        if proto != 1:
            lo, hi = int(min(pa[i], pb[i])), int(max(pa[i], pb[i]))
            if single[i]:
                hi = lo
            ports.append((lo, hi))
        rules[i]["port_end"] = len(ports)
    srcs_a = np.array(srcs, PREFIX_DTYPE)
    ports_a = np.array(ports, PORT_DTYPE) if ports else np.zeros(0, PORT_DTYPE)

    t0 = 1_700_000_000 * 1_000_000_000
    # outbound flows this node opens
    o_node = g.below(n_out, n_nodes)
    o_pw = g.below(n_out, 10)
    o_sport = g.below(n_out, 65535) + np.uint64(1)
    o_dport = g.below(n_out, 65535) + np.uint64(1)
    o_proto = np.where(o_pw < 6, 6, np.where(o_pw < 9, 17, 1)).astype(np.uint8)
    o_dst = nodes[o_node]
    outbound = _headers(o_proto, np.full(n_out, self_ip, np.uint64), o_dst, o_sport, o_dport)

    # inbound: 30 % replies, 5 % malformed, 65 % fresh traffic from random nodes
    cls = g.below(n_in, 100)
    pick = g.below(n_in, max(n_out, 1))
    i_node = g.below(n_in, n_nodes)
    i_pw = g.below(n_in, 10)
    i_sport = g.below(n_in, 65535) + np.uint64(1)
    i_dport = g.below(n_in, 65535) + np.uint64(1)
    bad_kind = g.below(n_in, 4)
    i_proto = np.where(i_pw < 6, 6, np.where(i_pw < 9, 17, 1)).astype(np.uint8)
    reply = cls < 30
    proto = np.where(reply, o_proto[pick], i_proto).astype(np.uint8)
    src = np.where(reply, o_dst[pick], nodes[i_node])
    sport = np.where(reply, o_dport[pick], i_sport)
    dport = np.where(reply, o_sport[pick], i_dport)
    inbound = _headers(proto, src, np.full(n_in, self_ip, np.uint64), sport, dport)
    in_len = np.full(n_in, 28, np.uint32)
    bad = (cls >= 30) & (cls < 35)
    k0, k1, k2, k3 = (bad & (bad_kind == k) for k in range(4))
    in_len[k0] = 22                    # transport header cut short
    inbound[k1, 0] = 0x65              # IPv6 version nibble
    inbound[k2, 0] = 0x44              # IHL below 5
    inbound[k3, 9] = 47                # GRE: not tcp/udp/icmp
    late_sel = np.flatnonzero(reply)[::50]  # 2 % of the replies, checked again after every TTL has run out
    late = inbound[late_sel].copy()
    return FilterWorkload(self_ip=self_ip, nodes=nodes, rules=rules, srcs=srcs_a, ports=ports_a, t0_ns=t0,
                          outbound=outbound, outbound_len=np.full(n_out, 28, np.uint32), inbound=inbound,
                          inbound_len=in_len, late=late, late_len=np.full(len(late), 28, np.uint32))


# ---------------------------------------------------------------------------------------
# configuration 4: bulk seal, sharded by peer
# ---------------------------------------------------------------------------------------
@dataclass
class BulkSealPlan:
    n_packets: int
    n_peers: int
    size: int
    stride: int
    key_seed: int
    payload_seed: int


def config4(n_packets: int = 1 << 20, n_peers: int = 1 << 16, size: int = 1420, rank: int = 0,
            world: int = 1) -> BulkSealPlan:
    """Weak-scaling shard `rank` of `world`: every rank holds n_peers peers (global peer index
    = local index * world + rank) and n_packets packets; packet i belongs to local peer i % n_peers
    with counter i // n_peers.  Keys are the first n_peers*32 bytes of SplitMix64(key_seed); the
    ring is filled by SplitMix64(payload_seed) from byte 0 (header room and tag room included)."""
    from .device import slot_size
    s = seed_for(4)
    return BulkSealPlan(n_packets=n_packets, n_peers=n_peers, size=size, stride=slot_size(size),
                        key_seed=(s * 0x10001 + 2 * rank) & _M64, payload_seed=(s * 0x10001 + 2 * rank + 1) & _M64)


def bulk_keys(plan: BulkSealPlan) -> np.ndarray:
    return SplitMix64(plan.key_seed).bytes(plan.n_peers * 32).reshape(plan.n_peers, 32)


def shard_of_peer(peer_index: int, world: int) -> int:
    """Which GPU owns a peer: all mutable per-peer state lives on exactly one device."""
    return peer_index % world


# ---------------------------------------------------------------------------------------
# configuration 5: GSO super-packets, Zipf peer popularity
# ---------------------------------------------------------------------------------------
@dataclass
class GsoWorkload:
    supers: list                 # byte strings: IPv4 + TCP header (40 B) + n_seg * mss payload bytes
    peer: np.ndarray             # [n_super] destination peer of each super-packet
    peer_ip: np.ndarray          # [n_peers] tunnel address of each peer
    self_ip: int
    keys: np.ndarray             # [n_peers, 32]
    mss: int
    hdr_len: int = 40
    csum_start: int = 20
    csum_offset: int = 16


def zipf_ranks(g: SplitMix64, n: int, n_items: int, s: float = 1.1) -> np.ndarray:
    """n draws from Zipf(s) over ranks 0..n_items-1 by inverse CDF on a 53-bit uniform."""
    w = 1.0 / np.power(np.arange(1, n_items + 1, dtype=np.float64), s)
    cdf = np.cumsum(w) / w.sum()
    u = (g.u64(n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    return np.minimum(np.searchsorted(cdf, u, side="left"), n_items - 1).astype(np.uint32)


def config5_peers(n_super: int, n_peers: int = 10_000, seed: int | None = None) -> np.ndarray:
    """Only the peer draws of config5 (same stream, same positions): what a dispatcher sees of a period of
    traffic when it measures the load per peer."""
    g = SplitMix64(seed_for(5) if seed is None else seed)
    g.bytes(n_peers * 32)
    return zipf_ranks(g, n_super, n_peers)


def config5(n_super: int = 64, n_peers: int = 10_000, n_seg: int = 47, mss: int = 1380, seed: int | None = None) -> GsoWorkload:
    """Draw order: n_peers*32 key bytes; n_super Zipf(1.1) peer draws; per super-packet: source port,
    destination port, sequence number, IP id (one u64 each), then n_seg*mss payload bytes.  Peer p has tunnel
    address 100.64.0.0 + 256 + p."""
    g = SplitMix64(seed_for(5) if seed is None else seed)
    keys = g.bytes(n_peers * 32).reshape(n_peers, 32)
    peer = zipf_ranks(g, n_super, n_peers)
    self_ip = ip4(100, 64, 0, 1)
    peer_ip = (ip4(100, 64, 0, 0) + 256 + np.arange(n_peers)).astype(np.uint64)
    supers = []
    for j in range(n_super):
        sport = 1024 + g.one_below(60000)
        dport = 1 + g.one_below(65535)
        seq = g.one_below(1 << 32)
        ipid = g.one_below(1 << 16)
        payload = g.bytes(n_seg * mss).tobytes()
        ip = bytearray(ipv4_header(6, self_ip, int(peer_ip[peer[j]]), 40 + len(payload)))
        ip[4], ip[5] = ipid >> 8, ipid & 0xFF
        tcp = bytearray(20)
        tcp[0:4] = bytes(l4_ports(sport, dport))
        tcp[4:8] = seq.to_bytes(4, "big")
        tcp[12] = 5 << 4
        tcp[13] = 0x18  # PSH | ACK
        supers.append(bytes(ip) + bytes(tcp) + payload)
    return GsoWorkload(supers=supers, peer=peer, peer_ip=peer_ip, self_ip=self_ip, keys=keys, mss=mss)
