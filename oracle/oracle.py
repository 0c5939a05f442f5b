"""ctypes binding of the CPU checker (oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark -- never by the bnk_b200 package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OK, AUTH_FAIL, REPLAY, FILTER_DENY, MALFORMED, KEEPALIVE, COUNTER_EXHAUSTED, BAD_DESC = range(8)
NO_KEYPAIR, BAD_INNER = 8, 9
REJECT_AFTER_MESSAGES = 0xFFFFFFFFFFFFDFFF


def build(force: bool = False) -> None:
    """Compile liboracle.so / libcpubaseline.so with gcc (seconds)."""
    targets = ["liboracle.so", "libcpubaseline.so"]
    srcs = {"liboracle.so": ["bnk_oracle.c", "bnk_oracle.h"], "libcpubaseline.so": ["cpu_baseline.c", "bnk_oracle.h"]}
    stale = force
    for t in targets:
        tp = os.path.join(_HERE, t)
        if not os.path.exists(tp):
            stale = True
            break
        for s in srcs[t]:
            if os.path.getmtime(os.path.join(_HERE, s)) > os.path.getmtime(tp):
                stale = True
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B", "all"], check=True, capture_output=True)


class Prefix(C.Structure):
    _fields_ = [("addr", C.c_uint32), ("bits", C.c_int32)]


class PortRange(C.Structure):
    _fields_ = [("first", C.c_uint16), ("last", C.c_uint16)]


class Rule(C.Structure):
    _fields_ = [
        ("proto", C.c_uint8),
        ("src_begin", C.c_uint32),
        ("src_end", C.c_uint32),
        ("port_begin", C.c_uint32),
        ("port_end", C.c_uint32),
    ]


def lib() -> C.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(_HERE, "liboracle.so")
    if not os.path.exists(path):
        build()
    L = C.CDLL(path)
    u8p, u32p, u64p = C.POINTER(C.c_uint8), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
    vp, sz = C.c_void_p, C.c_size_t
    L.bnko_chacha20_block.argtypes = [vp, C.c_uint32, vp, vp]
    L.bnko_chacha20_block.restype = None
    L.bnko_chacha20_xor.argtypes = [vp, C.c_uint32, vp, vp, vp, sz]
    L.bnko_chacha20_xor.restype = None
    L.bnko_poly1305.argtypes = [vp, vp, sz, vp]
    L.bnko_poly1305.restype = None
    L.bnko_aead_seal.argtypes = [vp, vp, vp, sz, vp, sz, vp]
    L.bnko_aead_seal.restype = None
    L.bnko_aead_open.argtypes = [vp, vp, vp, sz, vp, sz, vp]
    L.bnko_aead_open.restype = C.c_int
    L.bnko_wg_padded_len.argtypes = [sz, sz]
    L.bnko_wg_padded_len.restype = sz
    L.bnko_wg_seal.argtypes = [vp, C.c_uint32, C.c_uint64, vp, sz, sz, vp]
    L.bnko_wg_seal.restype = sz
    L.bnko_wg_open.argtypes = [vp, vp, sz, vp, C.POINTER(sz), u64p, u32p]
    L.bnko_wg_open.restype = C.c_int
    L.bnko_inner_check.argtypes = [vp, sz, C.c_uint32, C.POINTER(sz)]
    L.bnko_inner_check.restype = C.c_int
    L.bnko_classify_shape.argtypes = [vp, sz]
    L.bnko_classify_shape.restype = C.c_int
    L.bnko_gso_split.argtypes = [vp, sz, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint, vp, sz, vp, sz]
    L.bnko_gso_split.restype = C.c_int
    L.bnko_inet_checksum.argtypes = [vp, sz, C.c_uint32]
    L.bnko_inet_checksum.restype = C.c_uint16
    L.bnko_wg_seal_batch.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp, vp, vp, sz]
    L.bnko_wg_seal_batch.restype = None
    L.bnko_wg_open_batch.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz]
    L.bnko_wg_open_batch.restype = None
    L.bnko_replay_new.argtypes = [C.c_uint32]
    L.bnko_replay_new.restype = vp
    L.bnko_replay_free.argtypes = [vp]
    L.bnko_replay_free.restype = None
    L.bnko_replay_reset.argtypes = [vp]
    L.bnko_replay_reset.restype = None
    L.bnko_replay_validate.argtypes = [vp, C.c_uint64, C.c_uint64]
    L.bnko_replay_validate.restype = C.c_int
    L.bnko_replay_last.argtypes = [vp]
    L.bnko_replay_last.restype = C.c_uint64
    L.bnko_replay_ring.argtypes = [vp, vp]
    L.bnko_replay_ring.restype = None
    L.bnko_replay_load.argtypes = [vp, C.c_uint64, vp]
    L.bnko_replay_load.restype = None
    L.bnko_filter_new.argtypes = []
    L.bnko_filter_new.restype = vp
    L.bnko_filter_free.argtypes = [vp]
    L.bnko_filter_free.restype = None
    L.bnko_filter_set_rules.argtypes = [vp, vp, sz, vp, sz, vp, sz]
    L.bnko_filter_set_rules.restype = None
    L.bnko_filter_set_allow_all.argtypes = [vp]
    L.bnko_filter_set_allow_all.restype = None
    L.bnko_filter_check_inbound.argtypes = [vp, vp, sz, C.c_int64]
    L.bnko_filter_check_inbound.restype = C.c_int
    L.bnko_filter_note_outbound.argtypes = [vp, vp, sz, C.c_int64]
    L.bnko_filter_note_outbound.restype = None
    L.bnko_filter_flow_count.argtypes = [vp]
    L.bnko_filter_flow_count.restype = sz
    L.bnko_filter_flows_export.argtypes = [vp, vp, sz]
    L.bnko_filter_flows_export.restype = sz
    L.bnko_filter_check_batch.argtypes = [vp, vp, sz, vp, sz, C.c_int64, vp]
    L.bnko_filter_check_batch.restype = None
    L.bnko_filter_check_batch_mt.argtypes = [vp, vp, sz, vp, sz, C.c_int64, vp, C.c_int]
    L.bnko_filter_check_batch_mt.restype = None
    L.bnko_filter_note_batch.argtypes = [vp, vp, sz, vp, sz, C.c_int64]
    L.bnko_filter_note_batch.restype = None
    L.bnko_rule_match.argtypes = [vp, vp, vp, C.c_uint32, C.c_uint8, C.c_uint16]
    L.bnko_rule_match.restype = C.c_int
    L.bnko_filter_parse.argtypes = [vp, sz, vp]
    L.bnko_filter_parse.restype = C.c_int
    _LIB = L
    return L


def _buf(b: bytes):
    return C.create_string_buffer(bytes(b), max(len(b), 1))


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


# ---- RFC 8439 ---------------------------------------------------------------
def chacha20_block(key: bytes, counter: int, nonce: bytes) -> bytes:
    out = C.create_string_buffer(64)
    lib().bnko_chacha20_block(_buf(key), counter, _buf(nonce), out)
    return out.raw


def poly1305(key: bytes, msg: bytes) -> bytes:
    out = C.create_string_buffer(16)
    lib().bnko_poly1305(_buf(key), _buf(msg), len(msg), out)
    return out.raw


def aead_seal(key: bytes, nonce: bytes, pt: bytes, aad: bytes = b"") -> bytes:
    out = C.create_string_buffer(len(pt) + 16)
    lib().bnko_aead_seal(_buf(key), _buf(nonce), _buf(aad), len(aad), _buf(pt), len(pt), out)
    return out.raw


def aead_open(key: bytes, nonce: bytes, ct: bytes, aad: bytes = b""):
    out = C.create_string_buffer(max(len(ct) - 16, 1))
    ok = lib().bnko_aead_open(_buf(key), _buf(nonce), _buf(aad), len(aad), _buf(ct), len(ct), out)
    return out.raw[: max(len(ct) - 16, 0)] if ok else None


# ---- WireGuard transport ----------------------------------------------------
def wg_padded_len(n: int, mtu: int) -> int:
    return lib().bnko_wg_padded_len(n, mtu)


def wg_seal(key: bytes, receiver_index: int, counter: int, pt: bytes, mtu: int) -> bytes:
    out = C.create_string_buffer(len(pt) + 64)
    m = lib().bnko_wg_seal(_buf(key), receiver_index, counter, _buf(pt), len(pt), mtu, out)
    return out.raw[:m]


def wg_open(key: bytes, msg: bytes):
    """-> (status, plaintext, counter, receiver_index)"""
    out = C.create_string_buffer(max(len(msg), 1))
    pl = C.c_size_t(0)
    ctr = C.c_uint64(0)
    rx = C.c_uint32(0)
    st = lib().bnko_wg_open(_buf(key), _buf(msg), len(msg), out, C.byref(pl), C.byref(ctr), C.byref(rx))
    return st, out.raw[: pl.value], ctr.value, rx.value


def inner_check(pt: bytes, allowed_ip: int):
    """-> new length, or None when the packet is to be dropped."""
    nl = C.c_size_t(0)
    ok = lib().bnko_inner_check(_buf(pt), len(pt), allowed_ip, C.byref(nl))
    return nl.value if ok else None


def classify_shape(pkt: bytes) -> int:
    return lib().bnko_classify_shape(_buf(pkt), len(pkt))


def gso_split(pkt: bytes, hdr_len: int, gso_size: int, csum_start: int, csum_offset: int, proto: int):
    """-> list of segments (bytes), or None when the split is refused."""
    max_segs = max(1, (len(pkt) - hdr_len + gso_size - 1) // max(gso_size, 1)) + 1
    stride = hdr_len + gso_size + 8
    out = np.zeros(max_segs * stride, np.uint8)
    sizes = np.zeros(max_segs, np.uint32)
    n = lib().bnko_gso_split(_buf(pkt), len(pkt), hdr_len, gso_size, csum_start, csum_offset, proto, _ptr(out), stride,
                             _ptr(sizes), max_segs)
    if n < 0:
        return None
    return [out[i * stride:i * stride + int(sizes[i])].tobytes() for i in range(n)]


def inet_checksum(data: bytes, initial: int = 0) -> int:
    return lib().bnko_inet_checksum(_buf(data), len(data), initial)


def wg_seal_batch(keys, remote_index, mtu, ring, off, length, slot, counter):
    """In-place seal over a ring (numpy arrays).  -> (status u8[n], out_len u32[n])"""
    n = len(off)
    status = np.zeros(n, np.uint8)
    out_len = np.zeros(n, np.uint32)
    lib().bnko_wg_seal_batch(_ptr(keys), _ptr(remote_index), mtu, _ptr(ring), _ptr(off), _ptr(length), _ptr(slot),
                             _ptr(counter), _ptr(status), _ptr(out_len), n)
    return status, out_len


def wg_open_batch(keys, ring, off, length, slot):
    """In-place open over a ring.  -> (status, counter, pt_len); no replay check."""
    n = len(off)
    status = np.zeros(n, np.uint8)
    out_len = np.zeros(n, np.uint32)
    counter = np.zeros(n, np.uint64)
    lib().bnko_wg_open_batch(_ptr(keys), _ptr(ring), _ptr(off), _ptr(length), _ptr(slot), _ptr(counter),
                             _ptr(status), _ptr(out_len), n)
    return status, counter, out_len


# ---- OpenSSL-backed multi-threaded batch (the timed CPU baseline) ------------
_BASE = None


def baseline_lib() -> C.CDLL:
    global _BASE
    if _BASE is None:
        path = os.path.join(_HERE, "libcpubaseline.so")
        if not os.path.exists(path):
            build()
        B = C.CDLL(path)
        vp, sz = C.c_void_p, C.c_size_t
        B.bnkb_host_cores.restype = C.c_int
        B.bnkb_aead_batch.argtypes = [C.c_int, C.c_int, vp, vp, sz, vp, vp, vp, vp, vp, vp, vp, sz]
        B.bnkb_aead_batch.restype = C.c_double
        _BASE = B
    return _BASE


def host_cores() -> int:
    return baseline_lib().bnkb_host_cores()


def cpu_aead_batch(open_side: bool, threads: int, keys, remote_index, mtu, ring, off, length, slot, counter):
    """In-place seal/open of a ring with OpenSSL on `threads` host threads.
    -> (seconds, status, out_len); counter is read (seal) or written (open)."""
    n = len(off)
    status = np.zeros(n, np.uint8)
    out_len = np.zeros(n, np.uint32)
    secs = baseline_lib().bnkb_aead_batch(int(open_side), threads, _ptr(keys), _ptr(remote_index), mtu, _ptr(ring),
                                          _ptr(off), _ptr(length), _ptr(slot), _ptr(counter), _ptr(status),
                                          _ptr(out_len), n)
    return secs, status, out_len


# ---- replay window ----------------------------------------------------------
class Replay:
    def __init__(self, ring_blocks: int = 128):
        self.blocks = ring_blocks
        self._h = lib().bnko_replay_new(ring_blocks)
        if not self._h:
            raise ValueError("ring_blocks must be a power of two")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().bnko_replay_free(self._h)
            self._h = None

    def validate(self, counter: int, limit: int = REJECT_AFTER_MESSAGES) -> bool:
        return bool(lib().bnko_replay_validate(self._h, counter, limit))

    def reset(self):
        lib().bnko_replay_reset(self._h)

    @property
    def last(self) -> int:
        return lib().bnko_replay_last(self._h)

    def ring(self) -> np.ndarray:
        out = np.zeros(self.blocks, np.uint64)
        lib().bnko_replay_ring(self._h, _ptr(out))
        return out

    def load(self, last: int, ring: np.ndarray):
        ring = np.ascontiguousarray(ring, np.uint64)
        lib().bnko_replay_load(self._h, last, _ptr(ring))


# ---- filter -----------------------------------------------------------------
PROTO_ID = {"tcp": 6, "udp": 17, "icmp": 1}


class Filter:
    """Mirrors filter.Filter of the reference (internal/filter/filter.go:33-59)."""

    def __init__(self):
        self._h = lib().bnko_filter_new()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().bnko_filter_free(self._h)
            self._h = None

    def set_rules(self, rules):
        """rules: iterable of (srcs, proto, ports); srcs = [(addr_u32, bits)], ports = [(first, last)]."""
        rr, ss, pp = [], [], []
        for srcs, proto, ports in rules:
            r = Rule()
            r.proto = PROTO_ID.get(proto, 0) if isinstance(proto, str) else int(proto)
            r.src_begin = len(ss)
            ss.extend(srcs)
            r.src_end = len(ss)
            r.port_begin = len(pp)
            pp.extend(ports)
            r.port_end = len(pp)
            rr.append(r)
        ra = (Rule * max(len(rr), 1))(*rr)
        sa = (Prefix * max(len(ss), 1))(*[Prefix(a, b) for a, b in ss])
        pa = (PortRange * max(len(pp), 1))(*[PortRange(a, b) for a, b in pp])
        lib().bnko_filter_set_rules(self._h, ra, len(rr), sa, len(ss), pa, len(pp))

    def set_rules_arrays(self, rules: np.ndarray, srcs: np.ndarray, ports: np.ndarray):
        """Structured numpy arrays laid out like Rule / Prefix / PortRange."""
        lib().bnko_filter_set_rules(self._h, _ptr(rules), len(rules), _ptr(srcs), len(srcs), _ptr(ports), len(ports))

    def set_allow_all(self):
        lib().bnko_filter_set_allow_all(self._h)

    def check_inbound(self, pkt: bytes, now_ns: int) -> bool:
        pkt = pkt or b""
        return bool(lib().bnko_filter_check_inbound(self._h, _buf(pkt), len(pkt), now_ns))

    def note_outbound(self, pkt: bytes, now_ns: int) -> None:
        pkt = pkt or b""
        lib().bnko_filter_note_outbound(self._h, _buf(pkt), len(pkt), now_ns)

    def check_batch(self, hdr: np.ndarray, stride: int, length: np.ndarray, now_ns: int) -> np.ndarray:
        n = len(length)
        out = np.zeros(n, np.uint8)
        lib().bnko_filter_check_batch(self._h, _ptr(hdr), stride, _ptr(length), n, now_ns, _ptr(out))
        return out

    def check_batch_mt(self, hdr: np.ndarray, stride: int, length: np.ndarray, now_ns: int, threads: int = 0) -> np.ndarray:
        """check_batch with the (read-only) rule walk on `threads` host threads (0 = all cores); same result."""
        n = len(length)
        out = np.zeros(n, np.uint8)
        lib().bnko_filter_check_batch_mt(self._h, _ptr(hdr), stride, _ptr(length), n, now_ns, _ptr(out),
                                         threads or host_cores())
        return out

    def note_batch(self, hdr: np.ndarray, stride: int, length: np.ndarray, now_ns: int) -> None:
        lib().bnko_filter_note_batch(self._h, _ptr(hdr), stride, _ptr(length), len(length), now_ns)

    @property
    def flow_count(self) -> int:
        return lib().bnko_filter_flow_count(self._h)

    def flows(self) -> np.ndarray:
        """The map's entries as a FLOW_DTYPE array sorted by key."""
        n = self.flow_count
        out = np.zeros(max(n, 1), FLOW_DTYPE)
        got = lib().bnko_filter_flows_export(self._h, _ptr(out), n)
        assert got == n
        out = out[:n]
        return out[np.lexsort((out["lport"], out["rport"], out["remote"], out["proto"]))]


FLOW_DTYPE = np.dtype([("remote", "<u4"), ("rport", "<u2"), ("lport", "<u2"), ("proto", "u1"), ("reserved", "u1", 7),
                       ("exp", "<i8")])
RULE_DTYPE = np.dtype(Rule)
PREFIX_DTYPE = np.dtype(Prefix)
PORT_DTYPE = np.dtype(PortRange)
