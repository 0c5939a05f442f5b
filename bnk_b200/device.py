"""Host-side handles over the C ABI: one Context per GPU, Batches with pinned rings.

This is plumbing for tests, the benchmark and the Python mirror of the reference's
interfaces; all packet work happens in libbnkgpu.so's CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Sequence

import numpy as np

from . import _lib
from ._lib import (  # noqa: F401  (re-exported)
    F_ASSIGN_COUNTERS,
    F_CHECK_INBOUND,
    F_DEMUX_INDEX,
    F_INNER_CHECK,
    F_NO_D2H,
    F_NO_H2D,
    F_NOTE_OUTBOUND,
    F_REPLAY,
    F_SORT_BY_LENGTH,
    F_STATS,
    F_TIMED,
    F_USE_OUT_LEN,
    PKT_AUTH_FAIL,
    PKT_BAD_DESC,
    PKT_BAD_INNER,
    PKT_NO_KEYPAIR,
    PKT_COUNTER_EXHAUSTED,
    PKT_FILTER_DENY,
    PKT_KEEPALIVE,
    PKT_MALFORMED,
    PKT_OK,
    PKT_REPLAY,
    WAIT_FOREVER,
    BnkError,
)

ACL_TUPLE_DTYPE = np.dtype(_lib.AclTuple)
GSO_SUPER_DTYPE = np.dtype(_lib.GsoSuper)
FLOW_ENTRY_DTYPE = np.dtype(_lib.FlowEntry)


def _np_view(ptr: int, dtype, count: int) -> np.ndarray:
    nbytes = int(count) * np.dtype(dtype).itemsize
    buf = (C.c_uint8 * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype, count=count)


def slot_size(mtu: int) -> int:
    """Bytes one packet of up to `mtu` bytes needs in a ring: header room + padded payload + tag, 16-aligned."""
    return (16 + ((mtu + 15) & ~15) + 16 + 15) & ~15


class Context:
    """One GPU: keypair table, replay windows, ACL + flow tables."""

    def __init__(self, device_id: int = 0, max_keypairs: int = 1024, replay_ring_blocks: int = 128, mtu: int = 1420,
                 flow_capacity: int = 1 << 16, max_acl_tuples: int = 0):
        L = _lib.lib()
        cfg = _lib.Cfg(C.sizeof(_lib.Cfg), device_id, max_keypairs, replay_ring_blocks, mtu, flow_capacity,
                       max_acl_tuples, 0)
        h = C.c_void_p()
        _lib.check(L.bnk_ctx_create(C.byref(cfg), C.byref(h)))
        self._h = h
        self.cfg = cfg
        self._batches: list[Batch] = []

    # -- lifetime --
    def close(self):
        if getattr(self, "_h", None):
            for b in list(self._batches):
                b.close()
            _lib.lib().bnk_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _ck(self, code: int) -> int:
        return _lib.check(code, self._h)

    def synchronize(self):
        self._ck(_lib.lib().bnk_ctx_synchronize(self._h))

    # -- keypairs --
    def set_keypair(self, slot: int, send_key: bytes, recv_key: bytes, remote_index: int):
        self._ck(_lib.lib().bnk_keypair_set(self._h, slot, C.c_char_p(bytes(send_key)), C.c_char_p(bytes(recv_key)),
                                            remote_index))

    def set_keypairs(self, first_slot: int, send_keys: np.ndarray, recv_keys: np.ndarray, remote_index: np.ndarray):
        send_keys = np.ascontiguousarray(send_keys, np.uint8)
        recv_keys = np.ascontiguousarray(recv_keys, np.uint8)
        remote_index = np.ascontiguousarray(remote_index, np.uint32)
        n = len(remote_index)
        assert send_keys.size == 32 * n and recv_keys.size == 32 * n
        self._ck(_lib.lib().bnk_keypair_set_many(self._h, first_slot, n, send_keys.ctypes.data, recv_keys.ctypes.data,
                                                 remote_index.ctypes.data))

    def clear_keypair(self, slot: int):
        self._ck(_lib.lib().bnk_keypair_clear(self._h, slot))

    def send_counter(self, slot: int) -> int:
        v = C.c_uint64()
        self._ck(_lib.lib().bnk_send_counter_get(self._h, slot, C.byref(v)))
        return v.value

    def set_send_counter(self, slot: int, value: int):
        self._ck(_lib.lib().bnk_send_counter_set(self._h, slot, value))

    def index_set(self, local_index: int, slot: int):
        self._ck(_lib.lib().bnk_index_set(self._h, local_index, slot))

    def index_clear(self, local_index: int):
        self._ck(_lib.lib().bnk_index_clear(self._h, local_index))

    def set_allowed_ip(self, slot: int, ipv4: int):
        self._ck(_lib.lib().bnk_keypair_set_allowed_ip(self._h, slot, ipv4))

    def addr_set(self, addr16: bytes, port: int, peer_id: int):
        """byAddr[addr:port] = peer_id; addr16 is 16 bytes, IPv4 as ::ffff:a.b.c.d."""
        self._ck(_lib.lib().bnk_addr_set(self._h, C.c_char_p(bytes(addr16)), port, peer_id))

    def addr_clear(self, addr16: bytes, port: int):
        self._ck(_lib.lib().bnk_addr_clear(self._h, C.c_char_p(bytes(addr16)), port))

    def replay_export(self, slot: int):
        last = C.c_uint64()
        ring = np.zeros(self.cfg.replay_ring_blocks, np.uint64)
        self._ck(_lib.lib().bnk_replay_export(self._h, slot, C.byref(last), ring.ctypes.data))
        return last.value, ring

    def replay_import(self, slot: int, last: int, ring: np.ndarray):
        ring = np.ascontiguousarray(ring, np.uint64)
        assert len(ring) == self.cfg.replay_ring_blocks
        self._ck(_lib.lib().bnk_replay_import(self._h, slot, last, ring.ctypes.data))

    # -- ACL --
    def acl_set(self, enforce: bool, tuples: np.ndarray | None = None):
        if tuples is None or len(tuples) == 0:
            self._ck(_lib.lib().bnk_acl_set(self._h, int(enforce), None, 0))
            return
        tuples = np.ascontiguousarray(tuples, ACL_TUPLE_DTYPE)
        self._ck(_lib.lib().bnk_acl_set(self._h, int(enforce), tuples.ctypes.data, len(tuples)))

    def flows_clear(self):
        self._ck(_lib.lib().bnk_flows_clear(self._h))

    def flows_count(self) -> int:
        v = C.c_uint64()
        self._ck(_lib.lib().bnk_flows_count(self._h, C.byref(v)))
        return v.value

    def flows_export(self) -> np.ndarray:
        """The flow table's live entries as a FLOW_ENTRY_DTYPE array sorted by key."""
        n = C.c_size_t()
        self._ck(_lib.lib().bnk_flows_export(self._h, None, 0, C.byref(n)))
        out = np.zeros(max(n.value, 1), FLOW_ENTRY_DTYPE)
        self._ck(_lib.lib().bnk_flows_export(self._h, out.ctypes.data, n.value, C.byref(n)))
        out = out[:n.value]
        return out[np.lexsort((out["local_port"], out["remote_port"], out["remote_addr"], out["proto"]))]

    def flows_import(self, entries: np.ndarray):
        entries = np.ascontiguousarray(entries, FLOW_ENTRY_DTYPE)
        self._ck(_lib.lib().bnk_flows_import(self._h, entries.ctypes.data, len(entries)))

    def table_stats(self) -> "_lib.TableStats":
        v = _lib.TableStats()
        self._ck(_lib.lib().bnk_table_stats_get(self._h, C.byref(v)))
        return v

    # -- batches / measurement --
    def batch(self, max_pkts: int, ring_bytes: int) -> "Batch":
        return Batch(self, max_pkts, ring_bytes)

    def launch_count(self) -> int:
        v = C.c_uint64()
        self._ck(_lib.lib().bnk_kernel_launch_count(self._h, C.byref(v)))
        return v.value

    def probe_int_throughput(self, mix: int) -> float:
        v = C.c_double()
        self._ck(_lib.bench_lib().bnk_probe_int_throughput(self._h, mix, C.byref(v)))
        return v.value

    def probe_coissue(self, kind: int, k: int) -> float:
        v = C.c_double()
        self._ck(_lib.bench_lib().bnk_probe_coissue(self._h, kind, k, C.byref(v)))
        return v.value

    def probe_copy_rounds(self, threads: int, nbytes: int, rounds: int, directions: int = 3) -> float:
        """Copy rounds per second (nbytes up and/or down, then wait) over `threads` host threads: see the bench header."""
        v = C.c_double()
        self._ck(_lib.bench_lib().bnk_probe_copy_rounds(self._h, threads, nbytes, rounds, directions, C.byref(v)))
        return v.value

    def timer_start(self, batches: Sequence["Batch"]):
        arr = (C.c_void_p * len(batches))(*[b._h for b in batches])
        self._ck(_lib.bench_lib().bnk_timer_start(self._h, arr, len(batches)))

    def timer_stop(self, batches: Sequence["Batch"]) -> float:
        arr = (C.c_void_p * len(batches))(*[b._h for b in batches])
        ms = C.c_float()
        self._ck(_lib.bench_lib().bnk_timer_stop(self._h, arr, len(batches), C.byref(ms)))
        return ms.value


class Batch:
    """Pinned host ring + descriptors (numpy views) with a device mirror and a CUDA stream."""

    def __init__(self, ctx: Context, max_pkts: int, ring_bytes: int):
        self.ctx = ctx
        h = C.c_void_p()
        ctx._ck(_lib.lib().bnk_batch_create(ctx._h, max_pkts, ring_bytes, C.byref(h)))
        self._h = h
        v = _lib.BatchView()
        ctx._ck(_lib.lib().bnk_batch_view_get(h, C.byref(v)))
        self.max_pkts = max_pkts
        self.ring_bytes = ring_bytes
        self.ring = _np_view(v.ring, np.uint8, ring_bytes)
        self.off = _np_view(v.off, np.uint32, max_pkts)
        self.len = _np_view(v.len, np.uint32, max_pkts)
        self.slot = _np_view(v.slot, np.uint32, max_pkts)
        self.counter = _np_view(v.counter, np.uint64, max_pkts)
        self.out_len = _np_view(v.out_len, np.uint32, max_pkts)
        self.status = _np_view(v.status, np.uint8, max_pkts)
        self.src_addr = _np_view(v.src_addr, np.uint8, max_pkts * _lib.SRC_ADDR_STRIDE).reshape(max_pkts, _lib.SRC_ADDR_STRIDE)
        ctx._batches.append(self)

    def close(self):
        if getattr(self, "_h", None):
            # the numpy views alias pinned memory that is about to be freed
            for name in ("ring", "off", "len", "slot", "counter", "out_len", "status", "src_addr"):
                setattr(self, name, None)
            _lib.lib().bnk_batch_destroy(self._h)
            self._h = None
            if self in self.ctx._batches:
                self.ctx._batches.remove(self)

    def _ck(self, code: int) -> int:
        return _lib.check(code, self.ctx._h)

    # -- filling --
    def put_packets(self, packets: Iterable[bytes], stride: int | None = None, headroom: int = 16) -> int:
        """Lays packets out at fixed stride, payload at slot+headroom (headroom=0: whole messages). Returns n."""
        packets = list(packets)
        if stride is None:
            longest = max((len(p) for p in packets), default=0)
            stride = slot_size(longest)
        for i, p in enumerate(packets):
            o = i * stride
            self.off[i] = o
            self.len[i] = len(p)
            self.ring[o + headroom:o + headroom + len(p)] = np.frombuffer(bytes(p), np.uint8)
        return len(packets)

    def message(self, i: int) -> bytes:
        o = int(self.off[i])
        return self.ring[o:o + int(self.out_len[i])].tobytes()

    def payload(self, i: int, length: int | None = None) -> bytes:
        o = int(self.off[i]) + 16
        n = int(self.out_len[i]) if length is None else length
        return self.ring[o:o + n].tobytes()

    # -- work --
    def seal(self, n: int, flags: int = 0, now_ns: int = 0, wait: bool = True):
        self._ck(_lib.lib().bnk_seal_submit(self._h, n, flags, now_ns))
        if wait:
            self.wait()

    def open(self, n: int, flags: int = 0, now_ns: int = 0, wait: bool = True):
        self._ck(_lib.lib().bnk_open_submit(self._h, n, flags, now_ns))
        if wait:
            self.wait()

    def filter_note(self, n: int, now_ns: int, flags: int = 0, wait: bool = True):
        self._ck(_lib.lib().bnk_filter_note_submit(self._h, n, flags, now_ns))
        if wait:
            self.wait()

    def filter_check(self, n: int, now_ns: int, flags: int = 0, wait: bool = True):
        self._ck(_lib.lib().bnk_filter_check_submit(self._h, n, flags, now_ns))
        if wait:
            self.wait()

    def gso_split(self, supers: np.ndarray, n_pkts: int, flags: int = 0, wait: bool = True):
        """supers: array of GSO_SUPER_DTYPE; segment descriptors (off, len, slot) must already be filled."""
        supers = np.ascontiguousarray(supers, GSO_SUPER_DTYPE)
        self._ck(_lib.lib().bnk_gso_split_submit(self._h, supers.ctypes.data, len(supers), n_pkts, flags))
        if wait:
            self.wait()

    def classify(self, n: int, flags: int = 0, wait: bool = True):
        self._ck(_lib.lib().bnk_classify_submit(self._h, n, flags))
        if wait:
            self.wait()

    def upload(self, n: int, wait: bool = True):
        self._ck(_lib.lib().bnk_batch_upload(self._h, n))
        if wait:
            self.wait()

    def download(self, n: int, wait: bool = True):
        self._ck(_lib.lib().bnk_batch_download(self._h, n))
        if wait:
            self.wait()

    def wait(self, timeout_ns: int = WAIT_FOREVER):
        self._ck(_lib.lib().bnk_wait(self._h, timeout_ns))

    def try_wait(self, timeout_ns: int) -> bool:
        rc = _lib.lib().bnk_wait(self._h, timeout_ns)
        if rc == _lib.ETIMEDOUT:
            return False
        self._ck(rc)
        return True

    def last_kernel_ms(self) -> float:
        ms = C.c_float()
        self._ck(_lib.lib().bnk_batch_last_kernel_ms(self._h, C.byref(ms)))
        return ms.value

    def last_aead_ms(self) -> float:
        ms = C.c_float()
        self._ck(_lib.lib().bnk_batch_last_aead_ms(self._h, C.byref(ms)))
        return ms.value

    def fill_random(self, seed: int):
        self._ck(_lib.bench_lib().bnk_batch_fill_random(self._h, seed))

    def copy_only(self, n: int, up: bool = True, down: bool = True, wait: bool = True):
        """The copies a seal/open submit of n packets makes, and no kernel (measurement helper)."""
        self._ck(_lib.bench_lib().bnk_batch_copy_only(self._h, n, int(up), int(down)))
        if wait:
            self.wait()

    def stats(self) -> dict:
        """Counters of the last submit made with F_STATS (after wait): packets, bytes_out, by_status[16]."""
        v = _lib.BatchStats()
        self._ck(_lib.lib().bnk_batch_stats_get(self._h, C.byref(v)))
        return {"packets": v.packets, "bytes_out": v.bytes_out, "by_status": list(v.by_status)}


class Queue:
    """bnk_queue: many small caller batches packed into few large GPU batches (see include/bnk_gpu.h)."""

    def __init__(self, ctx: Context, open_side: bool, flags: int = 0, max_pkts: int = 4096, max_packet: int = 1420,
                 depth: int = 2):
        self.ctx = ctx
        self.open_side = open_side
        self.max_packet = max_packet
        cfg = _lib.QueueCfg(C.sizeof(_lib.QueueCfg), max_pkts, max_packet, depth, int(open_side), flags)
        h = C.c_void_p()
        ctx._ck(_lib.lib().bnk_queue_create(ctx._h, C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().bnk_queue_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def submit(self, packets: Sequence[bytes], slots=None, now_ns: int = 0):
        """-> ticket (opaque), or None when every GPU batch is taken (collect a ticket and try again)."""
        n = len(packets)
        lens = np.array([len(p) for p in packets], np.uint32)
        offs = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.uint64)
        src = np.frombuffer(b"".join(packets) + b"\0", np.uint8)
        ptrs = (np.uint64(src.ctypes.data) + offs).astype(np.uint64)
        sp = None
        if slots is not None:
            slots = np.ascontiguousarray(slots, np.uint32)
            sp = slots.ctypes.data
        t = C.c_uint64()
        rc = _lib.lib().bnk_queue_submit(self._h, ptrs.ctypes.data, lens.ctypes.data, sp, n, now_ns, C.byref(t))
        if rc == _lib.EBUSY:
            return None
        self.ctx._ck(rc)
        return (t.value, n)

    def wait(self, ticket):
        """-> (outputs: list[bytes], status, counters, slots)"""
        t, n = ticket
        stride = self.max_packet + 64
        dst = np.zeros(n * stride, np.uint8)
        ptrs = (np.uint64(dst.ctypes.data) + np.arange(n, dtype=np.uint64) * np.uint64(stride)).astype(np.uint64)
        out_len = np.zeros(n, np.uint32)
        counter = np.zeros(n, np.uint64)
        slot = np.zeros(n, np.uint32)
        status = np.zeros(n, np.uint8)
        self.ctx._ck(_lib.lib().bnk_queue_wait(self._h, t, ptrs.ctypes.data, out_len.ctypes.data, counter.ctypes.data,
                                               slot.ctypes.data, status.ctypes.data))
        outs = [dst[k * stride:k * stride + int(out_len[k])].tobytes() for k in range(n)]
        return outs, status, counter, slot

    # -- the same without host copies: the caller works on the pinned ring of the GPU batch itself --
    def _span_views(self, sp: "_lib.QueueSpan", n: int) -> dict:
        as_np = np.ctypeslib.as_array
        return {"data": as_np(sp.data, shape=(n, sp.stride)), "len": as_np(sp.len, shape=(n,)),
                "slot": as_np(sp.slot, shape=(n,)), "out_len": as_np(sp.out_len, shape=(n,)),
                "counter": as_np(sp.counter, shape=(n,)), "status": as_np(sp.status, shape=(n,))}

    def reserve(self, n: int, now_ns: int = 0):
        """-> (ticket, views) or None when every GPU batch is taken.  views["data"][k] is packet k's slot: a seal
        queue wants the plaintext from byte 16 on, an open queue the message from byte 0; set views["len"][k] and
        views["slot"][k], then commit(ticket)."""
        t, sp = C.c_uint64(), _lib.QueueSpan()
        rc = _lib.lib().bnk_queue_reserve(self._h, n, now_ns, C.byref(t), C.byref(sp))
        if rc == _lib.EBUSY:
            return None
        self.ctx._ck(rc)
        return (t.value, n), self._span_views(sp, n)

    def commit(self, ticket):
        self.ctx._ck(_lib.lib().bnk_queue_commit(self._h, ticket[0]))

    def wait_span(self, ticket) -> dict:
        """Blocks until the ticket's GPU batch is done -> views of the results in place (valid until release)."""
        sp = _lib.QueueSpan()
        self.ctx._ck(_lib.lib().bnk_queue_wait_span(self._h, ticket[0], C.byref(sp)))
        return self._span_views(sp, ticket[1])

    def release(self, ticket):
        self.ctx._ck(_lib.lib().bnk_queue_release(self._h, ticket[0]))

    def stats(self):
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self.ctx._ck(_lib.lib().bnk_queue_stats_get(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return {"gpu_batches": a.value, "packets": b.value, "caller_batches": c.value}
