"""Python handles over the multi-GPU part of the C ABI: the placement rule and the dispatcher.

Plumbing for tests and the benchmark; the routing, the per-GPU submits and every packet decision
happen in libbnkgpu.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib


def place_peers(load: np.ndarray | None, n_peers: int, n_gpus: int, max_per_gpu: int | None = None):
    """bnk_place_peers: peers to GPUs by measured load, heaviest first, each to the lightest GPU so far.
    -> (gpu_of[n_peers], slot_of[n_peers], load_per_gpu[n_gpus]).  Needs no GPU."""
    if max_per_gpu is None:
        max_per_gpu = n_peers
    gpu_of = np.zeros(n_peers, np.uint32)
    slot_of = np.zeros(n_peers, np.uint32)
    per_gpu = np.zeros(n_gpus, np.uint64)
    lp = None
    if load is not None:
        load = np.ascontiguousarray(load, np.uint64)
        assert len(load) == n_peers
        lp = load.ctypes.data
    rc = _lib.lib().bnk_place_peers(lp, n_peers, n_gpus, max_per_gpu, gpu_of.ctypes.data, slot_of.ctypes.data,
                                    per_gpu.ctypes.data)
    if rc < 0:
        raise _lib.BnkError(rc, "bnk_place_peers")
    return gpu_of, slot_of, per_gpu


def _pointers(buf: np.ndarray, offsets: np.ndarray) -> np.ndarray:
    return (np.uint64(buf.ctypes.data) + offsets.astype(np.uint64)).astype(np.uint64)


class MultiGpu:
    """One context per listed device behind bnk_mgpu_seal / bnk_mgpu_open."""

    def __init__(self, devices: Sequence[int], max_peers: int, max_pkts_per_gpu: int = 4096, max_packet: int = 1420,
                 max_keypairs_per_gpu: int | None = None, replay_ring_blocks: int = 128, mtu: int = 1420,
                 flow_capacity: int = 1 << 16):
        L = _lib.lib()
        devs = (C.c_int32 * len(devices))(*devices)
        ctx = _lib.Cfg(C.sizeof(_lib.Cfg), 0, max_keypairs_per_gpu or max_peers, replay_ring_blocks, mtu, flow_capacity, 0, 0)
        cfg = _lib.MgpuCfg(C.sizeof(_lib.MgpuCfg), len(devices), devs, max_pkts_per_gpu, max_packet, max_peers, 0, ctx)
        h = C.c_void_p()
        rc = L.bnk_mgpu_create(C.byref(cfg), C.byref(h))
        if rc < 0:
            raise _lib.BnkError(rc, L.bnk_last_error_string(None).decode(errors="replace"))
        self._h = h
        self.n_gpus = len(devices)
        self.max_peers = max_peers
        self.max_packet = max_packet

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().bnk_mgpu_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _ck(self, rc: int) -> int:
        if rc < 0:
            raise _lib.BnkError(rc, _lib.lib().bnk_mgpu_last_error_string(self._h).decode(errors="replace"))
        return rc

    def place(self, load: np.ndarray | None):
        lp = None
        if load is not None:
            load = np.ascontiguousarray(load, np.uint64)
            assert len(load) == self.max_peers
            lp = load.ctypes.data
        self._ck(_lib.lib().bnk_mgpu_place(self._h, lp))

    def locate(self, peer: int):
        g, s = C.c_uint32(), C.c_uint32()
        self._ck(_lib.lib().bnk_mgpu_locate(self._h, peer, C.byref(g), C.byref(s)))
        return g.value, s.value

    def peer_set(self, peer: int, send_key: bytes, recv_key: bytes, remote_index: int, local_index: int, allowed_ip: int = 0):
        self._ck(_lib.lib().bnk_mgpu_peer_set(self._h, peer, C.c_char_p(bytes(send_key)), C.c_char_p(bytes(recv_key)),
                                              remote_index, local_index, allowed_ip))

    def peer_clear(self, peer: int):
        self._ck(_lib.lib().bnk_mgpu_peer_clear(self._h, peer))

    def acl_set(self, enforce: bool, tuples: np.ndarray | None = None):
        if tuples is None or len(tuples) == 0:
            self._ck(_lib.lib().bnk_mgpu_acl_set(self._h, int(enforce), None, 0))
        else:
            tuples = np.ascontiguousarray(tuples, np.dtype(_lib.AclTuple))
            self._ck(_lib.lib().bnk_mgpu_acl_set(self._h, int(enforce), tuples.ctypes.data, len(tuples)))

    def loads(self, reset: bool = False):
        pk = np.zeros(self.max_peers, np.uint64)
        by = np.zeros(self.max_peers, np.uint64)
        pg = np.zeros(self.n_gpus, np.uint64)
        self._ck(_lib.lib().bnk_mgpu_loads_get(self._h, pk.ctypes.data, by.ctypes.data, pg.ctypes.data, int(reset)))
        return pk, by, pg

    def seal(self, packets: Sequence[bytes], peers: np.ndarray, flags: int = 0, now_ns: int = 0):
        """-> (messages: list[bytes], status, counters)"""
        n = len(packets)
        lens = np.array([len(p) for p in packets], np.uint32)
        in_off = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.uint64) if n else np.zeros(0, np.uint64)
        src = np.frombuffer(b"".join(packets) + b"\0", np.uint8).copy()
        stride = self.max_packet + 64
        dst = np.zeros(max(1, n * stride), np.uint8)
        out_off = np.arange(n, dtype=np.uint64) * np.uint64(stride)
        peers = np.ascontiguousarray(peers, np.uint32)
        out_len = np.zeros(n, np.uint32)
        counter = np.zeros(n, np.uint64)
        status = np.zeros(n, np.uint8)
        pin, pout = _pointers(src, in_off), _pointers(dst, out_off)
        self._ck(_lib.lib().bnk_mgpu_seal(self._h, pin.ctypes.data, lens.ctypes.data, peers.ctypes.data, n, flags, now_ns,
                                          pout.ctypes.data, out_len.ctypes.data, counter.ctypes.data, status.ctypes.data))
        msgs = [dst[int(o):int(o) + int(l)].tobytes() for o, l in zip(out_off, out_len)]
        return msgs, status, counter

    def open(self, messages: Sequence[bytes], flags: int = 0, now_ns: int = 0):
        """-> (plaintexts: list[bytes], status, counters, peers)"""
        n = len(messages)
        lens = np.array([len(p) for p in messages], np.uint32)
        in_off = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.uint64) if n else np.zeros(0, np.uint64)
        src = np.frombuffer(b"".join(messages) + b"\0", np.uint8).copy()
        stride = self.max_packet + 64
        dst = np.zeros(max(1, n * stride), np.uint8)
        out_off = np.arange(n, dtype=np.uint64) * np.uint64(stride)
        out_len = np.zeros(n, np.uint32)
        counter = np.zeros(n, np.uint64)
        peers = np.zeros(n, np.uint32)
        status = np.zeros(n, np.uint8)
        pin, pout = _pointers(src, in_off), _pointers(dst, out_off)
        self._ck(_lib.lib().bnk_mgpu_open(self._h, pin.ctypes.data, lens.ctypes.data, n, flags, now_ns, pout.ctypes.data,
                                          out_len.ctypes.data, counter.ctypes.data, peers.ctypes.data, status.ctypes.data))
        pts = [dst[int(o):int(o) + int(l)].tobytes() for o, l in zip(out_off, out_len)]
        return pts, status, counter, peers
