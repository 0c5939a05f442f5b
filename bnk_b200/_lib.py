"""ctypes binding of libbnkgpu.so (the C ABI in include/bnk_gpu.h).

There is no fallback: if the shared library is missing this module raises, and every
compute entry point fails with BNK_ECUDA when no sm_100 device is usable.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

SUCCESS, EINVAL, ENOMEM, ECUDA, ETIMEDOUT, EBUSY, EFULL = 0, -1, -2, -3, -4, -5, -6

PKT_OK, PKT_AUTH_FAIL, PKT_REPLAY, PKT_FILTER_DENY, PKT_MALFORMED, PKT_KEEPALIVE, PKT_COUNTER_EXHAUSTED, PKT_BAD_DESC = range(8)
PKT_NO_KEYPAIR, PKT_BAD_INNER = 8, 9

F_NO_H2D = 1 << 0
F_NO_D2H = 1 << 1
F_ASSIGN_COUNTERS = 1 << 2
F_NOTE_OUTBOUND = 1 << 3
F_REPLAY = 1 << 4
F_CHECK_INBOUND = 1 << 5
F_SORT_BY_LENGTH = 1 << 6
F_USE_OUT_LEN = 1 << 7
F_DEMUX_INDEX = 1 << 8
F_INNER_CHECK = 1 << 9
F_TIMED = 1 << 10
F_STATS = 1 << 11

WG_HEADER = 16
WG_TAG = 16
REJECT_AFTER_MESSAGES = 0xFFFFFFFFFFFFDFFF
WAIT_FOREVER = 0xFFFFFFFFFFFFFFFF
NOALLOC_MAX_PKTS = 16384


class Cfg(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("device_id", C.c_int32),
        ("max_keypairs", C.c_uint32),
        ("replay_ring_blocks", C.c_uint32),
        ("mtu", C.c_uint32),
        ("flow_capacity", C.c_uint32),
        ("max_acl_tuples", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class AclTuple(C.Structure):
    _fields_ = [
        ("addr", C.c_uint32),
        ("prefix_len", C.c_uint8),
        ("proto", C.c_uint8),
        ("port_first", C.c_uint16),
        ("port_last", C.c_uint16),
        ("reserved", C.c_uint16),
    ]


class GsoSuper(C.Structure):
    _fields_ = [
        ("src_off", C.c_uint32),
        ("src_len", C.c_uint32),
        ("first_pkt", C.c_uint32),
        ("n_pkts", C.c_uint32),
        ("hdr_len", C.c_uint16),
        ("gso_size", C.c_uint16),
        ("csum_start", C.c_uint16),
        ("csum_offset", C.c_uint16),
        ("proto", C.c_uint8),
        ("reserved", C.c_uint8 * 3),
    ]


class BatchView(C.Structure):
    _fields_ = [
        ("ring", C.c_void_p),
        ("off", C.c_void_p),
        ("len", C.c_void_p),
        ("slot", C.c_void_p),
        ("counter", C.c_void_p),
        ("out_len", C.c_void_p),
        ("status", C.c_void_p),
        ("ring_bytes", C.c_uint64),
        ("max_pkts", C.c_uint32),
        ("reserved", C.c_uint32),
        ("src_addr", C.c_void_p),
    ]


class FlowEntry(C.Structure):
    _fields_ = [("remote_addr", C.c_uint32), ("remote_port", C.c_uint16), ("local_port", C.c_uint16), ("proto", C.c_uint8),
                ("reserved", C.c_uint8 * 7), ("expiry_unix_ns", C.c_int64)]


class BatchStats(C.Structure):
    _fields_ = [("packets", C.c_uint64), ("bytes_out", C.c_uint64), ("by_status", C.c_uint64 * 16)]


class TableStats(C.Structure):
    _fields_ = [
        ("flow_live", C.c_uint64),
        ("flow_used", C.c_uint32 * 3),
        ("flow_dead", C.c_uint32 * 3),
        ("flow_capacity", C.c_uint32),
        ("index_live", C.c_uint32), ("index_dead", C.c_uint32), ("index_slots", C.c_uint32),
        ("addr_live", C.c_uint32), ("addr_dead", C.c_uint32), ("addr_slots", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class QueueCfg(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("max_pkts", C.c_uint32), ("max_packet", C.c_uint32), ("depth", C.c_uint32),
                ("open_side", C.c_uint32), ("flags", C.c_uint32), ("min_fill", C.c_uint32), ("reserved", C.c_uint32)]


class QueueSpan(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_uint8)), ("stride", C.c_uint32), ("reserved", C.c_uint32),
                ("len", C.POINTER(C.c_uint32)), ("slot", C.POINTER(C.c_uint32)), ("out_len", C.POINTER(C.c_uint32)),
                ("counter", C.POINTER(C.c_uint64)), ("status", C.POINTER(C.c_uint8))]


class MgpuCfg(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("n_devices", C.c_uint32),
        ("devices", C.POINTER(C.c_int32)),
        ("max_pkts_per_gpu", C.c_uint32),
        ("max_packet", C.c_uint32),
        ("max_peers", C.c_uint32),
        ("reserved", C.c_uint32),
        ("ctx", Cfg),
    ]


SRC_ADDR_STRIDE = 20
CLASS_WIREGUARD, CLASS_DISCO, CLASS_STUN, CLASS_STRANGER = 0, 10, 11, 12

# every symbol include/bnk_gpu.h declares: name -> (restype, argtypes)
_vp, _i, _u32, _u64, _i64, _sz = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64, C.c_int64, C.c_size_t
SYMBOLS = {
    "bnk_abi_version": (_i, []),
    "bnk_strerror": (C.c_char_p, [_i]),
    "bnk_device_count": (_i, []),
    "bnk_ctx_create": (_i, [C.POINTER(Cfg), C.POINTER(_vp)]),
    "bnk_ctx_destroy": (_i, [_vp]),
    "bnk_last_error_string": (C.c_char_p, [_vp]),
    "bnk_ctx_synchronize": (_i, [_vp]),
    "bnk_keypair_set": (_i, [_vp, _u32, _vp, _vp, _u32]),
    "bnk_keypair_set_many": (_i, [_vp, _u32, _u32, _vp, _vp, _vp]),
    "bnk_keypair_clear": (_i, [_vp, _u32]),
    "bnk_send_counter_get": (_i, [_vp, _u32, C.POINTER(_u64)]),
    "bnk_send_counter_set": (_i, [_vp, _u32, _u64]),
    "bnk_index_set": (_i, [_vp, _u32, _u32]),
    "bnk_index_clear": (_i, [_vp, _u32]),
    "bnk_keypair_set_allowed_ip": (_i, [_vp, _u32, _u32]),
    "bnk_replay_export": (_i, [_vp, _u32, C.POINTER(_u64), _vp]),
    "bnk_replay_import": (_i, [_vp, _u32, _u64, _vp]),
    "bnk_acl_set": (_i, [_vp, _i, _vp, _sz]),
    "bnk_flows_clear": (_i, [_vp]),
    "bnk_flows_count": (_i, [_vp, C.POINTER(_u64)]),
    "bnk_flows_export": (_i, [_vp, _vp, _sz, C.POINTER(_sz)]),
    "bnk_flows_import": (_i, [_vp, _vp, _sz]),
    "bnk_table_stats_get": (_i, [_vp, C.POINTER(TableStats)]),
    "bnk_batch_create": (_i, [_vp, _u32, _u64, C.POINTER(_vp)]),
    "bnk_batch_destroy": (_i, [_vp]),
    "bnk_batch_view_get": (_i, [_vp, C.POINTER(BatchView)]),
    "bnk_seal_submit": (_i, [_vp, _u32, _u32, _i64]),
    "bnk_open_submit": (_i, [_vp, _u32, _u32, _i64]),
    "bnk_filter_note_submit": (_i, [_vp, _u32, _u32, _i64]),
    "bnk_filter_check_submit": (_i, [_vp, _u32, _u32, _i64]),
    "bnk_addr_set": (_i, [_vp, _vp, C.c_uint16, _u32]),
    "bnk_addr_clear": (_i, [_vp, _vp, C.c_uint16]),
    "bnk_classify_submit": (_i, [_vp, _u32, _u32]),
    "bnk_gso_split_submit": (_i, [_vp, _vp, _u32, _u32, _u32]),
    "bnk_wait": (_i, [_vp, _u64]),
    "bnk_batch_stats_get": (_i, [_vp, C.POINTER(BatchStats)]),
    "bnk_batch_upload": (_i, [_vp, _u32]),
    "bnk_batch_download": (_i, [_vp, _u32]),
    "bnk_assign_counters_noalloc": (_i, [_vp, _vp, _vp, _u32, _vp]),
    "bnk_queue_create": (_i, [_vp, C.POINTER(QueueCfg), C.POINTER(_vp)]),
    "bnk_queue_destroy": (_i, [_vp]),
    "bnk_queue_submit": (_i, [_vp, _vp, _vp, _vp, _u32, _i64, C.POINTER(_u64)]),
    "bnk_queue_wait": (_i, [_vp, _u64, _vp, _vp, _vp, _vp, _vp]),
    "bnk_queue_reserve": (_i, [_vp, _u32, _i64, C.POINTER(_u64), C.POINTER(QueueSpan)]),
    "bnk_queue_commit": (_i, [_vp, _u64]),
    "bnk_queue_wait_span": (_i, [_vp, _u64, C.POINTER(QueueSpan)]),
    "bnk_queue_release": (_i, [_vp, _u64]),
    "bnk_queue_wait_room": (_i, [_vp, _u64]),
    "bnk_queue_stats_get": (_i, [_vp, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "bnk_place_peers": (_i, [_vp, _u32, _u32, _u32, _vp, _vp, _vp]),
    "bnk_mgpu_create": (_i, [C.POINTER(MgpuCfg), C.POINTER(_vp)]),
    "bnk_mgpu_destroy": (_i, [_vp]),
    "bnk_mgpu_last_error_string": (C.c_char_p, [_vp]),
    "bnk_mgpu_ctx": (_vp, [_vp, _u32]),
    "bnk_mgpu_place": (_i, [_vp, _vp]),
    "bnk_mgpu_locate": (_i, [_vp, _u32, C.POINTER(_u32), C.POINTER(_u32)]),
    "bnk_mgpu_peer_set": (_i, [_vp, _u32, _vp, _vp, _u32, _u32, _u32]),
    "bnk_mgpu_peer_clear": (_i, [_vp, _u32]),
    "bnk_mgpu_acl_set": (_i, [_vp, _i, _vp, _sz]),
    "bnk_mgpu_seal": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _i64, _vp, _vp, _vp, _vp]),
    "bnk_mgpu_open": (_i, [_vp, _vp, _vp, _u32, _u32, _i64, _vp, _vp, _vp, _vp, _vp]),
    "bnk_mgpu_loads_get": (_i, [_vp, _vp, _vp, _vp, _i]),
    "bnk_batch_last_kernel_ms": (_i, [_vp, C.POINTER(C.c_float)]),
    "bnk_batch_last_aead_ms": (_i, [_vp, C.POINTER(C.c_float)]),
    "bnk_kernel_launch_count": (_i, [_vp, C.POINTER(_u64)]),
}
# include/bnk_gpu_bench.h, exported by libbnkgpu_bench.so
BENCH_SYMBOLS = {
    "bnk_timer_start": (_i, [_vp, C.POINTER(_vp), _u32]),
    "bnk_timer_stop": (_i, [_vp, C.POINTER(_vp), _u32, C.POINTER(C.c_float)]),
    "bnk_probe_int_throughput": (_i, [_vp, _i, C.POINTER(C.c_double)]),
    "bnk_probe_coissue": (_i, [_vp, _i, _i, C.POINTER(C.c_double)]),
    "bnk_batch_fill_random": (_i, [_vp, _u64]),
    "bnk_batch_copy_only": (_i, [_vp, _u32, _i, _i]),
    "bnk_probe_copy_rounds": (_i, [_vp, _u32, _u64, _u32, _i, C.POINTER(C.c_double)]),
}

_LIB = None
_BENCH_LIB = None


class BnkError(RuntimeError):
    def __init__(self, code: int, detail: str = ""):
        self.code = code
        name = lib().bnk_strerror(code).decode() if _LIB is not None else str(code)
        super().__init__(f"libbnkgpu: {name} ({code}){': ' + detail if detail else ''}")


def lib_path() -> str:
    """Path of the shared library; BNK_B200_LIB points at another build of the same ABI."""
    return os.environ.get("BNK_B200_LIB") or _build.LIB_PATH


def lib() -> C.CDLL:
    """Loads libbnkgpu.so.  Raises if it has not been built: there is no other implementation."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m bnk_b200._build` (needs nvcc). "
            "bnk_b200 has no CPU fallback."
        )
    L = C.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def bench_lib() -> C.CDLL:
    """Loads libbnkgpu_bench.so (timers, probes, device-side fill, copy-only pass) after libbnkgpu.so."""
    global _BENCH_LIB
    if _BENCH_LIB is not None:
        return _BENCH_LIB
    lib()
    path = os.environ.get("BNK_B200_BENCH_LIB") or _build.BENCH_LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m bnk_b200._build` (needs nvcc).")
    L = C.CDLL(path)
    for name, (res, args) in BENCH_SYMBOLS.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _BENCH_LIB = L
    return L


def check(code: int, ctx=None) -> int:
    if code < 0:
        detail = lib().bnk_last_error_string(ctx).decode(errors="replace")
        raise BnkError(code, detail)
    return code
