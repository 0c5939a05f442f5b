"""Pins the CPU checker's filter against every case of the reference's own filter / ACL tests."""
import numpy as np
import pytest

from bnk_b200.filter import _prefix
from tests import reference_cases as RC


class OracleFilterAdapter:
    """Gives the CPU checker the reference's interface (rules as CompiledRule objects)."""

    def __init__(self, O):
        self.O = O
        self.f = O.Filter()

    def set_rules(self, rules):
        conv = []
        for r in rules:
            srcs = []
            for s in r.srcs:
                p = _prefix(s)
                srcs.append(p if p is not None else (0, -1))
            conv.append((srcs, r.proto, [(p.first, p.last) for p in r.ports]))
        self.f.set_rules(conv)

    def set_allow_all(self):
        self.f.set_allow_all()

    def check_inbound(self, pkt, now):
        return self.f.check_inbound(pkt, now)

    def note_outbound(self, pkt, now):
        self.f.note_outbound(pkt, now)


@pytest.mark.parametrize("case", RC.ALL_CASES, ids=lambda c: c.__name__)
def test_reference_cases(oracle, case):
    case(lambda: OracleFilterAdapter(oracle))


def test_sweep_above_4096_flows(oracle):
    """filter.go:202-208: once more than 4096 flows exist, a NoteOutbound sweeps the expired ones."""
    f = oracle.Filter()
    f.set_rules([])
    for i in range(4096):
        f.note_outbound(RC.udp(RC.SELF, RC.PEER, 1 + i, 7), RC.T0)
    assert f.flow_count == 4096
    f.note_outbound(RC.udp(RC.SELF, RC.PEER, 5000, 7), RC.T0 + 10 * RC.SEC)  # 4097 live, nothing expired yet
    assert f.flow_count == 4097
    f.note_outbound(RC.udp(RC.SELF, RC.PEER, 5001, 7), RC.T0 + 31 * RC.SEC)  # the first 4096 have expired
    assert f.flow_count == 2
    assert not f.check_inbound(RC.udp(RC.PEER, RC.SELF, 7, 1), RC.T0 + 5 * RC.SEC)  # swept, even at an earlier clock


def test_parse_fields(oracle):
    out = (np.zeros(6, np.uint32))
    pkt = RC.tcp(RC.PEER, RC.SELF, 0x1234, 0x5678)
    import ctypes

    assert oracle.lib().bnko_filter_parse(pkt, len(pkt), out.ctypes.data_as(ctypes.c_void_p)) == 1
    assert list(out) == [6, RC.PEER, RC.SELF, 0x1234, 0x5678, 0]


def test_threaded_batch_check_equals_the_sequential_one(oracle):
    """The full-size GPU comparisons use check_batch_mt (rule walk on all cores); it must be the same function."""
    import numpy as np

    from bnk_b200 import gen

    w = gen.config3(300, 800, 3000, 9000, seed=123)

    def fresh():
        f = oracle.Filter()
        f.set_rules_arrays(w.rules.astype(oracle.RULE_DTYPE), w.srcs.astype(oracle.PREFIX_DTYPE),
                           w.ports.astype(oracle.PORT_DTYPE))
        f.note_batch(np.ascontiguousarray(w.outbound), 28, w.outbound_len, w.t0_ns)
        return f

    a, b = fresh(), fresh()
    for hdr, lens, now in ((w.inbound, w.inbound_len, w.t0_ns + 10**9), (w.late, w.late_len, w.t0_ns + 600 * 10**9),
                           (w.late, w.late_len, w.t0_ns + 2 * 10**9)):
        va = a.check_batch(np.ascontiguousarray(hdr), 28, np.ascontiguousarray(lens), now)
        vb = b.check_batch_mt(np.ascontiguousarray(hdr), 28, np.ascontiguousarray(lens), now, threads=3)
        assert np.array_equal(va, vb)
        assert a.flow_count == b.flow_count
    allow = oracle.Filter()
    assert allow.check_batch_mt(np.ascontiguousarray(w.inbound), 28, np.ascontiguousarray(w.inbound_len), 0).all()
