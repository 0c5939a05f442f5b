"""ACL filter parity on the GPU: the reference's own cases through the Python mirror of its
interface, and configuration 3 against the CPU checker, verdict for verdict."""
import numpy as np
import pytest

from tests import reference_cases as RC

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(gpu_lib):
    from bnk_b200 import Context

    c = Context(max_keypairs=4, flow_capacity=1 << 14)
    yield c
    c.close()


@pytest.fixture()
def make(ctx):
    from bnk_b200.filter import Filter

    made = []

    def _make():
        ctx.flows_clear()
        f = Filter(ctx, batch_pkts=8)
        made.append(f)
        return f

    yield _make
    for f in made:
        f._batch.close()


@pytest.mark.parametrize("case", RC.ALL_CASES, ids=lambda c: c.__name__)
def test_reference_cases(make, case):
    case(make)


def test_wrap_tun_cases(make):
    from bnk_b200.filter import wrap_tun

    RC.tun_case_drops_denied_inbound_writes(make, wrap_tun)
    RC.tun_case_read_records_outbound_flows(make, wrap_tun)


def _load_headers(b, hdr, lens):
    from bnk_b200 import gen

    n = len(lens)
    stride = gen.HDR_STRIDE
    view = b.ring[:n * stride].reshape(n, stride)
    view[:, 16:16 + hdr.shape[1]] = hdr
    b.off[:n] = (np.arange(n, dtype=np.uint64) * stride).astype(np.uint32)
    b.len[:n] = lens
    return n


def _run_config3(oracle, n_rules, n_nodes, n_out, n_in, seed=None, flow_capacity=1 << 20):
    """Every verdict of the inbound batch, of a late batch after the TTLs have run out and of the same batch
    again, and the flow count, against the CPU checker (whose rule walk runs on all host cores)."""
    from bnk_b200 import Context, gen
    from bnk_b200.device import F_STATS, PKT_FILTER_DENY, PKT_OK
    from bnk_b200.filter import flatten_rule_arrays

    w = gen.config3(n_rules, n_nodes, n_out, n_in, seed=seed)
    # CPU checker
    f = oracle.Filter()
    f.set_rules_arrays(w.rules.astype(oracle.RULE_DTYPE), w.srcs.astype(oracle.PREFIX_DTYPE),
                       w.ports.astype(oracle.PORT_DTYPE))
    f.note_batch(np.ascontiguousarray(w.outbound), 28, w.outbound_len, w.t0_ns)
    want = f.check_batch_mt(np.ascontiguousarray(w.inbound), 28, np.ascontiguousarray(w.inbound_len), w.t0_ns + RC.SEC)
    want_late = f.check_batch_mt(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 10 * RC.MIN)
    want_again = f.check_batch_mt(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 2 * RC.SEC)
    want_flows = f.flow_count
    # GPU
    c = Context(max_keypairs=4, flow_capacity=flow_capacity)
    try:
        c.acl_set(True, flatten_rule_arrays(w.rules, w.srcs, w.ports))
        cap = max(n_out, n_in)
        b = c.batch(cap, cap * gen.HDR_STRIDE)
        n = _load_headers(b, w.outbound, w.outbound_len)
        b.filter_note(n, w.t0_ns)
        n = _load_headers(b, w.inbound, w.inbound_len)
        b.filter_check(n, w.t0_ns + RC.SEC, F_STATS)
        got = (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)
        stats = b.stats()
        assert stats["packets"] == n and stats["by_status"][PKT_OK] == int(got.sum())
        assert stats["by_status"][PKT_FILTER_DENY] == n - int(got.sum())
        n = _load_headers(b, w.late, w.late_len)
        b.filter_check(n, w.t0_ns + 10 * RC.MIN)
        got_late = (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)
        b.filter_check(n, w.t0_ns + 2 * RC.SEC)
        got_again = (np.array(b.status[:n]) == PKT_OK).astype(np.uint8)
        got_flows = c.flows_count()
        got_table = c.flows_export()
    finally:
        c.close()
    assert np.array_equal(got, want), f"{np.flatnonzero(got != want)[:10]} differ"
    assert np.array_equal(got_late, want_late)
    assert np.array_equal(got_again, want_again)
    assert got_flows == want_flows
    # not only the verdicts: the whole flow table, key for key and expiry for expiry, equals the checker's map
    from tests.helpers import flows_equal

    assert len(got_table) == want_flows and flows_equal(got_table, f.flows())
    return w, got, want_late


def test_config3_small(oracle):
    w, want, late = _run_config3(oracle, 500, 2000, 6000, 20000, seed=77, flow_capacity=1 << 14)
    assert 0.25 < want.mean() < 0.9      # both verdicts well represented
    assert late.sum() < len(late)        # replies whose flow ran out are refused


def test_config3_full_size(oracle):
    """BASELINE configuration 3 at its stated size: 10,000 rules, 300,000 noted flows, 1,000,000 inbound
    headers; all 1,000,000 verdicts, the late batch and the flow count equal the CPU checker's."""
    w, got, late = _run_config3(oracle, 10_000, 50_000, 300_000, 1_000_000)
    assert len(got) == 1_000_000 and got.sum() > 300_000
    # size-independent properties over all 1,000,000 verdicts: malformed headers never pass ...
    # (a header cut to 22 bytes still parses when it is icmp, which needs one body byte only)
    bad = ((w.inbound_len < 24) & (w.inbound[:, 9] != 1)) | (w.inbound[:, 0] != 0x45) | ~np.isin(w.inbound[:, 9], (1, 6, 17))
    assert bad.sum() > 40_000 and got[bad].sum() == 0
    # ... and every exact mirror of a noted flow passes while its TTL runs
    reply = np.zeros(len(got), bool)
    key_out = {bytes(h[9:10]) + bytes(h[16:20]) + bytes(h[22:24]) + bytes(h[20:22]) for h in w.outbound[::7]}
    for i in range(0, len(got), 97):
        h = w.inbound[i]
        if not bad[i] and bytes(h[9:10]) + bytes(h[12:16]) + bytes(h[20:24]) in key_out:
            reply[i] = True
    assert reply.sum() > 100 and got[reply].all()


def test_flow_sweep_and_count(ctx):
    """filter.go:202-208 through the batch path: counts and the >4096 sweep follow the reference."""
    from bnk_b200.filter import Filter

    ctx.flows_clear()
    f = Filter(ctx, batch_pkts=5000)
    f.set_rules([])
    f.note_outbound_batch([RC.udp(RC.SELF, RC.PEER, 1 + i, 7) for i in range(4096)], RC.T0)
    assert ctx.flows_count() == 4096
    f.note_outbound(RC.udp(RC.SELF, RC.PEER, 5000, 7), RC.T0 + 10 * RC.SEC)
    assert ctx.flows_count() == 4097
    f.note_outbound(RC.udp(RC.SELF, RC.PEER, 5001, 7), RC.T0 + 31 * RC.SEC)
    assert ctx.flows_count() == 2
    assert not f.check_inbound(RC.udp(RC.PEER, RC.SELF, 7, 1), RC.T0 + 5 * RC.SEC)
    # duplicates inside one batch count once; the all-ones key has its own slot
    ctx.flows_clear()
    f.note_outbound_batch([RC.udp(RC.SELF, RC.PEER, 9, 9)] * 100 + [RC.udp(RC.SELF, 0xFFFFFFFF, 65535, 65535)] * 3, RC.T0)
    assert ctx.flows_count() == 2
    assert f.check_inbound(RC.udp(0xFFFFFFFF, RC.SELF, 65535, 65535), RC.T0 + RC.SEC)
    assert not f.check_inbound(RC.tcp(0xFFFFFFFF, RC.SELF, 65535, 65535), RC.T0 + RC.SEC)
    f._batch.close()


def test_flow_table_full_is_reported(gpu_lib):
    from bnk_b200 import Context
    from bnk_b200.device import BnkError
    from bnk_b200.filter import Filter

    c = Context(max_keypairs=4, flow_capacity=16)
    try:
        f = Filter(c, batch_pkts=64)
        f.set_rules([])
        with pytest.raises(BnkError) as e:
            f.note_outbound_batch([RC.udp(RC.SELF, RC.PEER, 1 + i, 7) for i in range(40)], RC.T0)
        assert e.value.code == -6
    finally:
        c.close()


def test_policy_to_verdicts_end_to_end(make):
    """Policy document -> Compile -> netmap -> ApplyNetmap -> GPU verdicts, the route of the reference's
    internal/dataplane/acl_integration_test.go:20-80 (tcp/7777 allowed, tcp/8888 blocked, replies pass)."""
    from bnk_b200 import acl

    nodes = [acl.NodeInfo("a", "100.64.0.1"), acl.NodeInfo("b", "100.64.0.2"), acl.NodeInfo("c", "100.64.0.3")]
    policy = acl.Policy(rules=[acl.Rule(["a"], ["b"], ["tcp/7777"])])
    compiled = acl.compile_policy(policy, nodes)
    a, b, c = RC.ip("100.64.0.1"), RC.ip("100.64.0.2"), RC.ip("100.64.0.3")
    f = make()
    acl.apply_netmap_filter(f, {"filter_enabled": True, "filter": acl.rules_to_netmap(compiled.get("b", []))})
    assert f.check_inbound(RC.tcp(a, b, 40000, 7777), RC.T0)
    assert not f.check_inbound(RC.tcp(a, b, 40000, 8888), RC.T0)
    assert not f.check_inbound(RC.tcp(c, b, 40000, 7777), RC.T0)
    # node a has no inbound rule at all under this policy: deny all but replies to what it opened
    acl.apply_netmap_filter(f, {"filter_enabled": True, "filter": acl.rules_to_netmap(compiled.get("a", []))})
    assert not f.check_inbound(RC.tcp(b, a, 7777, 40000, False), RC.T0)
    f.note_outbound(RC.tcp(a, b, 40000, 7777), RC.T0)
    assert f.check_inbound(RC.tcp(b, a, 7777, 40000, False), RC.T0 + RC.SEC)
    # the policy is withdrawn: allow all (flows are kept, rules are gone)
    acl.apply_netmap_filter(f, {"filter_enabled": False})
    assert f.check_inbound(RC.tcp(c, a, 1, 2), RC.T0)


def test_flow_table_export_and_import(gpu_lib, oracle):
    """State hand-over: the entries exported from one context, imported into a fresh one, give the same verdicts
    and the same table there (all three protocol classes, the all-ones key, a deleted entry is not exported)."""
    from bnk_b200 import Context
    from bnk_b200.filter import Filter
    from tests.helpers import flows_equal

    a = Context(max_keypairs=4, flow_capacity=1 << 10)
    b = Context(max_keypairs=4, flow_capacity=1 << 12)
    o = oracle.Filter()
    o.set_rules([])
    try:
        fa, fb = Filter(a, batch_pkts=64), Filter(b, batch_pkts=64)
        fa.set_rules([])
        fb.set_rules([])
        out = ([RC.udp(RC.SELF, RC.PEER, 1000 + i, 53) for i in range(20)] + [RC.tcp(RC.SELF, RC.OTHER, 2000 + i, 443) for i in range(20)]
               + [RC.icmp_echo(RC.SELF, RC.PEER, False), RC.udp(RC.SELF, 0xFFFFFFFF, 65535, 65535)])
        fa.note_outbound_batch(out, RC.T0)
        for p in out:
            o.note_outbound(p, RC.T0)
        # one udp flow runs out and is deleted by a lookup
        late = RC.udp(RC.PEER, RC.SELF, 53, 1000)
        assert not fa.check_inbound(late, RC.T0 + 31 * RC.SEC) and not o.check_inbound(late, RC.T0 + 31 * RC.SEC)
        table = a.flows_export()
        assert len(table) == 41 and flows_equal(table, o.flows())
        b.flows_import(table)
        assert b.flows_count() == 41 and flows_equal(b.flows_export(), o.flows())
        for pkt, want in ((RC.udp(RC.PEER, RC.SELF, 53, 1001), True), (late, False),
                          (RC.tcp(RC.OTHER, RC.SELF, 443, 2005, False), True), (RC.icmp_echo(RC.PEER, RC.SELF, True), True),
                          (RC.udp(0xFFFFFFFF, RC.SELF, 65535, 65535), True), (RC.tcp(RC.OTHER, RC.SELF, 443, 2999, False), False)):
            assert fb.check_inbound(pkt, RC.T0 + RC.SEC) == want == o.check_inbound(pkt, RC.T0 + RC.SEC)
        assert flows_equal(b.flows_export(), o.flows())  # the refreshed expiries too
        b.flows_import(table[:3])                         # importing a key again only moves its expiry
        assert b.flows_count() == 41
        fa._batch.close()
        fb._batch.close()
    finally:
        a.close()
        b.close()


@pytest.mark.parametrize("shape", ["few_lengths_listed", "many_keys_per_length", "everything_listed", "default_route"])
def test_rule_tables_with_many_prefix_lengths(gpu_lib, oracle, shape):
    """Rule tables with several prefix lengths in very different numbers: every verdict equals the checker's rule
    walk (acl.go:149-172: any prefix of any length that contains the source, filter.go:131-135).  Shapes: a handful
    of hand-written prefixes beside thousands of /32s; hundreds of keys in each of four lengths; only a few prefixes;
    a /0 rule.  (The index probes one hash table per prefix length in use; a variant that kept the rare lengths in a
    short list in shared memory passed the same test and was no faster.)"""
    from bnk_b200 import Context
    from bnk_b200.filter import Filter, CompiledRule, PortRange

    rng = np.random.default_rng({"few_lengths_listed": 1, "many_keys_per_length": 2, "everything_listed": 3,
                                 "default_route": 4}[shape])
    base = RC.ip("100.64.0.0")

    def host(k):
        return base + int(k)

    def pfx(addr, bits):
        import ipaddress
        return f"{ipaddress.ip_address(addr & ((0xffffffff << (32 - bits)) & 0xffffffff) if bits else 0)}/{bits}"

    rules = []
    if shape in ("few_lengths_listed", "default_route"):
        for k in rng.integers(1, 1 << 20, 3000):
            rules.append(CompiledRule(srcs=[pfx(host(k), 32)], proto=str(rng.choice(["tcp", "udp"])),
                                      ports=[PortRange(1, int(rng.integers(1, 40000)))]))
        for bits in (8, 12, 16, 20, 24, 28, 30):
            for _ in range(int(rng.integers(1, 6))):
                rules.append(CompiledRule(srcs=[pfx(host(rng.integers(1, 1 << 20)), bits)], proto="udp",
                                          ports=[PortRange(50, 60)]))
        if shape == "default_route":
            rules.append(CompiledRule(srcs=["0.0.0.0/0"], proto="icmp", ports=[]))
    elif shape == "many_keys_per_length":
        for bits in (24, 26, 28, 32):
            for k in rng.integers(1, 1 << 20, 400):
                rules.append(CompiledRule(srcs=[pfx(host(k), bits)], proto="tcp", ports=[PortRange(1000, 2000)]))
    else:
        for bits in (10, 16, 24, 32):
            for _ in range(5):
                rules.append(CompiledRule(srcs=[pfx(host(rng.integers(1, 1 << 20)), bits)], proto="tcp",
                                          ports=[PortRange(22, 22), PortRange(80, 90)]))
    c = Context(max_keypairs=4, flow_capacity=1 << 10)
    try:
        f = Filter(c, batch_pkts=4096)
        f.set_rules(rules)
        chk = oracle.Filter()
        chk.set_rules([([(RC.ip(s.split("/")[0]), int(s.split("/")[1])) for s in r.srcs], r.proto,
                        [(p.first, p.last) for p in r.ports]) for r in rules])
        # sources: half of them taken from the rules' own prefixes (inside and just outside), half anywhere
        pool = [RC.ip(s.split("/")[0]) for r in rules for s in r.srcs]
        pkts = []
        for k in range(4096):
            src = int(pool[int(rng.integers(0, len(pool)))]) + int(rng.integers(0, 3)) if k % 2 else host(rng.integers(1, 1 << 20))
            src &= 0xffffffff
            kind = int(rng.integers(0, 3))
            port = int(rng.choice([22, 55, 85, 1500, 30000, int(rng.integers(1, 65535))]))
            if kind == 0:
                pkts.append(RC.tcp(src, RC.SELF, 40000, port))
            elif kind == 1:
                pkts.append(RC.udp(src, RC.SELF, 40000, port))
            else:
                pkts.append(RC.icmp_echo(src, RC.SELF, False))
        got = f.check_inbound_batch(pkts, RC.T0)
        want = [chk.check_inbound(p, RC.T0) for p in pkts]
        assert got == want
        assert 50 < sum(want) < 4000
        f._batch.close()
    finally:
        c.close()
