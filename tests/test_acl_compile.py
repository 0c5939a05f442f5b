"""acl.Compile restated on the host side: the reference's own cases (internal/acl/acl_test.go:15-81) and the path
from a policy document to the flattened device table."""
import json

import pytest

from bnk_b200 import acl
from bnk_b200.filter import flatten_rules

NODES = [acl.NodeInfo("laptop", "100.64.0.1"), acl.NodeInfo("desktop", "100.64.0.2"), acl.NodeInfo("nas", "100.64.0.3")]


def test_compile_group_rule_produces_inbound_rules_for_targets():  # acl_test.go:15-42
    p = acl.Policy(groups={"trusted": ["laptop", "desktop"], "servers": ["nas"]},
                   rules=[acl.Rule(["group:trusted"], ["group:servers"], ["tcp/22", "tcp/443", "icmp"])])
    compiled = acl.compile_policy(p, NODES)
    nas = compiled["nas"]
    assert len(nas) == 3
    assert all(len(r.srcs) == 2 for r in nas)
    assert not compiled.get("laptop") and not compiled.get("desktop")


def test_compile_wildcard_and_port_range():  # acl_test.go:44-68
    p = acl.Policy(rules=[acl.Rule(["*"], ["nas"], ["udp/6000-6100"])])
    rules = acl.compile_policy(p, NODES)["nas"]
    assert len(rules) == 1
    r = rules[0]
    assert r.proto == "udp" and [(q.first, q.last) for q in r.ports] == [(6000, 6100)]
    assert sorted(r.srcs) == ["100.64.0.1/32", "100.64.0.2/32"]  # every node but the destination itself


def test_compile_rejects_unknown_group_and_bad_port():  # acl_test.go:70-81
    with pytest.raises(acl.PolicyError, match="nope"):
        acl.compile_policy(acl.Policy(rules=[acl.Rule(["group:nope"], ["nas"], ["tcp/22"])]), NODES)
    with pytest.raises(acl.PolicyError):
        acl.compile_policy(acl.Policy(rules=[acl.Rule(["*"], ["nas"], ["tcp/notaport"])]), NODES)
    with pytest.raises(acl.PolicyError):
        acl.compile_policy(acl.Policy(rules=[acl.Rule(["ghost"], ["nas"], ["tcp/22"])]), NODES)
    for bad in ["icmp/1", "tcp", "udp/70000", "tcp/10-5", "sctp/5", "tcp/-1", "tcp/22-"]:
        with pytest.raises(acl.PolicyError):
            acl.parse_allow(bad)


def test_policy_document_to_device_table():
    doc = json.dumps({"groups": {"trusted": ["laptop", "desktop"], "servers": ["nas"]},
                      "rules": [{"from": ["group:trusted"], "to": ["group:servers"], "allow": ["tcp/22", "tcp/443", "icmp"]},
                                {"from": ["*"], "to": ["*"], "allow": ["icmp"]}]})
    compiled = acl.compile_policy(acl.Policy.from_json(doc), NODES)
    assert len(compiled["nas"]) == 4 and len(compiled["laptop"]) == 1
    netmap = {"filter_enabled": True, "filter": acl.rules_to_netmap(compiled["nas"])}
    enabled, rules = acl.rules_from_netmap(json.loads(json.dumps(netmap)))
    assert enabled and len(rules) == 4
    t = flatten_rules(rules)
    # tcp/22 and tcp/443 from two sources, icmp from two sources, twice (both policy rules grant it)
    assert len(t) == 2 * 2 + 2 + 2
    assert sorted(set(int(p) for p in t["proto"])) == [1, 6]
    assert acl.rules_from_netmap({}) == (False, [])
    assert acl.rules_from_netmap({"filter_enabled": True}) == (True, [])  # active policy, no rule: deny all inbound
