"""Policy -> per-node inbound rules -> device allowance table.

Restates, for the host side of the GPU filter, what the reference does per policy change (never per packet):
acl.Compile / parseAllow (internal/acl/acl.go:44-145) on the coordination server, the `filter` / `filter_enabled`
fields of the pushed netmap (internal/netmap/netmap.go:44-53), and the filter part of Engine.ApplyNetmap
(internal/dataplane/engine.go:279-283) on the client.  The result feeds Filter.set_rules, whose flattening builds
the prefix-indexed table the CheckInbound kernel probes.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Iterable

from .filter import CompiledRule, Filter, PortRange


@dataclass
class Rule:
    """acl.Rule: selectors are "*", "group:<name>" or a node name; allow entries "tcp/22", "udp/6000-6100", "icmp"."""
    frm: list
    to: list
    allow: list


@dataclass
class Policy:
    """acl.Policy (the admin-authored document, policy.example.json)."""
    rules: list
    groups: dict = field(default_factory=dict)

    @staticmethod
    def from_json(text: str) -> "Policy":
        doc = json.loads(text)
        return Policy(rules=[Rule(r.get("from", []), r.get("to", []), r.get("allow", [])) for r in doc.get("rules", [])],
                      groups=doc.get("groups", {}) or {})


@dataclass
class NodeInfo:
    name: str
    ip: str


class PolicyError(ValueError):
    """The error Compile returns: the policy is refused as a whole."""


def _parse_u16(text: str, what: str) -> int:
    if not text.isascii() or not text.isdigit():
        raise PolicyError(f"acl: bad port in {what!r}")
    v = int(text)
    if v > 65535:
        raise PolicyError(f"acl: bad port in {what!r}")
    return v


def parse_allow(s: str) -> CompiledRule:
    """parseAllow, acl.go:117-145."""
    proto, sep, spec = s.partition("/")
    if proto == "icmp":
        if sep:
            raise PolicyError(f"acl: icmp takes no port in {s!r}")
        return CompiledRule(srcs=[], proto="icmp", ports=[])
    if proto in ("tcp", "udp"):
        if not sep:
            raise PolicyError(f"acl: {s!r} needs a port like {proto}/22")
        first, dash, last = spec.partition("-")
        lo = _parse_u16(first, s)
        hi = lo
        if dash:
            hi = _parse_u16(last, s)
            if hi < lo:
                raise PolicyError(f"acl: bad port range in {s!r}")
        return CompiledRule(srcs=[], proto=proto, ports=[PortRange(lo, hi)])
    raise PolicyError(f"acl: unknown protocol in {s!r} (want tcp, udp, or icmp)")


def compile_policy(policy: Policy, nodes: Iterable[NodeInfo]) -> dict:
    """acl.Compile, acl.go:44-114: inbound rules keyed by destination node name.  Sources are always /32s, a node
    never appears as a source of its own rules, a destination with no remaining source gets no rule."""
    nodes = list(nodes)
    by_name = {n.name: n for n in nodes}

    def expand(selectors):
        out = {}
        for sel in selectors:
            if sel == "*":
                for n in nodes:
                    out[n.name] = True
            elif sel.startswith("group:"):
                name = sel[len("group:"):]
                if name not in policy.groups:
                    raise PolicyError(f"acl: unknown group {name!r}")
                for m in policy.groups[name]:
                    if m not in by_name:
                        raise PolicyError(f"acl: group {name!r} member {m!r} is not a known node")
                    out[m] = True
            else:
                if sel not in by_name:
                    raise PolicyError(f"acl: {sel!r} is not a known node, group, or *")
                out[sel] = True
        return out

    compiled: dict = {}
    for rule in policy.rules:
        froms, tos = expand(rule.frm), expand(rule.to)
        for dst in tos:
            srcs = [f"{by_name[src].ip}/32" for src in froms if src != dst]
            if not srcs:
                continue
            for allow in rule.allow:
                cr = parse_allow(allow)
                cr.srcs = list(srcs)
                compiled.setdefault(dst, []).append(cr)
    return compiled


def rules_from_netmap(netmap: dict) -> tuple:
    """-> (filter_enabled, [CompiledRule]) from a pushed netmap document (netmap.go:44-53)."""
    rules = []
    for r in netmap.get("filter") or []:
        rules.append(CompiledRule(srcs=list(r.get("srcs") or []), proto=r.get("proto", ""),
                                  ports=[PortRange(int(p["first"]), int(p["last"])) for p in (r.get("ports") or [])]))
    return bool(netmap.get("filter_enabled", False)), rules


def rules_to_netmap(rules: Iterable[CompiledRule]) -> list:
    """The JSON shape of acl.CompiledRule (acl.go:33-42)."""
    out = []
    for r in rules:
        d = {"srcs": list(r.srcs), "proto": r.proto}
        if r.ports:
            d["ports"] = [{"first": p.first, "last": p.last} for p in r.ports]
        out.append(d)
    return out


def apply_netmap_filter(f: Filter, netmap: dict) -> None:
    """The filter part of Engine.ApplyNetmap, engine.go:279-283: an active policy enforces its rules (an empty
    list means deny all inbound but replies), no policy means allow all.  The device table is rebuilt and swapped
    between batches; reply flows are kept."""
    enabled, rules = rules_from_netmap(netmap)
    if enabled:
        f.set_rules(rules)
    else:
        f.set_allow_all()
