"""Cluster topology files and the advisor that turns measured link shares into settings.

A topology file is JSON with ``//`` and ``/* */`` comments and trailing commas allowed:

    { "format": "idrak-topology/1",
      "nodes": [ { "name": "a", "address": "10.0.0.1", "gpus": [ { "device": 0, "memory": "180GiB" } ] } ],
      "links": { "intra-node": "nvlink", "inter-node": "tcp",
                 "overrides": [ { "between": ["a", "b"], "type": "rdma", "address": "10.1.0.1" } ] },
      "simulation": { "seed": 1, "failures": "slow-worker" } }

Unknown keys are refused by name; memory sizes need a unit in powers of 1,024 (KiB, MiB, GiB, TiB).

Reference: Topology.cs:103,399 (format, unknown keys), ClusterSettingAdvisor.cs:25 (advice from the exposed network
share of a step).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional

FORMAT = "idrak-topology/1"
_UNITS = {"KIB": 1 << 10, "MIB": 1 << 20, "GIB": 1 << 30, "TIB": 1 << 40}


def strip_json_comments(text: str) -> str:
    """Remove // and /* */ comments and trailing commas, leaving string literals untouched."""
    out, i, n = [], 0, len(text)
    in_str = False
    while i < n:
        c = text[i]
        if in_str:
            out.append(c)
            if c == "\\" and i + 1 < n:
                out.append(text[i + 1])
                i += 1
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True
            out.append(c)
        elif text.startswith("//", i):
            while i < n and text[i] != "\n":
                i += 1
            continue
        elif text.startswith("/*", i):
            end = text.find("*/", i + 2)
            if end < 0:
                raise ValueError("unterminated /* comment")
            i = end + 2
            continue
        else:
            out.append(c)
        i += 1
    return re.sub(r",(\s*[}\]])", r"\1", "".join(out))


def parse_memory(text) -> int:
    if not isinstance(text, str):
        raise ValueError(f"memory size {text!r} needs a unit (KiB, MiB, GiB, TiB)")
    m = re.fullmatch(r"\s*([0-9]+(?:\.[0-9]+)?)\s*([KMGT]iB)\s*", text)
    if not m:
        raise ValueError(f"memory size {text!r}: expected a number and a unit in powers of 1,024 (KiB, MiB, GiB, TiB)")
    return int(float(m.group(1)) * _UNITS[m.group(2).upper()])


def _only(obj: dict, allowed, where: str) -> None:
    if not isinstance(obj, dict):
        raise ValueError(f"{where}: expected an object")
    unknown = sorted(set(obj) - set(allowed))
    if unknown:
        raise ValueError(f"{where}: unknown key{'s' if len(unknown) > 1 else ''} {', '.join(repr(k) for k in unknown)}")


@dataclass
class Gpu:
    device: int
    memory: int


@dataclass
class Node:
    name: str
    address: str
    gpus: List[Gpu] = field(default_factory=list)


@dataclass
class LinkOverride:
    between: List[str]
    type: str
    address: Optional[str] = None


@dataclass
class Topology:
    nodes: List[Node]
    intra_node: str = "nvlink"
    inter_node: str = "tcp"
    overrides: List[LinkOverride] = field(default_factory=list)
    simulation: Dict[str, object] = field(default_factory=dict)

    @property
    def world(self) -> int:
        return sum(len(n.gpus) for n in self.nodes)

    def link_type(self, a: str, b: str) -> str:
        if a == b:
            return self.intra_node
        for o in self.overrides:
            if set(o.between) == {a, b}:
                return o.type
        return self.inter_node

    def ranks(self) -> List[dict]:
        out = []
        for n in self.nodes:
            for g in n.gpus:
                out.append({"rank": len(out), "node": n.name, "address": n.address, "device": g.device, "memory": g.memory})
        return out


def parse_topology(text: str) -> Topology:
    doc = json.loads(strip_json_comments(text))
    _only(doc, ("format", "nodes", "links", "simulation"), "topology")
    if doc.get("format") != FORMAT:
        raise ValueError(f"topology: format is {doc.get('format')!r}, expected '{FORMAT}'")
    nodes = []
    for i, n in enumerate(doc.get("nodes") or []):
        _only(n, ("name", "address", "gpus"), f"nodes[{i}]")
        gpus = []
        for j, g in enumerate(n.get("gpus") or []):
            _only(g, ("device", "memory"), f"nodes[{i}].gpus[{j}]")
            gpus.append(Gpu(int(g["device"]), parse_memory(g.get("memory"))))
        nodes.append(Node(str(n["name"]), str(n.get("address", "127.0.0.1")), gpus))
    if not nodes:
        raise ValueError("topology: no nodes")
    if len({n.name for n in nodes}) != len(nodes):
        raise ValueError("topology: node names must be unique")
    links = doc.get("links") or {}
    _only(links, ("intra-node", "inter-node", "overrides"), "links")
    overrides = []
    for i, o in enumerate(links.get("overrides") or []):
        _only(o, ("between", "type", "address"), f"links.overrides[{i}]")
        overrides.append(LinkOverride(list(o["between"]), str(o["type"]), o.get("address")))
    sim = doc.get("simulation") or {}
    _only(sim, ("seed", "failures"), "simulation")
    return Topology(nodes, links.get("intra-node", "nvlink"), links.get("inter-node", "tcp"), overrides, dict(sim))


def load_topology(path: str) -> Topology:
    with open(path, "r", encoding="utf-8") as f:
        return parse_topology(f.read())


@dataclass
class Advice:
    setting: str
    value: object
    why: str


def advise(step_seconds: float, exposed_network_seconds: float, gradient_bytes: int, link_bandwidth: float,
           link_latency: float = 5e-6, world: int = 8, bucket_bytes: int = 32 << 20, wire: str = "fp32",
           accumulation: int = 1, same_switch: bool = True) -> List[Advice]:
    """Suggestions from how much of a step the network is exposed (not hidden behind compute)."""
    out: List[Advice] = []
    share = exposed_network_seconds / step_seconds if step_seconds > 0 else 0.0
    if share < 0.05:
        return [Advice("none", None, f"the network is exposed for {share:.1%} of the step: nothing to gain")]
    if wire == "fp32":
        out.append(Advice("compression", "bf16", "halves the gradient bytes; sums stay in fp32"))
    transfer = gradient_bytes / max(link_bandwidth, 1.0)
    buckets = max(gradient_bytes // max(bucket_bytes, 1), 1)
    if buckets * link_latency > 0.2 * transfer:
        out.append(Advice("bucket_bytes", int(bucket_bytes * 4), "per-bucket latency is a large part of the transfer"))
    elif buckets < 4 and gradient_bytes > (64 << 20):
        out.append(Advice("bucket_bytes", int(max(bucket_bytes // 4, 1 << 20)), "too few buckets to overlap with backward"))
    if share > 0.3:
        k = max(2, int(round(share / 0.1)))
        out.append(Advice("accumulation", accumulation * 2, "one reduction per two micro-batches halves the exposed share"))
        if not same_switch:
            out.append(Advice("gradient_sync", f"local-sgd every {k}", "slow links: average weights every k steps instead"))
            out.append(Advice("compression", "top-k 1%", "with error feedback, for links far below the compute rate"))
    if not same_switch and world > 8:
        out.append(Advice("collectives", "hierarchical", "reduce inside each node over NVLink first, then between nodes"))
    return out
