"""The machine as a graph: nodes (machine, CPU packages, NUMA nodes, memory domains, accelerators, interconnect
endpoints) and typed links (contains, affine-to, peer-access, interconnect) that may carry transfer metrics with their
provenance (reported by the platform, measured here, or declared). ``validate`` refuses duplicate node ids and links to
missing nodes. ``probe_host_topology`` reads NUMA nodes, their CPUs and memory from sysfs; ``augment_accelerators`` adds
one accelerator node per GPU with its HBM domain, its NUMA affinity and peer links (NVLink through NVSwitch when every
pair can reach every other: one switch endpoint, 900 GB/s per direction per GPU declared). ``nvswitch_declared`` builds
the 8 x B200 node without a device for planning. ``canonical_topology_profile_bytes`` is the stable encoding.
Reference counterpart: scirust-compute/src/{topology,topology_probe,topology_augmentation,topology_provider,
profile_encoding}.rs.
"""
from __future__ import annotations

import enum
import glob
import os
from dataclasses import dataclass, field

from .contracts import DeviceId, MemorySpace
from .hardware import SupportLevel


class TopologyError(ValueError):
    pass


class NodeKind(enum.Enum):
    MACHINE = "machine"
    CPU_PACKAGE = "cpu-package"
    NUMA_NODE = "numa-node"
    PROCESSING_UNIT = "processing-unit"
    CACHE = "cache"
    MEMORY_DOMAIN = "memory-domain"
    ACCELERATOR = "accelerator"
    INTERCONNECT_ENDPOINT = "interconnect-endpoint"
    OTHER = "other"


class Relation(enum.Enum):
    CONTAINS = "contains"
    AFFINE_TO = "affine-to"
    PEER_ACCESS = "peer-access"
    COHERENT_WITH = "coherent-with"
    INTERCONNECT = "interconnect"


class InterconnectClass(enum.Enum):
    ON_CHIP = "on-chip"
    HOST_MEMORY_BUS = "host-memory-bus"
    PCIE = "pcie"
    HIGH_SPEED_PEER = "high-speed-peer"
    NETWORK_FABRIC = "network-fabric"
    OTHER = "other"


class MetricProvenance(enum.Enum):
    REPORTED = "reported"
    MEASURED = "measured"
    DECLARED = "declared"


@dataclass(frozen=True)
class TransferMetrics:
    bandwidth_bytes_per_second: int | None
    latency_nanoseconds: int | None
    provenance: MetricProvenance


@dataclass(frozen=True)
class CacheDescriptor:
    level: int
    size_bytes: int | None = None
    line_bytes: int | None = None


@dataclass(frozen=True)
class MemoryDomainDescriptor:
    space: MemorySpace
    capacity_bytes: int | None = None
    host_addressable: SupportLevel = SupportLevel.UNKNOWN


@dataclass
class TopologyNode:
    id: int
    kind: NodeKind
    name: str | None = None
    device: DeviceId | None = None
    cache: CacheDescriptor | None = None
    memory: MemoryDomainDescriptor | None = None


@dataclass
class TopologyLink:
    source: int
    to: int
    relation: Relation
    bidirectional: bool = False
    interconnect: InterconnectClass | None = None
    metrics: TransferMetrics | None = None


@dataclass
class SystemTopology:
    nodes: list = field(default_factory=list)
    links: list = field(default_factory=list)

    def validate(self) -> None:
        seen = set()
        for n in self.nodes:
            if n.id in seen:
                raise TopologyError(f"duplicate node id {n.id}")
            seen.add(n.id)
        for l in self.links:
            for end in (l.source, l.to):
                if end not in seen:
                    raise TopologyError(f"link endpoint {end} is not a node")

    def contains_node(self, i: int) -> bool:
        return any(n.id == i for n in self.nodes)

    def node(self, i: int):
        return next((n for n in self.nodes if n.id == i), None)

    def links_from(self, i: int):
        return [l for l in self.links if l.source == i]

    def adjacent_links(self, i: int):
        return [l for l in self.links if l.source == i or (l.bidirectional and l.to == i)]

    def next_id(self) -> int:
        return max((n.id for n in self.nodes), default=-1) + 1

    def accelerators(self):
        return [n for n in self.nodes if n.kind is NodeKind.ACCELERATOR]

    def peer_bandwidth(self, a: DeviceId, b: DeviceId):
        """Declared / measured bytes per second between two accelerators (direct link or through one switch)."""
        ia = next((n.id for n in self.accelerators() if n.device == a), None)
        ib = next((n.id for n in self.accelerators() if n.device == b), None)
        if ia is None or ib is None:
            return None
        for l in self.adjacent_links(ia):
            other = l.to if l.source == ia else l.source
            if other == ib and l.metrics:
                return l.metrics.bandwidth_bytes_per_second
            if self.node(other).kind is NodeKind.INTERCONNECT_ENDPOINT and l.metrics:
                if any((m.to if m.source == other else m.source) == ib for m in self.adjacent_links(other)):
                    return l.metrics.bandwidth_bytes_per_second
        return None


def _read(path, default=None):
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return default


def _cpulist(s: str):
    out = []
    for part in (s or "").split(","):
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        elif part.strip():
            out.append(int(part))
    return out


def probe_host_topology(sysfs: str = "/sys/devices/system/node") -> SystemTopology:
    t = SystemTopology([TopologyNode(0, NodeKind.MACHINE, os.uname().nodename if hasattr(os, "uname") else None)])
    numa_dirs = sorted(glob.glob(os.path.join(sysfs, "node[0-9]*")), key=lambda p: int(p.rsplit("node", 1)[1]))
    if not numa_dirs:
        numa_dirs = [None]
    for d in numa_dirs:
        nid = t.next_id()
        idx = 0 if d is None else int(d.rsplit("node", 1)[1])
        t.nodes.append(TopologyNode(nid, NodeKind.NUMA_NODE, f"numa{idx}"))
        t.links.append(TopologyLink(0, nid, Relation.CONTAINS))
        cap = None
        if d is not None:
            for line in (_read(os.path.join(d, "meminfo"), "") or "").splitlines():
                if "MemTotal" in line:
                    cap = int(line.split()[-2]) * 1024
        mid = t.next_id()
        t.nodes.append(TopologyNode(mid, NodeKind.MEMORY_DOMAIN, f"dram{idx}",
                                    memory=MemoryDomainDescriptor(MemorySpace.HOST, cap, SupportLevel.SUPPORTED)))
        t.links.append(TopologyLink(nid, mid, Relation.AFFINE_TO, True, InterconnectClass.HOST_MEMORY_BUS))
        cpus = _cpulist(_read(os.path.join(d, "cpulist"))) if d is not None else list(range(os.cpu_count() or 1))
        if cpus:
            pid = t.next_id()
            t.nodes.append(TopologyNode(pid, NodeKind.PROCESSING_UNIT, f"cpus {cpus[0]}-{cpus[-1]} ({len(cpus)})"))
            t.links.append(TopologyLink(nid, pid, Relation.CONTAINS))
    t.validate()
    return t


@dataclass(frozen=True)
class AcceleratorDescriptor:
    device: DeviceId
    name: str
    memory_bytes: int | None
    numa_index: int | None = None
    peers: tuple = ()                       # device ordinals reachable by load / store


NVLINK5_BYTES_PER_SECOND = 900 * 10 ** 9


def augment_accelerators(t: SystemTopology, accelerators, switch: bool | None = None) -> dict:
    """Adds the accelerators to ``t``; returns {device: node id}. ``switch`` None = one switch endpoint iff every
    accelerator reaches every other."""
    ids = {}
    numa = [n for n in t.nodes if n.kind is NodeKind.NUMA_NODE]
    for a in accelerators:
        if any(n.device == a.device for n in t.nodes):
            raise TopologyError(f"accelerator {a.device.record()} is already in the topology")
        nid = t.next_id()
        t.nodes.append(TopologyNode(nid, NodeKind.ACCELERATOR, a.name, a.device))
        mid = t.next_id()
        t.nodes.append(TopologyNode(mid, NodeKind.MEMORY_DOMAIN, f"hbm:{a.device.ordinal}",
                                    memory=MemoryDomainDescriptor(MemorySpace.DEVICE, a.memory_bytes, SupportLevel.UNSUPPORTED)))
        t.links.append(TopologyLink(nid, mid, Relation.AFFINE_TO, True, InterconnectClass.ON_CHIP))
        host = numa[a.numa_index] if a.numa_index is not None and a.numa_index < len(numa) else (numa[0] if numa else t.nodes[0])
        t.links.append(TopologyLink(host.id, nid, Relation.AFFINE_TO, True, InterconnectClass.PCIE))
        ids[a.device] = nid
    ords = {a.device.ordinal for a in accelerators}
    full = len(accelerators) > 1 and all(set(a.peers) >= ords - {a.device.ordinal} for a in accelerators)
    if switch is None:
        switch = full
    m = TransferMetrics(NVLINK5_BYTES_PER_SECOND, None, MetricProvenance.DECLARED)
    if switch and len(accelerators) > 1:
        sid = t.next_id()
        t.nodes.append(TopologyNode(sid, NodeKind.INTERCONNECT_ENDPOINT, "nvswitch"))
        for a in accelerators:
            t.links.append(TopologyLink(ids[a.device], sid, Relation.INTERCONNECT, True, InterconnectClass.HIGH_SPEED_PEER, m))
    else:
        done = set()
        for a in accelerators:
            for p in a.peers:
                pd = next((b.device for b in accelerators if b.device.ordinal == p), None)
                if pd is not None and (p, a.device.ordinal) not in done:
                    t.links.append(TopologyLink(ids[a.device], ids[pd], Relation.PEER_ACCESS, True, InterconnectClass.HIGH_SPEED_PEER, m))
                    done.add((a.device.ordinal, p))
    t.validate()
    return ids


def probe_cuda_accelerators():
    import torch
    out = []
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        peers = tuple(j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j))
        out.append(AcceleratorDescriptor(DeviceId.cuda(i), p.name, p.total_memory, None, peers))
    return out


def probe_system_topology() -> SystemTopology:
    t = probe_host_topology()
    acc = probe_cuda_accelerators()
    if acc:
        augment_accelerators(t, acc)
    return t


def nvswitch_declared(n_gpus: int = 8, numa_nodes: int = 2) -> SystemTopology:
    t = SystemTopology([TopologyNode(0, NodeKind.MACHINE, "hgx-b200")])
    for k in range(numa_nodes):
        t.nodes.append(TopologyNode(k + 1, NodeKind.NUMA_NODE, f"numa{k}"))
        t.links.append(TopologyLink(0, k + 1, Relation.CONTAINS))
    acc = [AcceleratorDescriptor(DeviceId.cuda(i), "NVIDIA B200", 180 * 10 ** 9, i * numa_nodes // n_gpus,
                                 tuple(j for j in range(n_gpus) if j != i)) for i in range(n_gpus)]
    augment_accelerators(t, acc)
    return t


def canonical_topology_profile_bytes(t: SystemTopology) -> bytes:
    t.validate()
    rows = [b"scirust-b200-topology-v1"]
    for n in sorted(t.nodes, key=lambda n: n.id):
        mem = "" if n.memory is None else f"{n.memory.space.value}:{n.memory.capacity_bytes}:{n.memory.host_addressable.value}"
        rows.append(f"n{n.id};{n.kind.value};{n.device.record() if n.device else ''};{mem}".encode())
    for l in sorted(t.links, key=lambda l: (l.source, l.to, l.relation.value)):
        met = "" if l.metrics is None else f"{l.metrics.bandwidth_bytes_per_second}:{l.metrics.latency_nanoseconds}:{l.metrics.provenance.value}"
        rows.append(f"l{l.source}>{l.to};{l.relation.value};{int(l.bidirectional)};{l.interconnect.value if l.interconnect else ''};{met}".encode())
    return b"\n".join(rows)
