"""Compute contracts: value types, three-valued hardware facts, requirement matching and implementation selection,
topology graph, transfers and workspaces, the reference backend, and the evidence-based autotuner."""
import struct
import time

import pytest
import torch

from scirust_b200.compute import autotune as AT
from scirust_b200.compute import backend as B
from scirust_b200.compute import contracts as C
from scirust_b200.compute import hardware as H
from scirust_b200.compute import requirements as R
from scirust_b200.compute import topology as T
from scirust_b200.compute import transfer as X


def test_value_types_validate():
    assert [d.size_bytes() for d in (C.DType.BOOL, C.DType.BF16, C.DType.F32, C.DType.F64, C.DType.F8E4M3)] == [1, 2, 4, 8, 1]
    assert C.DType.BF16.torch_dtype() is torch.bfloat16
    assert C.DeviceId.cuda(0) != C.DeviceId.cuda(1) and C.DeviceId.cpu() != C.DeviceId(C.DeviceKind.CUDA, 0)
    spec = C.TensorSpec.contiguous(C.DType.BF16, C.Shape((4, 6, 8)), C.DeviceId.cuda(0))
    assert spec.strides.elems == (48, 8, 1) and spec.checked_byte_len() == 384 and spec.tma_ok()
    assert not C.TensorSpec.contiguous(C.DType.BF16, C.Shape((4, 7)), C.DeviceId.cuda(0)).tma_ok()       # 14-byte rows
    assert not C.TensorSpec(C.DType.F32, C.Shape((4, 8)), C.Strides((1, 4)), C.Layout.STRIDED, C.DeviceId.cuda(0)).tma_ok()
    with pytest.raises(C.ComputeError):
        C.Shape((2, -1))
    with pytest.raises(C.ComputeError):
        C.Shape((1 << 40, 1 << 40)).checked_num_elements()
    m = C.KernelModule(C.KernelFormat.CUDA_C, "main", "__global__ void main() {}")
    assert m.code.startswith(b"__global__")
    for bad in (("", b"x"), ("main", b"")):
        with pytest.raises(C.ComputeError):
            C.KernelModule(C.KernelFormat.PTX, *bad)
    assert C.LaunchConfig((8, 1, 1), (32, 1, 1)).cluster == (1, 1, 1)
    assert C.LaunchConfig((8, 2, 1), (128, 1, 1), 1024, (2, 1, 1)).shared_memory_bytes == 1024
    for bad in (((0, 1, 1), (32, 1, 1)), ((1, 1, 1), (0, 1, 1)), ((3, 1, 1), (32, 1, 1), 0, (2, 1, 1)), ((1, 1), (1, 1, 1))):
        with pytest.raises(C.ComputeError):
            C.LaunchConfig(*bad)


def test_capability_sets_and_profiles():
    s = H.CapabilitySet()
    assert s.is_empty() and s.support_level("x") is H.SupportLevel.UNKNOWN
    s.set_support("x", H.SupportLevel.SUPPORTED)
    s.set_support("y", H.SupportLevel.UNSUPPORTED)
    s.set_support("x", H.SupportLevel.UNSUPPORTED)                 # re-stating a fact replaces it
    assert not s.supports("x") and s.unsupported_values() == ["y", "x"]
    s.set_support("y", H.SupportLevel.UNKNOWN)
    assert s.support_level("y") is H.SupportLevel.UNKNOWN
    base = H.DeviceCapabilities.reference_cpu().hardware_baseline()
    assert base.isa.features.is_empty() and base.isa.vector_model is H.VectorModel.UNKNOWN      # nothing optional is invented
    assert base.execution.async_execution is H.SupportLevel.UNSUPPORTED and base.matrix.accelerated is H.SupportLevel.UNKNOWN
    assert base.numeric.storage_dtypes.supports(C.DType.F32) and not base.numeric.storage_dtypes.supports(C.DType.F64)
    b200 = H.b200_declared()
    for f in (H.IsaFeature.TCGEN05, H.IsaFeature.TMEM, H.IsaFeature.TMA, H.IsaFeature.CTA_PAIR, H.IsaFeature.FP4_MMA, H.IsaFeature.NVLINK_P2P):
        assert b200.isa.supports(f)
    assert b200.isa.features.support_level(H.IsaFeature.WGMMA) is H.SupportLevel.UNSUPPORTED
    assert b200.execution.multiprocessors == 148 and b200.memory.tensor_memory_per_sm == 256 * 1024
    hopper = H._nvidia_profile(C.DeviceId.cuda(0), "H100", (9, 0), 132, 80 * 10 ** 9, 227 * 1024, 50 * 2 ** 20, H.SupportLevel.SUPPORTED)
    assert hopper.isa.supports(H.IsaFeature.WGMMA) and hopper.isa.supports(H.IsaFeature.TMA) and not hopper.isa.supports(H.IsaFeature.TCGEN05)
    cpu = H.probe_host_cpu()
    assert cpu.device == C.DeviceId.cpu() and cpu.memory.spaces.supports(C.MemorySpace.HOST)
    # canonical bytes: independent of the order facts were stated in, sensitive to every fact
    a, b = H.b200_declared(), H.b200_declared()
    b.isa.features.set_support(H.IsaFeature.TMA, H.SupportLevel.SUPPORTED)        # moves TMA to the end of the list
    assert H.canonical_hardware_profile_bytes(a) == H.canonical_hardware_profile_bytes(b)
    b.isa.features.set_support(H.IsaFeature.TMA, H.SupportLevel.UNSUPPORTED)
    assert H.canonical_hardware_profile_bytes(a) != H.canonical_hardware_profile_bytes(b)
    assert H.canonical_hardware_profile_bytes(H.b200_declared(peers=False)) != H.canonical_hardware_profile_bytes(a)


def _hw():
    hw = H.HardwareCapabilities(C.DeviceId.cpu(), H.Architecture.current_host())
    hw.isa.features = H.CapabilitySet([H.IsaFeature.AVX2], [H.IsaFeature.AVX512F])
    hw.isa.vector_model, hw.isa.min_vector_bits, hw.isa.max_vector_bits = H.VectorModel.FIXED_WIDTH, 128, 256
    for cs in (hw.numeric.storage_dtypes, hw.numeric.arithmetic_dtypes, hw.numeric.accumulation_dtypes):
        cs.set_support(C.DType.F32, H.SupportLevel.SUPPORTED)
        cs.set_support(C.DType.F64, H.SupportLevel.UNSUPPORTED)
    hw.matrix.accelerated = H.SupportLevel.UNSUPPORTED
    hw.memory.spaces = H.CapabilitySet([C.MemorySpace.HOST], [C.MemorySpace.DEVICE])
    hw.execution.async_execution, hw.execution.atomic_i64 = H.SupportLevel.UNSUPPORTED, H.SupportLevel.SUPPORTED
    hw.reproducibility.modes.set_support(H.ReproducibilityLevel.BIT_EXACT, H.SupportLevel.SUPPORTED)
    return hw


def test_requirement_matching_is_three_valued():
    hw = _hw()
    ok = R.KernelRequirements(storage_dtypes=[C.DType.F32], required_isa=[H.IsaFeature.AVX2], vector=R.VectorRequirement("fixed", 256),
                              memory_spaces=[C.MemorySpace.HOST], atomic_i64=R.SupportRequirement.REQUIRED,
                              matrix_acceleration=R.SupportRequirement.FORBIDDEN, reproducibility=H.ReproducibilityLevel.BIT_EXACT)
    rep = R.match_requirements(ok, hw)
    assert rep.is_compatible() and rep.issues == []
    bad = R.KernelRequirements(storage_dtypes=[C.DType.F64], required_isa=[H.IsaFeature.AVX512F], vector=R.VectorRequirement("fixed", 512),
                               memory_spaces=[C.MemorySpace.DEVICE], async_execution=R.SupportRequirement.REQUIRED,
                               matrix_acceleration=R.SupportRequirement.REQUIRED)
    rep = R.match_requirements(bad, hw)
    kinds = [i.kind for i in rep.issues]
    assert rep.is_incompatible() and kinds == ["storage-dtype-unsupported", "isa-unsupported", "memory-space-unsupported",
                                               "vector-width-insufficient", "matrix-acceleration-mismatch", "async-execution-mismatch"]
    unk = R.KernelRequirements(storage_dtypes=[C.DType.BF16], required_isa=[H.IsaFeature.AMX_TILE],
                               subgroup_operations=R.SupportRequirement.REQUIRED, reproducibility=H.ReproducibilityLevel.DETERMINISTIC)
    rep = R.match_requirements(unk, hw)
    assert rep.disposition is R.MatchDisposition.INDETERMINATE and all(i.kind.endswith("-unknown") for i in rep.issues) and len(rep.issues) == 4
    # a single known violation outweighs any number of unknowns
    unk.memory_spaces = [C.MemorySpace.DEVICE]
    assert R.match_requirements(unk, hw).is_incompatible()
    assert R.match_requirements(R.KernelRequirements(vector=R.VectorRequirement("scalable")), hw).is_incompatible()
    hw.isa.vector_model = H.VectorModel.UNKNOWN
    assert R.match_requirements(R.KernelRequirements(vector=R.VectorRequirement("vectorized")), hw).disposition is R.MatchDisposition.INDETERMINATE


def test_candidate_and_implementation_selection():
    req = R.KernelRequirements(storage_dtypes=[C.DType.BF16], matrix_acceleration=R.SupportRequirement.REQUIRED)
    cands = [R.ExecutionCandidate("cpu", 0, _hw()), R.ExecutionCandidate("gpu-b", 5, H.b200_declared(1)),
             R.ExecutionCandidate("gpu-a", 5, H.b200_declared(0))]
    assert R.select_candidate(req, cands).name == "gpu-a"                     # cpu incompatible; equal priority: name decides
    assert R.select_candidate(R.KernelRequirements(memory_spaces=[C.MemorySpace.UNIFIED]), cands[:1]) is None
    loose = R.KernelRequirements(required_isa=[H.IsaFeature.AMX_TILE])
    assert R.select_candidate(loose, cands[:1]) is None
    assert R.select_candidate(loose, cands[:1], R.PlannerPolicy(True)).report.disposition is R.MatchDisposition.INDETERMINATE
    # the framework's own GEMM paths on three machines
    pick = lambda hw, lim, pol=R.PlannerPolicy(): getattr(R.select_implementation(hw, lim, R.GEMM_CANDIDATES, pol), "name", None)
    assert pick(H.b200_declared(), H.b200_limits()) == "tcgen05-cta-pair"
    assert pick(H.b200_declared(), H.ExecutionLimits((1024, 1024, 64), 1024, 227 * 1024, 1)) == "tcgen05-single-cta"   # no clusters
    assert pick(H.b200_declared(), H.ExecutionLimits((1024, 1024, 64), 1024, 48 * 1024, 16)) == "library-gemm"          # small shared memory
    hopper = H._nvidia_profile(C.DeviceId.cuda(0), "H100", (9, 0), 132, 80 * 10 ** 9, 227 * 1024, 50 * 2 ** 20, H.SupportLevel.SUPPORTED)
    assert pick(hopper, H.b200_limits()) == "library-gemm"
    assert pick(H.probe_host_cpu(), H.ExecutionLimits()) == "host-fp32-fixed-order"
    # unknown limits make a launch-shape requirement indeterminate, never satisfied
    rep = R.match_implementation(R.GEMM_CANDIDATES[0].requirements, H.b200_declared(), H.ExecutionLimits())
    assert rep.disposition is R.MatchDisposition.INDETERMINATE and {i.kind for i in rep.issues} == {
        "workgroup-x-limit-unknown", "shared-memory-limit-unknown", "cluster-size-limit-unknown"}
    k = R.KernelRequirements()
    r = R.ImplementationRequirements(k).with_workgroup(R.WorkgroupRequirement.x(64))
    assert R.match_implementation(r, _hw(), H.ExecutionLimits((64, 1, 1))).disposition is R.MatchDisposition.COMPATIBLE
    assert R.match_implementation(r, _hw(), H.ExecutionLimits((32, 1, 1))).disposition is R.MatchDisposition.INCOMPATIBLE


def test_topology_graph():
    t = T.SystemTopology([T.TopologyNode(0, T.NodeKind.MACHINE), T.TopologyNode(1, T.NodeKind.NUMA_NODE),
                          T.TopologyNode(2, T.NodeKind.MEMORY_DOMAIN, memory=T.MemoryDomainDescriptor(C.MemorySpace.HOST, 64 << 30, H.SupportLevel.SUPPORTED)),
                          T.TopologyNode(3, T.NodeKind.ACCELERATOR, device=C.DeviceId.cuda(0))],
                         [T.TopologyLink(0, 1, T.Relation.CONTAINS), T.TopologyLink(1, 2, T.Relation.AFFINE_TO, True, T.InterconnectClass.HOST_MEMORY_BUS),
                          T.TopologyLink(1, 3, T.Relation.AFFINE_TO, True, T.InterconnectClass.PCIE)])
    t.validate()
    assert len(t.adjacent_links(3)) == 1 and len(t.links_from(1)) == 2 and t.node(9) is None
    t.links[2].metrics = T.TransferMetrics(24_000_000_000, None, T.MetricProvenance.MEASURED)
    t.validate()
    with pytest.raises(T.TopologyError):
        T.SystemTopology([T.TopologyNode(7, T.NodeKind.CPU_PACKAGE), T.TopologyNode(7, T.NodeKind.NUMA_NODE)]).validate()
    with pytest.raises(T.TopologyError):
        T.SystemTopology([T.TopologyNode(0, T.NodeKind.MACHINE)], [T.TopologyLink(0, 5, T.Relation.CONTAINS)]).validate()
    node = T.nvswitch_declared(8)
    acc = node.accelerators()
    assert len(acc) == 8 and sum(n.kind is T.NodeKind.INTERCONNECT_ENDPOINT for n in node.nodes) == 1
    assert node.peer_bandwidth(C.DeviceId.cuda(0), C.DeviceId.cuda(7)) == 900 * 10 ** 9
    assert node.peer_bandwidth(C.DeviceId.cuda(0), C.DeviceId.cuda(9)) is None
    hbm = [n for n in node.nodes if n.kind is T.NodeKind.MEMORY_DOMAIN and n.memory.space is C.MemorySpace.DEVICE]
    assert len(hbm) == 8 and all(n.memory.capacity_bytes == 180 * 10 ** 9 for n in hbm)
    # partial peer access: direct links, no switch
    base = T.SystemTopology([T.TopologyNode(0, T.NodeKind.MACHINE)])
    ids = T.augment_accelerators(base, [T.AcceleratorDescriptor(C.DeviceId.cuda(0), "a", 1, None, (1,)),
                                        T.AcceleratorDescriptor(C.DeviceId.cuda(1), "b", 1, None, (0,)),
                                        T.AcceleratorDescriptor(C.DeviceId.cuda(2), "c", 1, None, ())])
    assert len(ids) == 3 and sum(l.relation is T.Relation.PEER_ACCESS for l in base.links) == 1
    assert base.peer_bandwidth(C.DeviceId.cuda(0), C.DeviceId.cuda(1)) and base.peer_bandwidth(C.DeviceId.cuda(0), C.DeviceId.cuda(2)) is None
    with pytest.raises(T.TopologyError):
        T.augment_accelerators(base, [T.AcceleratorDescriptor(C.DeviceId.cuda(0), "again", 1)])
    host = T.probe_host_topology()
    kinds = [n.kind for n in host.nodes]
    assert kinds[0] is T.NodeKind.MACHINE and T.NodeKind.NUMA_NODE in kinds and T.NodeKind.MEMORY_DOMAIN in kinds
    assert T.probe_host_topology("/nonexistent").nodes[1].kind is T.NodeKind.NUMA_NODE          # falls back to one node
    a, b = T.canonical_topology_profile_bytes(node), T.canonical_topology_profile_bytes(T.nvswitch_declared(8))
    assert a == b and a != T.canonical_topology_profile_bytes(T.nvswitch_declared(4))
    assert T._cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]


def test_transfers_and_workspaces():
    dev = C.DeviceId.cuda(1)
    r = X.TransferRequest(X.TensorResidency.host_pinned(), X.TensorResidency.on(dev), C.DType.F32, 4096, X.TransferMode.on_stream(C.StreamId(7)))
    assert r.canonical_record() == ("scirust-transfer-v1;dtype_version=1;dtype=f32;bytes=4096;source=host-pinned;"
                                    "destination=device:cuda:1;mode=async;stream=7")
    assert not r.crosses_nvlink() and not r.wants_pinned_host()
    assert X.TransferRequest(X.TensorResidency.host(), X.TensorResidency.on(dev), C.DType.I8, 8, X.TransferMode.on_stream(C.StreamId(1))).wants_pinned_host()
    p2p = X.TransferRequest(X.TensorResidency.on(C.DeviceId.cuda(0)), X.TensorResidency(C.MemorySpace.PEER_DEVICE, dev), C.DType.BF16, 64)
    assert p2p.crosses_nvlink() and "mode=sync;stream=none" in p2p.canonical_record()
    with pytest.raises(X.TransferRequestError):
        X.TransferRequest(X.TensorResidency.on(dev), X.TensorResidency.on(dev), C.DType.F32, 16)
    with pytest.raises(X.TransferRequestError):
        X.TransferRequest(X.TensorResidency.host(), X.TensorResidency.on(dev), C.DType.F32, 6)
    for bad in (lambda: X.TensorResidency(C.MemorySpace.DEVICE), lambda: X.TensorResidency(C.MemorySpace.HOST, dev),
                lambda: X.TransferMode(X.TransferKind.ASYNCHRONOUS), lambda: X.TransferMode(X.TransferKind.SYNCHRONOUS, C.StreamId(1))):
        with pytest.raises(C.ComputeError):
            bad()
    a, b = X.WorkspaceSpec(100, 16), X.WorkspaceSpec(64, 64)
    both = a.then(b)
    assert (both.size_bytes, both.align_bytes, a.offset_of_next(b)) == (192, 64, 128) and X.WorkspaceSpec.empty().is_empty()
    for bad in ((8, 0), (8, 3), (-1, 4)):
        with pytest.raises(X.WorkspaceError):
            X.WorkspaceSpec(*bad)
    buf = torch.zeros(1024, dtype=torch.uint8)
    off = (-buf.data_ptr()) % 64
    ws = X.KernelWorkspace(buf[off:], X.WorkspaceSpec(128, 64))
    ws.view()[127] = 7
    assert len(ws) == 128 and int(buf[off + 127]) == 7
    with pytest.raises(X.WorkspaceError, match="too small"):
        X.KernelWorkspace(buf[:64], X.WorkspaceSpec(128, 1))
    with pytest.raises(X.WorkspaceError, match="not aligned"):
        X.KernelWorkspace(buf[off + 1:], X.WorkspaceSpec(128, 64))
    assert len(X.KernelWorkspace(bytearray(16), X.WorkspaceSpec(16, 1))) == 16


def test_reference_backend_runs_and_refuses():
    be = B.ReferenceBackend()
    assert be.capabilities().name == "reference-cpu" and be.execution_limits().max_workgroup_size == (1, 1, 1)
    x, y = be.allocate(16, 4, C.MemorySpace.HOST), be.allocate(16, 4, C.MemorySpace.HOST)
    be.write(x, 0, struct.pack("4f", 1, 2, 3, 4))
    be.write(y, 0, struct.pack("4f", 10, 10, 10, 10))
    k = be.compile(C.KernelModule(C.KernelFormat.REFERENCE, "main", b"axpy_f32"))
    s = be.create_stream()
    cfg = C.LaunchConfig((1, 1, 1), (4, 1, 1))
    bind = lambda slot, buf, off, n, acc: C.BufferBinding(slot, buf, off, n, acc)
    ev = be.launch(k, s, cfg, [bind(0, x, 0, 16, C.BufferAccess.READ_ONLY), bind(1, y, 0, 16, C.BufferAccess.READ_WRITE)], (2.0,))
    be.wait(ev)
    be.synchronize(s)
    assert struct.unpack("4f", be.read(y, 0, 16)) == (12.0, 14.0, 16.0, 18.0) and be.launches == 1      # a kernel really ran
    # sub-ranges of one allocation: disjoint is fine, overlapping a written range is refused before anything runs
    z = be.allocate(32)
    be.write(z, 0, struct.pack("8f", *range(8)))
    relu = be.compile(C.KernelModule(C.KernelFormat.REFERENCE, "main", b"relu_f32"))
    be.launch(relu, s, cfg, [bind(0, z, 0, 16, C.BufferAccess.READ_ONLY), bind(1, z, 16, 16, C.BufferAccess.WRITE_ONLY)])
    assert struct.unpack("8f", be.read(z, 0, 32))[4:] == (0.0, 1.0, 2.0, 3.0)
    with pytest.raises(C.ComputeError, match="aliasing"):
        be.launch(relu, s, cfg, [bind(0, z, 0, 16, C.BufferAccess.READ_ONLY), bind(1, z, 8, 16, C.BufferAccess.WRITE_ONLY)])
    be.launch(relu, s, cfg, [bind(0, z, 0, 16, C.BufferAccess.READ_ONLY), bind(1, y, 0, 16, C.BufferAccess.WRITE_ONLY)])   # two readers may overlap
    for bad in ([bind(0, x, 8, 16, C.BufferAccess.READ_ONLY)], [bind(0, x, 0, 0, C.BufferAccess.READ_ONLY)],
                [bind(0, x, 0, 8, C.BufferAccess.READ_ONLY), bind(0, y, 0, 8, C.BufferAccess.WRITE_ONLY)]):
        with pytest.raises(C.ComputeError):
            be.launch(relu, s, cfg, bad)
    assert be.launches == 3
    for bad in (lambda: be.allocate(0), lambda: be.allocate(8, 3), lambda: be.allocate(8, 1, C.MemorySpace.DEVICE),
                lambda: be.write(x, 12, b"12345678"), lambda: be.read(x, 8, 16),
                lambda: be.compile(C.KernelModule(C.KernelFormat.CUDA_C, "main", b"x")),
                lambda: be.compile(C.KernelModule(C.KernelFormat.REFERENCE, "main", b"nope"))):
        with pytest.raises(C.ComputeError):
            bad()
    # a read-only binding cannot be written through
    @B.ReferenceBackend.register("scribble")
    def _scribble(config, views):
        views[0][0] = 1
    with pytest.raises(ValueError):
        be.launch(be.compile(C.KernelModule(C.KernelFormat.REFERENCE, "main", b"scribble")), s, cfg, [bind(0, x, 0, 16, C.BufferAccess.READ_ONLY)])


def _cand(i, scratch=0, det=True):
    return AT.ElasticCandidate.new("sgemm-f32", b"rev1", {"path": i}, det, scratch)


def _ev(c, med, p95=None, p99=None, mad=0):
    return AT.ElasticEvidence(c, b"ok", AT.ElasticMeasurement(8, med, p95 or med, p99 or p95 or med, mad))


def test_autotuner_ranking_statistics_and_racing():
    hw, prob = AT.HardwareProfile.from_capabilities(H.b200_declared()), AT.ProblemClass.gemm(4096, 4096, 4096)
    tuner = AT.ElasticAutoTuner(AT.ElasticConfig(AT.ElasticMode.LEARN, max_ranked_candidates=3))
    space = lambda h, p: [_cand(3), _cand(1), _cand(2), _cand(1), _cand(4, det=False), _cand(5)]
    ranked = tuner.rank_candidates(hw, prob, space, lambda h, p, c: c.param("path") != 5, lambda h, p, c, o: 10 if c.param("path") < 3 else 5)
    assert [r.candidate.param("path") for r in ranked] == [3, 4, 1]            # cost first, then the candidate; duplicates and rejects gone
    det = AT.ElasticAutoTuner(AT.ElasticConfig(objective=AT.ElasticObjective.DETERMINISTIC_ONLY))
    assert all(r.candidate.deterministic for r in det.rank_candidates(hw, prob, space, lambda *a: True, lambda *a: 0))
    with pytest.raises(AT.ElasticError, match="duplicate tuning parameter"):
        AT.ElasticCandidate.new("f", b"r", [("a", 1), ("a", 2)], True, 0)
    proto = AT.MeasurementProtocol(2, 8, AT.TimingSource.HOST_WALL_CLOCK)
    m = proto.summarize([10, 12, 11, 13, 100, 12, 11, 12])
    assert (m.median_ns, m.p95_ns, m.p99_ns, m.mad_ns, m.sample_count) == (12, 100, 100, 1, 8)
    assert AT.MeasurementProtocol(0, 4).summarize([1, 2, 4, 7]).median_ns == 3 and AT._median_sorted([2 ** 63, 2 ** 63 + 1]) == 2 ** 63
    assert len(proto.canonical_bytes()) == 15 and proto.canonical_bytes()[12:] == bytes([0, 0, 0])
    for bad in (lambda: AT.MeasurementProtocol(1, 0).validate(), lambda: proto.summarize([1, 2]),
                lambda: AT.MeasurementProtocol(1, 1, schema_version=9).validate()):
        with pytest.raises(AT.ElasticError):
            bad()
    calls = []
    got = AT.MeasurementProtocol(2, 5, AT.TimingSource.HOST_WALL_CLOCK).measure(lambda: calls.append(1), flush=lambda: calls.append(0))
    assert got.sample_count == 5 and calls.count(1) == 7 and calls.count(0) == 5 and got.median_ns >= 1
    # one racing round: half survive, ordered by latency; ties fall back to p95, then to the original rank
    ranked = [AT.RankedCandidate(0, _cand(i)) for i in range(4)]
    ev = [_ev(ranked[0].candidate, 50), _ev(ranked[1].candidate, 30, 40), _ev(ranked[2].candidate, 30, 35), _ev(ranked[3].candidate, 90)]
    pol = AT.RacingPolicy()
    assert [r.candidate.param("path") for r in pol.race_round(tuner, ranked, ev)] == [2, 1]
    assert len(AT.RacingPolicy(4, 3).race_round(tuner, ranked, ev)) == 3 and pol.protocol_for_round(proto, 3).measured_iterations == 64
    with pytest.raises(AT.ElasticError, match="missing racing evidence"):
        pol.race_round(tuner, ranked, ev[:3])
    with pytest.raises(AT.ElasticError, match="duplicate evidence"):
        pol.race_round(tuner, ranked, ev + [ev[0]])
    for bad in (AT.RacingPolicy(1), AT.RacingPolicy(2, 0), AT.RacingPolicy(2, 1, 0)):
        with pytest.raises(AT.ElasticError):
            bad.validate()
    with pytest.raises(AT.ElasticError, match="overflowed"):
        AT.RacingPolicy(2, 1, 2 ** 16).protocol_for_round(proto, 2)
    # objectives
    mem = [_ev(_cand(0, 4096), 10), _ev(_cand(1, 0), 30), _ev(_cand(2, 1024), 12), _ev(_cand(3, 8192), 40)]
    rk = [AT.RankedCandidate(0, e.candidate) for e in mem]
    pick = lambda obj: AT.ElasticAutoTuner(AT.ElasticConfig(AT.ElasticMode.LEARN, obj)).select_measured_evidence(rk, mem).candidate.param("path")
    assert pick(AT.ElasticObjective.MIN_LATENCY) == 0 and pick(AT.ElasticObjective.MIN_TEMPORARY_MEMORY) == 1
    assert pick(AT.ElasticObjective.BALANCED_LATENCY_MEMORY) == 0              # Pareto front {0, 1, 2}; fastest of it
    assert tuner.select_measured_evidence(rk, mem[1:2]).candidate.param("path") == 1     # only measured candidates compete
    for bad in (lambda: tuner.select_measured_evidence([], mem), lambda: tuner.select_measured_evidence(rk, []),
                lambda: tuner.plan_from_evidence(hw, prob, AT.ElasticEvidence(_cand(0), b"", mem[0].measurement)),
                lambda: _ev(_cand(0), 10, 5).validate(), lambda: _ev(_cand(0), 10, 20, 30, 31).validate(),
                lambda: AT.ElasticEvidence(_cand(0), b"ok", AT.ElasticMeasurement(0, 1, 1, 1, 0)).validate(),
                lambda: det.plan_from_evidence(hw, prob, _ev(_cand(0, det=False), 5))):
        with pytest.raises(AT.ElasticError):
            bad()
    # the whole loop on a host-timed toy: the fastest callable wins and slow ones are measured less often
    counts = {}

    def run(c):
        def f():
            counts[c.param("path")] = counts.get(c.param("path"), 0) + 1
            time.sleep(0.0002 * (1 + c.param("path")))
        return f
    win, last = AT.race(tuner, ranked, run, AT.MeasurementProtocol(0, 2, AT.TimingSource.HOST_WALL_CLOCK),
                        correctness=lambda c: b"" if c.param("path") == 0 else b"max_err=0")
    assert win.candidate.param("path") == 1 and 0 not in counts and counts[1] > counts[3] and win.correctness_evidence == b"max_err=0"
    with pytest.raises(AT.ElasticError, match="forbidden in cold"):
        AT.race(AT.ElasticAutoTuner(), ranked, run, proto)


def test_autotuner_modes_and_persistence(tmp_path):
    hw, prob = AT.HardwareProfile.from_capabilities(H.b200_declared()), AT.ProblemClass.gemm(1024, 1024, 1024)
    learn = AT.ElasticAutoTuner(AT.ElasticConfig(AT.ElasticMode.LEARN))
    plan = learn.plan_from_evidence(hw, prob, _ev(_cand(7, 512), 1000, 1100, 1200, 20))
    key = plan.key()
    modes = {m: AT.ElasticAutoTuner(AT.ElasticConfig(m)) for m in AT.ElasticMode}
    assert [modes[m].startup_strategy(True) for m in AT.ElasticMode] == ["qualified-heuristic", "persisted-then-explore", "persisted-only", "audit-only"]
    assert modes[AT.ElasticMode.LEARN].startup_strategy(False) == "qualified-heuristic-then-explore"
    with pytest.raises(AT.ElasticError, match="locked mode requires"):
        modes[AT.ElasticMode.LOCKED].startup_strategy(False)
    p = modes[AT.ElasticMode.AUDIT].mode_permissions()
    assert p.may_measure and p.audit_replay and not p.may_mutate_selection and not p.may_explore
    store = AT.PersistedPlanStore(tmp_path / "plans")
    for m in (AT.ElasticMode.COLD, AT.ElasticMode.LOCKED, AT.ElasticMode.AUDIT):
        with pytest.raises(AT.ElasticError, match="mutation is forbidden"):
            modes[m].store_plan_for_mode(store, key, plan)
    assert learn.load_plan_for_mode(store, key) is None
    with pytest.raises(AT.ElasticError):
        modes[AT.ElasticMode.LOCKED].load_plan_for_mode(store, key)
    learn.store_plan_for_mode(store, key, plan)
    assert modes[AT.ElasticMode.LOCKED].load_plan_for_mode(store, key) == plan and modes[AT.ElasticMode.COLD].load_plan_for_mode(store, key) is None
    for m, fn in ((AT.ElasticMode.LOCKED, "require_measurement"), (AT.ElasticMode.AUDIT, "require_exploration"), (AT.ElasticMode.COLD, "require_measurement")):
        with pytest.raises(AT.ElasticError):
            getattr(modes[m], fn)()
    learn.require_exploration()
    # a plan stored under the wrong key, or for other hardware, is refused
    other = AT.PlanKey(hw, AT.ProblemClass.gemm(2048, 1024, 1024), plan.objective)
    with pytest.raises(AT.ElasticError, match="does not match"):
        learn.store_plan_for_mode(AT.InMemoryPlanCache(), other, plan)
    assert AT.PlanKey(AT.HardwareProfile.from_capabilities(H.b200_declared(peers=False)), prob, plan.objective).digest() != key.digest()
    # the file format: round trip, checksum, malformed input is a typed refusal, never a crash
    blob = AT.encode_plan(plan)
    assert AT.decode_plan(blob) == plan
    path = next((tmp_path / "plans").glob("*.plan"))
    assert path.read_bytes() == blob and path.stem == key.digest()
    for bad in (blob[:-3], blob.replace(b'"objective"', b'"objectiv3"'), b"", b"SBPLAN2\nx\n{}", blob.replace(b"1000", b"1001", 1)):
        with pytest.raises(AT.ElasticError):
            AT.decode_plan(bad)
    path.write_bytes(blob[:40])
    with pytest.raises(AT.ElasticError):
        modes[AT.ElasticMode.LOCKED].load_plan_for_mode(store, key)
