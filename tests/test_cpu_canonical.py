"""Canonical tensor facade on CPU: shape checks, grad (against torch autograd), vmap, memory-plan reuse, JIT cache,
SPMD session, conformance cases."""
import pytest
import torch

from scirust_b200.canonical import (Graph, GraphError, ReferenceJitSession, ReferencePlanRuntime, ReferenceSpmdSession,
                                    grad, lower, plan_execution, plan_memory, run_conformance, vmap)
from scirust_b200.parallel.mesh import DeviceMesh, PartitionSpec


def _mlp_graph(n=6, d=5, h=4):
    g = Graph()
    x, w1, b1, w2 = g.input("x", (n, d)), g.input("w1", (d, h)), g.input("b1", (h,)), g.input("w2", (h, 1))
    hid = g.relu(g.add(g.matmul(x, w1), g.broadcast_to(b1, (n, h))))
    y = g.matmul(g.checkpoint(hid), w2)
    loss = g.reduce_sum_to(g.mul(y, y), (1, 1))
    return g, (x, w1, b1, w2), loss


def test_shape_inference_rejects_bad_graphs():
    g = Graph()
    a, b = g.input("a", (2, 3)), g.input("b", (3, 2))
    with pytest.raises(GraphError):
        g.add(a, b)
    with pytest.raises(GraphError):
        g.matmul(a, a)
    with pytest.raises(GraphError):
        g.reshape(a, (4, 2))
    with pytest.raises(GraphError):
        g.transpose(a, (0, 0))
    with pytest.raises(GraphError):
        g.broadcast_to(a, (3, 3))
    with pytest.raises(GraphError):
        g.reduce_sum_to(a, (2,))
    with pytest.raises(GraphError):
        g.input("a", (1,))
    other = Graph()
    with pytest.raises(GraphError):
        g.relu(other.input("z", (2, 3)))
    with pytest.raises(GraphError):
        plan_execution(g)                      # no outputs


def test_grad_matches_autograd_and_second_order_works():
    g, (x, w1, b1, w2), loss = _mlp_graph()
    gs = grad(g, loss, [w1, b1, w2, x])
    g.set_outputs(loss, *gs)
    gen = torch.Generator().manual_seed(0)
    feeds = {"x": torch.randn(6, 5, generator=gen), "w1": torch.randn(5, 4, generator=gen),
             "b1": torch.randn(4, generator=gen), "w2": torch.randn(4, 1, generator=gen)}
    out = ReferencePlanRuntime().run(lower(g), feeds)
    t = {k: v.clone().requires_grad_(True) for k, v in feeds.items()}
    ref = ((torch.relu(t["x"] @ t["w1"] + t["b1"]) @ t["w2"]) ** 2).sum()
    ref.backward()
    assert torch.allclose(out[0].reshape(()), ref.detach(), rtol=1e-5)
    for got, name in zip(out[1:], ("w1", "b1", "w2", "x")):
        assert torch.allclose(got, t[name].grad, rtol=1e-4, atol=1e-5), name
    # d/dx of sum(x^3) twice: 6x
    g2 = Graph()
    a = g2.input("a", (4,))
    cube = g2.mul(g2.mul(a, a), a)
    (d1,) = grad(g2, cube, [a])
    (d2,) = grad(g2, d1, [a])
    g2.set_outputs(d2)
    v = torch.tensor([1.0, -2.0, 0.5, 3.0])
    assert torch.allclose(ReferencePlanRuntime().run(lower(g2), {"a": v})[0], 6 * v)
    # stop_gradient blocks, unrelated inputs get zeros
    g3 = Graph()
    p, q = g3.input("p", (3,)), g3.input("q", (3,))
    out3 = g3.mul(g3.stop_gradient(p), p)
    dp, dq = grad(g3, out3, [p, q])
    g3.set_outputs(dp, dq)
    r = ReferencePlanRuntime().run(lower(g3), {"p": torch.tensor([1.0, 2.0, 3.0]), "q": torch.ones(3)})
    assert r[0].tolist() == [1.0, 2.0, 3.0] and r[1].tolist() == [0.0, 0.0, 0.0]


def test_vmap_lifts_matmul_to_batch_matmul():
    g = Graph()
    x, w = g.input("x", (3, 4)), g.input("w", (4, 2))
    g.set_outputs(g.relu(g.matmul(x, w)), g.reduce_sum_to(x, (4,)))
    vg = vmap(g, 5, {"x"})
    assert any(n.op == "BatchMatMul" for n in vg.nodes) and vg.batched_outputs == [True, True]
    gen = torch.Generator().manual_seed(1)
    xs, wv = torch.randn(5, 3, 4, generator=gen), torch.randn(4, 2, generator=gen)
    out = ReferencePlanRuntime().run(lower(vg), {"x": xs, "w": wv})
    for i in range(5):
        one = ReferencePlanRuntime().run(lower(g), {"x": xs[i], "w": wv})
        assert torch.equal(out[0][i], one[0]) and torch.equal(out[1][i], one[1])


def test_memory_plan_reuses_buffers_and_aliases_views():
    g = Graph()
    a = g.input("a", (64, 64))
    v = a
    for _ in range(12):
        v = g.relu(g.scale(v, 1.01))
    r = g.reshape(v, (4096,))
    g.set_outputs(r)
    ep = plan_execution(g)
    mp = plan_memory(ep)
    assert mp.arena_bytes <= 3 * 64 * 64 * 4 < mp.naive_bytes       # a chain needs two live buffers (+ the input)
    assert mp.offsets[r.id] == mp.offsets[v.id]                     # reshape is a view
    out = ReferencePlanRuntime().run(lower(g), {"a": torch.ones(64, 64)})[0]
    assert torch.allclose(out, torch.full((4096,), 1.01 ** 12), rtol=1e-5)
    # unused nodes are not executed
    g.exp(a)
    assert len(plan_execution(g).order) == len(ep.order)
    # checkpoint marks its producers recomputable
    g2, _, loss = _mlp_graph()
    g2.set_outputs(loss)
    assert plan_execution(g2).recomputable


def test_jit_session_caches_by_structure_and_spmd_session_checks_replicas():
    sess = ReferenceJitSession()

    def build():
        g = Graph()
        a = g.input("a", (4, 4))
        g.set_outputs(g.relu(g.scale(a, 2.0)))
        return g
    x = torch.randn(4, 4)
    r1, r2 = sess.run(build(), {"a": x}), sess.run(build(), {"a": x})
    assert sess.compilations == 1 and torch.equal(r1[0], r2[0])

    mesh = DeviceMesh(("dp",), (4,))
    spmd = ReferenceSpmdSession(mesh)

    def local(shapes):
        g = Graph()
        xs, w = g.input("x", shapes["x"]), g.input("w", shapes["w"])
        y = g.matmul(xs, w)
        g.set_outputs(y, g.scale(w, 2.0))
        return g
    gen = torch.Generator().manual_seed(2)
    X, W = torch.randn(8, 3, generator=gen), torch.randn(3, 2, generator=gen)
    y, w2 = spmd.run(local, {"x": X, "w": W}, {"x": PartitionSpec("dp", None), "w": PartitionSpec(None, None)},
                     [PartitionSpec("dp", None), PartitionSpec(None, None)])
    assert torch.allclose(y, X @ W, atol=1e-6) and torch.equal(w2, W * 2)
    with pytest.raises(GraphError, match="replicated"):
        spmd.run(local, {"x": X, "w": W}, {"x": PartitionSpec("dp", None), "w": PartitionSpec(None, None)},
                 [PartitionSpec(None, None), PartitionSpec(None, None)])


def test_conformance_cases_run_on_cpu_and_are_repeatable():
    a, b = run_conformance("cpu"), run_conformance("cpu")
    assert set(a) == {"elementwise", "matmul_permute_reshape", "broadcast_reduce", "batch_matmul"}
    for k in a:
        for x, y in zip(a[k], b[k]):
            assert torch.equal(x.view(torch.int32), y.view(torch.int32))


def test_fusion_pass_groups_elementwise_trees_keeps_bits_and_shrinks_the_arena():
    from scirust_b200.canonical import (Graph, ReferenceJitSession, cuda_source, find_groups, lower, lower_fused,
                                        plan_execution, run_conformance)
    g = Graph()
    a, b = g.input("x", (64, 33)), g.input("y", (64, 33))
    t = g.div(g.mul(g.add(a, b), g.sub(a, b)), g.scale(b, 0.3))
    r = g.relu(t)
    w = g.input("w", (33, 5))
    mm = g.matmul(r, w)                      # r feeds a matmul: the tree above ends at r
    tail = g.scale(g.relu(mm), 2.0)
    g.set_outputs(tail, g.relu_grad(a, b))
    groups = find_groups(plan_execution(g))
    sizes = sorted(len(m) for m in groups.values())
    assert sizes == [2, 6]                   # {relu(mm), scale} and {add, sub, mul, scale, div, relu}
    plain, fused = lower(g), lower_fused(g)
    n_plain = sum(k.kind != "alias" for k in plain.kernels)
    n_fused = sum(k.kind != "alias" for k in fused.kernels)
    assert n_fused == n_plain - 6 and fused.memory.arena_bytes < plain.memory.arena_bytes
    gen = torch.Generator().manual_seed(0)
    feeds = {"x": torch.randn(64, 33, generator=gen), "y": torch.randn(64, 33, generator=gen),
             "w": torch.randn(33, 5, generator=gen)}
    feeds["x"][0, 0], feeds["x"][0, 1], feeds["y"][0, 2] = float("nan"), -0.0, float("inf")
    o1 = ReferenceJitSession("cpu").run(g, feeds)
    o2 = ReferenceJitSession("cpu", fuse=True).run(g, feeds)
    # "w" is declared after values that are dead by the time it is used: a feed must still own its storage from the
    # start, since every input is written before the first kernel runs
    xs, ys = torch.nan_to_num(feeds["x"][1:]), feeds["y"][1:]
    want = torch.relu(torch.relu((xs + ys) * (xs - ys) / (ys * 0.3)) @ feeds["w"]) * 2.0
    assert torch.allclose(o1[0][1:], want, rtol=1e-4, atol=1e-4)
    for p, q in zip(o1, o2):
        nan = torch.isnan(p)
        assert torch.equal(torch.isnan(q), nan) and torch.equal(p.view(torch.int32)[~nan], q.view(torch.int32)[~nan])
    # a value with two consumers, or a graph output, is never swallowed
    g2 = Graph()
    x = g2.input("x", (8,))
    s = g2.scale(x, 2.0)
    g2.set_outputs(g2.add(s, x), g2.relu(s))
    assert find_groups(plan_execution(g2)) == {}
    # the conformance suite gives the same words with the pass switched on
    c0, c1 = run_conformance("cpu"), run_conformance("cpu", fuse=True)
    for name in c0:
        for p, q in zip(c0[name], c1[name]):
            nan = torch.isnan(p)
            assert torch.equal(p.view(torch.int32)[~nan], q.view(torch.int32)[~nan]), name
    # generated device source: individually rounded intrinsics, never a bare * or +
    k = [k for k in fused.kernels if k.kind == "fused_elementwise" and len(k.attrs["program"]) == 6][0]
    src = cuda_source(k.attrs["program"], len(k.inputs))
    assert "__fdiv_rn" in src and "__fmul_rn" in src and "__fadd_rn" in src and " * " not in src.split("{", 1)[1].replace("blockIdx.x * (long long)blockDim.x", "")
