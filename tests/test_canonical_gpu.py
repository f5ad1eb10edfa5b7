"""Canonical operators: the CUDA kernels agree with the CPU statement word for word."""
import pytest
import torch

from scirust_b200.ops import canonical as K

pytestmark = pytest.mark.gpu


def _special(n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * 3
    x[:8] = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1e-45, -1e-45, 3.4e38])
    bits = x.view(torch.int32)
    bits[4] = 0x7FC12345          # NaN with a payload
    return x


@pytest.mark.parametrize("op", ["relu", "scale", "add", "sub", "mul", "div", "copy"])
def test_elementwise_bits(op):
    a, b = _special(100003, 1), _special(100003, 2).flip(0)
    kw = {"factor": 0.3} if op == "scale" else {}
    ref = K.run(op, a, b if K.ARITY[op] == 2 else None, **kw)
    out = K.run(op, a.cuda(), b.cuda() if K.ARITY[op] == 2 else None, **kw).cpu()
    r, o = ref.view(torch.int32), out.view(torch.int32)
    nan = torch.isnan(ref)
    assert torch.equal(r[~nan], o[~nan])
    assert torch.equal(torch.isnan(out), nan)
    if op in ("relu", "copy"):
        assert torch.equal(r, o)          # words move untouched, NaN payloads included


@pytest.mark.parametrize("shape,perm", [((7, 5), (1, 0)), ((3, 4, 5), (2, 0, 1)), ((2, 3, 4, 5, 6), (4, 2, 0, 3, 1))])
def test_permute_and_reshape_copy(shape, perm):
    x = torch.randn(*shape)
    out = K.run("permute", x.cuda(), perm=perm).cpu()
    assert torch.equal(out, x.permute(perm).contiguous())
    flat = K.run("copy", x.cuda(), shape=(x.numel(),)).cpu()
    assert torch.equal(flat, x.reshape(-1))


def test_refusals():
    x = torch.ones(4)
    with pytest.raises(K.Unsupported):
        K.run("exp", x)
    with pytest.raises(K.Unsupported):
        K.run("log", x)
    with pytest.raises(K.Unsupported):
        K.run("tanh", x)


def test_raw_runtime_compiles_and_launches_with_validated_bindings():
    """Raw runtime on the device: strict-IEEE NVRTC kernel, launch through validated bindings, refusal of an
    aliased read/write pair before anything is launched."""
    import ctypes as C
    import numpy as np
    from scirust_b200.runtime import RawAccess, RawBinding, RawError, RawLaunchConfig, RawRuntime
    rt = RawRuntime(0)
    k = rt.compile('extern "C" __global__ void axpy(float* y, const float* x, float a, int n) {'
                   ' int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) y[i] = a * x[i] + y[i]; }', "axpy")
    n = 5000
    x = np.arange(n, dtype=np.float32) * 0.25
    y = np.ones(n, dtype=np.float32)
    bx, by = rt.allocate(4 * n), rt.allocate(4 * n)
    rt.write(bx, x.tobytes())
    rt.write(by, y.tobytes())
    cfg = RawLaunchConfig(((n + 255) // 256, 1, 1), (256, 1, 1))
    ev = rt.launch(k, cfg, [RawBinding(by, RawAccess.READ_WRITE), RawBinding(bx, RawAccess.READ)],
                   scalars=[C.c_float(3.0), C.c_int(n)])
    ev.synchronize()
    got = np.frombuffer(rt.read(by), dtype=np.float32)
    assert np.array_equal(got, np.float32(3.0) * x + y)          # mul then add, each rounded: no contraction
    with pytest.raises(RawError, match="alias"):
        rt.launch(k, cfg, [RawBinding(by, RawAccess.READ_WRITE), RawBinding(by, RawAccess.READ)],
                  scalars=[C.c_float(1.0), C.c_int(n)])
    with pytest.raises(RawError, match="threads"):
        rt.launch(k, RawLaunchConfig((1, 1, 1), (32, 64, 1)), [RawBinding(by, RawAccess.READ_WRITE),
                                                                 RawBinding(bx, RawAccess.READ)],
                  scalars=[C.c_float(1.0), C.c_int(n)])


def test_canonical_facade_conformance_device_equals_cpu_bit_for_bit():
    """Every conformance graph (element-wise with NaN / -0 / inf operands, matmul + permute + reshape, broadcast +
    ordered reduce, batched matmul) gives the CPU adapter's bits on the device adapter; exp / log are refused there."""
    from scirust_b200.canonical import Graph, ReferenceJitSession, run_conformance
    cpu, dev = run_conformance("cpu"), run_conformance("cuda")
    for name in cpu:
        for a, b in zip(cpu[name], dev[name]):
            nan = torch.isnan(a)                      # arithmetic NaNs agree in position; their payload is not defined
            assert torch.equal(torch.isnan(b), nan), name
            assert torch.equal(a.view(torch.int32)[~nan], b.view(torch.int32)[~nan]), name
    g = Graph()
    g.set_outputs(g.exp(g.input("x", (4,))))
    with pytest.raises(K.Unsupported):
        ReferenceJitSession("cuda").run(g, {"x": torch.zeros(4)})
    assert torch.allclose(ReferenceJitSession("cpu").run(g, {"x": torch.zeros(4)})[0], torch.ones(4))


def test_fused_elementwise_groups_run_as_one_generated_kernel_with_the_unfused_bits():
    """The fusion pass on the device adapter: each element-wise tree is ONE NVRTC-compiled kernel launched on views of
    the plan's arena; outputs equal the CPU adapter (fused or not) word for word, NaN positions included."""
    from scirust_b200.canonical import Graph, ReferenceJitSession, run_conformance
    g = Graph()
    a, b = g.input("x", (300, 77)), g.input("y", (300, 77))
    t = g.div(g.mul(g.add(a, b), g.sub(a, b)), g.scale(b, 0.3))
    r = g.relu(t)
    w = g.input("w", (77, 9))
    tail = g.scale(g.relu(g.matmul(r, w)), 2.0)
    g.set_outputs(tail, g.relu_grad(a, b), r)
    gen = torch.Generator().manual_seed(0)
    feeds = {"x": torch.randn(300, 77, generator=gen), "y": torch.randn(300, 77, generator=gen),
             "w": torch.randn(77, 9, generator=gen)}
    feeds["x"][0, 0], feeds["x"][0, 1], feeds["y"][0, 2] = float("nan"), -0.0, float("inf")
    cpu = ReferenceJitSession("cpu").run(g, feeds)
    sess = ReferenceJitSession("cuda", fuse=True)
    dev = [o.cpu() for o in sess.run(g, feeds)]
    assert sess.runtime._fused is not None and sess.runtime._fused.compiled == 2
    for p, q in zip(cpu, dev):
        nan = torch.isnan(p)
        assert torch.equal(torch.isnan(q), nan) and torch.equal(p.view(torch.int32)[~nan], q.view(torch.int32)[~nan])
    c0, c1 = run_conformance("cpu"), run_conformance("cuda", fuse=True)
    for name in c0:
        for p, q in zip(c0[name], c1[name]):
            nan = torch.isnan(p)
            assert torch.equal(torch.isnan(q), nan) and torch.equal(p.view(torch.int32)[~nan], q.view(torch.int32)[~nan])
