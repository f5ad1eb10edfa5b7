"""tcgen05 GEMM against a plain fp32 PyTorch reference, all operand forms."""
import pytest
import torch

from scirust_b200 import ops
from scirust_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _mk(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(torch.bfloat16)


def _check(y, ref, K):
    """Per-element bound: one bf16 rounding of the result (relative 2^-8, taken with a factor two) plus the fp32
    accumulation slack, which grows with sum |a||b| ~ 0.16 K for the N(0, 0.5^2) operands of these tests. A kernel
    that drops one 64-deep k-step is off by ~2 per element and fails this at any K; a bound on max|ref| would not."""
    _lib.check_status()
    err = (y.float() - ref).abs()
    tol = ref.abs() * 2.0 ** -7 + 2.0 ** -14 * 0.16 * K
    bad = err > tol
    assert not bool(bad.any()), f"{int(bad.sum())} elements off, worst {float((err - tol).max()):.4g} over its bound"


def _ints(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-2, 3, shape, generator=g, device="cuda").to(torch.bfloat16)


@pytest.mark.parametrize("pair", ["0", "1"])
@pytest.mark.parametrize("M,N", [(256, 256), (384, 520)])
def test_small_integer_operands_are_exact_in_every_form(pair, M, N, monkeypatch):
    """K = 64 with operands in {-2..2} (and all ones): every product and partial sum is an integer below 256,
    exact in fp32 and in bf16, so each operand form must return the integers themselves."""
    from scirust_b200.ops import gemm
    monkeypatch.setattr(gemm, "PAIR_MODE", pair)
    K = 64
    for mk in (_ints, lambda shape, seed: torch.ones(shape, dtype=torch.bfloat16, device="cuda")):
        a, b, at, bt = mk((M, K), 1), mk((K, N), 2), mk((K, M), 3), mk((N, K), 4)
        assert torch.equal(ops.matmul_nn(a, b).float(), a.float() @ b.float())
        assert torch.equal(ops.matmul_nt(a, bt).float(), a.float() @ bt.float().t())
        assert torch.equal(ops.matmul_tn(at, b, splits=1).float(), at.float().t() @ b.float())
        assert torch.equal(ops.matmul_tt_a(at, bt).float(), at.float().t() @ bt.float().t())
    _lib.check_status()


SHAPES = [(128, 128, 64), (256, 256, 256), (384, 512, 1024), (200, 264, 136), (2048, 1536, 1024), (1000, 5632, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_nn(M, N, K):
    x, w = _mk((M, K), 1), _mk((K, N), 2)
    _check(ops.matmul_nn(x, w), x.float() @ w.float(), K)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_nt(M, N, K):
    a, b = _mk((M, K), 3), _mk((N, K), 4)
    _check(ops.matmul_nt(a, b), a.float() @ b.float().t(), K)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_tn(M, N, K):
    a, b = _mk((K, M), 5), _mk((K, N), 6)
    _check(ops.matmul_tn(a, b, splits=1), a.float().t() @ b.float(), K)


@pytest.mark.parametrize("M,N,K", SHAPES[:4])
def test_tt_a(M, N, K):
    a, b = _mk((K, M), 7), _mk((N, K), 8)
    _check(ops.matmul_tt_a(a, b), a.float().t() @ b.float().t(), K)


def test_residual_and_bn128():
    x, w, r = _mk((512, 1024), 1), _mk((1024, 1024), 2), _mk((512, 1024), 9)
    ref = x.float() @ w.float() + r.float()
    _check(ops.matmul_nn(x, w, residual=r), ref, 1024)
    _check(ops.matmul_nn(x, w, residual=r, bn=128), ref, 1024)


def test_splitk_fixed_order_is_repeatable():
    a, b, r = _mk((8192, 1024), 5), _mk((8192, 1536), 6), _mk((1024, 1536), 3)
    ref = a.float().t() @ b.float() + r.float()
    y1 = ops.matmul_tn(a, b, residual=r, splits=8)
    y2 = ops.matmul_tn(a, b, residual=r, splits=8)
    _check(y1, ref, 8192)
    assert torch.equal(y1, y2)
    y3 = ops.matmul_tn(a, b, residual=r)  # heuristic split
    _check(y3, ref, 8192)


def test_strided_views():
    big = _mk((512, 3072), 11)
    x = big[:, 1024:2048]  # pitch 3072, offset 2048 bytes
    w = _mk((1024, 256), 12)
    out = torch.zeros((512, 1024), dtype=torch.bfloat16, device="cuda")
    ops.matmul_nn(x, w, out=out[:, 512:768])
    _lib.check_status()
    ref = x.float() @ w.float()
    assert (out[:, 512:768].float() - ref).abs().max().item() < 0.3
    assert out[:, :512].abs().max().item() == 0 and out[:, 768:].abs().max().item() == 0


PAIR_SHAPES = [(256, 256, 64), (512, 768, 512), (304, 264, 1000), (4096, 1536, 1024), (2176, 2816, 520)]


@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
@pytest.mark.parametrize("form", ["nn", "nt", "tn", "tt"])
def test_cta_pair_kernel_all_forms(M, N, K, form, monkeypatch):
    """The cta_group::2 kernel (256 x 256 tiles over two SMs) against fp32, same answers as the
    single-CTA kernel's contract; odd sizes exercise the zero-filled edges of both CTAs."""
    from scirust_b200.ops import gemm
    monkeypatch.setattr(gemm, "PAIR_MODE", "1")
    r = _mk((M, N), 11)
    if form == "nn":
        a, b = _mk((M, K), 1), _mk((K, N), 2)
        y, ref = ops.matmul_nn(a, b, residual=r), a.float() @ b.float()
    elif form == "nt":
        a, b = _mk((M, K), 3), _mk((N, K), 4)
        y, ref = ops.matmul_nt(a, b, residual=r), a.float() @ b.float().t()
    elif form == "tn":
        a, b = _mk((K, M), 5), _mk((K, N), 6)
        y, ref = ops.matmul_tn(a, b, residual=r, splits=1), a.float().t() @ b.float()
    else:
        a, b = _mk((K, M), 7), _mk((N, K), 8)
        y, ref = ops.matmul_tt_a(a, b, residual=r), a.float().t() @ b.float().t()
    _check(y, ref + r.float(), K)


def test_cta_pair_kernel_is_bitwise_repeatable_and_matches_single_cta(monkeypatch):
    from scirust_b200.ops import gemm
    x, w = _mk((4096, 1024), 1), _mk((1024, 2816), 2)
    monkeypatch.setattr(gemm, "BALANCED", False)
    monkeypatch.setattr(gemm, "PAIR_MODE", "1")
    y1 = ops.matmul_nn(x, w)
    y2 = ops.matmul_nn(x, w)
    monkeypatch.setattr(gemm, "PAIR_MODE", "0")
    y0 = ops.matmul_nn(x, w)
    _lib.check_status()
    assert torch.equal(y1, y2)
    # same K order and fp32 accumulation in both kernels: identical results
    assert torch.equal(y1, y0)


@pytest.mark.parametrize("M,N,K", [(16384, 1024, 1024), (1024, 1536, 16384), (2816, 1024, 8192), (200, 264, 136),
                                   (19072, 256, 512), (16, 6144, 4096)])
def test_balanced_schedule_matches_plain_schedule_bitwise(M, N, K, monkeypatch):
    """Whole waves one tile per CTA, the last partial wave dealt out in k-blocks and summed by the
    fix-up pass in k order: fp32 partial sums are added in a fixed order, so two runs agree bit for
    bit, and the result matches fp32 within bf16 rounding for every operand form."""
    from scirust_b200.ops import gemm
    monkeypatch.setattr(gemm, "PAIR_MODE", "0")
    monkeypatch.setattr(gemm, "BALANCED", True)
    monkeypatch.setattr(gemm, "_BALANCED_MIN_K", 0)
    x, w, r = _mk((M, K), 1), _mk((K, N), 2), _mk((M, N), 3)
    y1 = ops.matmul_nn(x, w, residual=r)
    y2 = ops.matmul_nn(x, w, residual=r)
    assert torch.equal(y1, y2)
    _check(y1, x.float() @ w.float() + r.float(), K)
    a, b = _mk((K, M), 5), _mk((K, N), 6)
    _check(ops.matmul_tn(a, b), a.float().t() @ b.float(), K)
    bt = _mk((N, K), 7)
    _check(ops.matmul_nt(x, bt), x.float() @ bt.float().t(), K)


@pytest.mark.parametrize("M,N,K", [(1024, 1536, 16384), (2816, 1024, 8192), (5632, 1024, 4096), (300, 520, 704)])
def test_cta_pair_kernel_with_balanced_schedule(M, N, K, monkeypatch):
    from scirust_b200.ops import gemm
    monkeypatch.setattr(gemm, "PAIR_MODE", "1")
    monkeypatch.setattr(gemm, "BALANCED", True)
    monkeypatch.setattr(gemm, "_BALANCED_MIN_K", 0)
    Mt = (M + 7) // 8 * 8
    a, b, r = _mk((K, Mt), 5), _mk((K, N), 6), _mk((Mt, N), 3)
    y1 = ops.matmul_tn(a, b, residual=r)
    y2 = ops.matmul_tn(a, b, residual=r)
    assert torch.equal(y1, y2)
    _check(y1, a.float().t() @ b.float() + r.float(), K)
    x, w = _mk((M, K), 1), _mk((K, N), 2)
    _check(ops.matmul_nn(x, w), x.float() @ w.float(), K)


@pytest.mark.parametrize("pair", ["0", "1"])
def test_bias_epilogue(pair, monkeypatch):
    from scirust_b200.ops import gemm
    monkeypatch.setattr(gemm, "PAIR_MODE", pair)
    x, w, b = _mk((640, 512), 1), _mk((512, 768), 2), _mk((768,), 3)
    _check(ops.matmul_nn(x, w, bias=b), x.float() @ w.float() + b.float()[None, :], 512)
    wt = _mk((768, 512), 4)
    _check(ops.matmul_nt(x, wt, bias=b), x.float() @ wt.float().t() + b.float()[None, :], 512)
    with pytest.raises(ValueError):
        ops.matmul_nn(x, w, bias=b, residual=_mk((640, 768), 5))


@pytest.mark.parametrize("M,K,ff", [(512, 256, 128), (4096, 1024, 2816), (1000, 512, 264)])
def test_swiglu_epilogue_is_bitwise_the_unfused_path(M, K, ff, monkeypatch):
    from scirust_b200.ops import basic, gemm
    monkeypatch.setattr(gemm, "FUSE_SWIGLU", True)
    x, wgu = _mk((M, K), 1), _mk((K, 2 * ff), 2)
    gu, act = ops.matmul_nn_swiglu(x, wgu)
    _lib.check_status()
    monkeypatch.setattr(gemm, "PAIR_MODE", "0")
    monkeypatch.setattr(gemm, "BALANCED", False)
    gu0 = ops.matmul_nn(x, wgu)
    act0 = basic.swiglu_fwd(gu0)
    assert torch.equal(gu, gu0)
    assert torch.equal(act, act0)
    _check(gu, x.float() @ wgu.float(), K)


@pytest.mark.parametrize("M,d,ff", [(512, 256, 128), (4096, 1024, 2816), (1000, 512, 264)])
def test_swiglu_backward_epilogue_is_bitwise_the_unfused_path(M, d, ff, monkeypatch):
    from scirust_b200.ops import basic, gemm
    monkeypatch.setattr(gemm, "FUSE_SWIGLU", True)
    dy, wd, gu = _mk((M, d), 1), _mk((ff, d), 2), _mk((M, 2 * ff), 3)
    dgu = ops.matmul_nt_swiglu_bwd(dy, wd, gu)
    _lib.check_status()
    monkeypatch.setattr(gemm, "PAIR_MODE", "0")
    monkeypatch.setattr(gemm, "BALANCED", False)
    ref = basic.swiglu_bwd(gu, ops.matmul_nt(dy, wd))
    assert torch.equal(dgu, ref)
