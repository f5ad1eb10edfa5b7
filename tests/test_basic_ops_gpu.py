"""Bandwidth-bound kernels against the fp32 PyTorch statement of the same op (the CPU path of
each op in scirust_b200.ops.basic is that statement)."""
import pytest
import torch

from scirust_b200 import ops

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _r(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF)


def _close(a, b, tol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    lim = tol * max(1.0, b.abs().max().item())
    assert err <= lim, f"max err {err} > {lim}"


@pytest.mark.parametrize("rows,cols", [(7, 256), (1000, 1024), (33, 4096), (5, 264)])
def test_rmsnorm_fwd_bwd(rows, cols):
    x, w, dy, dres = _r((rows, cols), 1), _r((cols,), 2), _r((rows, cols), 3), _r((rows, cols), 4)
    y_ref, inv_ref = ops.rmsnorm_fwd(x, w)
    y, inv = ops.rmsnorm_fwd(x.cuda(), w.cuda())
    _close(y, y_ref)
    assert torch.allclose(inv.cpu(), inv_ref, rtol=1e-4, atol=1e-6)
    dx_ref, dw_ref = ops.rmsnorm_bwd(dy, x, w, inv_ref, dres=dres)
    dx, dw = ops.rmsnorm_bwd(dy.cuda(), x.cuda(), w.cuda(), inv, dres=dres.cuda())
    _close(dx, dx_ref)
    assert torch.allclose(dw.cpu(), dw_ref, rtol=2e-3, atol=2e-2 * max(1.0, dw_ref.abs().max().item()) * 0.05)
    dx2, dw2 = ops.rmsnorm_bwd(dy.cuda(), x.cuda(), w.cuda(), inv, dres=dres.cuda())
    assert torch.equal(dw, dw2) and torch.equal(dx, dx2)


@pytest.mark.parametrize("dh", [64, 128])
def test_rope_roundtrip_and_reference(dh):
    rows, heads, kv = 96, 4, 2
    ld = (heads + 2 * kv) * dh
    x = _r((rows, ld), 5)
    cos_t, sin_t = ops.rope_table(64, dh, 10000.0, "cpu")
    ref = ops.rope_(x.clone(), heads + kv, dh, 32, cos_t, sin_t, offset=3)
    xg = x.cuda()
    cg, sg = ops.rope_table(64, dh, 10000.0, "cuda")
    ops.rope_(xg, heads + kv, dh, 32, cg, sg, offset=3)
    _close(xg, ref, 1e-2)
    assert torch.equal(xg[:, (heads + kv) * dh:].cpu(), x[:, (heads + kv) * dh:])  # v untouched
    ops.rope_(xg, heads + kv, dh, 32, cg, sg, offset=3, backward=True)
    _close(xg, x, 2e-2)
    pos = torch.randint(0, 64, (rows,), dtype=torch.int32)
    ref2 = ops.rope_(x.clone(), heads, dh, 32, cos_t, sin_t, positions=pos)
    x2 = x.cuda()
    ops.rope_(x2, heads, dh, 32, cg, sg, positions=pos.cuda())
    _close(x2, ref2, 1e-2)


def test_swiglu_and_add():
    gu, dh = _r((130, 2 * 2816), 6), _r((130, 2816), 7)
    _close(ops.swiglu_fwd(gu.cuda()), ops.swiglu_fwd(gu))
    _close(ops.swiglu_bwd(gu.cuda(), dh.cuda()), ops.swiglu_bwd(gu, dh))
    a, b = _r((64, 1024), 8), _r((64, 1024), 9)
    _close(ops.add(a.cuda(), b.cuda()), ops.add(a, b), 1e-2)


def test_embedding_fwd_bwd_deterministic():
    V, d, n = 500, 256, 4096
    table = _r((V, d), 10)
    tok = torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(0))
    tok[:100] = 7  # a long segment
    out = ops.embed_fwd(table.cuda(), tok.cuda())
    assert torch.equal(out.cpu(), table[tok])
    dy = _r((n, d), 11, 0.1)
    base = _r((V, d), 12, 0.1)
    ref = ops.embed_bwd(dy, tok, base.clone())
    g1 = ops.embed_bwd(dy.cuda(), tok.cuda(), base.clone().cuda())
    g2 = ops.embed_bwd(dy.cuda(), tok.cuda(), base.clone().cuda())
    assert torch.equal(g1, g2)
    _close(g1, ref, 2e-2)


@pytest.mark.parametrize("rows,cols", [(64, 32000), (17, 1000), (9, 128256)])
def test_cross_entropy(rows, cols):
    logits = _r((rows, cols), 13, 2.0)
    tgt = torch.randint(0, cols, (rows,), generator=torch.Generator().manual_seed(1))
    tgt[0] = cols + 5  # clamps
    tgt[1] = -1        # ignored
    loss_ref, d_ref = ops.ce_fwd_bwd(logits.clone(), tgt, 1.0 / rows)
    lg = logits.cuda()
    loss, d = ops.ce_fwd_bwd(lg, tgt.cuda(), 1.0 / rows)
    assert d.data_ptr() == lg.data_ptr()
    assert torch.allclose(loss.cpu(), loss_ref, rtol=1e-3, atol=1e-3)
    assert (d.float().cpu() - d_ref.float()).abs().max().item() <= 1e-2 / rows + 1e-6
    assert torch.allclose(ops.ce_loss_only(logits.cuda(), tgt.cuda()).cpu(), loss_ref, rtol=1e-3, atol=1e-3)


def test_sumsq_and_optimizer():
    n = 1_000_003
    g = _r((n,), 14, 0.01)
    s = ops.sumsq(g.cuda())
    assert abs(s.item() - g.float().pow(2).sum().item()) <= 1e-3 * s.item()
    assert torch.equal(s, ops.sumsq(g.cuda()))
    for mode in ("adamw", "adam", "sgd"):
        p = torch.randn(n, generator=torch.Generator().manual_seed(3))
        m, v = torch.zeros(n), torch.zeros(n)
        pg, mg, vg = p.cuda(), m.cuda(), v.cuda()
        pb = torch.empty(n, dtype=BF, device="cuda")
        for step in (1, 2):
            kw = dict(lr=1e-2, weight_decay=0.1, step=step, decay_end=n // 2, max_grad_norm=0.5, mode=mode)
            ops.optim_step(p, m, v, g, None, grad_sumsq=g.float().pow(2).sum().reshape(1), **kw)
            ops.optim_step(pg, mg, vg, g.cuda(), pb, grad_sumsq=s, **kw)
        assert torch.allclose(pg.cpu(), p, rtol=1e-4, atol=1e-5), mode
        assert torch.equal(pb.cpu(), pg.cpu().to(BF))
    # non-finite gradient norm skips the update
    before = pg.clone()
    ops.optim_step(pg, mg, vg, g.cuda(), pb, lr=1e-2, grad_sumsq=torch.tensor([float("nan")], device="cuda"))
    assert torch.equal(before, pg)


def test_deferred_status_raises_collective_timeout_one_poll_late():
    """A bounded wait that runs out leaves a code in the status word; the non-blocking reader used by the
    trainers turns it into CollectiveTimeout on the following poll, and the word is cleared."""
    import ctypes as C
    from scirust_b200.ops import _lib
    _lib.register("sb_wait_probe", [_lib.vp, _lib.i32, C.c_uint32, _lib.i32, _lib.vp, _lib.vp])
    dev = torch.device("cuda", 0)
    ds = _lib.DeferredStatus(dev)
    ds.poll()
    ds.poll()                                   # nothing recorded: no error
    flags = torch.zeros(16, dtype=torch.int32, device=dev)
    st = _lib.status_word(dev)
    _lib.call("sb_wait_probe", flags.data_ptr(), 2, 7, 50, st.data_ptr(), _lib.stream())   # waits 50 ms for nothing
    ds.poll()                                   # queues the copy behind the probe
    with pytest.raises(_lib.CollectiveTimeout):
        ds.poll()
    assert int(st.item()) == 0
    ds.poll()
    ds.poll()
