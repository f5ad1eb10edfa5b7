"""Op-graph fusion pass, fused linear bodies, Medusa / EAGLE drafting, tensor-train compression, CTC and the audio encoder."""
import pytest
import torch
import torch.nn.functional as F

from scirust_b200 import fusion as FU
from scirust_b200.nn import fused_ops as FO
from scirust_b200.nn import tensor_train as TT
from scirust_b200.nn.audio import AudioEncoder, CTCLossLastBlank, ctc_loss
from scirust_b200.nn.modules import Linear
from scirust_b200.nn.rng import PcgEngine
from scirust_b200.nn.speculative import EagleHead, MedusaHeads, generate_eagle, generate_greedy, generate_medusa
from scirust_b200.nn.zoo import NdDecoderLM


def test_fused_bodies_match_the_unfused_statement():
    torch.manual_seed(0)
    x, w, b = torch.randn(5, 8), torch.randn(8, 12), torch.randn(12)
    y = x @ w + b
    assert torch.allclose(FO.matmul_silu(x, w, b), F.silu(y), atol=1e-6)
    assert torch.allclose(FO.matmul_relu(x, w, b), y.clamp_min(0))
    assert torch.allclose(FO.matmul_gelu(x, w, b), F.gelu(y, approximate="tanh"), atol=1e-6)
    g, be = torch.randn(12), torch.randn(12)
    assert torch.allclose(FO.matmul_layernorm(x, w, b, g, be, 1e-5), F.layer_norm(y, (12,), g, be, 1e-5), atol=1e-5)
    w2, b2, g2, be2 = torch.randn(12, 6), torch.randn(6), torch.randn(6), torch.randn(6)
    ref = F.layer_norm(F.silu(y) @ w2 + b2, (6,), g2, be2, 1e-5)
    assert torch.allclose(FO.matmul_silu_layernorm(x, w, w2, b, b2, g2, be2), ref, atol=1e-5)
    s = torch.rand(12)
    assert torch.allclose(FO.matmul_scale(x, w, s), (x @ w) * s)
    assert torch.allclose(FO.run(FO.FusedKernelOp.MATMUL_RELU, x, w, b), y.clamp_min(0))
    # the reference's golden vectors: relu([1,2] @ [[1,0],[0,-1]]) = [1,0]; layernorm of [2,4] with gamma/beta
    assert FO.matmul_relu(torch.tensor([[1.0, 2.0]]), torch.tensor([[1.0, 0.0], [0.0, -1.0]])).tolist() == [[1.0, 0.0]]
    out = FO.matmul_layernorm(torch.tensor([[1.0, 1.0]]), torch.tensor([[2.0, 4.0], [0.0, 0.0]]), None,
                              torch.tensor([2.0, 3.0]), torch.tensor([10.0, 20.0]), 0.0)
    assert torch.allclose(out, torch.tensor([[8.0, 23.0]]))


def _mlp_graph():
    g = FU.OpGraph()
    x, w, b, ga, be = (g.add_input() for _ in range(5))
    lin = g.add(FU.OpKind.LINEAR, x, w, b)
    act = g.add(FU.OpKind.SILU, lin)
    ln = g.add(FU.OpKind.LAYERNORM, act, ga, be, constant=1e-5)
    w2 = g.add_input()
    mm = g.add(FU.OpKind.MATMUL, ln, w2)
    out = g.add(FU.OpKind.RELU, mm)
    feeds = {x: torch.randn(4, 8), w: torch.randn(8, 16), b: torch.randn(16), ga: torch.randn(16), be: torch.randn(16),
             w2: torch.randn(16, 5)}
    return g, feeds, (lin, act, ln, mm, out)


def test_fusion_pass_finds_chains_and_preserves_values():
    torch.manual_seed(1)
    g, feeds, (lin, act, ln, mm, out) = _mlp_graph()
    kernels = FU.FusionPipeline().fuse(g)
    assert [(k.kernel_type, k.group) for k in kernels] == [
        (FU.KernelType.MATMUL_SILU_LAYERNORM, [lin, act, ln]), (FU.KernelType.MATMUL_RELU, [mm, out])]
    assert kernels[0].inputs == [0, 1, 2, 3, 4] and kernels[0].op_count() == 3
    fused, plain = FU.execute(g, feeds, True), FU.execute(g, feeds, False)
    assert fused.keys() == plain.keys() == {out}
    assert torch.allclose(fused[out], plain[out], atol=1e-5)


def test_fusion_pass_keeps_observable_intermediates():
    g = FU.OpGraph()
    x, w = g.add_input(), g.add_input()
    mm = g.add(FU.OpKind.MATMUL, x, w)
    r = g.add(FU.OpKind.RELU, mm)
    g.mark_output(mm)                                   # the pre-activation is wanted: do not swallow it
    assert FU.FusionPipeline().fuse(g) == []
    # two consumers of the product: not fusable either
    g2 = FU.OpGraph()
    x, w = g2.add_input(), g2.add_input()
    mm = g2.add(FU.OpKind.MATMUL, x, w)
    g2.add(FU.OpKind.RELU, mm)
    g2.add(FU.OpKind.SILU, mm)
    assert FU.FusionPipeline().fuse(g2) == []
    feeds = {0: torch.randn(2, 3), 1: torch.randn(3, 4)}
    res = FU.execute(g2, feeds)
    assert torch.allclose(res[3], (feeds[0] @ feeds[1]).clamp_min(0))
    with pytest.raises(ValueError):
        g2.add(FU.OpKind.RELU, 99)
    with pytest.raises(KeyError):
        FU.execute(g2, {0: feeds[0]})


def test_fusion_patterns_residual_mlp_scale_norm_act_and_scan():
    torch.manual_seed(2)
    g = FU.OpGraph()
    x, w1, w2 = g.add_input(), g.add_input(), g.add_input()
    m1 = g.add(FU.OpKind.MATMUL, x, w1)
    m2 = g.add(FU.OpKind.MATMUL, m1, w2)
    res = g.add(FU.OpKind.ADD, m2, x)
    sc = g.add(FU.OpKind.SCALE, res, constant=0.5)      # add -> scale is not a pattern: stays separate
    ks = FU.FusionPipeline().fuse(g)
    assert [k.kernel_type for k in ks] == [FU.KernelType.TWO_LAYER_MLP] and ks[0].group == [m1, m2, res]
    feeds = {x: torch.randn(3, 6), w1: torch.randn(6, 7), w2: torch.randn(7, 6)}
    assert torch.allclose(FU.execute(g, feeds)[sc], ((feeds[x] @ feeds[w1] @ feeds[w2]) + feeds[x]) * 0.5, atol=1e-5)

    g = FU.OpGraph()
    x, w, ga, be = (g.add_input() for _ in range(4))
    s = g.add(FU.OpKind.SCALE, g.add(FU.OpKind.MATMUL, x, w), constant=3.0)
    a = g.add(FU.OpKind.TANH, g.add(FU.OpKind.LAYERNORM, s, ga, be))
    ks = FU.FusionPipeline().fuse(g)
    assert [k.kernel_type for k in ks] == [FU.KernelType.MATMUL_SCALE, FU.KernelType.LAYERNORM_ACTIVATION]
    feeds = {x: torch.randn(3, 4), w: torch.randn(4, 5), ga: torch.randn(5), be: torch.randn(5)}
    ref = torch.tanh(F.layer_norm(feeds[x] @ feeds[w] * 3.0, (5,), feeds[ga], feeds[be], 1e-5))
    assert torch.allclose(FU.execute(g, feeds)[a], ref, atol=1e-5)
    assert torch.allclose(FU.execute(g, feeds, False)[a], ref, atol=1e-5)

    # diagonal state-space scan: h <- a h + b x_t, y_t = c . h
    g = FU.OpGraph()
    xs, a_, b_, c_ = (g.add_input() for _ in range(4))
    y1 = g.add(FU.OpKind.SSM_STEP, xs, a_, b_, c_)
    y2 = g.add(FU.OpKind.SSM_STEP, y1, a_, b_, c_)
    ks = FU.FusionPipeline().fuse(g)
    assert [k.kernel_type for k in ks] == [FU.KernelType.SSM_SCAN]
    feeds = {xs: torch.tensor([1.0, 0.0, 0.0]), a_: torch.tensor([0.5, 0.25]), b_: torch.tensor([1.0, 1.0]), c_: torch.tensor([1.0, 2.0])}
    one = FU.execute(g, {**feeds}, False)
    assert torch.allclose(FU.execute(g, feeds)[y2], one[y2])
    # impulse response of the first scan: c.(a^t b) = 3, 1, 0.375
    g1 = FU.OpGraph()
    ins = [g1.add_input() for _ in range(4)]
    y = g1.add(FU.OpKind.SSM_STEP, *ins)
    assert torch.allclose(FU.execute(g1, dict(zip(ins, feeds.values())))[y], torch.tensor([3.0, 1.0, 0.375]))
    assert "matmul_silu_layernorm" in FU.high_gain_patterns(60.0) and "ssm_scan" not in FU.high_gain_patterns(1.0)
    assert FU.match_sequence([FU.OpKind.LINEAR, FU.OpKind.GELU]).kernel == FU.KernelType.MATMUL_GELU
    assert FU.match_sequence([FU.OpKind.ADD, FU.OpKind.MUL]) is None


def _trained_lm():
    torch.manual_seed(0)
    m = NdDecoderLM(12, 32, 2)
    seq = [1, 2, 3, 4, 5, 6, 7, 8] * 6
    t = torch.tensor([seq])
    opt = torch.optim.Adam(m.parameters(), 3e-3)
    for _ in range(150):
        opt.zero_grad()
        F.cross_entropy(m(t)[0, :-1], t[0, 1:]).backward()
        opt.step()
    return m, seq


def test_medusa_and_eagle_reproduce_greedy_with_fewer_forwards():
    m, seq = _trained_lm()
    greedy = generate_greedy(m, [1, 2, 3], 20)
    assert greedy[:5] == [4, 5, 6, 7, 8]
    blind = MedusaHeads(3, 32, 12, PcgEngine(5))
    out, f_blind = generate_medusa(m, blind, [1, 2, 3], 20)
    assert out == greedy                                         # verification makes any heads exact
    heads = MedusaHeads(3, 32, 12, PcgEngine(5))
    heads.fit(m, seq, 200, 1e-2)
    out, f = generate_medusa(m, heads, [1, 2, 3], 20)
    assert out == greedy and f < f_blind and heads.num_heads() == 3
    assert len(heads.propose(torch.zeros(32))) == 3
    eagle = EagleHead(32, PcgEngine(6))
    out0, f0 = generate_eagle(m, eagle, [1, 2, 3], 20, 4)
    eagle.fit(m, seq, 300, 1e-2)
    out1, f1 = generate_eagle(m, eagle, [1, 2, 3], 20, 4)
    assert out0 == greedy and out1 == greedy and f1 < f0
    out_k1, f_k1 = generate_eagle(m, eagle, [1, 2, 3], 7, 1)
    assert out_k1 == greedy[:7]
    with pytest.raises(ValueError):
        generate_eagle(m, eagle, [1], 3, 0)
    with pytest.raises(ValueError):
        generate_medusa(m, heads, [], 3)
    with pytest.raises(ValueError):
        MedusaHeads(0, 8, 8)


def test_tensor_train_decomposition():
    lin = Linear(6, 4)
    with torch.no_grad():
        lin.weight.copy_(torch.sin(torch.arange(24.0)).reshape(6, 4))
        lin.bias.copy_(torch.arange(4.0).reshape(1, 4))
    tt = TT.tt_decompose(lin, [2, 3], [2, 2], 100, 0.0)
    assert float((tt.full_weight() - lin.weight).detach().norm() / lin.weight.detach().norm()) < 1e-5
    x = torch.randn(3, 6)
    assert torch.allclose(tt(x), lin(x), atol=1e-5)
    lin2 = Linear(8, 16)
    with torch.no_grad():
        lin2.weight.copy_(torch.cos(torch.arange(128.0) * 0.13).reshape(8, 16))
    auto = TT.tt_decompose_auto(lin2, 2, 100, 0.0)
    assert auto.in_modes == [2, 4] and auto.out_modes == [4, 4]
    assert float((auto.full_weight() - lin2.weight).norm() / lin2.weight.norm()) < 1e-5
    # rank truncation trades error for parameters, monotonically
    errs, sizes = [], []
    torch.manual_seed(0)
    with torch.no_grad():
        lin2.weight.copy_(torch.randn(8, 16))
    for r in (1, 2, 4, 8):
        t = TT.tt_decompose_auto(lin2, 2, r, 0.0)
        errs.append(float((t.full_weight() - lin2.weight).norm()))
        sizes.append(TT.num_params(t))
    assert errs == sorted(errs, reverse=True) and sizes == sorted(sizes) and errs[-1] < 1e-4
    assert TT.compression_ratio(TT.tt_decompose_auto(lin2, 2, 1, 0.0)) > 3
    # a torch.nn.Linear ([out, in]) is accepted too; the tolerance drops negligible singular values
    tl = torch.nn.Linear(6, 4)
    t3 = TT.tt_decompose(tl, [2, 3], [2, 2], 100, 1e-6)
    assert torch.allclose(t3(x), tl(x), atol=1e-5)
    low = Linear(9, 9)
    with torch.no_grad():
        low.weight.copy_(torch.kron(torch.randn(3, 3), torch.randn(3, 3)))      # TT rank 1 by construction
    assert TT.tt_decompose(low, [3, 3], [3, 3], 100, 1e-5).ranks == [1, 1, 1]
    assert TT.auto_factorize(12, 2) == [3, 4] and TT.auto_factorize(7, 3) == [1, 1, 7] and TT.auto_factorize(64, 3) == [4, 4, 4]
    with pytest.raises(ValueError):
        TT.tt_decompose(lin, [2, 2], [2, 2], 4)


def test_ctc_matches_library_and_handles_edge_cases():
    torch.manual_seed(0)
    T, V = 12, 6
    lg = torch.randn(T, V, requires_grad=True)
    tg = torch.tensor([1, 1, 3, 0])
    loss = CTCLossLastBlank()(lg, tg)
    loss.backward()
    ref_in = lg.detach().clone().requires_grad_(True)
    ref = F.ctc_loss(torch.log_softmax(ref_in, -1)[:, None, :], tg[None], [T], [4], blank=V - 1, reduction="sum")
    ref.backward()
    assert float(loss) == pytest.approx(float(ref), rel=1e-5)
    assert torch.allclose(lg.grad, ref_in.grad, atol=1e-5)
    # batched, ragged
    lgb = torch.randn(3, T, V, requires_grad=True)
    tgb = torch.tensor([[1, 2, 3, 0], [2, 2, 0, 0], [4, 0, 0, 0]])
    il, tl = [12, 9, 5], [4, 2, 1]
    lb = ctc_loss(lgb, tgb, il, tl)
    lb.sum().backward()
    xb = lgb.detach().clone().requires_grad_(True)
    rb = F.ctc_loss(torch.log_softmax(xb, -1).transpose(0, 1), tgb, il, tl, blank=V - 1, reduction="none")
    rb.sum().backward()
    assert torch.allclose(lb, rb, rtol=1e-5) and torch.allclose(lgb.grad, xb.grad, atol=1e-5)
    # empty target: probability of all blanks
    e = ctc_loss(lg.detach(), torch.zeros(0, dtype=torch.int64))
    assert float(e) == pytest.approx(-float(torch.log_softmax(lg.detach(), -1)[:, V - 1].sum()), rel=1e-5)
    # three equal labels need five frames: two are not enough, the loss is infinite and the gradient zero
    short = torch.randn(2, V, requires_grad=True)
    inf = ctc_loss(short, torch.tensor([1, 1, 1]))
    inf.backward()
    assert torch.isinf(inf) and float(short.grad.abs().sum()) == 0.0
    # a sharply peaked alignment has near-zero loss
    peaked = torch.full((5, 4), -20.0)
    for t, k in enumerate([0, 3, 1, 3, 2]):
        peaked[t, k] = 20.0
    assert float(ctc_loss(peaked, torch.tensor([0, 1, 2]))) < 1e-3


def test_audio_encoder_shapes_and_state_dict():
    enc = AudioEncoder(1, 4, 8, 16, 20, PcgEngine(2))
    x = torch.randn(2, 320)
    y = enc(x)
    assert y.shape == (2, 8 * 4 * 5) and enc.out_hw(16, 20) == (4, 5) and float(y.min()) >= 0.0
    sd = enc.state_dict_ref()
    assert set(sd) == {"conv1.weight", "conv1.bias", "conv2.weight", "conv2.bias"} and sd["conv1.weight"].shape == (4, 9)
    other = AudioEncoder(1, 4, 8, 16, 20, PcgEngine(9))
    assert not torch.allclose(other(x), y)
    other.load_state_dict_ref(sd)
    assert torch.allclose(other(x), y)
    with pytest.raises(KeyError):
        other.load_state_dict_ref({"conv1.weight": sd["conv1.weight"]})
    with pytest.raises(ValueError):
        other.load_state_dict_ref({**sd, "conv2.weight": torch.zeros(3, 3)})
    y.sum().backward()
    assert enc.conv1.weight.grad is not None
