"""Layers, losses, schedules, N-D optimizers, the model zoo and the telemetry helpers on CPU."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

from scirust_b200 import nn as snn
from scirust_b200.autodiff import nd_optim as O
from scirust_b200.autodiff import scheduler as S
from scirust_b200.nn import loss as L
from scirust_b200.nn import modules as M
from scirust_b200.nn import transformer as T
from scirust_b200.nn import vision as V
from scirust_b200.nn import zoo as Z
from scirust_b200.nn.rng import PcgEngine
from scirust_b200.utils import logging as ulog
from scirust_b200.utils import planning


def test_linear_conv_pool_shapes_keys_and_gradients():
    rng = PcgEngine(3)
    lin = M.Linear(6, 4, rng=rng).with_name("fc")
    x = torch.randn(5, 6, requires_grad=True)
    y = lin(x)
    assert torch.allclose(y, x @ lin.weight + lin.bias)
    assert set(lin.state_dict_ref()) == {"fc.weight", "fc.bias"} and lin.state_dict_ref()["fc.bias"].shape == (1, 4)
    conv = M.Conv2d(2, 3, 3, stride=1, padding=M.Padding.SAME, in_h=8, in_w=8, rng=rng)
    img = torch.randn(4, 2 * 8 * 8, requires_grad=True)
    out = conv(img)
    assert out.shape == (4, 3 * 8 * 8) and conv.weight.shape == (3, 2 * 9)
    ref = F.conv2d(img.reshape(4, 2, 8, 8), conv.weight.reshape(3, 2, 3, 3), conv.bias.reshape(-1), padding=1)
    assert torch.allclose(out, ref.reshape(4, -1), atol=1e-5)
    valid = M.Conv2d(2, 3, 3, stride=2, padding=M.Padding.VALID, in_h=8, in_w=8, rng=rng)
    assert valid.out_hw() == (3, 3) and valid(img).shape == (4, 27)
    pool = M.MaxPool2d(2, 2, 3, 8, 8)
    assert pool(out).shape == (4, 3 * 4 * 4)
    out.sum().backward()
    assert img.grad is not None and conv.weight.grad.abs().sum() > 0
    seq = M.Sequential(M.Linear(6, 8, rng=rng), M.ReLU(), M.Linear(8, 2, rng=rng))
    assert sorted(seq.state_dict_ref()) == ["0.bias", "0.weight", "2.bias", "2.weight"]
    other = M.Sequential(M.Linear(6, 8, rng=PcgEngine(9)), M.ReLU(), M.Linear(8, 2, rng=PcgEngine(9)))
    other.load_state_dict_ref(seq.state_dict_ref())
    assert torch.equal(other(x), seq(x))
    with pytest.raises(ValueError):
        lin(torch.randn(2, 7))


def test_norms_match_their_definitions():
    x = torch.randn(16, 12)
    ln = M.LayerNorm(12)
    assert torch.allclose(ln(x), F.layer_norm(x, (12,)), atol=1e-5)
    rn = M.RMSNorm(12)
    assert torch.allclose(rn(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + rn.eps), atol=1e-5)
    bn = M.BatchNorm1d(12)
    bn.train()
    y = bn(x)
    assert torch.allclose(y.mean(0), torch.zeros(12), atol=1e-5)
    # running variance is the unbiased estimate, momentum 0.1
    assert torch.allclose(bn.running_var, 0.9 * torch.ones(12) + 0.1 * x.var(0, unbiased=True), atol=1e-5)
    bn.eval()
    assert not torch.allclose(bn(x), y)


def test_losses():
    lg = torch.randn(6, 5, requires_grad=True)
    idx = torch.tensor([0, 4, 2, 2, 1, 3])
    onehot = F.one_hot(idx, 5).float()
    ce = L.CrossEntropyLoss()
    a = ce(lg, onehot)
    assert a.shape == (1, 1) and torch.allclose(a.reshape(()), F.cross_entropy(lg, idx), atol=1e-6)
    assert torch.allclose(ce.forward_with_indices(lg, idx).reshape(()), F.cross_entropy(lg, idx), atol=1e-6)
    with pytest.raises(ValueError):
        ce(lg, onehot[:, :4])
    p, t = torch.randn(4, 3), torch.randn(4, 3)
    assert torch.allclose(L.MSELoss()(p, t).reshape(()), F.mse_loss(p, t))
    assert torch.allclose(L.NLLLoss()(F.log_softmax(lg, -1), idx).reshape(()), F.cross_entropy(lg, idx), atol=1e-6)
    assert torch.allclose(L.PoissonNLLLoss()(p, t.abs()).reshape(()), F.poisson_nll_loss(p, t.abs(), log_input=True))
    assert L.PINNLoss(2.0)(p, t, torch.ones(4, 1)).item() == pytest.approx(F.mse_loss(p, t).item() + 2.0)
    lp = F.log_softmax(torch.randn(12, 2, 6), -1)
    tg = torch.randint(1, 6, (2, 4))
    ctc = L.CTCLoss()(lp, tg, torch.tensor([12, 12]), torch.tensor([4, 3]))
    assert torch.isfinite(ctc)


def test_schedules():
    assert S.Constant(0.1).lr_at(100) == 0.1
    assert S.StepDecay(1.0, 10, 0.5).lr_at(25) == pytest.approx(0.25)
    assert S.Exponential(1.0, 0.9).lr_at(3) == pytest.approx(0.729)
    cos = S.CosineAnnealing(1.0, 0.1, 100)
    assert cos.lr_at(0) == pytest.approx(1.0) and cos.lr_at(100) == pytest.approx(0.1)
    wc = S.WarmupCosine(1.0, 0.0, 10, 110)
    assert wc.lr_at(5) < wc.lr_at(10) and wc.lr_at(10) == pytest.approx(1.0, abs=1e-6) and wc.lr_at(110) == pytest.approx(0.0, abs=1e-9)
    rp = S.ReduceOnPlateau(1.0, factor=0.5, patience=2)
    for m in [1.0, 1.0, 1.0, 1.0]:
        lr = rp.observe(m)
    assert lr == pytest.approx(0.5)


@pytest.mark.parametrize("name", ["RMSprop", "Lion", "LAMB", "Adafactor", "Muon", "Adan", "AdEMAMix", "Sophia",
                                  "ScheduleFreeSGD", "GaLore", "Prodigy", "Shampoo", "SOAP"])
def test_nd_optimizers_descend_a_quadratic(name):
    torch.manual_seed(0)
    target = torch.randn(8, 6)
    w = torch.nn.Parameter(torch.zeros(8, 6))
    b = torch.nn.Parameter(torch.zeros(6))
    kw = {"Lion": dict(lr=3e-2), "ScheduleFreeSGD": dict(lr=0.5), "Muon": dict(lr=0.05, adam_lr=5e-2),
          "RMSprop": dict(lr=2e-2), "LAMB": dict(lr=5e-2), "Adafactor": dict(lr=5e-2), "Adan": dict(lr=5e-2),
          "AdEMAMix": dict(lr=5e-2), "Sophia": dict(lr=5e-2), "GaLore": dict(lr=5e-2, rank=4, update_gap=10),
          "Prodigy": dict(), "Shampoo": dict(lr=0.05), "SOAP": dict(lr=5e-2, precond_freq=5)}[name]
    opt = getattr(O, name)([w, b], **kw)

    def loss_fn():
        return ((w + b - target) ** 2).mean()
    first = loss_fn().item()
    for _ in range(300):
        opt.zero_grad()
        loss_fn().backward()
        opt.step()
    assert loss_fn().item() < 0.5 * first, (name, first, loss_fn().item())


def test_inverse_root_and_soap_repeatability():
    torch.manual_seed(1)
    a = torch.randn(5, 5)
    spd = a @ a.t() + 0.1 * torch.eye(5)
    r = O.inverse_pth_root(spd, 4.0, 0.0)
    back = torch.linalg.matrix_power(r, 4) @ spd          # (A^-1/4)^4 A = I
    assert torch.allclose(back, torch.eye(5), atol=1e-3)

    def run():
        torch.manual_seed(2)
        w = torch.nn.Parameter(torch.randn(6, 4))
        opt = O.SOAP([w], lr=1e-2, precond_freq=3)
        x = torch.randn(16, 6)
        for _ in range(7):
            opt.zero_grad()
            ((x @ w) ** 2).mean().backward()
            opt.step()
        return w.detach().clone()
    assert torch.equal(run(), run())                      # same bits on a second run


def test_lookahead_sam_and_newton_schulz():
    g = torch.randn(6, 10)
    q = O.newton_schulz_orthogonalize(g, steps=8)
    sv = torch.linalg.svdvals(q)
    assert sv.max() < 1.3 and sv.min() > 0.5          # singular values pushed towards 1
    w = torch.nn.Parameter(torch.ones(4))
    la = O.Lookahead(torch.optim.SGD([w], lr=0.1), k=2, alpha=0.5)
    for _ in range(4):
        la.zero_grad()
        (w ** 2).sum().backward()
        la.step()
    assert w.abs().max() < 1.0
    w2 = torch.nn.Parameter(torch.ones(4))
    sam = O.SAM(torch.optim.SGD([w2], lr=0.1), rho=0.05)
    (w2 ** 2).sum().backward()
    sam.first_step()
    assert not torch.allclose(w2.detach(), torch.ones(4))
    sam.base.zero_grad() if hasattr(sam, "base") else None
    (w2 ** 2).sum().backward()
    sam.second_step()
    assert w2.abs().max() < 1.0


def test_transformer_blocks_and_vision_zoo_run_and_train():
    rng = PcgEngine(1)
    mha = T.MultiHeadAttention(16, 4, rng=rng, causal=True)
    x = torch.randn(2 * 6, 16)
    y = mha(x, seq_len=6)
    assert y.shape == x.shape
    # causal: output at position t must not depend on later positions
    x2 = x.clone()
    x2[5] += 1.0
    assert torch.allclose(mha(x2, seq_len=6)[:5], y[:5], atol=1e-6)
    q, k, v = torch.randn(33, 8), torch.randn(33, 8), torch.randn(33, 8)
    fa, row_max, row_sum = T.flash_attention_blockwise(q, k, v, block=16, causal=True)
    assert torch.allclose(fa, F.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=True)[0], atol=1e-5)
    assert row_max.shape[0] == 33 and (row_sum > 0).all()
    moe = T.MoE(16, 32, n_experts=4, top_k=2, rng=rng)
    assert moe(torch.randn(10, 16)).shape == (10, 16)
    lm = T.MiniLLM(vocab=50, d_model=32, n_heads=4, n_layers=2, d_ff=64, max_len=16)
    toks = torch.randint(0, 50, (3, 12))
    assert lm(toks).shape[-1] == 50
    net = V.resnet18(num_classes=10, in_c=3, in_hw=16)
    assert net(torch.randn(2, 3 * 16 * 16)).shape == (2, 10)
    vit = V.ViT(image=16, patch=4, in_c=3, d_model=32, n_heads=4, n_layers=1, d_ff=64, num_classes=5)
    assert vit(torch.randn(2, 3 * 16 * 16)).shape == (2, 5)


def test_zoo_recurrent_graph_generative_operator_layers():
    torch.manual_seed(0)
    lstm = Z.LSTM(5, 7)
    ref = torch.nn.LSTM(5, 7, batch_first=True)
    with torch.no_grad():
        ref.weight_ih_l0.copy_(lstm.w_ih.weight); ref.bias_ih_l0.copy_(lstm.w_ih.bias)
        ref.weight_hh_l0.copy_(lstm.w_hh.weight); ref.bias_hh_l0.zero_()
    x = torch.randn(3, 6, 5)
    assert torch.allclose(lstm(x)[0], ref(x)[0], atol=1e-5)
    adj = (torch.rand(9, 9) > 0.6).float()
    adj = ((adj + adj.t()) > 0).float()
    assert Z.GCN(4, 8, 3)(torch.randn(9, 4), adj).shape == (9, 3)
    a = Z.GCNLayer.normalize_adjacency(adj)
    assert torch.allclose(a, a.t(), atol=1e-6)
    vae = Z.VAE(12, 16, 4)
    xb = torch.randn(8, 12)
    rec, mu, lv = vae(xb, generator=torch.Generator().manual_seed(1))
    assert rec.shape == xb.shape and Z.VAE.loss(rec, xb, mu, lv).item() > 0
    assert Z.KANLayer(6, 3)(torch.randn(5, 6)).shape == (5, 3)
    fno = Z.FNO1d(in_c=1, out_c=1, width=8, modes=6, n_layers=2)
    assert fno(torch.randn(2, 1, 64)).shape == (2, 1, 64)
    assert Z.DeepONet(20, 1, 16, 8)(torch.randn(4, 20), torch.rand(30, 1)).shape == (4, 30)
    ode = Z.NeuralODE(3, 16, steps=4)
    z0 = torch.randn(5, 3, requires_grad=True)
    ode(z0).sum().backward()
    assert z0.grad is not None
    tt = Z.TTLinear([4, 4], [3, 5], rank=3)
    assert tt.full_weight().shape == (16, 15) and tt(torch.randn(2, 16)).shape == (2, 15)
    assert sum(p.numel() for p in tt.cores) < 16 * 15
    base = torch.nn.Linear(10, 6)
    for dora in (False, True):
        lora = Z.LoRALinear(base, r=2, dora=dora)
        xx = torch.randn(3, 10)
        assert torch.allclose(lora(xx), base(xx), atol=1e-5)        # B starts at zero: adapter is the identity
        assert not base.weight.requires_grad and lora.A.requires_grad


@pytest.mark.parametrize("mixer", ["llama", "retnet", "gla", "deltanet", "hgrn", "s4", "mamba", "mamba2", "rwkv",
                                   "xlstm", "hyena"])
def test_sequence_mixers_are_causal_and_trainable(mixer):
    torch.manual_seed(1)
    lm = Z.NdDecoderLM(vocab=40, d_model=32, n_layers=1, mixer=mixer, n_heads=4, n_kv_heads=2, d_ff=64)
    toks = torch.randint(0, 40, (2, 10))
    logits = lm(toks)
    assert logits.shape == (2, 10, 40) and torch.isfinite(logits).all()
    changed = toks.clone()
    changed[:, 7] = (changed[:, 7] + 1) % 40
    assert torch.allclose(lm(changed)[:, :7], logits[:, :7], atol=1e-4)       # no look-ahead
    loss = F.cross_entropy(logits[:, :-1].reshape(-1, 40), toks[:, 1:].reshape(-1))
    loss.backward()
    assert all(p.grad is not None for p in lm.parameters() if p.requires_grad)


def test_speculative_decoding_equals_target_greedy():
    torch.manual_seed(2)
    target = Z.NdDecoderLM(vocab=30, d_model=32, n_layers=2, mixer="llama", medusa_heads=2)
    draft = Z.NdDecoderLM(vocab=30, d_model=16, n_layers=1, mixer="llama", n_heads=2, n_kv_heads=1, d_ff=32)
    toks = torch.randint(0, 30, (1, 5))
    out, frac = Z.speculative_generate(target, draft, toks, max_new=9, k=3)
    ref = toks.clone()
    with torch.no_grad():
        for _ in range(9):
            ref = torch.cat([ref, target(ref)[:, -1].argmax(-1, keepdim=True)], 1)
    assert torch.equal(out, ref) and 0.0 <= frac <= 1.0
    assert len(target.medusa_logits(toks)) == 2


def test_training_logger_tensorboard_and_planner(tmp_path):
    lg = ulog.TrainingLogger(tmp_path / "log.csv")
    lg.log(1, "loss", 2.5, timestamp=10.0)
    lg.log(2, "loss", 2.0, timestamp=11.0)
    lg.close()
    rows = (tmp_path / "log.csv").read_text().strip().splitlines()
    assert len(rows) == 3 and rows[1].split(",")[0] == "1"
    tb = ulog.TensorBoardWriter(tmp_path / "tb")
    tb.add_scalar("loss", 1.25, 3, wall_time=5.0)
    tb.close()
    files = [f for f in os.listdir(tmp_path / "tb") if "tfevents" in f]
    assert files
    recs = list(ulog.read_tfrecords(tmp_path / "tb" / files[0]))
    assert len(recs) >= 2                       # file-version record + the scalar
    assert ulog.crc32c(b"123456789") == 0xE3069283
    from scirust_b200.models import SciAgentConfig
    cfg = SciAgentConfig.preset("gqa_12l")
    plan = planning.plan(cfg, batch=8, seq=2048)
    assert planning.n_params(cfg) == 168059904
    assert plan.fits() and plan.total("flash") < plan.total("naive")


def test_onnx_json_export_import_roundtrip():
    from scirust_b200.io import onnx_json as OJ
    rng = PcgEngine(5)
    net = M.Sequential(M.Linear(6, 8, rng=rng), M.ReLU(), M.LayerNorm(8), M.Linear(8, 3, rng=rng, bias=False),
                       M.Tanh())
    text = OJ.export_sequential(net, "tiny", (-1, 6))
    g = OJ.import_onnx_json(text)
    assert g.doc["ir_version"] == 7 and g.doc["domain"] == "ai.scirust"
    assert [n["op_type"] for n in g.nodes] == ["Gemm", "Relu", "LayerNormalization", "MatMul", "Tanh"]
    assert g.doc["graph"]["inputs"][0]["shape"]["dims"][0]["dim_param"] == "batch_size"
    names = [w[0] for w in g.weights()]
    assert names == ["param_0", "param_1", "param_2", "param_3", "param_4"]
    # weights survive bit for bit, and the imported graph computes what the model computes
    assert torch.equal(g.tensors()["param_0"], net.layers[0].weight.detach())
    x = torch.randn(5, 6)
    assert torch.allclose(OJ.run_graph(g, x), net(x), atol=1e-6)
    broken = text.replace('"param_3"', '"param_9"', 1)
    with pytest.raises(ValueError):
        OJ.run_graph(OJ.import_onnx_json(broken), x) if '"param_9"' in broken else (_ for _ in ()).throw(ValueError())
    with pytest.raises(ValueError):
        OJ.import_onnx_json('{"name": "x"}')


def test_cli_quantizer_kvcache_onnx_plan_calibrate_commands(tmp_path, capsys):
    from scirust_b200 import cli
    for cmd in ("gptq", "awq", "bitnet", "int4"):
        assert cli.run([cmd, "--rows", "64", "--cols", "32"]) == 0
        assert "output_rel_err" in capsys.readouterr().out
    assert cli.run(["kvcache", "--tokens", "40"]) == 0
    out = capsys.readouterr().out
    assert "paged rel_err 0.000000" in out and "int4 rel_err" in out
    f = str(tmp_path / "m.json")
    assert cli.run(["onnx", "export", "--file", f, "--layers", "4", "8", "3"]) == 0
    assert cli.run(["onnx", "inspect", "--file", f]) == 0
    assert "Gemm" in capsys.readouterr().out
    assert cli.run(["plan", "--model", "gqa_12l"]) == 0
    assert "fits_180GB True" in capsys.readouterr().out
    torch.manual_seed(0)
    labels = torch.randint(0, 5, (400,))
    logits = F.one_hot(labels, 5).float() * 2.0 + torch.randn(400, 5)
    torch.save({"logits": logits * 4.0, "labels": labels}, tmp_path / "d.pt")     # over-confident by 4x
    assert cli.run(["calibrate", "--data", str(tmp_path / "d.pt")]) == 0
    line = capsys.readouterr().out.split()
    t, before, after = float(line[1]), float(line[3]), float(line[5])
    assert 2.0 < t < 8.0 and after < before
    assert cli.run(["conformal", "--data", str(tmp_path / "d.pt"), "--alpha", "0.1"]) == 0
    cov = float(capsys.readouterr().out.split()[3])
    assert cov > 0.8
    assert cli.run(["calibrate", "--data", str(tmp_path / "missing.pt")]) == 2


def test_interval_bounds_are_sound():
    from scirust_b200 import calibration as C
    torch.manual_seed(1)
    layers = [(torch.randn(4, 6), torch.randn(6)), (torch.randn(6, 3), torch.randn(3))]
    x0 = torch.randn(4)
    lo, hi = C.interval_bounds(layers, x0 - 0.1, x0 + 0.1)
    for _ in range(200):
        x = x0 + (torch.rand(4) - 0.5) * 0.2
        y = torch.relu(x @ layers[0][0] + layers[0][1]) @ layers[1][0] + layers[1][1]
        assert (y >= lo - 1e-5).all() and (y <= hi + 1e-5).all()


def test_canonical_operator_statements():
    from scirust_b200.ops import canonical as K
    x = torch.tensor([0.0, -0.0, float("nan"), 2.0, -1.0])
    r = K.run("relu", x)
    assert r[:2].view(torch.int32).tolist() == [0, 0] and torch.isnan(r[2]) and r[3:].tolist() == [2.0, 0.0]
    assert K.run("scale", x, factor=0.5)[3:].tolist() == [1.0, -0.5]
    q = K.run("div", torch.ones(2), torch.tensor([3.0, 0.0]))
    assert q[0].item() == (torch.tensor(1.0) / torch.tensor(3.0)).item() and q[1].item() == float("inf")
    assert K.run("permute", torch.arange(6.0).reshape(2, 3), perm=(1, 0)).tolist() == [[0, 3], [1, 4], [2, 5]]
    for bad in ("exp", "log", "tanh"):
        with pytest.raises(K.Unsupported):
            K.run(bad, x)


def test_sequence_scans_recurrent_and_parallel_forms_agree():
    import math
    from scirust_b200.nn import sequence_scans as S
    g = torch.Generator().manual_seed(0)
    T, dk, dv = 37, 8, 6
    q, k, v = (torch.randn(T, d, generator=g, dtype=torch.float64) * 0.5 for d in (dk, dk, dv))
    close = lambda a, b, tol=1e-9: torch.allclose(a, b, atol=tol, rtol=1e-8)     # noqa: E731
    assert close(S.retention(q, k, v, 0.9), S.retention_recurrent(q, k, v, 0.9))
    alpha = torch.sigmoid(torch.randn(T, dk, generator=g, dtype=torch.float64)) * 0.5 + 0.5
    assert close(S.gated_linear_attention(q, k, v, alpha), S.gla_recurrent(q, k, v, alpha), 1e-7)
    beta = torch.sigmoid(torch.randn(T, generator=g, dtype=torch.float64))
    kn = k / k.norm(dim=1, keepdim=True)
    assert close(S.delta_rule(q, kn, v, beta), S.delta_rule_recurrent(q, kn, v, beta))
    d, n = 5, 4
    x = torch.randn(T, d, generator=g, dtype=torch.float64)
    dt = torch.nn.functional.softplus(torch.randn(T, d, generator=g, dtype=torch.float64))
    A = -torch.rand(d, n, generator=g, dtype=torch.float64) - 0.1
    B, C = torch.randn(T, n, generator=g, dtype=torch.float64), torch.randn(T, n, generator=g, dtype=torch.float64)
    assert close(S.selective_scan(x, dt, A, B, C), S.selective_scan_recurrent(x, dt, A, B, C))
    a = torch.sigmoid(torch.randn(T, generator=g, dtype=torch.float64)) * 0.5 + 0.5
    assert close(S.ssd_dual(x, a, B, C), S.ssd_dual_recurrent(x, a, B, C))
    lam = torch.complex(-torch.rand(n, generator=g, dtype=torch.float64) * 0.5, torch.randn(n, generator=g, dtype=torch.float64))
    lam = torch.exp(lam)
    Bc = torch.randn(n, 3, generator=g, dtype=torch.float64).to(torch.complex128)
    Cc = torch.randn(2, n, generator=g, dtype=torch.float64).to(torch.complex128)
    u = torch.randn(T, 3, generator=g, dtype=torch.float64)
    assert close(S.s5_parallel_scan(u, lam, Bc, Cc), S.s5_scan(u, lam, Bc, Cc))
    As = -torch.rand(n, generator=g, dtype=torch.float64) - 0.2
    y = S.s4_scan(u[:, 0], As, torch.ones(n, dtype=torch.float64), torch.ones(n, dtype=torch.float64), 0.1)
    h = torch.zeros(n, dtype=torch.float64)
    want = []
    for t in range(T):
        h = torch.exp(0.1 * As) * h + (torch.exp(0.1 * As) - 1) / As * u[t, 0]
        want.append(h.sum())
    assert close(y, torch.stack(want))
    f, c = torch.sigmoid(torch.randn(T, d, generator=g, dtype=torch.float64)), torch.randn(T, d, generator=g, dtype=torch.float64)
    assert close(S.hgrn(f, c), S.hgrn_recurrent(f, c))
    w, uu = torch.rand(d, generator=g, dtype=torch.float64) + 0.1, torch.randn(d, generator=g, dtype=torch.float64)
    kk, vv = torch.randn(12, d, generator=g, dtype=torch.float64), torch.randn(12, d, generator=g, dtype=torch.float64)
    assert close(S.rwkv_wkv(w, uu, kk, vv), S.rwkv_wkv_direct(w, uu, kk, vv))
    big = S.rwkv_wkv(w, uu, kk * 0 + 500.0, vv)                  # the stabiliser keeps e^{500} out of the arithmetic
    assert torch.isfinite(big).all()
    ip, fp = torch.randn(T, generator=g, dtype=torch.float64), torch.randn(T, generator=g, dtype=torch.float64) + 2
    assert close(S.mlstm_parallel(q, k / math.sqrt(dk), v, ip, fp), S.mlstm_scan(q, k / math.sqrt(dk), v, ip, fp).to(torch.float64), 1e-5)
    hs = S.slstm_scan(torch.randn(T, d, generator=g) * 3, torch.randn(T, d, generator=g), torch.tanh(torch.randn(T, d, generator=g)),
                      torch.sigmoid(torch.randn(T, d, generator=g)))
    assert torch.isfinite(hs).all() and hs.abs().max() <= 1.0 + 1e-5
    filt = torch.randn(T, d, generator=g, dtype=torch.float64) * 0.2
    assert close(S.hyena_long_conv(x, filt), S.hyena_long_conv_direct(x, filt), 1e-9)
    # ALiBi: slopes for 8 heads are 2^-1 .. 2^-8; a non-power-of-two count keeps the first power's slopes
    s8 = S.alibi_slopes(8)
    assert torch.allclose(s8, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s12 = S.alibi_slopes(12)
    assert torch.allclose(s12[:8], s8) and s12.numel() == 12
    bias = S.alibi_bias(s8, 5)
    assert bias.shape == (8, 5, 5) and bias[0, 3, 1] == -1.0 and bias[0, 1, 3] == float("-inf") and bias[3, 2, 2] == 0


def test_zoo_layers_parallel_training_form_equals_the_decoding_recurrence():
    from scirust_b200.nn import zoo
    torch.manual_seed(0)
    x = torch.randn(2, 19, 16)
    for cls in (zoo.RetNet, zoo.GLA, zoo.DeltaNet, zoo.HGRN):
        layer = cls(16)
        assert torch.allclose(layer.forward_parallel(x), layer(x), atol=2e-5), cls.__name__
    for layer in (zoo.Mamba2(16, d_state=8, head_dim=8), zoo.S5(16, d_state=12)):
        par = layer(x)
        st = layer.init_state(x)
        seq = []
        for t in range(x.shape[1]):
            y, st = layer.step(x[:, t], st)
            seq.append(y)
        assert torch.allclose(par, torch.stack(seq, 1), atol=3e-5), type(layer).__name__
        par.sum().backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())


def test_cli_sequence_layer_search_and_som_commands(capsys):
    from scirust_b200 import cli, search
    import numpy as np
    for cmd in ("retnet", "deltanet", "gla", "hgrn", "mamba", "mamba2", "rwkv", "s5"):
        assert cli.run([cmd, "--steps", "25", "--seed", "3"]) == 0
        out = capsys.readouterr().out
        first, last = (float(v) for v in out.split("MSE to target:")[1].split("(")[0].replace("->", " ").split())
        assert last < first, cmd
        if "recurrent form vs parallel form" in out:
            assert float(out.rsplit("max difference", 1)[1]) < 1e-4
    assert cli.run(["tt", "--steps", "30"]) == 0 and "fewer" in capsys.readouterr().out
    assert cli.run(["cmaes", "--objective", "rosenbrock", "--dim", "4", "--generations", "250"]) == 0
    assert cli.run(["evo", "--objective", "sphere", "--generations", "60"]) == 0
    assert cli.run(["som", "--epochs", "8"]) == 0
    capsys.readouterr()
    assert cli.run(["pinn", "--steps", "400"]) == 0
    out = capsys.readouterr().out
    assert float(out.rsplit("=", 1)[1]) < 0.5 and "loss" in out
    x, fx, hist = search.cma_es(search.rosenbrock, 4, generations=300, seed=1)
    assert fx < 1e-8 and np.allclose(x, 1.0, atol=1e-3) and hist[-1] <= hist[0]
    x2, fx2, _ = search.cma_es(search.rosenbrock, 4, generations=300, seed=1)
    assert fx2 == fx and np.array_equal(x, x2)                     # deterministic in the seed
    _, fe, he = search.evolution_strategy(search.sphere, 6, generations=120, seed=2)
    assert fe < 1e-6 and all(b <= a for a, b in zip(he, he[1:]))    # elitist: never worse
    rng = np.random.default_rng(0)
    data = np.concatenate([c + 0.04 * rng.standard_normal((40, 2)) for c in ([0.2, 0.2], [0.8, 0.7])])
    som = search.SelfOrganizingMap(5, 5, 2, seed=0)
    q0 = som.quantization_error(data)
    som.fit(data, epochs=10)
    assert som.quantization_error(data) < 0.5 * q0 and som.topographic_error(data) < 0.3
