"""The benchmark's reference arm: the reference's own CUDA-C kernels (read from baseline/_ref at run time,
NVRTC-compiled) driven in the reference's call order must reproduce a plain fp32 PyTorch statement of the
same decoder, and its training step must lower the loss."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from baseline import reference_replay as R  # noqa: E402

pytestmark = pytest.mark.gpu

needs_ref = pytest.mark.skipif(not (R.REF_ROOT / "scirust-cuda" / "src" / "chain.rs").exists(),
                               reason="reference sources are not staged under baseline/_ref")


def _torch_loss(model, tokens, targets, B, S):
    cfg = model.cfg
    dh = cfg.d_model // cfg.n_heads
    x = model.embedding.float()[tokens.long().cuda()]
    pos = torch.arange(S, device="cuda").float()
    freq = cfg.theta ** (-2.0 * torch.arange(dh // 2, device="cuda").float() / dh)
    ang = pos[:, None] * freq[None, :]
    cos, sin = ang.cos(), ang.sin()

    def rope(t, nh):
        t = t.view(B, S, nh, dh // 2, 2)
        x0, x1 = t[..., 0], t[..., 1]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).view(B, S, nh, dh)

    def norm(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float().view(-1)
    for b in model.blocks:
        xn = norm(x, b["norm1"])
        q = rope(xn @ b["wq"].float(), cfg.n_heads)
        k = rope(xn @ b["wk"].float(), cfg.n_kv_heads)
        v = (xn @ b["wv"].float()).view(B, S, cfg.n_kv_heads, dh)
        rep = cfg.n_heads // cfg.n_kv_heads
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        sc = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(dh)
        sc = sc.masked_fill(torch.triu(torch.ones(S, S, device="cuda", dtype=torch.bool), 1), float("-inf"))
        ctx = torch.einsum("bhqk,bkhd->bqhd", sc.softmax(-1), v).reshape(B * S, cfg.d_model)
        x = x + ctx @ b["wo"].float()
        hn = norm(x, b["norm2"])
        x = x + (torch.nn.functional.silu(hn @ b["wg"].float()) * (hn @ b["wu"].float())) @ b["wd"].float()
    logits = norm(x, model.final_norm) @ model.embedding.float().t()
    return torch.nn.functional.cross_entropy(logits, targets.long().cuda()).item()


@needs_ref
def test_replay_forward_matches_fp32_statement_and_training_lowers_loss():
    chain = R.Chain()
    cfg = R.PRESETS["tiny"]
    model = R.RefModel(cfg, chain, seed=3, std=0.08)
    B, S = 2, 32
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab, (B, S + 1), generator=g)
    tokens = tok[:, :-1].reshape(-1).to(torch.int32)
    targets = tok[:, 1:].reshape(-1).to(torch.int32)
    want = _torch_loss(model, tokens, targets, B, S)
    logits, _ = model.forward_train(tokens, B, S)
    loss_rows, _ = chain.cross_entropy_loss_grad_resident(logits, targets)
    got = R.RefTrainer.finish_step_diagnostics(loss_rows)
    assert abs(got - want) < 0.03 * want, (got, want)
    trainer = R.RefTrainer(model, lr=3e-3)
    losses = []
    for _ in range(6):
        rows, _ = trainer.train_step_batch_deferred(tokens, targets, B, S)
        losses.append(trainer.finish_step_diagnostics(rows))
    assert losses[-1] < losses[0] - 0.05, losses


@needs_ref
def test_replay_cached_decode_equals_full_recompute():
    chain = R.Chain()
    cfg = R.PRESETS["tiny"]
    model = R.RefModel(cfg, chain, seed=5, std=0.08, masters=False)
    prompt = torch.randint(1, cfg.vocab, (24,), generator=torch.Generator().manual_seed(1)).to(torch.int32)
    toks = model.generate_cached(prompt, 6)
    # full recompute through the cached-attention kernels (the reference's parity contract: same tokens)
    seq = prompt.tolist()
    for _ in range(6):
        L = cfg.n_layers
        logits = model.prefill_cached(torch.tensor(seq, dtype=torch.int32), [None] * L, [None] * L)
        seq.append(model.greedy(logits))
    assert toks == seq
