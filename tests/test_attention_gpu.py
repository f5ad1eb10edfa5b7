"""tcgen05 flash attention against the dense fp32 PyTorch reference."""
import pytest
import torch

from scirust_b200.ops import _lib, attention as A

pytestmark = pytest.mark.gpu


def _qkv(B, S, H, Hkv, dh, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(B * S, (H + 2 * Hkv) * dh, generator=g, device="cuda").to(torch.bfloat16)


CASES = [(1, 128, 1, 1, 64), (2, 256, 4, 2, 64), (1, 1000, 4, 1, 64), (2, 2048, 16, 4, 64), (1, 384, 4, 2, 128),
         (1, 200, 2, 2, 128)]


@pytest.mark.parametrize("B,S,H,Hkv,dh", CASES)
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("two_tiles", [True, False])
def test_forward(B, S, H, Hkv, dh, causal, two_tiles, monkeypatch):
    # two_tiles: the head-dimension-64 kernel with two query tiles per CTA; otherwise the one-tile kernel
    if dh != 64 and two_tiles:
        pytest.skip("the two-tile kernel covers head dimension 64")
    monkeypatch.setattr(A, "FWD_TWO_TILES", two_tiles)
    qkv = _qkv(B, S, H, Hkv, dh)
    o, lse = A.attention_fwd(qkv, B, S, H, Hkv, dh, causal=causal)
    _lib.check_status()
    o_ref, lse_ref = A.attention_ref(qkv, B, S, H, Hkv, dh, causal=causal)
    assert (o.float() - o_ref).abs().max().item() < 3e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2
    o2, _ = A.attention_fwd(qkv, B, S, H, Hkv, dh, causal=causal)
    assert torch.equal(o, o2)


@pytest.mark.parametrize("causal", [True, False])
def test_forward_growing_maxima(causal, monkeypatch):
    # keys grow along the sequence, so row maxima rise by more than 2^8 from block to block and the
    # output accumulator in tensor memory is rescaled many times
    monkeypatch.setattr(A, "FWD_TWO_TILES", True)
    B, S, H, Hkv, dh = 2, 1024, 4, 2, 64
    qkv = _qkv(B, S, H, Hkv, dh, seed=5).float().reshape(B, S, H + 2 * Hkv, dh)
    ramp = (1.0 + 6.0 * torch.arange(S, device="cuda") / S).reshape(1, S, 1, 1)
    qkv[:, :, H:H + Hkv] *= ramp
    qkv = qkv.reshape(B * S, -1).to(torch.bfloat16)
    o, lse = A.attention_fwd(qkv, B, S, H, Hkv, dh, causal=causal)
    _lib.check_status()
    o_ref, lse_ref = A.attention_ref(qkv, B, S, H, Hkv, dh, causal=causal)
    assert (o.float() - o_ref).abs().max().item() < 3e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2
    monkeypatch.setattr(A, "FWD_TWO_TILES", False)
    o1, lse1 = A.attention_fwd(qkv, B, S, H, Hkv, dh, causal=causal)
    assert (o.float() - o1.float()).abs().max().item() < 2e-2 and (lse - lse1).abs().max().item() < 1e-3


@pytest.mark.parametrize("B,S,H,Hkv,dh", CASES)
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("spill", [True, False])
def test_backward(B, S, H, Hkv, dh, causal, spill, monkeypatch):
    # spill: dQ streams the dS tiles stored by the dK/dV kernel; otherwise it recomputes the scores
    monkeypatch.setattr(A, "DS_SCRATCH_LIMIT_BYTES", (4 << 30) if spill else 0)
    qkv = _qkv(B, S, H, Hkv, dh, seed=1)
    g = torch.Generator(device="cuda").manual_seed(2)
    do = torch.randn(B * S, H * dh, generator=g, device="cuda").to(torch.bfloat16)
    o, lse = A.attention_fwd(qkv, B, S, H, Hkv, dh, causal=causal)
    d = A.attention_bwd(qkv, o, lse, do, B, S, H, Hkv, dh, causal=causal)
    _lib.check_status()
    ref = A.attention_bwd_ref(qkv, do, B, S, H, Hkv, dh, causal=causal)
    err = (d.float() - ref).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.abs().max().item()), err
    d2 = A.attention_bwd(qkv, o, lse, do, B, S, H, Hkv, dh, causal=causal)
    assert torch.equal(d, d2)
