"""Fixed-point tensors: rounding / overflow rules against exact rational arithmetic, order-independent reductions,
integer transcendental functions within an ulp or two, and a whole integer MLP (CPU)."""
from fractions import Fraction

import pytest
import torch

from scirust_b200 import fixed as FX
from scirust_b200.fixed import FixedOverflow, FixedTensor


def _round(fr: Fraction, mode: str) -> int:
    fl = fr.numerator // fr.denominator
    rem = fr - fl
    if mode == "floor" or rem == 0:
        return fl
    if mode == "ceil":
        return fl + 1
    if mode == "toward_zero":
        return fl + 1 if fr < 0 else fl
    return fl + 1 if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2) else fl


def test_round_shift_and_narrow_follow_the_four_rounding_and_three_overflow_modes():
    vals = torch.tensor([-13, -12, -11, -10, -9, -8, -1, 0, 1, 8, 9, 10, 11, 12, 13], dtype=torch.int64)
    for mode in FX.ROUNDINGS:
        got = FX.round_shift(vals, 2, mode).tolist()
        assert got == [_round(Fraction(int(v), 4), mode) for v in vals], mode
    wide = torch.tensor([FX.I32_MAX + 5, FX.I32_MIN - 5, 7], dtype=torch.int64)
    assert FX.narrow(wide, "saturate").tolist() == [FX.I32_MAX, FX.I32_MIN, 7]
    assert FX.narrow(wide, "wrap").tolist() == [FX.I32_MIN + 4, FX.I32_MAX - 4, 7]
    with pytest.raises(FixedOverflow):
        FX.narrow(wide, "checked")
    with pytest.raises(FixedOverflow):
        FixedTensor.from_float(torch.tensor([1e6]), 16)
    assert FixedTensor.from_float(torch.tensor([0.5 / 65536, 1.5 / 65536]), 16).raw.tolist() == [0, 2]   # ties to even


def test_mul_and_div_round_the_exact_result_once():
    g = torch.Generator().manual_seed(0)
    a = FixedTensor(torch.randint(-(1 << 20), 1 << 20, (200,), generator=g, dtype=torch.int32), 12)
    b = FixedTensor(torch.randint(1 << 10, 1 << 20, (200,), generator=g, dtype=torch.int32) * (1 - 2 * torch.randint(0, 2, (200,), generator=g, dtype=torch.int32)), 12)
    for mode in FX.ROUNDINGS:
        m = a.mul(b, mode, "checked").raw.tolist()
        d = a.div(b, mode, "checked").raw.tolist()
        for i in range(200):
            x, y = int(a.raw[i]), int(b.raw[i])
            assert m[i] == _round(Fraction(x * y, 1 << 12), mode)
            assert d[i] == _round(Fraction(x << 12, y), mode)
    with pytest.raises(ZeroDivisionError):
        a.div(FixedTensor(torch.zeros(200, dtype=torch.int32), 12))
    with pytest.raises(ValueError):
        a.add(a.rescale(10))
    assert a.rescale(20).rescale(12) == a                                        # widening is exact
    assert (a + b - b) == a and (-a).neg() == a


def test_dot_and_matmul_do_not_depend_on_order_or_tiling():
    g = torch.Generator().manual_seed(1)
    a = FixedTensor.from_float(torch.randn(7, 300, generator=g, dtype=torch.float64), 16)
    b = FixedTensor.from_float(torch.randn(300, 5, generator=g, dtype=torch.float64), 16)
    ref = a.matmul(b, chunk=300)
    assert a.matmul(b, chunk=7) == ref and a.matmul(b, chunk=64) == ref
    perm = torch.randperm(300, generator=g)
    assert FixedTensor(a.raw[:, perm], 16).matmul(FixedTensor(b.raw[perm], 16)) == ref
    col = FixedTensor(b.raw[:, 2].contiguous(), 16)
    assert torch.equal(FixedTensor(a.raw[3], 16).dot(col).raw, ref.raw[3, 2])
    assert float((ref.to_float() - a.to_float() @ b.to_float()).abs().max()) < 300 * 2.0 ** -16
    assert a.sum(-1) == FixedTensor(a.raw[:, perm], 16).sum(-1)


def test_integer_transcendentals_stay_within_two_units_in_the_last_place():
    for frac, lim, top in ((16, 8.0, 30000.0), (24, 3.0, 100.0)):
        u = 2.0 ** -frac
        x = FixedTensor.from_float(torch.linspace(-lim, lim, 2001, dtype=torch.float64), frac)
        p = FixedTensor.from_float(torch.linspace(0.001, top, 2001, dtype=torch.float64), frac)
        xf, pf = x.to_float(), p.to_float()
        for got, want in ((x.exp(), xf.exp()), (x.exp2(), xf.exp2()), (p.ln(), pf.log()), (p.log2(), pf.log2()),
                          (x.sin(), xf.sin()), (x.cos(), xf.cos()), (x.sigmoid(), xf.sigmoid()), (x.tanh(), xf.tanh()),
                          (p.sqrt(), pf.sqrt())):
            assert float((got.to_float() - want).abs().max()) <= 2 * u
    ext = FixedTensor.from_float(torch.tensor([-30000.0, -50.0, 20.0, 30000.0]), 16)
    assert ext.exp().raw.tolist() == [0, 0, FX.I32_MAX, FX.I32_MAX]               # underflow to zero, saturation
    assert ext.tanh().to_float().tolist() == [-1.0, -1.0, 1.0, 1.0]
    assert float((ext.sin().to_float() - ext.to_float().sin()).abs().max()) < 1e-3      # range reduction of large angles
    bad = FixedTensor.from_float(torch.tensor([0.0, -1.0]), 16)
    assert bad.ln().raw.tolist() == [FX.I32_MIN, FX.I32_MIN] and bad.sqrt().raw.tolist() == [0, 0]
    sq = FixedTensor.from_int(torch.tensor([0, 1, 4, 9, 144]), 16).sqrt()
    assert sq.to_float().tolist() == [0.0, 1.0, 2.0, 3.0, 12.0]                   # perfect squares are exact


def test_softmax_norms_and_an_integer_mlp_track_the_float_model():
    g = torch.Generator().manual_seed(2)
    z = torch.randn(6, 33, generator=g, dtype=torch.float64) * 3
    sm = FixedTensor.from_float(z, 20).softmax()
    assert float((sm.to_float() - torch.softmax(z, -1)).abs().max()) < 4 * 2.0 ** -20
    assert float((sm.to_float().sum(-1) - 1).abs().max()) < 40 * 2.0 ** -20
    x = FixedTensor.from_float(z, 16)
    gam = FixedTensor.from_float(torch.rand(33, generator=g, dtype=torch.float64) + 0.5, 16)
    bet = FixedTensor.from_float(torch.randn(33, generator=g, dtype=torch.float64), 16)
    ln_ref = torch.nn.functional.layer_norm(x.to_float(), (33,), gam.to_float(), bet.to_float(), 1e-5)
    assert float((FX.layer_norm(x, gam, bet).to_float() - ln_ref).abs().max()) < 2e-3
    rms_ref = x.to_float() / torch.sqrt((x.to_float() ** 2).mean(-1, keepdim=True) + 1e-5) * gam.to_float()
    assert float((FX.rmsnorm(x, gam).to_float() - rms_ref).abs().max()) < 2e-3
    torch.manual_seed(3)
    seq = torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.ReLU(), torch.nn.Linear(32, 16), torch.nn.Tanh(),
                              torch.nn.Linear(16, 4), torch.nn.Softmax(-1)).double()
    inp = torch.randn(9, 12, generator=g, dtype=torch.float64)
    fm = FX.FixedMlp.from_float(seq, 16)
    out = fm(inp)
    assert float((out.to_float() - seq(inp)).abs().max()) < 2e-3
    assert torch.equal(out.argmax(-1), seq(inp).argmax(-1))
    assert fm(inp) == out                                                        # same bits every time
    with pytest.raises(ValueError):
        FX.FixedMlp.from_float(torch.nn.Sequential(torch.nn.GELU()))
