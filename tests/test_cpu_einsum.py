"""Planned einsum: every pattern class against torch.einsum, the planner's costs, and input validation (CPU)."""
import pytest
import torch

from scirust_b200.einsum import ContractionPlan, EinsumError, einsum, parse_pattern

CASES = [("ij,jk->ik", [(3, 4), (4, 5)]), ("ij,jk", [(3, 4), (4, 5)]), ("ii->i", [(4, 4)]), ("ii", [(4, 4)]), ("ij->ji", [(3, 4)]),
         ("ij->", [(3, 4)]), ("bij,bjk->bik", [(2, 3, 4), (2, 4, 5)]), ("i,j->ij", [(3,), (4,)]), ("ij,ij->", [(3, 4), (3, 4)]),
         ("ijk,jl,kl->il", [(3, 4, 5), (4, 6), (5, 6)]), ("ab,bc,cd,de->ae", [(8, 2), (2, 9), (9, 3), (3, 7)]),
         ("bhqd,bhkd->bhqk", [(2, 3, 4, 5), (2, 3, 6, 5)]), ("iij,jk->ik", [(3, 3, 4), (4, 5)]), ("ij,k->ijk", [(2, 3), (4,)]),
         ("abc,cde,efg,gha->bdfh", [(2, 3, 4), (4, 2, 3), (3, 2, 4), (4, 3, 2)]), ("i,i,i->i", [(5,), (5,), (5,)]),
         ("ij,jk,kl,lm,mn,no,op->ip", [(2, 3), (3, 4), (4, 5), (5, 2), (2, 3), (3, 4), (4, 2)]), ("ijk->kj", [(2, 3, 4)]),
         ("ij,j->i", [(3, 4), (4,)]), (" i j , j k -> i k ", [(2, 3), (3, 2)])]


@pytest.mark.parametrize("pattern,shapes", CASES)
def test_matches_torch_einsum_under_every_planner(pattern, shapes):
    g = torch.Generator().manual_seed(len(pattern))
    ts = [torch.randn(*s, dtype=torch.float64, generator=g) for s in shapes]
    ref = torch.einsum(pattern.replace(" ", ""), *ts)
    for method in ("auto", "greedy", "left"):
        got = einsum(pattern, *ts, method=method)
        assert got.shape == ref.shape and torch.allclose(got, ref, atol=1e-10), method


def test_planner_picks_the_cheap_order_and_reports_costs():
    shapes = [(1000, 2), (2, 1000), (1000, 3)]
    best, left = ContractionPlan.new("ab,bc,cd->ad", shapes), ContractionPlan.new("ab,bc,cd->ad", shapes, "left")
    assert best.method == "optimal" and (best.flops, best.peak_elements) == (12000, 3000)
    assert (left.flops, left.peak_elements) == (5_000_000, 1_000_000)
    assert [(s.left, s.right) for s in best.steps] == [(1, 2), (0, 1)]
    assert ContractionPlan.new("ab,bc,cd->ad", shapes, "greedy").flops == 12000
    chain = ContractionPlan.new("ab,bc,cd,de,ef,fg,gh->ah", [(4, 50), (50, 3), (3, 60), (60, 2), (2, 70), (70, 5), (5, 9)])
    assert chain.method == "greedy" and chain.flops < ContractionPlan.new("ab,bc,cd,de,ef,fg,gh->ah", [(4, 50), (50, 3), (3, 60), (60, 2), (2, 70), (70, 5), (5, 9)], "left").flops
    plan = ContractionPlan.new("bij,bjk->bik", [(2, 3, 4), (2, 4, 5)])
    a, b = torch.randn(2, 3, 4), torch.randn(2, 4, 5)
    assert torch.allclose(plan.execute(a, b), torch.bmm(a, b), atol=1e-6)       # a plan is reusable across calls
    nc = a.transpose(1, 2).contiguous().transpose(1, 2)                         # non-contiguous operand, same values
    assert torch.allclose(plan.execute(nc, b), torch.bmm(a, b), atol=1e-6)


def test_gradients_flow_through_the_lowered_products():
    a = torch.randn(3, 4, dtype=torch.float64, requires_grad=True)
    b = torch.randn(4, 5, dtype=torch.float64, requires_grad=True)
    c = torch.randn(5, 3, dtype=torch.float64, requires_grad=True)
    einsum("ij,jk,ki->", a, b, c).backward()
    ga, gb, gc = a.grad.clone(), b.grad.clone(), c.grad.clone()
    for t in (a, b, c):
        t.grad = None
    torch.einsum("ij,jk,ki->", a, b, c).backward()
    assert torch.allclose(ga, a.grad) and torch.allclose(gb, b.grad) and torch.allclose(gc, c.grad)


def test_malformed_patterns_and_shapes_are_rejected():
    assert parse_pattern("ij,jk", 2) == ([["i", "j"], ["j", "k"]], ["i", "k"])
    a, b = torch.zeros(2, 3), torch.zeros(4, 5)
    for pattern, ops in (("ij,jk->ik", (a, b)), ("ij->ik", (a,)), ("ij,jk->ik", (a,)), ("ijk->i", (a,)), ("ij->ii", (a,)), ("i1->i", (a,))):
        with pytest.raises(EinsumError):
            einsum(pattern, *ops)
    with pytest.raises(EinsumError):
        ContractionPlan.new("ij,jk->ik", [(2, 3), (3, 4)]).execute(torch.zeros(2, 3))
    with pytest.raises(EinsumError):
        ContractionPlan.new("ij,jk->ik", [(2, 3), (3, 4)], "random")
