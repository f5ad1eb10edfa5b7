"""Measured selection of a GEMM configuration with the evidence-based autotuner.

    python examples/autotune_gemm.py --m 16384 --n 1024 --k 1024 --plans ./plans --mode learn

Candidates are the router's own choice plus explicit (column tile, split-K) settings of the single-CTA tcgen05 kernel
(``splits = 0`` is the balanced last-wave schedule). Every candidate is first checked against an fp32 product (the
check's summary becomes the plan's correctness evidence), then raced by successive halving under a device-timestamp
protocol with an L2 flush before every sample. The winning plan is stored under a key made of the hardware profile, the
problem class and the objective; ``--mode locked`` replays a stored plan without measuring. On a machine without a
GPU the products run through the fp32 statement and all candidates tie (useful only to see the flow).
"""
import argparse
import hashlib
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from scirust_b200.compute import autotune as AT
from scirust_b200.compute import hardware as H
from scirust_b200.ops import gemm as G


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--plans", default="./plans")
    ap.add_argument("--mode", default="learn", choices=[m.value for m in AT.ElasticMode])
    ap.add_argument("--iters", type=int, default=8)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev = "cuda" if cuda else "cpu"
    hw = AT.HardwareProfile.from_capabilities(H.probe_cuda(0) if cuda else H.probe_host_cpu())
    prob = AT.ProblemClass.gemm(a.m, a.n, a.k)
    tuner = AT.ElasticAutoTuner(AT.ElasticConfig(AT.ElasticMode(a.mode)))
    store = AT.PersistedPlanStore(a.plans)
    key = AT.PlanKey(hw, prob, tuner.config.objective)
    plan = tuner.load_plan_for_mode(store, key)
    if plan is not None and not tuner.mode_permissions().may_explore:
        c = plan.evidence.candidate
        print(f"stored plan: {dict(c.parameters)} median {plan.evidence.measurement.median_ns / 1e3:.1f} us")
        return
    torch.manual_seed(0)
    x = torch.randn(a.m, a.k, device=dev).to(torch.bfloat16)
    w = torch.randn(a.k, a.n, device=dev).to(torch.bfloat16)
    ref = x[:256].float() @ w.float()
    flush_buf = torch.empty(160 << 20, dtype=torch.uint8, device=dev) if cuda else None

    def space(_hw, _prob):
        yield AT.ElasticCandidate.new("gemm-bf16", b"router", {"bn": 0, "splits": -1}, True, 0)
        for bn in (128, 256):
            for splits in (0, 1, 2, 4):
                if splits > 1 and a.k // splits < 256:
                    continue
                tmp = 4 * a.m * a.n * splits if splits > 1 else 148 * 3 * 128 * 256 * 4 if splits == 0 else 0
                yield AT.ElasticCandidate.new("gemm-bf16", b"single-cta", {"bn": bn, "splits": splits}, True, tmp)

    def run(c):
        bn, splits = c.param("bn") or None, c.param("splits")
        return lambda: G.matmul_nn(x, w, bn=bn, splits=None if splits < 0 else splits)

    def correctness(c):
        y = run(c)()[:256].float()
        err = float((y - ref).abs().max() / ref.abs().max())
        return f"rel_max_err={err:.3e}".encode() if err < 2e-2 else b""

    ranked = tuner.rank_candidates(hw, prob, space, lambda *_: True,
                                   lambda _h, _p, c, _o: 0 if c.kernel_revision == b"router" else 1 + c.param("splits"))
    proto = AT.MeasurementProtocol(3, a.iters, AT.TimingSource.DEVICE_TIMESTAMP if cuda else AT.TimingSource.HOST_WALL_CLOCK)
    win, last = AT.race(tuner, ranked, run, proto, correctness=correctness) if not cuda else _race_flushed(tuner, ranked, run, proto, correctness, flush_buf)
    for e in sorted(last, key=lambda e: e.measurement.median_ns):
        print(f"  {dict(e.candidate.parameters)}  median {e.measurement.median_ns / 1e3:8.1f} us  p95 {e.measurement.p95_ns / 1e3:8.1f}  {e.correctness_evidence.decode()}")
    plan = tuner.plan_from_evidence(hw, prob, win)
    tuner.store_plan_for_mode(store, key, plan)
    tf = 2 * a.m * a.n * a.k / win.measurement.median_ns / 1e3
    print(f"winner {dict(win.candidate.parameters)}: {win.measurement.median_ns / 1e3:.1f} us ({tf:.0f} TFLOP/s); "
          f"plan {key.digest()[:12]} stored in {a.plans}; protocol {hashlib.sha256(proto.canonical_bytes()).hexdigest()[:8]}")


def _race_flushed(tuner, ranked, run, base, correctness, flush_buf):
    """The library's race with an L2 flush (a write larger than the cache) before every timed sample."""
    policy = AT.RacingPolicy()
    alive, evidence = list(ranked), []
    for rnd in range(8):
        proto = policy.protocol_for_round(base, rnd)
        evidence, still = [], []
        for r in alive:
            proof = correctness(r.candidate)
            if proof:
                evidence.append(AT.ElasticEvidence(r.candidate, proof, proto.measure(run(r.candidate), flush=flush_buf.zero_)))
                still.append(r)
        alive = policy.race_round(tuner, still, evidence)
        if len(alive) == 1:
            break
    return tuner.select_measured_evidence(alive, evidence), evidence


if __name__ == "__main__":
    main()
