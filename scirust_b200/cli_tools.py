"""Additional `scirust` commands: data preparation, fine-tuning, held-out evaluation and the model-assurance tools.

`byte-shard` (scirust-sciagent/src/bin/byte-shard.rs), `eval-shards` (bin/sciagent-eval.rs), `sft` (train/sft.rs); the
rest demonstrate library functions on seeded synthetic inputs in the style of the reference's `certify` / `guard`
commands: `robust` (DeepPoly branch and bound + randomised smoothing + Lipschitz radius), `watermark`, `prune`,
`dp-sgd`, `conformal-sets`, `ensemble`, `fuse`. Registered by ``cli.build_parser``; exit codes follow ``cli``.
"""
from __future__ import annotations

import sys

EXIT_OK, EXIT_USAGE, EXIT_VALIDATION = 0, 2, 3


def cmd_byte_shard(a):
    from .data.corpus import byte_shard
    n, paths = byte_shard(a.input, a.output, a.extension, a.recursive, a.tokens_per_shard, a.max_files, a.u32)
    print(f"Total files: {n}")
    for p in paths:
        print(f"{p.name}: {p.stat().st_size // (4 if a.u32 else 1)} tokens")
    print(f"Done: {len(paths)} shards written to {a.output}")
    return EXIT_OK


def cmd_eval_shards(a):
    from .io import checkpoint as CK
    from .train.evaluate import evaluate_shards
    from . import cli
    model, meta = CK.load_sciagent_checkpoint(a.checkpoint, device=cli._device(a.device))
    rep = evaluate_shards(model, a.data_dir, a.batch_size, a.max_batches, a.seq_len or None)
    print("=== SCIAGENT eval ===")
    print(f"Checkpoint: step {meta['step']} (train loss {meta['loss']:.4f})")
    print(f"Eval set: {rep.tokens} tokens, {rep.sequences} sequences")
    print(f"Batches: {rep.batches} | mean cross-entropy {rep.mean_loss:.4f} | perplexity {rep.perplexity:.2f}")
    return EXIT_OK


def cmd_sft(a):
    from . import cli
    from .io import checkpoint as CK
    from .models import GQADecoder, SciAgentConfig
    from .train import sft as SFT
    tok = cli._load_tokenizer(a.tokenizer)
    ds = SFT.SftDataset.from_jsonl(a.data)
    if ds.is_empty():
        sys.stderr.write("error: the SFT file holds no examples\n")
        return EXIT_VALIDATION
    dev = cli._device(a.device)
    if a.checkpoint:
        model, _ = CK.load_sciagent_checkpoint(a.checkpoint, device=dev)
    else:
        model = GQADecoder(SciAgentConfig.preset(a.model), device=dev, seed=a.seed)
    hist = SFT.sft_train(model, ds, tok, a.lr, a.epochs, a.batch_size, a.max_seq_len, not a.train_on_prompt, log=print)
    if a.out:
        CK.save_sciagent_checkpoint(model, a.out, a.epochs, hist[-1], a.lr)
        print(f"saved {a.out}")
    return EXIT_OK


def cmd_robust(a):
    import torch
    from .certify import IbpLinear, IbpMlp, Interval, certified_robust
    from .nn.lipschitz import GloroClassifier
    from .nn.rng import PcgEngine
    from .nn.smoothing import SmoothedClassifier
    from .verify import verify_robustness
    if not a.eps > 0:
        sys.stderr.write("error: --eps must be positive\n")
        return EXIT_USAGE
    g = torch.Generator().manual_seed(a.seed)
    layers = [IbpLinear(torch.randn(2, 8, generator=g), torch.randn(8, generator=g) * 0.3),
              IbpLinear(torch.randn(8, 3, generator=g), torch.randn(3, generator=g) * 0.3)]
    net = IbpMlp(layers)
    x = torch.tensor([0.3, -0.2])
    cls = int(net.forward(x).argmax())
    box = Interval.around(x, a.eps)
    print(f"Robustness of a seeded 2->8->3 ReLU net at {[round(v, 3) for v in x.tolist()]} (class {cls}), eps = {a.eps}")
    for name, out in (("IBP", net.certify(box)), ("zonotope", net.certify_zonotope(box)), ("DeepPoly", net.certify_deeppoly(box))):
        print(f"  {name:<9} total width {float(out.width().sum()):.4f}  {'CERTIFIED' if certified_robust(out, cls) else 'not certified'}")
    r = verify_robustness(layers, box, cls, 1e-5, a.max_boxes)
    extra = f" counterexample {[round(v, 4) for v in r.counterexample.tolist()]}" if r.counterexample is not None else ""
    print(f"  branch and bound: {r.status.upper()} after {r.boxes} boxes{extra}")
    cert = SmoothedClassifier(a.sigma).certify_cohen(lambda X: net.forward(X).argmax(1), x, 100, a.samples, 3, 0.001, PcgEngine(a.seed))
    print(f"  randomised smoothing (sigma {a.sigma}): class {cert.cls}, " +
          ("abstains" if cert.abstained else f"L2 radius {cert.radius:.4f} (p_A >= {cert.p_a_lower:.4f})"))
    head = GloroClassifier(layers[1].w.t().contiguous(), 3, 8)
    hcls, hr = head.certify(torch.relu(layers[0].forward(x)))
    print(f"  Lipschitz bound of the head: {head.lipschitz():.4f} (estimate {head.lipschitz_estimate():.4f}), feature-space radius {hr:.4f}")
    return EXIT_OK


def cmd_watermark(a):
    from .nn import watermark as W
    from .nn.rng import PcgEngine
    rng = PcgEngine(a.seed)
    plain, marked = [0], [0]
    for _ in range(a.tokens):
        plain.append(int(rng.float() * a.vocab))
        row = rng.fill_normal((a.vocab,))
        W.apply_green_bias(row, a.key, marked[-1], a.gamma, a.delta)
        marked.append(int(row.argmax()))
    print(f"Green-list watermark: vocab {a.vocab}, gamma {a.gamma}, delta {a.delta}, {a.tokens} tokens")
    print(f"  unmarked text   z = {W.detect_z(a.key, plain, a.gamma):+.2f}")
    print(f"  watermarked     z = {W.detect_z(a.key, marked, a.gamma):+.2f}  (p = {W.detect_p_value(a.key, marked, a.gamma):.2e})")
    print(f"  wrong key       z = {W.detect_z(a.key + 1, marked, a.gamma):+.2f}")
    return EXIT_OK


def cmd_prune(a):
    import torch
    from . import pruning as P
    if not 0.0 <= a.sparsity <= 1.0:
        sys.stderr.write("error: --sparsity must be in [0, 1]\n")
        return EXIT_USAGE
    g = torch.Generator().manual_seed(a.seed)
    W = torch.randn(a.rows, a.cols, generator=g)
    X = torch.randn(256, a.cols, generator=g) * torch.linspace(0.1, 2.0, a.cols)
    ref = X @ W.t()
    print(f"Pruning a seeded {a.rows}x{a.cols} weight at sparsity {a.sparsity} (output error on 256 calibration rows)")
    variants = {"magnitude": P.prune_magnitude(W.clone(), a.sparsity),
                "wanda": P.prune_wanda(W.clone(), X.norm(dim=0), a.sparsity),
                "columns": P.prune_structured_columns(W.clone(), sparsity=a.sparsity),
                "rows": P.prune_structured_rows(W.clone(), sparsity=a.sparsity)}
    if a.cols % 4 == 0:
        variants["2:4"] = P.prune_n_of_m(W.clone())
    for name, Wp in variants.items():
        err = float((X @ Wp.t() - ref).norm() / ref.norm())
        print(f"  {name:<10} sparsity {P.sparsity_ratio(Wp):.3f}  relative output error {err:.4f}")
    return EXIT_OK


def cmd_dp_sgd(a):
    import torch
    import torch.nn.functional as F
    from . import privacy as D
    cfg = D.DpSgdConfig(a.clip, a.noise, a.delta)
    cfg.validate()
    g = torch.Generator().manual_seed(a.seed)
    X = torch.cat([torch.randn(128, 4, generator=g) + 1.5, torch.randn(128, 4, generator=g) - 1.5])
    Y = torch.cat([torch.zeros(128), torch.ones(128)]).long()
    torch.manual_seed(a.seed)
    clf = torch.nn.Linear(4, 2)
    opt = D.DpSgd(clf, F.cross_entropy, a.lr, cfg, torch.Generator().manual_seed(a.seed + 1))
    print(f"DP-SGD: clip {a.clip}, noise multiplier {a.noise}, delta {a.delta}")
    for step in range(1, a.steps + 1):
        opt.step(X, Y)
        if step % max(a.steps // 5, 1) == 0 or step == a.steps:
            acc = float((clf(X).argmax(1) == Y).float().mean())
            print(f"  step {step:4d}  accuracy {acc:.3f}  epsilon {opt.epsilon:.2f}")
    return EXIT_OK


def cmd_conformal_sets(a):
    import torch
    from . import conformal as CF
    if not 0.0 < a.alpha < 1.0:
        sys.stderr.write("error: --alpha must be in (0, 1)\n")
        return EXIT_USAGE
    g = torch.Generator().manual_seed(a.seed)
    probs = torch.softmax(torch.randn(4000, a.classes, generator=g) * 2, 1)
    y = torch.multinomial(probs, 1, generator=g).squeeze(1)
    cal, test = slice(0, 2000), range(2000, 4000)
    print(f"Conformal classification, {a.classes} classes, target coverage {1 - a.alpha:.2f}")
    for name, clf in (("threshold", CF.ConformalClassifier.calibrate(probs[cal], y[cal], a.alpha)),
                      ("APS", CF.AdaptivePredictionSets.calibrate(probs[cal], y[cal], a.alpha)),
                      ("RAPS", CF.AdaptivePredictionSets.calibrate_raps(probs[cal], y[cal], a.alpha, 2, 0.05))):
        cov = sum(clf.covers(probs[i], int(y[i])) for i in test) / 2000
        size = sum(len(clf.predict_set(probs[i])) for i in test) / 2000
        print(f"  {name:<10} coverage {cov:.4f}  mean set size {size:.2f}")
    risks = [max(0.5 - 0.1 * i, 0.0) for i in range(8)]
    print(f"  RCPS over 8 nested predictors: lambda index {CF.rcps_select(risks, 2000, a.alpha, 0.05)}; "
          f"learn-then-test keeps {CF.learn_then_test(risks, 2000, a.alpha, 0.05)}")
    return EXIT_OK


def cmd_ensemble(a):
    import torch
    from .nn.ensemble import DeepEnsemble
    xs = torch.linspace(-1, 1, 40)
    ens = DeepEnsemble.train(xs, torch.sin(3 * xs), a.members, a.hidden, a.steps, a.lr, a.seed)
    print(f"Deep ensemble of {len(ens)} MLPs (hidden {a.hidden}) on sin(3x), x in [-1, 1]")
    for x in (-0.5, 0.0, 0.75, 2.0, 4.0):
        m, s = ens.predict(x)
        print(f"  x = {x:+.2f}  mean {m:+.4f}  spread {s:.4f}{'   (outside the data)' if abs(x) > 1 else ''}")
    return EXIT_OK


def cmd_fuse(a):
    import torch
    from . import fusion as FU
    g = FU.OpGraph()
    x, w1, b1, ga, be, w2 = (g.add_input() for _ in range(6))
    h = g.add(FU.OpKind.LAYERNORM, g.add(FU.OpKind.SILU, g.add(FU.OpKind.LINEAR, x, w1, b1)), ga, be)
    out = g.add(FU.OpKind.RELU, g.add(FU.OpKind.MATMUL, h, w2))
    kernels = FU.FusionPipeline().fuse(g)
    print(f"Graph of {len(g)} nodes -> {len(kernels)} fused kernels")
    for k in kernels:
        print(f"  {k.kernel_type.value:<24} nodes {k.group}  external inputs {k.inputs}")
    gen = torch.Generator().manual_seed(a.seed)
    feeds = {x: torch.randn(4, 8, generator=gen), w1: torch.randn(8, 16, generator=gen), b1: torch.randn(16, generator=gen),
             ga: torch.ones(16), be: torch.zeros(16), w2: torch.randn(16, 5, generator=gen)}
    diff = float((FU.execute(g, feeds, True)[out] - FU.execute(g, feeds, False)[out]).abs().max())
    print(f"  fused vs unfused max difference {diff:.2e}")
    return EXIT_OK


def cmd_pretrain(a):
    """The SCIAGENT_* environment harness (flags override the environment)."""
    import os
    from .train.pretrain import run_from_env
    env = dict(os.environ)
    for flag, key in (("config", "SCIAGENT_CONFIG"), ("text", "SCIAGENT_TEXT"), ("shards", "SCIAGENT_SHARDS"), ("ckpt", "SCIAGENT_CKPT"),
                      ("steps", "SCIAGENT_STEPS"), ("seq", "SCIAGENT_SEQ"), ("batch", "SCIAGENT_BATCH"), ("lr", "SCIAGENT_LR"),
                      ("save", "SCIAGENT_SAVE"), ("val_frac", "SCIAGENT_VAL_FRAC"), ("telemetry", "SCIAGENT_TELEMETRY")):
        v = getattr(a, flag)
        if v not in (None, ""):
            env[key] = str(v)
    if a.preflight_only:
        env["SCIAGENT_PREFLIGHT_ONLY"] = "1"
    if a.require_fresh:
        env["SCIAGENT_REQUIRE_FRESH"] = "1"
    from . import cli
    return run_from_env(env, device=cli._device(a.device))


def register(sub):
    p = sub.add_parser("pretrain")
    for flag in ("config", "text", "shards", "ckpt", "steps", "seq", "batch", "lr", "save", "val-frac", "telemetry"):
        p.add_argument(f"--{flag}", default=None)
    p.add_argument("--preflight-only", action="store_true")
    p.add_argument("--require-fresh", action="store_true")
    p.add_argument("--device", default="auto")
    p.set_defaults(fn=cmd_pretrain)
    p = sub.add_parser("byte-shard")
    p.add_argument("--input", "-i", nargs="+", required=True)
    p.add_argument("--output", "-o", default="./shards")
    p.add_argument("--extension", default="rs")
    p.add_argument("--recursive", action="store_true")
    p.add_argument("--tokens-per-shard", type=int, default=1_000_000)
    p.add_argument("--max-files", type=int, default=0)
    p.add_argument("--u32", action="store_true", help="little-endian u32 tokens (the training loader's format)")
    p.set_defaults(fn=cmd_byte_shard)
    p = sub.add_parser("eval-shards")
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--data-dir", required=True)
    p.add_argument("--batch-size", type=int, default=8)
    p.add_argument("--max-batches", type=int, default=0)
    p.add_argument("--seq-len", type=int, default=0)
    p.add_argument("--device", default="auto")
    p.set_defaults(fn=cmd_eval_shards)
    p = sub.add_parser("sft")
    p.add_argument("--data", required=True)
    p.add_argument("--tokenizer", default="bpe.json")
    p.add_argument("--checkpoint", default="")
    p.add_argument("--model", default="debug")
    p.add_argument("--out", default="")
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--batch-size", type=int, default=2)
    p.add_argument("--max-seq-len", type=int, default=128)
    p.add_argument("--train-on-prompt", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--device", default="auto")
    p.set_defaults(fn=cmd_sft)
    p = sub.add_parser("robust")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--eps", type=float, default=0.05)
    p.add_argument("--sigma", type=float, default=0.25)
    p.add_argument("--samples", type=int, default=2000)
    p.add_argument("--max-boxes", type=int, default=5000)
    p.set_defaults(fn=cmd_robust)
    p = sub.add_parser("watermark")
    p.add_argument("--key", type=int, default=1)
    p.add_argument("--seed", type=int, default=5)
    p.add_argument("--vocab", type=int, default=200)
    p.add_argument("--tokens", type=int, default=300)
    p.add_argument("--gamma", type=float, default=0.3)
    p.add_argument("--delta", type=float, default=4.0)
    p.set_defaults(fn=cmd_watermark)
    p = sub.add_parser("prune")
    p.add_argument("--rows", type=int, default=64)
    p.add_argument("--cols", type=int, default=128)
    p.add_argument("--sparsity", type=float, default=0.5)
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(fn=cmd_prune)
    p = sub.add_parser("dp-sgd")
    p.add_argument("--clip", type=float, default=1.0)
    p.add_argument("--noise", type=float, default=1.0)
    p.add_argument("--delta", type=float, default=1e-5)
    p.add_argument("--lr", type=float, default=0.5)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(fn=cmd_dp_sgd)
    p = sub.add_parser("conformal-sets")
    p.add_argument("--alpha", type=float, default=0.1)
    p.add_argument("--classes", type=int, default=6)
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(fn=cmd_conformal_sets)
    p = sub.add_parser("ensemble")
    p.add_argument("--members", type=int, default=5)
    p.add_argument("--hidden", type=int, default=16)
    p.add_argument("--steps", type=int, default=400)
    p.add_argument("--lr", type=float, default=0.02)
    p.add_argument("--seed", type=int, default=100)
    p.set_defaults(fn=cmd_ensemble)
    p = sub.add_parser("fuse")
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(fn=cmd_fuse)
