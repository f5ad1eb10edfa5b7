"""``scirust``-style command line (scirust-cli/src/lib.rs:631-760; exit-code contract
docs/CLI_CONTRACT.md:20-34: 0 ok, 1 domain failure, 2 usage / IO, 3 validation, 5 numerical,
6 cancelled, 7 internal). Standard output is byte-deterministic for a given command line; timing
goes to stderr and only when stderr is a terminal (lib.rs:626-651).

    python -m scirust_b200.cli quickstart
    python -m scirust_b200.cli train --model debug --steps 20 --data shards/*.bin --checkpoint-dir ckpt
    python -m scirust_b200.cli infer --checkpoint ckpt/step_20 --prompt "fn main" --max-new 32
    python -m scirust_b200.cli sciagent info|generate|quantize|attest ...
    python -m scirust_b200.cli bpe train|encode|decode ...
    python -m scirust_b200.cli verify emit|verify ...
"""
from __future__ import annotations

import argparse
import glob
import hashlib
import json
import math
import sys
import time

EXIT_OK, EXIT_FAIL, EXIT_USAGE, EXIT_VALIDATION, EXIT_NUMERICAL, EXIT_CANCELLED, EXIT_INTERNAL = 0, 1, 2, 3, 5, 6, 7


class _Parser(argparse.ArgumentParser):
    def error(self, message):
        raise SystemExit(self._usage_exit(message))

    def _usage_exit(self, message):
        sys.stderr.write(f"error: {message}\n")
        return EXIT_USAGE


def _device(name):
    import torch
    if name == "auto":
        return "cuda" if torch.cuda.is_available() else "cpu"
    return name


def cmd_version(a):
    from . import __version__
    print(f"scirust_b200 {__version__}")
    return EXIT_OK


def cmd_info(a):
    import torch
    from . import __version__
    from ._build import CUDA_LIB, RT_LIB
    print(f"scirust_b200 {__version__}")
    print(f"torch {torch.__version__}")
    print(f"cuda_available {torch.cuda.is_available()}")
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        print(f"device {p.name} sm_{p.major}{p.minor} {p.total_memory // (1 << 20)} MiB x{torch.cuda.device_count()}")
    print(f"native_cuda_lib {'present' if CUDA_LIB.exists() else 'missing'}")
    print(f"native_rt_lib {'present' if RT_LIB.exists() else 'missing'}")
    from .utils import capability_registry as CR
    CR.register_default_capabilities(probe=False)
    print(f"compute_paths {CR.capability_summary()}")
    return EXIT_OK


def cmd_quickstart(a):
    from .models.mlp_cpu import train_gaussian_mlp
    model, hist = train_gaussian_mlp(epochs=a.epochs, seed=a.seed, fma=a.fma, log=print)
    loss, acc = hist[-1]
    print(f"final loss {loss:.6f} accuracy {acc:.4f} fingerprint {model.fingerprint():016x}")
    if loss != loss:
        return EXIT_NUMERICAL
    return EXIT_OK if acc >= 0.9 else EXIT_FAIL


def _load_tokenizer(path):
    from .tokenizer import BpeTokenizer
    return BpeTokenizer.load_json(path)


def cmd_bpe(a):
    from .tokenizer import BpeTrainer
    if a.action == "train":
        texts = [open(p, encoding="utf-8").read() for p in a.inputs]
        tok = BpeTrainer(a.vocab_size, a.min_frequency).train(texts)
        tok.save_json(a.out)
        print(f"vocab {tok.vocab_size()} merges {len(tok.merges)} -> {a.out}")
    elif a.action == "encode":
        print(" ".join(str(i) for i in _load_tokenizer(a.tokenizer).encode(a.text)))
    else:
        print(_load_tokenizer(a.tokenizer).decode([int(t) for t in a.text.split()]))
    return EXIT_OK


def cmd_train(a):
    import torch
    from .data.datasets import TokenShardDataset
    from .io import checkpoint as CK
    from .models import GQADecoder, SciAgentConfig
    from .train import Trainer, TrainerConfig
    dev = _device(a.device)
    cfg = SciAgentConfig.preset(a.model)
    paths = sorted(p for pat in a.data for p in glob.glob(pat))
    start = 0
    if a.resume:
        last = CK.latest_checkpoint(a.checkpoint_dir)
        if last is None:
            sys.stderr.write("error: --resume given but no checkpoint found\n")
            return EXIT_USAGE
        model, meta = CK.load_sciagent_checkpoint(last, device=dev)
        cfg, start = model.cfg, meta["step"]
    else:
        model = GQADecoder(cfg, device=dev, seed=a.seed)
    tc = TrainerConfig(lr=a.lr, min_lr=a.min_lr, warmup_steps=a.warmup_steps, total_steps=a.total_steps,
                       max_grad_norm=a.max_grad_norm, weight_decay=a.weight_decay)
    tr = Trainer(model, tc)
    if a.resume:
        CK.load_optimizer_state(model, tr, last)
    if paths:
        ds = TokenShardDataset(paths, a.seq_len, cfg.vocab_size, val_frac=a.val_frac, seed=a.seed)
        get = lambda s: ds.batch(s, a.batch_size)  # noqa: E731
    else:
        def get(s):
            g = torch.Generator().manual_seed(a.seed * 1000003 + s)
            return torch.randint(0, cfg.vocab_size, (a.batch_size, a.seq_len + 1), generator=g)
    t0 = time.time()
    loss = float("nan")
    for step in range(start, a.steps):
        loss = float(tr.train_step(get(step)).item())
        if loss != loss:
            sys.stderr.write(f"error: loss is NaN at step {step}\n")
            return EXIT_NUMERICAL
        if (step + 1) % a.log_interval == 0 or step + 1 == a.steps:
            print(f"[step {step + 1}] {a.batch_size}x{a.seq_len} loss {loss:.4f} | lr {tr.schedule.lr_at(step):.3e} | "
                  f"gnorm {tr.grad_norm():.3f}")
        if a.checkpoint_dir and a.save_interval and (step + 1) % a.save_interval == 0:
            CK.save_sciagent_checkpoint(model, f"{a.checkpoint_dir}/step_{step + 1}", step + 1, loss,
                                        tr.schedule.lr_at(step), trainer=tr)
            if a.keep_last:
                CK.prune_checkpoints(a.checkpoint_dir, a.keep_last)
    if a.checkpoint_dir:
        CK.save_sciagent_checkpoint(model, f"{a.checkpoint_dir}/step_{a.steps}", a.steps, loss,
                                    tr.schedule.lr_at(max(a.steps - 1, 0)), trainer=tr)
    if sys.stderr.isatty():
        dt = time.time() - t0
        sys.stderr.write(f"{(a.steps - start) * a.batch_size * a.seq_len / max(dt, 1e-9):.0f} tok/s\n")
    return EXIT_OK


def cmd_infer(a):
    import torch
    from .generate import SamplingParams
    from .io import checkpoint as CK
    from .models.infer import InferenceEngine
    dev = _device(a.device)
    model, meta = CK.load_sciagent_checkpoint(a.checkpoint, device=dev)
    if a.tokenizer:
        tok = _load_tokenizer(a.tokenizer)
        ids = tok.encode(a.prompt)
    else:
        tok, ids = None, [int(t) for t in a.prompt.split()]
    if not ids:
        sys.stderr.write("error: empty prompt\n")
        return EXIT_VALIDATION
    eng = InferenceEngine(model, quant=a.quant, max_batch=1, max_seq=len(ids) + a.max_new + 1)
    params = SamplingParams(a.temperature, a.top_k, a.top_p, a.repetition_penalty)
    out = eng.generate(torch.tensor([ids]), a.max_new, params, seed=a.seed)[0].tolist()
    if 0 in out:
        out = out[:out.index(0)]      # token 0 stops generation
    print(tok.decode(out) if tok else " ".join(str(t) for t in out))
    return EXIT_OK


def cmd_sciagent(a):
    from .io import checkpoint as CK
    if a.action == "info":
        meta = CK.read_meta(a.checkpoint)
        print(json.dumps({"step": meta["step"], "loss": meta["loss"], "lr": meta["lr"], "config": meta["config"].to_dict()},
                         indent=2, sort_keys=True))
        return EXIT_OK
    if a.action == "generate":
        return cmd_infer(a)
    if a.action == "quantize":
        import torch
        from . import quantization as Q
        model, _ = CK.load_sciagent_checkpoint(a.checkpoint)
        sd = model.reference_state_dict()
        blob, index, off = [], {}, 0
        for k in sorted(sd):
            packed, scale, shape, pad = Q.int4_group_quantize(sd[k], a.group)
            raw = packed.numpy().tobytes() + scale.numpy().astype("<f4").tobytes()
            index[k] = {"shape": list(shape), "pad": pad, "offset": off, "codes": packed.numel(), "groups": scale.numel()}
            blob.append(raw)
            off += len(raw)
        hdr = json.dumps({"format": "SCIAGENT-INT4-1", "group": a.group, "tensors": index}).encode()
        with open(a.out, "wb") as f:
            f.write(len(hdr).to_bytes(8, "little") + hdr + b"".join(blob))
        print(f"wrote {a.out}: {off + len(hdr) + 8} bytes ({sum(v.numel() for v in sd.values()) * 4} fp32 bytes)")
        return EXIT_OK
    if a.action == "attest":
        from pathlib import Path
        mb = (Path(a.checkpoint) / "model.safetensors").read_bytes()
        from .io import execution_attestation as EA
        tok_sha = EA.file_sha256(a.tokenizer) if a.tokenizer else EA.sha256_hex(b"")
        model_sha = hashlib.sha256(mb).hexdigest()
        rec = {"model_sha256": model_sha, "model_bytes": len(mb),
               "model_semantics_version": CK.MODEL_SEMANTICS_VERSION,
               "training_route": json.loads(EA.build_training_route_attestation(model_sha, tok_sha).to_json()),
               "decode_route": json.loads(EA.build_decode_route_attestation(model_sha, tok_sha).to_json())}
        if a.tokenizer:
            rec["tokenizer_sha256"] = tok_sha
        print(json.dumps(rec, indent=2, sort_keys=True))
        return EXIT_OK
    return EXIT_USAGE


def cmd_verify(a):
    from pathlib import Path
    from .io import proof
    art = Path(a.artifact).read_bytes()
    if a.action == "emit":
        try:
            text = proof.build_bundle(art, a.batch, a.seeds)
        except ValueError as e:
            sys.stderr.write(f"error: {e}\n")
            return EXIT_VALIDATION
        if a.out:
            Path(a.out).write_text(text)
        else:
            sys.stdout.write(text)
        return EXIT_OK
    errs = proof.verify_bundle(Path(a.bundle).read_text(), art)
    for e in errs:
        print(f"MISMATCH {e}")
    print("VERIFIED" if not errs else f"FAILED ({len(errs)} mismatches)")
    return EXIT_OK if not errs else EXIT_FAIL


def _matrix(a):
    """Weight matrix for the quantiser commands: a tensor of a safetensors file, or seeded noise."""
    import torch
    if a.weights:
        from .io.safetensors import load_file
        sd = load_file(a.weights)
        key = a.tensor or sorted(sd)[0]
        return torch.as_tensor(sd[key]).float()
    g = torch.Generator().manual_seed(a.seed)
    return torch.randn(a.rows, a.cols, generator=g) * 0.05


def cmd_quantizer(a):
    """gptq / awq / bitnet / int4: quantise one matrix, report the reconstruction error."""
    import torch
    from . import quantization as Q
    w = _matrix(a)
    g = torch.Generator().manual_seed(a.seed + 1)
    x = torch.randn(256, w.shape[0], generator=g)
    if a.cmd == "gptq":
        wq = Q.gptq_quantize(w, x, bits=a.bits)
    elif a.cmd == "awq":
        wq, _scales = Q.awq_quantize(w, x, bits=a.bits)
    elif a.cmd == "bitnet":
        t, scale = Q.ternary_quantize(w)
        wq = t.float() * scale
    else:
        packed, scale, shape, pad = Q.int4_group_quantize(w, group=a.group)
        wq = Q.int4_group_dequantize(packed, scale, shape, pad, group=a.group)
    wq = torch.as_tensor(wq).float().reshape(w.shape)
    werr = ((wq - w).norm() / w.norm()).item()
    yerr = ((x @ wq - x @ w).norm() / (x @ w).norm()).item()
    print(f"{a.cmd} shape {tuple(w.shape)} weight_rel_err {werr:.6f} output_rel_err {yerr:.6f}")
    return EXIT_OK if math.isfinite(yerr) else EXIT_NUMERICAL


def cmd_kvcache(a):
    """Attention error and bytes per token of every KV-cache backend on seeded data."""
    import torch
    from .nn import kv_cache as KV
    g = torch.Generator().manual_seed(a.seed)
    d = a.head_dim
    ks, vs, q = torch.randn(a.tokens, d, generator=g), torch.randn(a.tokens, d, generator=g), torch.randn(d, generator=g)
    ref = KV.PlainKvCache(d)
    caches = {"plain": KV.PlainKvCache(d), "paged": KV.PagedKvCache(d, page=16), "int8": KV.QuantKvCache(d, bits=8),
              "int4": KV.QuantKvCache(d, bits=4), "latent": KV.LatentKvCache(d, rank=max(4, d // 2))}
    for t in range(a.tokens):
        ref.append(ks[t], vs[t])
        for c in caches.values():
            c.append(ks[t], vs[t])
    want = ref.decode_step(q)
    for name, c in caches.items():
        err = ((c.decode_step(q) - want).norm() / want.norm()).item()
        print(f"{name} rel_err {err:.6f} bytes_per_token {c.nbytes() / max(len(c), 1):.1f}")
    return EXIT_OK


def cmd_onnx(a):
    from .io import onnx_json as OJ
    from .nn import modules as M
    from .nn.rng import PcgEngine
    if a.action == "export":
        rng = PcgEngine(a.seed)
        dims = a.layers
        layers = []
        for i in range(len(dims) - 1):
            layers.append(M.Linear(dims[i], dims[i + 1], rng=rng))
            if i + 2 < len(dims):
                layers.append(M.ReLU())
        text = OJ.export_sequential(M.Sequential(*layers), a.name, (-1, dims[0]))
        with open(a.file, "w") as f:
            f.write(text)
        print(f"wrote {a.file} ({len(text)} bytes)")
        return EXIT_OK
    g = OJ.import_onnx_json(open(a.file).read())
    print(f"{g.doc['name']}: {len(g.nodes)} nodes, {len(g.weights())} initializers")
    for n in g.nodes:
        print(f"  {n['op_type']} {n['inputs']} -> {n['outputs']}")
    return EXIT_OK


def cmd_plan(a):
    from .models import SciAgentConfig
    from .utils import planning
    cfg = SciAgentConfig.preset(a.model)
    pl = planning.plan(cfg, a.batch, a.seq, tp=a.tp)
    print(f"{a.model}: {planning.n_params(cfg)} parameters, batch {a.batch} x seq {a.seq}, tp {a.tp}")
    for mode in ("flash", "naive"):
        print(f"  {mode}: {pl.total(mode) / (1 << 30):.2f} GiB  fits_180GB {pl.fits(mode)}")
    return EXIT_OK


def cmd_calibrate(a):
    """calibrate / conformal on a ``.pt`` file holding {"logits": [N, C], "labels": [N]}."""
    import torch
    from . import calibration as C
    d = torch.load(a.data)
    logits, labels = d["logits"].float(), d["labels"].long()
    if logits.dim() != 2 or labels.shape[0] != logits.shape[0]:
        raise ValueError("expected logits [N, C] and labels [N]")
    n = logits.shape[0] // 2
    if a.cmd == "calibrate":
        t = C.fit_temperature(logits[:n], labels[:n])
        before = C.expected_calibration_error(torch.softmax(logits[n:], -1), labels[n:])
        after = C.expected_calibration_error(torch.softmax(logits[n:] / t, -1), labels[n:])
        print(f"temperature {t:.4f} ece_before {before:.4f} ece_after {after:.4f}")
    else:
        thr = C.conformal_threshold(torch.softmax(logits[:n], -1), labels[:n], a.alpha)
        sets = C.conformal_sets(torch.softmax(logits[n:], -1), thr)
        cover = sets.gather(1, labels[n:, None]).float().mean().item()
        print(f"threshold {thr:.4f} coverage {cover:.4f} mean_set_size {sets.float().sum(1).mean().item():.3f}")
    return EXIT_OK



def cmd_lm(a):
    """Next-token training of a one-block decoder on a token sequence with a chosen optimizer of the zoo
    (scirust-cli/src/nlp.rs:214-330)."""
    import torch
    from .autodiff import nd_optim as NO
    from .nn.zoo import NdDecoderLM
    try:
        toks = [int(t) for t in a.tokens.split(",") if t.strip()]
    except ValueError:
        sys.stderr.write("error: tokens must be non-negative integers\n")
        return EXIT_USAGE
    if len(toks) < 2 or min(toks) < 0:
        sys.stderr.write("error: need at least 2 non-negative tokens for next-token training\n")
        return EXIT_USAGE
    torch.manual_seed(a.seed)
    vocab = max(toks) + 1
    model = NdDecoderLM(vocab, d_model=16, n_layers=1, n_heads=2, n_kv_heads=1, d_ff=32)
    table = {"adam": lambda p: torch.optim.Adam(p, lr=a.lr), "adamw": lambda p: torch.optim.AdamW(p, lr=a.lr),
             "lion": lambda p: NO.Lion(p, lr=a.lr * 0.3), "lamb": lambda p: NO.LAMB(p, lr=a.lr),
             "adan": lambda p: NO.Adan(p, lr=a.lr), "adafactor": lambda p: NO.Adafactor(p, lr=a.lr),
             "ademamix": lambda p: NO.AdEMAMix(p, lr=a.lr), "soap": lambda p: NO.SOAP(p, lr=a.lr),
             "shampoo": lambda p: NO.Shampoo(p, lr=a.lr), "prodigy": lambda p: NO.Prodigy(p),
             "galore": lambda p: NO.GaLore(p, lr=a.lr), "schedule-free": lambda p: NO.ScheduleFreeSGD(p, lr=a.lr * 10),
             "muon": lambda p: NO.Muon(p, lr=a.lr), "sophia": lambda p: NO.Sophia(p, lr=a.lr),
             "lookahead": lambda p: NO.Lookahead(torch.optim.Adam(p, lr=a.lr))}
    if a.opt not in table:
        sys.stderr.write(f"error: unknown optimizer {a.opt!r}; known: {sorted(table)}\n")
        return EXIT_USAGE
    opt = table[a.opt](list(model.parameters()))
    x = torch.tensor([toks[:-1]])
    y = torch.tensor(toks[1:])
    first = last = None
    for step in range(a.steps):
        logits = model(x)[0]
        loss = torch.nn.functional.cross_entropy(logits, y)
        if step == 0:
            first = float(loss.detach())
        if hasattr(opt, "zero_grad"):
            opt.zero_grad()
        loss.backward()
        opt.step()
        last = float(loss.detach())
    pred = model(x)[0].argmax(-1).tolist()
    acc = sum(int(p_ == t) for p_, t in zip(pred, toks[1:])) / len(pred)
    print(f"lm: {len(toks)} tokens, vocab {vocab}, optimizer {a.opt}, seed {a.seed}")
    print(f"  loss {first:.4f} -> {last:.4f} after {a.steps} steps; next-token accuracy {acc:.2f}")
    print(f"  predicted continuation: {pred}")
    return EXIT_OK if last == last else EXIT_NUMERICAL


_SEQ_LAYERS = {"deltanet": ("DeltaNet", "delta-rule linear attention (fast-weight recurrence)"),
               "retnet": ("RetNet", "retention with decay 0.9 (recurrent form = parallel form)"),
               "gla": ("GLA", "gated linear attention (data-dependent per-key decay)"),
               "hgrn": ("HGRN", "hierarchically gated recurrence"),
               "mamba": ("Mamba", "selective state space (input-dependent dt, B, C)"),
               "mamba2": ("Mamba2", "Mamba-2: scalar decay per head, quadratic dual form"),
               "rwkv": ("RWKVTimeMix", "RWKV time mixing (stabilised wkv recurrence)"),
               "s5": ("S5", "S5: one MIMO diagonal state space, parallel prefix scan")}


def cmd_seq_layer(a):
    """``deltanet | retnet | gla | hgrn | mamba | mamba2 | rwkv | s5 [--seed N] [--steps S]``: train one sequence-mixing
    layer to fit a fixed target sequence (x = sin(0.3 i - 1), target = cos(0.2 i), Adam lr 0.05) and report the MSE
    reduction; where the layer has both forms, also the gap between the recurrence and the parallel form
    (scirust-cli/src/nlp.rs: run_deltanet / run_retnet / run_gla / run_hgrn / run_mamba / run_rwkv)."""
    import torch
    from .nn import zoo
    cls_name, what = _SEQ_LAYERS[a.cmd]
    torch.manual_seed(a.seed)
    T, d = 6, 8
    kw = {"gamma": 0.9} if a.cmd == "retnet" else {"d_state": 4, "head_dim": 4} if a.cmd == "mamba2" else \
        {"d_state": 8} if a.cmd in ("s5",) else {"d_state": 4} if a.cmd == "mamba" else {}
    layer = getattr(zoo, cls_name)(d, **kw)
    i = torch.arange(T * d, dtype=torch.float32)
    x, target = torch.sin(i * 0.3 - 1.0).view(1, T, d), torch.cos(i * 0.2).view(1, T, d)
    opt = torch.optim.Adam(layer.parameters(), lr=0.05)
    fwd = layer.forward_parallel if hasattr(layer, "forward_parallel") else layer
    first = last = float("nan")
    for step in range(a.steps):
        loss = ((fwd(x) - target) ** 2).sum()
        if step == 0:
            first = float(loss)
        last = float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    print(f"{cls_name} layer - deterministic (seed {a.seed})")
    print(f"  {what}; d_model {d}, sequence length {T}; {a.steps} Adam steps")
    print(f"  MSE to target: {first:.4f} -> {last:.4f}  ({100.0 * last / first:.1f}% of initial)")
    if hasattr(layer, "forward_parallel"):
        with torch.no_grad():
            gap = float((layer.forward_parallel(x) - layer(x)).abs().max())
        print(f"  recurrent form vs parallel form: max difference {gap:.2e}")
    return 0


def cmd_tt(a):
    """``tt``: a tensor-train linear layer against the dense layer it replaces: parameter count and fit error."""
    import torch
    from .nn import zoo
    torch.manual_seed(a.seed)
    layer = zoo.TTLinear([4, 4, 4], [4, 4, 4], rank=a.rank)
    dense = torch.nn.Linear(64, 64)
    x = torch.randn(256, 64)
    y = dense(x).detach()
    opt = torch.optim.Adam(layer.parameters(), lr=0.02)
    first = last = 0.0
    for step in range(a.steps):
        loss = ((layer(x) - y) ** 2).mean()
        first = float(loss) if step == 0 else first
        last = float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    n_tt, n_dense = sum(p.numel() for p in layer.parameters()), sum(p.numel() for p in dense.parameters())
    print(f"tensor-train linear 64 -> 64, modes 4x4x4, rank {a.rank}: {n_tt} parameters against {n_dense} dense "
          f"({n_dense / n_tt:.1f}x fewer)")
    print(f"  fit of a random dense layer: MSE {first:.4f} -> {last:.4f} in {a.steps} Adam steps")
    return 0


def cmd_search(a):
    """``evo`` / ``cmaes``: minimise a test function (sphere, rosenbrock, rastrigin) without gradients."""
    from . import search
    f = search.OBJECTIVES[a.objective]
    if a.cmd == "cmaes":
        x, fx, hist = search.cma_es(f, a.dim, generations=a.generations, seed=a.seed)
        name = "CMA-ES"
    else:
        x, fx, hist = search.evolution_strategy(f, a.dim, generations=a.generations, seed=a.seed)
        name = "(mu + lambda) evolution strategy"
    print(f"{name} on {a.objective} ({a.dim} dimensions, seed {a.seed}): best {hist[0]:.4g} -> {fx:.4g} "
          f"after {len(hist)} generations")
    print("  x* =", " ".join(f"{v:.4f}" for v in x[:8]), "..." if a.dim > 8 else "")
    return 0


def cmd_pinn(a):
    """``pinn``: a physics-informed network for u'' + pi^2 u = 0 on [0, 1] with u(0) = 0, u'(0) = pi (solution
    sin(pi x)): data loss on the two boundary conditions plus the mean squared residual at collocation points
    (``nn.loss.PINNLoss``); derivatives of the network by automatic differentiation."""
    import math
    import torch
    from .nn.loss import PINNLoss
    torch.manual_seed(a.seed)
    net = torch.nn.Sequential(torch.nn.Linear(1, 24), torch.nn.Tanh(), torch.nn.Linear(24, 24), torch.nn.Tanh(),
                              torch.nn.Linear(24, 1))
    opt = torch.optim.Adam(net.parameters(), lr=5e-3)
    lossf = PINNLoss(residual_weight=a.weight)
    xs = torch.linspace(0, 1, 64).reshape(-1, 1).requires_grad_()
    x0 = torch.zeros(1, 1, requires_grad=True)
    first = last = 0.0
    for step in range(a.steps):
        u = net(xs)
        du = torch.autograd.grad(u.sum(), xs, create_graph=True)[0]
        d2u = torch.autograd.grad(du.sum(), xs, create_graph=True)[0]
        u0 = net(x0)
        du0 = torch.autograd.grad(u0.sum(), x0, create_graph=True)[0]
        pred = torch.cat([u0, du0], 1)
        loss = lossf(pred, torch.tensor([[0.0, math.pi]]), d2u + math.pi ** 2 * u)
        loss = (loss if isinstance(loss, torch.Tensor) else loss.t).reshape(())
        first = float(loss) if step == 0 else first
        last = float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    with torch.no_grad():
        grid = torch.linspace(0, 1, 101).reshape(-1, 1)
        err = float((net(grid) - torch.sin(math.pi * grid)).abs().max())
    print(f"physics-informed network for u'' + pi^2 u = 0, u(0) = 0, u'(0) = pi (seed {a.seed})")
    print(f"  loss {first:.4f} -> {last:.6f} in {a.steps} Adam steps; max |u - sin(pi x)| on [0, 1] = {err:.4f}")
    return 0


def cmd_som(a):
    """``som``: fit a self-organising map to three Gaussian clusters; quantisation and topographic error."""
    import numpy as np
    from . import search
    rng = np.random.default_rng(a.seed)
    centres = np.array([[0.2, 0.2], [0.8, 0.3], [0.5, 0.8]])
    data = np.concatenate([c + 0.05 * rng.standard_normal((60, 2)) for c in centres])
    som = search.SelfOrganizingMap(a.rows, a.cols, 2, seed=a.seed)
    q0 = som.quantization_error(data)
    som.fit(data, epochs=a.epochs, seed=a.seed)
    print(f"self-organising map {a.rows} x {a.cols} on 180 points from 3 clusters (seed {a.seed})")
    print(f"  quantisation error {q0:.4f} -> {som.quantization_error(data):.4f}; topographic error "
          f"{som.topographic_error(data):.3f}")
    return 0


def cmd_certify(a):
    """IBP and CROWN output bounds of a seeded 4->8->3 ReLU MLP over an L-infinity box
    (scirust-cli/src/learning.rs:46-120)."""
    import torch
    from .certify import IbpLinear, IbpMlp, Interval, certified_robust, crown_bounds
    if not (a.eps > 0 and a.eps == a.eps and a.eps != float("inf")):
        sys.stderr.write("usage: scirust certify [--seed N] [--eps E]\nerror: --eps must be a positive number\n")
        return EXIT_USAGE
    g = torch.Generator().manual_seed(a.seed)
    l1 = IbpLinear(torch.randn(4, 8, generator=g) * 0.5, torch.zeros(8))
    l2 = IbpLinear(torch.randn(8, 3, generator=g) * 0.5, torch.zeros(3))
    centre = [0.2, -0.5, 0.7, -0.1]
    box = Interval.around(centre, a.eps)
    mlp = IbpMlp([l1, l2])
    pred = mlp.forward(centre)
    cls = int(pred.argmax())
    ibp, crown = mlp.certify(box), crown_bounds(l1, l2, box)
    print(f"Certified bounds (seed {a.seed}): MLP 4->8->3 (ReLU), input {centre} -> class {cls}, eps = {a.eps}")
    for name, out in (("IBP  ", ibp), ("CROWN", crown)):
        verdict = (f"CERTIFIED: class {cls} cannot change in the box" if certified_robust(out, cls)
                   else "not certified at this eps")
        print(f"  {name} avg width {float(out.width().mean()):.4f}  {verdict}")
        for c in range(3):
            print(f"      y[{c}] in [{float(out.lo[c]):+.4f}, {float(out.hi[c]):+.4f}]")
    return EXIT_OK


def cmd_guard(a):
    """Calibrate the statistical guard on synthetic 3-class probabilities and report coverage and verdicts
    (scirust-cli/src/synergy.rs:90-160)."""
    import torch
    from .certify import StatisticalGuard
    if not (0.0 < a.alpha < 1.0):
        sys.stderr.write("usage: scirust guard [--seed N] [--alpha A]\nerror: --alpha must be in (0, 1)\n")
        return EXIT_USAGE
    g = torch.Generator().manual_seed(a.seed)

    def sample(n):
        y = torch.randint(0, 3, (n,), generator=g)
        lg = torch.rand(n, 3, generator=g) * 2 - 1
        lg[torch.arange(n), y] += 1.5
        return torch.softmax(lg, -1), y
    cp, cy = sample(2000)
    guard = StatisticalGuard.calibrate(cp, cy, a.alpha)
    tp, ty = sample(5000)
    covered = sum(guard.covers(p_, int(t)) for p_, t in zip(tp, ty))
    print(f"Statistical guard (seed {a.seed}): target coverage >= {1 - a.alpha:.2f}, "
          f"empirical {covered / 5000:.4f} on 5000 fresh samples")
    for name, p_ in (("confident", [0.92, 0.05, 0.03]), ("ambiguous", [0.48, 0.46, 0.06]),
                     ("flat", [0.34, 0.33, 0.33])):
        verdict, cls = guard.decide(p_)
        text = {"accept": f"ACCEPT class {cls}", "abstain": "ABSTAIN (ambiguous: flag for review)",
                "reject": "REJECT (out of distribution)"}[verdict]
        print(f"  {name:<10} {p_} -> {text}")
    return EXIT_OK


def cmd_attest(a):
    """Verified inferences chained into an attestation log; a forged output is refused and an altered event changes
    the chain head (scirust-cli/src/synergy.rs:163-230)."""
    import random
    from .io.attest import AttestationLog, P, VModel, attest_and_record
    rng = random.Random(a.seed)
    out, inn, batch = 4, 6, 3
    model = VModel([rng.randrange(P) for _ in range(out * inn)], out, inn)
    log = AttestationLog()
    for _ in range(4):
        x = [rng.randrange(P) for _ in range(inn * batch)]
        attest_and_record(log, model, x, batch, model.infer(x, batch), 2)
    x = [rng.randrange(P) for _ in range(inn * batch)]
    forged = model.infer(x, batch)
    forged[0] = (forged[0] + 1) % P
    rejected = attest_and_record(log, model, x, batch, forged, 2) is None
    heads = []
    for tamper in (False, True):
        alt = AttestationLog()
        for i in range(4):
            xx = [(i * 7 + j) % P for j in range(inn * batch)]
            yy = model.infer(xx, batch)
            if tamper and i == 1:
                yy[0] = (yy[0] + 1) % P
            alt.record(model.commit(), xx, yy)
        heads.append(alt.head.hex())
    print(f"Attestation log (seed {a.seed}): model commitment {model.commit().hex()[:16]}..")
    print(f"  {len(log)} verified inferences chained, head {log.head.hex()[:16]}.., chain valid: {log.verify_chain()}")
    print(f"  forged output refused: {rejected}")
    print(f"  altered event changes the head: {heads[0] != heads[1]}")
    return EXIT_OK if rejected and log.verify_chain() and heads[0] != heads[1] else EXIT_VALIDATION


def _sciagent_reply(a, prompt_text, max_new):
    import torch
    from .generate import SamplingParams
    from .io import checkpoint as CK
    from .models.infer import InferenceEngine
    dev = _device(a.device)
    model, _ = CK.load_sciagent_checkpoint(a.checkpoint, device=dev)
    tok = _load_tokenizer(a.tokenizer) if a.tokenizer else None
    ids = tok.encode(prompt_text) if tok else [b for b in prompt_text.encode()][:model.cfg.max_seq_len]
    ids = [min(i, model.cfg.vocab_size - 1) for i in ids][-(model.cfg.max_seq_len - max_new - 1):]
    if not ids:
        raise ValueError("empty prompt")
    eng = InferenceEngine(model, quant=a.quant, max_batch=1, max_seq=len(ids) + max_new + 1)
    params = SamplingParams(a.temperature, a.top_k, a.top_p, a.repetition_penalty)
    out = eng.generate(torch.tensor([ids]), max_new, params, seed=a.seed)[0].tolist()
    if 0 in out:
        out = out[:out.index(0)]
    return tok.decode(out) if tok else bytes(t % 256 for t in out).decode("utf-8", "replace")


def cmd_sciagent_text(a):
    """`sciagent ask <prompt>`, `chat` (one reply per input line until end of input) and `explain <path>`
    (scirust-cli/src/sciagent.rs:137-260). Without a tokenizer file, text is fed as bytes."""
    if a.action == "ask":
        if not a.prompt:
            sys.stderr.write("usage: scirust sciagent ask --prompt TEXT --checkpoint PATH\n")
            return EXIT_USAGE
        print(_sciagent_reply(a, a.prompt, a.max_new))
        return EXIT_OK
    if a.action == "explain":
        from pathlib import Path
        if not a.path:
            sys.stderr.write("usage: scirust sciagent explain --path FILE [--lines N-M] --checkpoint PATH\n")
            return EXIT_USAGE
        content = Path(a.path).read_text(errors="replace")
        if a.lines:
            lo, _, hi = a.lines.partition("-")
            start = int(lo or 1)
            end = int(hi) if hi else start + 30
            excerpt = "\n".join(content.splitlines()[max(start - 1, 0):end])
        else:
            excerpt = content[:2000]
        print(_sciagent_reply(a, "Explain the following code:\n" + excerpt + "\nExplanation:", a.max_new))
        return EXIT_OK
    history = ""
    print("SCIAGENT chat (end of input to exit)")
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        history += line + "\n"
        reply = _sciagent_reply(a, history, a.max_new)
        history += reply + "\n"
        print(reply)
    return EXIT_OK


def build_parser():
    p = _Parser(prog="scirust", description="scirust_b200 command line")
    sub = p.add_subparsers(dest="cmd")
    sub.add_parser("version").set_defaults(fn=cmd_version)
    sub.add_parser("info").set_defaults(fn=cmd_info)
    q = sub.add_parser("quickstart")
    q.add_argument("--epochs", type=int, default=100)
    q.add_argument("--seed", type=int, default=42)
    q.add_argument("--fma", action="store_true")
    q.set_defaults(fn=cmd_quickstart)
    b = sub.add_parser("bpe")
    b.add_argument("action", choices=["train", "encode", "decode"])
    b.add_argument("--inputs", nargs="*", default=[])
    b.add_argument("--vocab-size", type=int, default=8192)
    b.add_argument("--min-frequency", type=int, default=2)
    b.add_argument("--out", default="bpe.json")
    b.add_argument("--tokenizer", default="bpe.json")
    b.add_argument("--text", default="")
    b.set_defaults(fn=cmd_bpe)
    t = sub.add_parser("train")
    t.add_argument("--model", default="debug")
    t.add_argument("--data", nargs="*", default=[])
    t.add_argument("--steps", type=int, default=10)
    t.add_argument("--batch-size", type=int, default=2)
    t.add_argument("--seq-len", type=int, default=128)
    t.add_argument("--lr", type=float, default=3e-4)
    t.add_argument("--min-lr", type=float, default=3e-5)
    t.add_argument("--warmup-steps", type=int, default=0)
    t.add_argument("--total-steps", type=int, default=0)
    t.add_argument("--max-grad-norm", type=float, default=1.0)
    t.add_argument("--weight-decay", type=float, default=0.1)
    t.add_argument("--val-frac", type=float, default=0.0)
    t.add_argument("--seed", type=int, default=0)
    t.add_argument("--checkpoint-dir", default="")
    t.add_argument("--save-interval", type=int, default=0)
    t.add_argument("--keep-last", type=int, default=0)
    t.add_argument("--log-interval", type=int, default=10)
    t.add_argument("--resume", action="store_true")
    t.add_argument("--device", default="auto")
    t.set_defaults(fn=cmd_train)

    def gen_args(sp):
        sp.add_argument("--checkpoint", required=True)
        sp.add_argument("--tokenizer", default="")
        sp.add_argument("--prompt", default="")
        sp.add_argument("--max-new", type=int, default=32)
        sp.add_argument("--temperature", type=float, default=0.0)
        sp.add_argument("--top-k", type=int, default=0)
        sp.add_argument("--top-p", type=float, default=1.0)
        sp.add_argument("--repetition-penalty", type=float, default=1.0)
        sp.add_argument("--seed", type=int, default=0)
        sp.add_argument("--quant", default=None, choices=[None, "int8"])
        sp.add_argument("--device", default="auto")
    i = sub.add_parser("infer")
    gen_args(i)
    i.set_defaults(fn=cmd_infer)
    s = sub.add_parser("sciagent")
    s.add_argument("action", choices=["info", "generate", "quantize", "attest", "ask", "chat", "explain"])
    gen_args(s)
    s.add_argument("--out", default="model.int4.bin")
    s.add_argument("--group", type=int, default=32)
    s.add_argument("--path", default="")
    s.add_argument("--lines", default="")
    s.set_defaults(fn=lambda a: cmd_sciagent_text(a) if a.action in ("ask", "chat", "explain") else cmd_sciagent(a))
    lm = sub.add_parser("lm")
    lm.add_argument("tokens", nargs="?", default="1,2,3,4,2,5")
    lm.add_argument("--seed", type=int, default=123)
    lm.add_argument("--steps", type=int, default=200)
    lm.add_argument("--lr", type=float, default=0.05)
    lm.add_argument("--opt", default="adam")
    lm.set_defaults(fn=cmd_lm)
    for name in _SEQ_LAYERS:
        sq = sub.add_parser(name)
        sq.add_argument("--seed", type=int, default=7)
        sq.add_argument("--steps", type=int, default=150)
        sq.set_defaults(fn=cmd_seq_layer)
    tt = sub.add_parser("tt")
    tt.add_argument("--seed", type=int, default=0)
    tt.add_argument("--rank", type=int, default=4)
    tt.add_argument("--steps", type=int, default=200)
    tt.set_defaults(fn=cmd_tt)
    for name in ("evo", "cmaes"):
        sr = sub.add_parser(name)
        sr.add_argument("--objective", default="rosenbrock", choices=["sphere", "rosenbrock", "rastrigin"])
        sr.add_argument("--dim", type=int, default=5)
        sr.add_argument("--generations", type=int, default=300)
        sr.add_argument("--seed", type=int, default=0)
        sr.set_defaults(fn=cmd_search)
    pn = sub.add_parser("pinn")
    pn.add_argument("--seed", type=int, default=0)
    pn.add_argument("--steps", type=int, default=1500)
    pn.add_argument("--weight", type=float, default=0.1)
    pn.set_defaults(fn=cmd_pinn)
    so = sub.add_parser("som")
    so.add_argument("--rows", type=int, default=6)
    so.add_argument("--cols", type=int, default=6)
    so.add_argument("--epochs", type=int, default=20)
    so.add_argument("--seed", type=int, default=0)
    so.set_defaults(fn=cmd_som)
    ce = sub.add_parser("certify")
    ce.add_argument("--seed", type=int, default=1)
    ce.add_argument("--eps", type=float, default=0.05)
    ce.set_defaults(fn=cmd_certify)
    gd = sub.add_parser("guard")
    gd.add_argument("--seed", type=int, default=1)
    gd.add_argument("--alpha", type=float, default=0.1)
    gd.set_defaults(fn=cmd_guard)
    at = sub.add_parser("attest")
    at.add_argument("--seed", type=int, default=1)
    at.set_defaults(fn=cmd_attest)
    for name in ("gptq", "awq", "bitnet", "int4"):
        qz = sub.add_parser(name)
        qz.add_argument("--weights", default="")
        qz.add_argument("--tensor", default="")
        qz.add_argument("--rows", type=int, default=128)
        qz.add_argument("--cols", type=int, default=64)
        qz.add_argument("--bits", type=int, default=4)
        qz.add_argument("--group", type=int, default=32)
        qz.add_argument("--seed", type=int, default=0)
        qz.set_defaults(fn=cmd_quantizer)
    kc = sub.add_parser("kvcache")
    kc.add_argument("--tokens", type=int, default=64)
    kc.add_argument("--head-dim", type=int, default=32)
    kc.add_argument("--seed", type=int, default=0)
    kc.set_defaults(fn=cmd_kvcache)
    ox = sub.add_parser("onnx")
    ox.add_argument("action", choices=["export", "inspect"])
    ox.add_argument("--file", required=True)
    ox.add_argument("--name", default="model")
    ox.add_argument("--layers", type=int, nargs="*", default=[4, 8, 2])
    ox.add_argument("--seed", type=int, default=0)
    ox.set_defaults(fn=cmd_onnx)
    pl = sub.add_parser("plan")
    pl.add_argument("--model", default="gqa_12l")
    pl.add_argument("--batch", type=int, default=8)
    pl.add_argument("--seq", type=int, default=2048)
    pl.add_argument("--tp", type=int, default=1)
    pl.set_defaults(fn=cmd_plan)
    for name in ("calibrate", "conformal"):
        cb = sub.add_parser(name)
        cb.add_argument("--data", required=True)
        cb.add_argument("--alpha", type=float, default=0.1)
        cb.set_defaults(fn=cmd_calibrate)
    v = sub.add_parser("verify")
    v.add_argument("action", choices=["emit", "verify"])
    v.add_argument("--artifact", required=True)
    v.add_argument("--bundle", default="")
    v.add_argument("--batch", type=int, default=1)
    v.add_argument("--seeds", type=int, nargs="*", default=[1, 2, 3])
    v.add_argument("--out", default="")
    v.set_defaults(fn=cmd_verify)
    from . import cli_tools
    cli_tools.register(sub)
    from . import cli_math
    cli_math.register(sub)
    return p


def run(argv) -> int:
    """Entry point returning the exit code (never raises for user errors)."""
    p = build_parser()
    try:
        a = p.parse_args(list(argv))
    except SystemExit as e:
        return int(e.code) if isinstance(e.code, int) else EXIT_USAGE
    if not getattr(a, "fn", None):
        p.print_help()
        return EXIT_OK
    try:
        return int(a.fn(a))
    except KeyboardInterrupt:
        return EXIT_CANCELLED
    except (FileNotFoundError, PermissionError, IsADirectoryError) as e:
        sys.stderr.write(f"error: {e}\n")
        return EXIT_USAGE
    except (ValueError, KeyError) as e:
        sys.stderr.write(f"error: {e}\n")
        return EXIT_VALIDATION
    except Exception as e:  # noqa: BLE001
        sys.stderr.write(f"internal error: {type(e).__name__}: {e}\n")
        return EXIT_INTERNAL


def main():
    sys.exit(run(sys.argv[1:]))


if __name__ == "__main__":
    main()
