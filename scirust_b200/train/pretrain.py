"""The pretraining loop: windows of a token stream, warm-up + cosine schedule, deferred telemetry, held-out evaluation,
checkpoints by step count or wall-clock, best-model tracking, pruning, and EXACT resume.

* Window order: the train / validation split is a pure function of (stream length, sequence length, fraction); the order
  of epoch ``e`` is a pure function of (split, ``e``): a 64-bit LCG Fisher-Yates shuffle seeded by a constant xor ``e``.
  A resumed run rebuilds (epoch, cursor) from ``start_step * batch`` windows already consumed, so an interrupted and an
  uninterrupted run see the same next windows; together with the optimizer sidecar the resumed step is bit-identical.
* Telemetry: losses stay on the device; they are read back every ``telemetry_interval`` steps or when a log line, an
  evaluation or a checkpoint needs them, so the steady state has no host synchronisation per step.
* Input pipeline: batches are assembled in pinned host buffers (two in flight) and copied on a side stream while the
  previous step computes.
* ``PretrainConfig.from_env`` reads the reference's ``SCIAGENT_*`` variables (CONFIG / TEXT / SHARDS / CKPT / STEPS /
  TOTAL_STEPS / SEQ / BATCH / LR / WARMUP / CLIP / EPS / SAVE / SAVE_HOURS / KEEP / VAL_FRAC / SHUFFLE / TELEMETRY /
  MAX_TOKENS / REQUIRE_FRESH / PREFLIGHT_ONLY / EXPECT_*), ``run_from_env`` is the harness around them (fresh-directory
  gate, corpus identity gates, preflight line).
Reference counterparts: scirust-sciagent/src/cuda_model.rs:1960-2225 (``CudaTrainer::pretrain``), :2298-2350 (shuffle,
pruning), :2355-2444 (``CudaPretrainConfig``); scirust-sciagent/examples/cuda_pretrain.rs (environment harness).
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..data.corpus import distributed_window_split
from ..io import checkpoint as CK
from .schedule import WarmupCosineSchedule

WINDOW_SPLIT_VERSION = 1
_SHUFFLE_KEY = 0x5343494147454E54
_M64 = (1 << 64) - 1


def shuffle_windows(order: list, seed: int) -> None:
    """In-place Fisher-Yates driven by a 64-bit LCG (multiplier 6364136223846793005, increment 1442695040888963407)."""
    state = (seed * 6364136223846793005 + 1442695040888963407) & _M64
    for i in range(len(order) - 1, 0, -1):
        state = (state * 6364136223846793005 + 1442695040888963407) & _M64
        j = (state >> 33) % (i + 1)
        order[i], order[j] = order[j], order[i]


def epoch_order(base_order, epoch: int, shuffle: bool) -> list:
    order = list(base_order)
    if shuffle:
        shuffle_windows(order, _SHUFFLE_KEY ^ epoch)
    return order


def corpus_fnv64(tokens) -> int:
    """FNV-1a over the little-endian u32 bytes of the whole token stream (corpus identity gate)."""
    h = 0xCBF29CE484222325
    data = np.asarray(tokens, dtype="<u4").tobytes()
    for i in range(0, len(data), 1 << 20):
        for b in data[i:i + (1 << 20)]:
            h = ((h ^ b) * 0x100000001B3) & _M64
    return h


@dataclass
class PretrainConfig:
    base_lr: float = 3e-4
    min_lr: float = 3e-5
    warmup_steps: int = 0
    total_steps: int = 300
    start_step: int = 0
    betas: tuple = (0.9, 0.95)
    adam_eps: float = 1e-8
    weight_decay: float = 0.1
    seq_len: int = 128
    batch_size: int = 1
    telemetry_interval: int = 25
    log_interval: int = 25
    save_interval: int = 0
    save_interval_seconds: int = 0
    checkpoint_dir: str = "checkpoints/cuda"
    max_grad_norm: float = 1.0
    val_frac: float = 0.0
    eval_interval: int = 0
    eval_windows: int = 16
    keep_last: int = 0
    corpus_tokens: int = 0
    corpus_hash: int = 0
    shuffle: bool = True

    @staticmethod
    def from_env(env=None) -> "PretrainConfig":
        e = os.environ if env is None else env
        c = PretrainConfig()
        geti = lambda k, d: int(e[k]) if e.get(k) not in (None, "") else d
        getf = lambda k, d: float(e[k]) if e.get(k) not in (None, "") else d
        steps = geti("SCIAGENT_STEPS", c.total_steps)
        c.total_steps = geti("SCIAGENT_TOTAL_STEPS", steps)
        c.seq_len, c.batch_size = geti("SCIAGENT_SEQ", c.seq_len), geti("SCIAGENT_BATCH", c.batch_size)
        c.base_lr = getf("SCIAGENT_LR", c.base_lr)
        c.min_lr = c.base_lr * 0.1
        c.warmup_steps = geti("SCIAGENT_WARMUP", max(c.total_steps // 20, 1))
        c.max_grad_norm, c.adam_eps = getf("SCIAGENT_CLIP", c.max_grad_norm), getf("SCIAGENT_EPS", c.adam_eps)
        c.telemetry_interval = geti("SCIAGENT_TELEMETRY", c.telemetry_interval)
        c.log_interval = c.telemetry_interval
        c.checkpoint_dir = e.get("SCIAGENT_CKPT") or c.checkpoint_dir
        if e.get("SCIAGENT_SAVE") not in (None, ""):
            c.save_interval = int(e["SCIAGENT_SAVE"])                    # an explicit step cadence
        else:
            c.save_interval_seconds = int(getf("SCIAGENT_SAVE_HOURS", 6.0) * 3600)
        c.keep_last = geti("SCIAGENT_KEEP", 3)
        c.val_frac = getf("SCIAGENT_VAL_FRAC", 0.0)
        if c.val_frac > 0:
            c.eval_interval = max(c.total_steps // 10, 1)
        c.shuffle = e.get("SCIAGENT_SHUFFLE", "1") != "0"
        return c


class PretrainError(RuntimeError):
    pass


class _Uploader:
    """Two pinned staging buffers; ``put`` fills one and starts its copy to the device on a side stream."""

    def __init__(self, batch, width, device):
        from ..utils.pinned import DoubleBufferedUploader
        self.up = DoubleBufferedUploader(batch * width, torch.int64, device)

    def put(self, host):
        return self.up.submit(host)

    def get(self, ticket):
        return self.up.take(ticket)


def _window_batch(tokens: torch.Tensor, starts, s: int) -> torch.Tensor:
    return torch.stack([tokens[a:a + s + 1] for a in starts])


@torch.no_grad()
def evaluate_windows(model, tokens: torch.Tensor, val_windows, s: int, batch: int, max_windows: int) -> float:
    """Mean next-token loss over (at most ``max_windows``) held-out windows, in their fixed order."""
    use = list(val_windows[:max_windows]) if max_windows else list(val_windows)
    if not use:
        return math.nan
    dev = model.flat.device
    total, rows = 0.0, 0
    for i in range(0, len(use), batch):
        w = _window_batch(tokens, use[i:i + batch], s).to(dev)
        total += float(model(w[:, :-1].contiguous(), w[:, 1:].contiguous())) * w.shape[0]
        rows += w.shape[0]
    return total / rows


def pretrain(trainer, tokens, cfg: PretrainConfig, log=print, clock=time.monotonic) -> list:
    """Train ``trainer.model`` on the token stream; returns the per-step losses (in step order)."""
    model = trainer.model
    tok = torch.as_tensor(np.asarray(tokens, dtype=np.int64))
    s, batch = cfg.seq_len, max(cfg.batch_size, 1)
    telemetry = max(cfg.telemetry_interval, 1)
    losses: list = []
    if tok.numel() <= s:
        log(f"pretrain: token stream ({tok.numel()}) shorter than a single window ({s + 1}); nothing to do")
        return losses
    base_order, val_windows = distributed_window_split(tok.numel(), s, cfg.val_frac)
    n_windows = len(base_order)
    if n_windows == 0:
        return losses
    if val_windows:
        log(f"held-out validation: {len(val_windows)} distributed windows ({cfg.val_frac * 100:.1f}% target, split-v{WINDOW_SPLIT_VERSION})")
    trainer.schedule = WarmupCosineSchedule(cfg.base_lr, cfg.min_lr, cfg.warmup_steps, cfg.total_steps)
    tc = trainer.cfg
    tc.beta1, tc.beta2, tc.eps, tc.weight_decay, tc.max_grad_norm = cfg.betas[0], cfg.betas[1], cfg.adam_eps, cfg.weight_decay, cfg.max_grad_norm
    if trainer.step != cfg.start_step:
        raise PretrainError(f"trainer is at step {trainer.step}, the run starts at {cfg.start_step}: load the optimizer state first")
    step = cfg.start_step
    consumed = cfg.start_step * batch
    epoch, wi = consumed // n_windows, consumed % n_windows
    order = epoch_order(base_order, epoch, cfg.shuffle)
    sel = Path(cfg.checkpoint_dir) / "best" / "selection.json"
    best_val, best_step = math.inf, None
    if sel.exists():
        import json
        prev = json.loads(sel.read_text())
        best_val, best_step = float(prev.get("metric", math.inf)), prev.get("step")
        log(f"restored best validation: {best_val:.4f} @ step {best_step}")
    t0 = clock()
    last_ckpt_at, last_ckpt_step = t0, None
    checkpointing = cfg.save_interval > 0 or cfg.save_interval_seconds > 0
    pending: list = []
    last_loss = math.nan
    up = _Uploader(batch, s + 1, model.flat.device)

    def next_starts():
        nonlocal epoch, wi, order
        out = []
        for _ in range(batch):
            if wi >= len(order):
                epoch += 1
                order = epoch_order(base_order, epoch, cfg.shuffle)
                wi = 0
            out.append(order[wi])
            wi += 1
        return out

    def save(at_step, lr):
        nonlocal last_ckpt_at, last_ckpt_step
        trainer.check_status()
        CK.save_sciagent_checkpoint(model, Path(cfg.checkpoint_dir) / f"step_{at_step}", at_step, last_loss, lr, trainer=trainer,
                                    extra_opt={"corpus_tokens": cfg.corpus_tokens, "corpus_hash": cfg.corpus_hash, "seq_len": s,
                                               "batch_size": batch, "shuffle": cfg.shuffle, "window_split_version": WINDOW_SPLIT_VERSION})
        if cfg.keep_last:
            CK.prune_checkpoints(cfg.checkpoint_dir, cfg.keep_last)
        last_ckpt_at, last_ckpt_step = clock(), at_step

    ticket = up.put(_window_batch(tok, next_starts(), s)) if step < cfg.total_steps else None
    while step < cfg.total_steps:
        dev_batch = up.get(ticket)
        lr = trainer.schedule.lr_at(step)
        pending.append(trainer.train_step(dev_batch))
        step += 1
        if step < cfg.total_steps:
            ticket = up.put(_window_batch(tok, next_starts(), s))          # staged while this step's kernels run
        need_log = cfg.log_interval > 0 and step % cfg.log_interval == 0
        need_eval = cfg.eval_interval > 0 and bool(val_windows) and step % cfg.eval_interval == 0
        need_save = (cfg.save_interval > 0 and step % cfg.save_interval == 0) or \
                    (cfg.save_interval_seconds > 0 and clock() - last_ckpt_at >= cfg.save_interval_seconds)
        if len(pending) >= telemetry or need_log or need_eval or need_save or step == cfg.total_steps:
            for l in pending:
                last_loss = float(l)
                losses.append(last_loss)
            pending.clear()
            if last_loss != last_loss:
                raise PretrainError(f"loss is NaN at step {step}")
        if need_log:
            tps = (step - cfg.start_step) * s * batch / max(clock() - t0, 1e-9)
            log(f"[step {step:>6}] B{batch}xT{s} loss {last_loss:>9.4f} | lr {lr:.3e} | gnorm {trainer.grad_norm():>7.2f} | {tps:>8.0f} tok/s")
        if need_eval:
            v = evaluate_windows(model, tok, val_windows, s, batch, cfg.eval_windows)
            gap = v - last_loss
            log(f"[step {step:>6}] validation loss {v:.4f} (train {last_loss:.4f}, gap {gap:+.4f})")
            if v < best_val:
                best_val, best_step = v, step
                CK.save_best(model, cfg.checkpoint_dir, step, v)
                log(f"[step {step:>6}] new best validation {v:.4f}")
        if need_save and checkpointing:
            save(step, lr)
    if checkpointing and last_ckpt_step != step and step > cfg.start_step:
        save(step, trainer.schedule.lr_at(max(step - 1, 0)))
    return losses


# ------------------------------------------------------------------ environment harness
def _ingest_bytes(path) -> np.ndarray:
    p = Path(path)
    files = [p] if p.is_file() else sorted(q for q in p.rglob("*") if q.is_file())
    buf = bytearray()
    for f in files:
        try:
            buf.extend(f.read_bytes())
        except OSError:
            continue
        buf.append(0xFF)
    return np.frombuffer(bytes(buf), dtype=np.uint8).astype(np.int64)


def run_from_env(env=None, log=print, device=None) -> int:
    """The ``SCIAGENT_*`` harness. Returns a process exit code (0 ok, 2 usage / IO, 3 validation)."""
    from ..data.corpus import ShardLoader
    from ..models import GQADecoder, SciAgentConfig
    from .trainer import Trainer, TrainerConfig
    e = dict(os.environ if env is None else env)
    cfg = PretrainConfig.from_env(e)
    fresh = e.get("SCIAGENT_REQUIRE_FRESH") == "1"
    ckpt = Path(cfg.checkpoint_dir)
    if fresh:
        if ckpt.exists() and any(ckpt.iterdir()):
            log(f"error: SCIAGENT_REQUIRE_FRESH=1 but {ckpt} is not empty")
            return 3
        if e.get("SCIAGENT_MAX_TOKENS") or e.get("SCIAGENT_ALLOW_NONEXACT_RESUME") == "1":
            log("error: SCIAGENT_REQUIRE_FRESH=1 refuses SCIAGENT_MAX_TOKENS and non-exact resume overrides")
            return 3
    preset = e.get("SCIAGENT_CONFIG")
    if e.get("SCIAGENT_SHARDS"):
        loader = ShardLoader()
        loader.load_dir(e["SCIAGENT_SHARDS"])
        tokens, n_shards = loader.tokens().astype(np.int64), len(list(Path(e["SCIAGENT_SHARDS"]).glob("*.bin")))
        preset = preset or "small"
    elif e.get("SCIAGENT_TEXT"):
        tokens, n_shards = _ingest_bytes(e["SCIAGENT_TEXT"]), 0
        preset = preset or "byte"
    else:
        g = np.random.default_rng(0)
        tokens, n_shards = g.integers(1, 256, size=max(4 * cfg.seq_len * cfg.batch_size, 4096)).astype(np.int64), 0
        preset = preset or "byte"
    if tokens.size == 0:
        log("error: the corpus is empty")
        return 2
    if e.get("SCIAGENT_MAX_TOKENS"):
        cap = int(e["SCIAGENT_MAX_TOKENS"])
        if cap < tokens.size:
            log(f"corpus capped to its first {cap} of {tokens.size} tokens (a prefix, not a sample)")
            tokens = tokens[:cap]
    cfg.corpus_tokens, cfg.corpus_hash = int(tokens.size), corpus_fnv64(tokens)
    for key, have in (("SCIAGENT_EXPECT_SHARDS", n_shards), ("SCIAGENT_EXPECT_CORPUS_TOKENS", cfg.corpus_tokens),
                      ("SCIAGENT_EXPECT_CORPUS_FNV64", cfg.corpus_hash)):
        if e.get(key):
            want = int(e[key], 0)
            if want != have:
                log(f"error: {key} = {want}, the corpus has {have}")
                return 3
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    last = CK.latest_checkpoint(ckpt) if ckpt.exists() else None
    if last is not None:
        model, meta = CK.load_sciagent_checkpoint(last, device=device)
        mcfg = model.cfg
        cfg.start_step = int(meta["step"])
    else:
        mcfg = SciAgentConfig.preset(preset)
        model = GQADecoder(mcfg, device=device, seed=0)
    if int(tokens.max()) >= mcfg.vocab_size:
        log(f"error: token id {int(tokens.max())} >= vocab_size {mcfg.vocab_size}: shards tokenised for another vocabulary")
        return 3
    trainer = Trainer(model, TrainerConfig(lr=cfg.base_lr, min_lr=cfg.min_lr, warmup_steps=cfg.warmup_steps, total_steps=cfg.total_steps,
                                           max_grad_norm=cfg.max_grad_norm, eps=cfg.adam_eps))
    if last is not None:
        CK.load_optimizer_state(model, trainer, last)
        log(f"resumed from {last} at step {cfg.start_step}")
    if e.get("SCIAGENT_PREFLIGHT_ONLY") == "1":
        log(f"SCIAGENT_PREFLIGHT_OK config={preset} device={device} corpus_tokens={cfg.corpus_tokens} "
            f"corpus_fnv64={cfg.corpus_hash:#018x} start_step={cfg.start_step} total_steps={cfg.total_steps}")
        return 0
    losses = pretrain(trainer, tokens, cfg, log=log)
    if losses:
        log(f"done: {len(losses)} steps, first loss {losses[0]:.4f}, last loss {losses[-1]:.4f}")
    return 0
